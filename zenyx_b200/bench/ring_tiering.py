"""KV tiering under the ring: every rank's K/V shards of all layers live in a
``BeladyKVCacheTieringManager`` (capped HBM budget, the rest in pinned host DRAM or a file), and the ring
attention kernels read them from the peer-visible slots, forward over the layers and backward in reverse.

    python -m torch.distributed.run --nproc-per-node 8 -m zenyx_b200.bench.ring_tiering --hbm-gb 2
    python -m zenyx_b200.bench.ring_tiering --seq-len 131072 --hbm-gb 0.5          # one GPU, ring degree 1

Per layer and phase a rank (1) acquires the tier blocks of its shard from the manager, in the order of the
manager's plan, and copies them into its K/V slot (device-to-device; a block that is not resident comes from
the host first, prefetched under the previous layers' attention when the plan foresaw it), (2) tells the
manager about the R - 1 further reads of the same blocks by its peers, which are hits and keep the plan's
cursor in step, (3) runs the ring attention of the layer, whose kernels pull the peers' slots over NVLink.
A slot is reused two layers later, like in the training engine, so one barrier per layer call orders
everything. One JSON line from rank 0: step time (CUDA events, maximum over ranks), exposed stalls and bytes
per tier of the slowest rank's manager, hit rate, attention TFLOP/s.

The reference describes this component in its README only (README.md:150-154, "516 GB of KV through 16 GB of
HBM"); its stock ``KVTierManager`` (zenyx/streaming/kv_tiering.py:36-66) places blocks by capacity and is not
connected to any attention.
"""
from __future__ import annotations

import argparse
import json
import math

import torch
import torch.distributed as dist


def acquire_order(ring_degree: int, layers: int, blocks_per_layer: int):
    """(layer, block) of every ``acquire`` one step of this benchmark makes, in order: forward over the layers, then
    backward in reverse; per layer the rank's own pass over its blocks followed by one pass per peer. This is the
    order of ``RingAttentionAccessSequence.block_ids(rank)``, which is what keeps the manager on its plan."""
    out = []
    for order in (range(layers), reversed(range(layers))):
        for layer in order:
            for _ in range(ring_degree):
                out.extend((layer, b) for b in range(blocks_per_layer))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq-len", type=int, default=1 << 20)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--block-tokens", type=int, default=4096)
    ap.add_argument("--hbm-gb", type=float, default=16.0, help="HBM budget of the KV tier per rank")
    ap.add_argument("--dram-gb", type=float, default=None)
    ap.add_argument("--nvme-path", default=None)
    ap.add_argument("--steps", type=int, default=2)
    args = ap.parse_args(argv)
    from zenyx_b200.ops import _ext
    from zenyx_b200.ops.attention import MaskSpec, RingContext, ring_attn_backward, ring_attn_forward
    from zenyx_b200.parallel.communication import init_distributed_from_env
    from zenyx_b200.train.belayd_kv_cache_tiering import BeladyKVCacheTieringManager

    ctx = init_distributed_from_env()
    R, r, dev = ctx.world_size, ctx.rank, ctx.device
    B, S, Hq, Hkv, D, L, bt = 1, args.seq_len, 32, 8, 128, args.layers, args.block_tokens
    Sl = S // R
    assert S % (R * bt) == 0, "the local shard must be a whole number of tier blocks"
    nb = Sl // bt
    scale = 1.0 / math.sqrt(D)
    mgr = BeladyKVCacheTieringManager(num_devices=R, context_length=S, num_layers=L, num_kv_heads=Hkv, head_dim=D,
                                      tier_block_tokens=bt, hbm_budget_bytes=int(args.hbm_gb * (1 << 30)),
                                      dram_budget_bytes=None if args.dram_gb is None else int(args.dram_gb * (1 << 30)),
                                      nvme_path=args.nvme_path, simulate=False, rank=r)
    assert mgr.blocks_per_layer == nb, (mgr.blocks_per_layer, nb)
    plan = mgr.plan()
    g = torch.Generator(device=dev).manual_seed(100 + r)
    for layer in range(L):
        for b in range(nb):
            mgr.register(layer, b, torch.randn(2, bt, Hkv, D, device=dev, generator=g).bfloat16())
    q = torch.randn(B, Sl, Hq, D, device=dev, generator=g).bfloat16()
    do = torch.randn(B, Sl, Hq, D, device=dev, generator=g).bfloat16()
    peer = None
    if R > 1:
        from zenyx_b200.parallel.peer import RingBuffers

        peer = RingBuffers((B, Sl, Hkv, D), group=None)
        slots = [peer.kv_views(r, s) for s in (0, 1)]
    else:
        slots = [(torch.empty(B, Sl, Hkv, D, device=dev, dtype=torch.bfloat16),
                  torch.empty(B, Sl, Hkv, D, device=dev, dtype=torch.bfloat16)) for _ in (0, 1)]
    ring = RingContext(rank=r, degree=R, seq_len=S, peer=peer, mask=MaskSpec(True, 0, 0))

    def stage(layer: int):
        """This rank's K/V of `layer` into slot layer % 2, block by block through the manager."""
        ks, vs = slots[layer % 2]
        for b in range(nb):
            blk = mgr.acquire(layer, b).view(2, bt, Hkv, D)
            ks[0, b * bt:(b + 1) * bt].copy_(blk[0])
            vs[0, b * bt:(b + 1) * bt].copy_(blk[1])
        for _ in range(1, R):          # the peers' pulls of the same blocks, in the plan's order: hits
            for b in range(nb):
                mgr.acquire(layer, b)
        return ks, vs

    def step():
        mgr.step_begin()
        kept = []
        for layer in range(L):
            ks, vs = stage(layer)
            kept.append(ring_attn_forward(ring, q, ks, vs, scale, layer % 2))
        for layer in reversed(range(L)):
            ks, vs = stage(layer)
            o, lse = kept[layer]
            ring_attn_backward(ring, q, ks, vs, o, do, lse, scale, layer % 2)
        mgr.step_end()

    def sync():
        if R > 1:
            dist.barrier()
        torch.cuda.synchronize()

    times = []
    for _ in range(args.steps):
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        sync()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if R > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t.item()))
    _ext.check_status()
    st = mgr.stats()
    # the rank with the longest exposed stall reports its manager's counters
    stall = torch.tensor([st.exposed_stall_ms, float(r)], device=dev, dtype=torch.float64)
    if R > 1:
        allst = [torch.zeros_like(stall) for _ in range(R)]
        dist.all_gather(allst, stall)
        worst = int(max(allst, key=lambda x: float(x[0]))[1].item())
    else:
        worst = 0
    ms = min(times)
    flops = L * 3.5 * (4.0 * S * S * D * Hq * 0.5)
    if r == worst:
        print(json.dumps({
            "metric": "ring attention over tiered KV, fwd+bwd step time", "value": round(ms, 2), "unit": "ms",
            "higher_is_better": False, "step_ms_all": [round(t, 2) for t in times], "ring_degree": R, "seq_len": S,
            "layers": L, "block_tokens": bt, "share_kv_bytes": mgr.total_kv_bytes(),
            "hbm_budget_bytes": mgr.hbm_budget_bytes, "accesses_per_step": len(plan.ids),
            "plan": {"hits": plan.hits, "misses": plan.misses, "hit_rate": round(plan.hit_rate, 4),
                     "lru_misses": mgr.lru_baseline()["misses"], "bytes_loaded": plan.bytes_loaded},
            "measured_on_rank": r,
            "measured": {"hits": st.hits, "misses": st.misses, "prefetched": st.prefetched, "bytes_h2d": st.bytes_h2d,
                         "bytes_d2h": st.bytes_d2h, "bytes_nvme_read": st.bytes_nvme_read,
                         "bytes_nvme_write": st.bytes_nvme_write,
                         "exposed_stall_ms_total": round(st.exposed_stall_ms, 2), "peak_hbm_bytes": st.peak_hbm_bytes},
            "attention_tflops_whole_job": round(flops / ms / 1e9, 1), "steps": args.steps,
            "timing": "CUDA events around one forward + backward pass over the layers, max over ranks, best step",
        }), flush=True)
    mgr.close()
    if peer is not None:
        peer.close()
    if R > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
