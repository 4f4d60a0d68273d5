"""KV tiering stress: one rank's share of a long-context ring, its KV blocks spilling from a capped HBM
budget to pinned host DRAM (and a file, when ``--nvme-path`` is given), residency driven by the
Belady-optimal plan computed from the ring schedule.

    python -m zenyx_b200.bench.kv_tiering                      # 1M tokens, 8 layers, ring of 8, rank 0's share
    python -m zenyx_b200.bench.kv_tiering --hbm-gb 1           # force spilling (the share is 4.3 GB)

Each access of the plan (every reader of the ring touching one of this rank's blocks, forward order)
acquires the block through ``BeladyKVCacheTieringManager.acquire`` and runs the flash-attention
forward kernel of ``--q-tokens`` queries against it, so host-to-device copies overlap real tensor-core
work. One JSON line: step time (CUDA events), exposed stall (host-measured waits on copies that had
not landed), bytes per tier, hit rate, and the miss count an LRU policy takes on the same trace.
The reference only describes this component (README.md:150-154); its stock tier manager is
``KVTierManager`` (zenyx/streaming/kv_tiering.py:36-66), a capacity-ordered placement without a schedule.
"""
from __future__ import annotations

import argparse
import json
import math

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--context", type=int, default=1 << 20)
    ap.add_argument("--ring", type=int, default=8)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--block-tokens", type=int, default=4096)
    ap.add_argument("--hbm-gb", type=float, default=16.0)
    ap.add_argument("--q-tokens", type=int, default=8192)
    ap.add_argument("--nvme-path", default=None)
    ap.add_argument("--dram-gb", type=float, default=None)
    ap.add_argument("--steps", type=int, default=2)
    args = ap.parse_args(argv)
    from zenyx_b200.ops import _ext
    from zenyx_b200.train.belayd_kv_cache_tiering import BeladyKVCacheTieringManager

    C = _ext.C()
    Hq, Hkv, D = 32, 8, 128
    mgr = BeladyKVCacheTieringManager(num_devices=args.ring, context_length=args.context, num_layers=args.layers,
                                      num_kv_heads=Hkv, head_dim=D, tier_block_tokens=args.block_tokens,
                                      hbm_budget_bytes=int(args.hbm_gb * (1 << 30)),
                                      dram_budget_bytes=None if args.dram_gb is None else int(args.dram_gb * (1 << 30)),
                                      nvme_path=args.nvme_path, simulate=False, rank=0)
    plan = mgr.plan()
    bt = args.block_tokens
    gen = torch.Generator(device="cuda").manual_seed(0)
    for layer in range(args.layers):
        for b in range(mgr.blocks_per_layer):
            kv = torch.randn(2, bt, Hkv, D, device="cuda", generator=gen).bfloat16()
            mgr.register(layer, b, kv)
    torch.cuda.synchronize()
    q = torch.randn(1, args.q_tokens, Hq, D, device="cuda", generator=gen).bfloat16()
    o = torch.empty_like(q)
    lse = torch.empty(1, Hq, args.q_tokens, device="cuda", dtype=torch.float32)
    scale = 1.0 / math.sqrt(D)
    n_acc = len(plan.ids)
    times = []
    for _ in range(args.steps):
        mgr.step_begin()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i, bid in enumerate(plan.ids):
            layer, b = divmod(bid, mgr.blocks_per_layer)
            blk = mgr.acquire(layer, b).view(2, 1, bt, Hkv, D)
            # non-causal block attention, merged into the running output after the first block of a layer pass
            C.attn_fwd(q, blk[0], blk[1], o, lse, scale, False, 0, 0, [0], [0], i % mgr.blocks_per_layer != 0, 0, 0, 0)
        e1.record()
        torch.cuda.synchronize()
        mgr.step_end()
        times.append(e0.elapsed_time(e1))
    _ext.check_status()
    st = mgr.stats()
    lru = mgr.lru_baseline()
    flops = 4.0 * args.q_tokens * bt * D * Hq * n_acc
    ms = min(times)
    print(json.dumps({
        "metric": "KV tiering stress step time", "value": round(ms, 2), "unit": "ms", "higher_is_better": False,
        "step_ms_all": [round(t, 2) for t in times],
        "context_tokens": args.context, "ring": args.ring, "layers": args.layers, "block_tokens": bt,
        "share_kv_bytes": mgr.total_kv_bytes(), "hbm_budget_bytes": mgr.hbm_budget_bytes, "accesses_per_step": n_acc,
        "plan": {"hits": plan.hits, "misses": plan.misses, "hit_rate": round(plan.hit_rate, 4), "lru_misses": lru["misses"],
                 "bytes_loaded": plan.bytes_loaded},
        "measured": {"hits": st.hits, "misses": st.misses, "prefetched": st.prefetched, "bytes_h2d": st.bytes_h2d,
                     "bytes_d2h": st.bytes_d2h, "bytes_nvme_read": st.bytes_nvme_read, "bytes_nvme_write": st.bytes_nvme_write,
                     "exposed_stall_ms_total": round(st.exposed_stall_ms, 2), "peak_hbm_bytes": st.peak_hbm_bytes},
        "attention_tflops": round(flops / ms / 1e9, 1), "steps": args.steps, "timing": "CUDA events around one pass over the plan",
    }), flush=True)
    mgr.close()


if __name__ == "__main__":
    main()
