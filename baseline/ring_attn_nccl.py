"""Same-box NCCL + library baseline for the ring-attention benchmark (``zenyx_b200.bench.ring_attn``):
context-parallel causal attention built only from ``torch.distributed`` point-to-point calls and stock
PyTorch attention, the way the reference's stack would do it (its transport is
zenyx/distributed/communication.py:136-171; it has no attention op of its own, its models call
``torch.nn.functional.scaled_dot_product_attention``).

    python -m torch.distributed.run --nproc-per-node R -m baseline.ring_attn_nccl [--seq-len 131072]

Scheme (the all-gather form of context parallelism): every rank keeps its zigzag shard of Q; K and V travel
around the ring with ``batch_isend_irecv`` (R - 1 hops) until every rank holds the whole sequence; each of a
rank's two query chunks then runs ONE library attention call against the keys up to its own end with a
lower-right-aligned causal mask; backward is autograd through that call followed by a ring reduce-scatter of
dK/dV (R - 1 hops, fp32 accumulation). Nothing of this package's kernels or peer memory is used: only
``zenyx_b200.ops.comm`` (thin wrappers over ``batch_isend_irecv``) and the shard arithmetic.
Prints one JSON line with the same fields as the benchmark it is the baseline for.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq-len", type=int, default=131072)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    args = ap.parse_args(argv)
    from torch.nn.attention.bias import causal_lower_right

    from zenyx_b200.ops.attention import shard_positions
    from zenyx_b200.ops.comm import ring_all_gather, ring_reduce_scatter

    R = int(os.environ.get("WORLD_SIZE", "1"))
    r = int(os.environ.get("RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    if R > 1:
        dist.init_process_group("nccl")
    B, S, Hq, Hkv, D = 1, args.seq_len, 32, 8, 128
    Sl, L = S // R, S // (2 * R)
    scale = 1 / math.sqrt(D)
    g = torch.Generator(device=dev).manual_seed(100 + r)
    q = torch.randn(B, Sl, Hq, D, device=dev, generator=g).bfloat16().requires_grad_(True)
    do = torch.randn(B, Sl, Hq, D, device=dev, generator=g).bfloat16()
    k = torch.randn(B, Sl, Hkv, D, device=dev, generator=g).bfloat16()
    v = torch.randn(B, Sl, Hkv, D, device=dev, generator=g).bfloat16()
    my_pos = shard_positions(r, R, S) if R > 1 else [0]
    chunk = L if R > 1 else S

    def gather_global(x):
        """[B, S, Hkv, D] in global token order from every rank's zigzag shard (NCCL ring hops)."""
        if R == 1:
            return x
        parts = ring_all_gather(x)
        full = torch.empty(B, S, Hkv, D, device=dev, dtype=x.dtype)
        for owner, part in enumerate(parts):
            for ci, p0 in enumerate(shard_positions(owner, R, S)):
                full[:, p0: p0 + L] = part[:, ci * L: (ci + 1) * L]
        return full

    def forward(kk, vv):
        kg, vg = gather_global(kk), gather_global(vv)
        kg.requires_grad_(True)
        vg.requires_grad_(True)
        outs = []
        for ci, p0 in enumerate(my_pos):
            end = p0 + chunk
            qc = q[:, ci * chunk: (ci + 1) * chunk].transpose(1, 2)
            o = F.scaled_dot_product_attention(qc, kg[:, :end].transpose(1, 2), vg[:, :end].transpose(1, 2),
                                               attn_mask=causal_lower_right(chunk, end), scale=scale, enable_gqa=True)
            outs.append(o.transpose(1, 2))
        return torch.cat(outs, dim=1), kg, vg

    def backward(o, kg, vg):
        q.grad = None
        o.backward(do)
        if R == 1:
            return q.grad, kg.grad, vg.grad
        # this rank's contribution to every owner's dK/dV, then W - 1 hops of reduce-scatter
        dks, dvs = [], []
        for owner in range(R):
            idx = [slice(p0, p0 + L) for p0 in shard_positions(owner, R, S)]
            dks.append(torch.cat([kg.grad[:, sl] for sl in idx], dim=1))
            dvs.append(torch.cat([vg.grad[:, sl] for sl in idx], dim=1))
        return q.grad, ring_reduce_scatter(dks), ring_reduce_scatter(dvs)

    def sync():
        if R > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_ms(ms):
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        if R > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    try:
        fwd_ms, bwd_ms = [], []
        for it in range(args.warmup + args.iters):
            sync()
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            e0.record()
            o, kg, vg = forward(k, v)
            e1.record()
            backward(o, kg, vg)
            e2.record()
            sync()
            if it >= args.warmup:
                fwd_ms.append(max_ms(e0.elapsed_time(e1)))
                bwd_ms.append(max_ms(e1.elapsed_time(e2)))
            del o, kg, vg
    except Exception as e:  # noqa: BLE001
        if r == 0:
            print(json.dumps({"impl": "nccl+sdpa baseline", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}), flush=True)
        if R > 1:
            dist.destroy_process_group()
        return
    fwd_ms.sort()
    bwd_ms.sort()
    ms_f, ms_b = fwd_ms[len(fwd_ms) // 2], bwd_ms[len(bwd_ms) // 2]
    f_fwd = 4.0 * S * S * D * Hq * 0.5
    f_bwd = 2.5 * f_fwd
    rec = {"metric": "ring-attn fwd+bwd TFLOP/s", "impl": "nccl ring hops (batch_isend_irecv) + library SDPA", "ring_degree": R,
           "seq_len": S, "heads": [Hq, Hkv], "head_dim": D, "layout": "zigzag", "mask": "causal",
           "fwd_ms": round(ms_f, 3), "bwd_ms": round(ms_b, 3), "fwd_tflops": round(f_fwd / ms_f / 1e9, 1),
           "bwd_tflops": round(f_bwd / ms_b / 1e9, 1), "value": round((f_fwd + f_bwd) / (ms_f + ms_b) / 1e9, 1),
           "unit": "TFLOP/s (whole job)", "per_gpu_tflops": round((f_fwd + f_bwd) / (ms_f + ms_b) / 1e9 / R, 1),
           "timing": "CUDA events, max over ranks, median of %d" % args.iters}
    if r == 0:
        print(json.dumps(rec), flush=True)
    if R > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
