"""Benchmark of the GEMMs fused with their collective against the unfused sequence (NCCL collective,
then the same GEMM kernel), on the MLP shapes of a tensor-parallel Llama-3-8B layer at 32K tokens.

    python -m torch.distributed.run --nproc-per-node N -m zenyx_b200.bench.fused_collective

One JSON line per operation from rank 0. Times are CUDA-event times on the launching stream, maximum
over ranks, after warm-up; the operands (tens to hundreds of MB) exceed L2. The roofline is the slower
of FLOPs / measured GEMM peak and bytes that must cross NVLink / 770 GB/s (measured peer copy rate).
The reference has no counterpart (its tensor-parallel layers call ``dist.all_reduce`` /
``dist.all_gather`` around ``F.linear``, zenyx/distributed/tensor_parallel.py:48-50, 96-114).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time(fn, warmup=3, iters=10):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    args = ap.parse_args(argv)
    from zenyx_b200.bench.kernels import peaks
    from zenyx_b200.ops import _ext
    from zenyx_b200.ops.gemm import gemm
    from zenyx_b200.parallel.communication import init_distributed_from_env
    from zenyx_b200.parallel.fused_collective import FusedCollectiveContext, allgather_gemm, gemm_reduce_scatter

    ctx = init_distributed_from_env(timeout_seconds=120)
    R, r = ctx.world_size, ctx.rank
    T, D, Fd = args.tokens, args.d_model, args.ffn
    m = T // R
    n_col = 2 * Fd // R            # gate|up, this rank's features
    k_row = Fd // R                # down projection, this rank's input features
    fc = FusedCollectiveContext(m, D, max(D, n_col))
    x_local = torch.randn(m, D, device="cuda").bfloat16()
    w_col = (torch.randn(n_col, D, device="cuda") / 64).bfloat16()
    a_full = torch.randn(T, k_row, device="cuda").bfloat16()
    w_row = (torch.randn(D, k_row, device="cuda") / 64).bfloat16()
    pk = peaks()
    link = 770e9

    def unfused_ag():
        parts = torch.empty(T, D, device="cuda", dtype=torch.bfloat16)
        dist.all_gather_into_tensor(parts, x_local)
        return gemm(parts, w_col)

    def unfused_rs():
        y = gemm(a_full, w_row)
        out = torch.empty(m, D, device="cuda", dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(out, y)
        return out

    rows = []
    for name, fused, unfused, flops, wire in (
        ("allgather_gemm", lambda: allgather_gemm(x_local, w_col, fc, fused=True), unfused_ag,
         2.0 * T * D * n_col, (R - 1) * m * D * 2),
        ("gemm_reduce_scatter", lambda: gemm_reduce_scatter(a_full, w_row, fc, fused=True), unfused_rs,
         2.0 * T * k_row * D, (R - 1) * m * D * 4),
    ):
        ms_f = _time(fused)
        _ext.check_status()
        ms_u = _time(unfused)
        roof_ms = max(flops / (pk["tflops"] * 1e12), wire / link) * 1e3
        rows.append({"op": name, "ranks": R, "tokens": T, "shape_per_rank": {"m": m, "d_model": D, "n_col": n_col, "k_row": k_row},
                     "fused_ms": round(ms_f, 3), "nccl_then_gemm_ms": round(ms_u, 3), "speedup": round(ms_u / ms_f, 3),
                     "tflops_per_gpu": round(flops / ms_f / 1e9, 1), "nvlink_bytes_per_gpu": int(wire),
                     "roofline_ms": round(roof_ms, 3), "frac_of_roofline": round(roof_ms / ms_f, 3),
                     "peaks": pk["source"], "timing": "CUDA events, max over ranks, 10 iterations after 3 warm-up"})
    if r == 0:
        for row in rows:
            print(json.dumps(row), flush=True)
    fc.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    main()
