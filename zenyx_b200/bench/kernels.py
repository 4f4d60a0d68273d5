"""Device-timed microbenchmarks of the hot kernels against the measured roofline.

``python -m zenyx_b200.bench.kernels [--quick]`` prints one JSON line per kernel with the achieved
TFLOP/s (or GB/s) and the fraction of the measured peak (``MEASURED_PEAKS.json`` at the repository
root when present, otherwise 1.59 PFLOP/s / 6.65 TB/s). Timing: CUDA events on the launching
stream, 3 warm-up launches, an L2 flush (a 256 MB write) between timed launches.
The reference project's ``zenyx/bench`` package was deleted from its tree; only its name survives
(ZENYX_2_0_PHASE_1_SUMMARY.md:27).
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import torch


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"tflops": d.get("bf16_tflops", 1590.0), "tflops_sustained": d.get("bf16_tflops_sustained", 1400.0),
                "gbs": d.get("hbm_gbs", 6650.0), "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "gbs": 6650.0, "source": "fallback"}


_flush = None


def time_cuda(fn, iters=10, warmup=3, flush_l2=True):
    global _flush
    if flush_l2 and _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush_l2:
            _flush.zero_()
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def bench_gemm(M, N, K, a_t=False, b_t=False, compare=True):
    from zenyx_b200.ops import _ext

    C = _ext.C()
    a = torch.randn((K, M) if a_t else (M, K), device="cuda").bfloat16()
    b = torch.randn((K, N) if b_t else (N, K), device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ms = time_cuda(lambda: C.gemm(a, b, out, a_t, b_t, None))
    _ext.check_status()
    tf = 2.0 * M * N * K / ms / 1e9
    rec = {"kernel": "gemm_bf16", "M": M, "N": N, "K": K, "a_t": a_t, "b_t": b_t, "ms": round(ms, 4),
           "tflops": round(tf, 1), "frac_of_peak": round(tf / peaks()["tflops"], 3), "peak": peaks()["source"]}
    if compare:
        am = a.t() if a_t else a
        bm = b if b_t else b.t()
        ms_ref = time_cuda(lambda: torch.matmul(am, bm, out=out))
        rec["cublas_ms"] = round(ms_ref, 4)
        rec["cublas_tflops"] = round(2.0 * M * N * K / ms_ref / 1e9, 1)
    return rec


def bench_attn(S, Hq=32, Hkv=8, B=1, causal=True, bwd=True, iters=5, warmup=3):
    from zenyx_b200.ops import _ext

    C = _ext.C()
    D = 128
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    o = torch.empty_like(q)
    lse = torch.empty(B, Hq, S, device="cuda", dtype=torch.float32)
    scale = 1.0 / math.sqrt(D)
    ms_f = time_cuda(lambda: C.attn_fwd(q, k, v, o, lse, scale, causal, 0, 0, [0], [0], False, 0, 0, 0), iters=iters,
                     warmup=warmup)
    _ext.check_status()
    flops_f = 4.0 * B * Hq * S * S * D * (0.5 if causal else 1.0)
    rec = {"kernel": "attn_fwd", "S": S, "Hq": Hq, "Hkv": Hkv, "B": B, "causal": causal, "ms": round(ms_f, 3),
           "tflops": round(flops_f / ms_f / 1e9, 1), "frac_of_peak": round(flops_f / ms_f / 1e9 / peaks()["tflops"], 3)}
    out = [rec]
    if bwd:
        do = torch.randn_like(q)
        delta = torch.empty_like(lse)
        dq = torch.empty(B, S, Hq, D, device="cuda")
        dk = torch.zeros(B, S, Hkv, D, device="cuda")
        dv = torch.zeros(B, S, Hkv, D, device="cuda")
        ms_b = time_cuda(lambda: C.attn_bwd(q, k, v, o, do, lse, delta, dq, dk, dv, scale, causal, 0, 0, [0], [0],
                                            True, False, 0, 0, 0), iters=iters, warmup=warmup)
        _ext.check_status()
        flops_b = 2.5 * flops_f
        out.append({"kernel": "attn_bwd", "S": S, "Hq": Hq, "Hkv": Hkv, "B": B, "causal": causal,
                    "ms": round(ms_b, 3), "tflops": round(flops_b / ms_b / 1e9, 1),
                    "frac_of_peak": round(flops_b / ms_b / 1e9 / peaks()["tflops"], 3)})
    return out


def bench_zero(n_params=64 << 20):
    """The sharded-optimizer step on one GPU (no peers): per parameter it reads an fp32 gradient, the bf16 + int16
    halves of the master weight and fp32 m, v, writes all but the gradient back and clears the gradient: 32 bytes."""
    from zenyx_b200.models.llama import FlatBuffers
    from zenyx_b200.ops import _ext
    from zenyx_b200.parallel.zero import ZeroAdamW

    rows = n_params // 8192
    flat = FlatBuffers([("w", (rows, 8192), True)], "cuda")
    opt = ZeroAdamW(flat, lr=1e-3)
    flat.grads.normal_()
    ms = time_cuda(lambda: opt.step(), iters=10)
    _ext.check_status()
    gbs = flat.total * 32 / ms / 1e6
    return {"kernel": "zero_adamw step (1 GPU)", "params": flat.total, "ms": round(ms, 4), "gbs": round(gbs, 1),
            "frac_of_copy_rate": round(gbs / peaks()["gbs"], 3), "peak": peaks()["source"]}


def bench_fused(tokens=32768, H=4096, F=14336, Hq=32, Hkv=8, D=128):
    """Achieved HBM rate of the bandwidth-bound kernels of a Llama block at the 8B shape (algorithmic bytes / time)."""
    from zenyx_b200.ops import _ext, fused

    out = []
    gbs_peak = peaks()["gbs"]

    def rec(name, nbytes, fn):
        ms = time_cuda(fn, iters=10)
        _ext.check_status()
        out.append({"kernel": name, "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1),
                    "frac_of_copy_rate": round(nbytes / ms / 1e6 / gbs_peak, 3)})

    x = torch.randn(tokens, H, device="cuda").bfloat16()
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    y, rstd = fused.rmsnorm_fwd(x, w, 1e-5)
    rec("rmsnorm_fwd", 2 * x.numel() * 2, lambda: fused.rmsnorm_fwd(x, w, 1e-5))
    dw = torch.zeros(H, device="cuda")
    rec("rmsnorm_bwd (+residual gradient)", 4 * x.numel() * 2, lambda: fused.rmsnorm_bwd(y, x, w, rstd, dw, x))
    gu = torch.randn(tokens, 2 * F, device="cuda").bfloat16()
    h = fused.swiglu_fwd(gu)
    rec("swiglu_fwd", 3 * tokens * F * 2, lambda: fused.swiglu_fwd(gu))
    rec("swiglu_bwd", 5 * tokens * F * 2, lambda: fused.swiglu_bwd(gu, h))
    qkv = torch.randn(tokens, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    cos, sin = fused.rope_tables(torch.arange(tokens, device="cuda"), D, 500000.0)
    rec("rope_qkv (in place)", 2 * tokens * (Hq + Hkv) * D * 2, lambda: fused.rope_qkv_(qkv, cos, sin, Hq, Hkv, D, tokens))
    dq = torch.randn(tokens, Hq, D, device="cuda")
    dk = torch.randn(tokens, Hkv, D, device="cuda")
    dv = torch.randn(tokens, Hkv, D, device="cuda")
    rec("rope_bwd_pack (fp32 dq, dk, dv -> bf16 dqkv)", tokens * (Hq + 2 * Hkv) * D * 6,
        lambda: fused.rope_bwd_pack(dq, dk, dv, cos, sin, Hq, Hkv, D, tokens))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--no-attn", action="store_true")
    ap.add_argument("--no-gemm", action="store_true")
    ap.add_argument("--no-bwd", action="store_true")
    ap.add_argument("--seq", type=int, nargs="*", default=None, help="attention sequence lengths (default 8192 32768)")
    ap.add_argument("--attn-iters", type=int, default=5, help="timed attention launches (1 for a profiler capture)")
    ap.add_argument("--attn-warmup", type=int, default=3)
    ap.add_argument("--zero", action="store_true", help="also time the optimizer step kernel")
    ap.add_argument("--fused", action="store_true", help="also time the bandwidth-bound kernels of a Llama block")
    args = ap.parse_args(argv)
    shapes = [(8192, 8192, 8192, False, False)]
    if not args.quick:
        shapes += [
            (32768, 6144, 4096, False, False),   # QKV projection
            (32768, 28672, 4096, False, False),  # gate|up projection
            (32768, 4096, 14336, False, False),  # down projection
            (32768, 4096, 6144, False, True),    # dgrad of QKV
            (28672, 4096, 32768, True, True),    # wgrad of gate|up
        ]
    for M, N, K, at, bt in ([] if args.no_gemm else shapes):
        print(json.dumps(bench_gemm(M, N, K, at, bt)), flush=True)
    if args.zero:
        print(json.dumps(bench_zero()), flush=True)
    if args.fused:
        for rec in bench_fused():
            print(json.dumps(rec), flush=True)
    if not args.no_attn:
        for S in (args.seq or ([8192] if args.quick else [8192, 32768])):
            for rec in bench_attn(S, bwd=not args.no_bwd, iters=args.attn_iters, warmup=args.attn_warmup):
                print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
