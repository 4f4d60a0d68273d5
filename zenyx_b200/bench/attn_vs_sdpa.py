"""Attention and GEMM kernels of this package beside the stock library paths (cuDNN attention through
``scaled_dot_product_attention``, cuBLAS through ``torch.matmul``), each run back to back for a few
seconds while the SM clock and board power are read through NVML (read-only).

    python -m zenyx_b200.bench.attn_vs_sdpa [--seq-len 32768] [--seconds 3]

One line per kernel: time of the first launch after warm-up, mean time over the sustained run, median
SM clock and power over the second half of the run. The library rows are the yardstick the
reference arm of ``bench.py`` runs on (its model calls SDPA and ``nn.Linear``).
"""
from __future__ import annotations

import argparse
import math
import threading
import time

import torch
import torch.nn.functional as F


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq-len", type=int, default=32768)
    ap.add_argument("--seconds", type=float, default=3.0)
    args = ap.parse_args(argv)
    import pynvml

    from zenyx_b200.ops import _ext

    C = _ext.C()
    pynvml.nvmlInit()
    h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())

    def sample(stop, out):
        while not stop.is_set():
            out.append((pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM), pynvml.nvmlDeviceGetPowerUsage(h) / 1000))
            time.sleep(0.05)

    def run(name, fn, flops):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record(); torch.cuda.synchronize()
        one = e0.elapsed_time(e1)
        n = max(3, int(args.seconds * 1e3 / one))
        stop, out = threading.Event(), []
        th = threading.Thread(target=sample, args=(stop, out))
        th.start()
        e0.record()
        for _ in range(n):
            fn()
        e1.record(); torch.cuda.synchronize(); stop.set(); th.join()
        ms = e0.elapsed_time(e1) / n
        tail = out[len(out) // 2:] or [(0, 0.0)]
        clk = sorted(c for c, _ in tail)[len(tail) // 2]
        pw = sorted(p for _, p in tail)[len(tail) // 2]
        print(f"{name:34s} first {one:8.3f} ms   sustained {ms:8.3f} ms ({flops / ms / 1e9:7.1f} TFLOP/s)   "
              f"SM {clk} MHz   {pw:.0f} W", flush=True)
        time.sleep(1.0)

    B, S, Hq, Hkv, D = 1, args.seq_len, 32, 8, 128
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    o = torch.empty_like(q)
    lse = torch.empty(B, Hq, S, device="cuda")
    scale = 1 / math.sqrt(D)
    f_fwd = 4.0 * S * S * D * Hq / 2
    run("attention forward (this package)", lambda: C.attn_fwd(q, k, v, o, lse, scale, True, 0, 0, [0], [0], False, 0, 0, 0), f_fwd)
    do = torch.randn_like(q)
    delta = torch.empty_like(lse)
    dq = torch.empty(B, S, Hq, D, device="cuda")
    dk = torch.zeros(B, S, Hkv, D, device="cuda")
    dv = torch.zeros(B, S, Hkv, D, device="cuda")
    run("attention backward (this package)",
        lambda: C.attn_bwd(q, k, v, o, do, lse, delta, dq, dk, dv, scale, True, 0, 0, [0], [0], True, False, 0, 0, 0), 2.5 * f_fwd)
    qt = q.transpose(1, 2).detach().requires_grad_(True)
    kt = k.transpose(1, 2).detach().requires_grad_(True)
    vt = v.transpose(1, 2).detach().requires_grad_(True)
    run("SDPA forward (library)", lambda: F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, scale=scale, enable_gqa=True), f_fwd)

    def fb():
        F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, scale=scale, enable_gqa=True).backward(do.transpose(1, 2))

    run("SDPA forward+backward (library)", fb, 3.5 * f_fwd)
    a = torch.randn(32768, 4096, device="cuda").bfloat16()
    w = torch.randn(28672, 4096, device="cuda").bfloat16()
    out = torch.empty(32768, 28672, device="cuda", dtype=torch.bfloat16)
    f_mm = 2.0 * 32768 * 28672 * 4096
    run("GEMM 32768x28672x4096 (this package)", lambda: C.gemm(a, w, out, False, False, None), f_mm)
    run("GEMM same shape (cuBLAS)", lambda: torch.matmul(a, w.t(), out=out), f_mm)
    _ext.check_status()


if __name__ == "__main__":
    main()
