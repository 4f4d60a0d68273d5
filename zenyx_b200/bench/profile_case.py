"""Small, self-terminating workloads for profiler captures: ``python -m zenyx_b200.bench.profile_case
<case>`` launches one kernel family a few times on inputs larger than L2 but well under a few GB.

cases: attn_fwd, attn_bwd (S=8192, 32/8 heads, causal), gemm (8192x8192x4096), gemm_wgrad, zero (64M parameters)
"""
from __future__ import annotations

import math
import sys

import torch


def main(case: str, iters: int = 3) -> None:
    from zenyx_b200.ops import _ext

    C = _ext.C()
    torch.manual_seed(0)
    if case in ("attn_fwd", "attn_bwd"):
        B, S, Hq, Hkv, D = 1, 8192, 32, 8, 128
        q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
        k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
        v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
        o = torch.empty_like(q)
        lse = torch.empty(B, Hq, S, device="cuda")
        scale = 1 / math.sqrt(D)
        C.attn_fwd(q, k, v, o, lse, scale, True, 0, 0, [0], [0], False, 0, 0, 0)
        if case == "attn_fwd":
            for _ in range(iters):
                C.attn_fwd(q, k, v, o, lse, scale, True, 0, 0, [0], [0], False, 0, 0, 0)
        else:
            do = torch.randn_like(q)
            delta = torch.empty_like(lse)
            dq = torch.empty(B, S, Hq, D, device="cuda")
            dk = torch.zeros(B, S, Hkv, D, device="cuda")
            dv = torch.zeros(B, S, Hkv, D, device="cuda")
            for _ in range(iters):
                C.attn_bwd(q, k, v, o, do, lse, delta, dq, dk, dv, scale, True, 0, 0, [0], [0], True, False, 0, 0, 0)
    elif case in ("gemm", "gemm_wgrad"):
        M, N, K = (8192, 8192, 4096) if case == "gemm" else (8192, 4096, 16384)
        at = bt = case == "gemm_wgrad"
        a = torch.randn((K, M) if at else (M, K), device="cuda").bfloat16()
        b = torch.randn((K, N) if bt else (N, K), device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for _ in range(iters + 1):
            C.gemm(a, b, out, at, bt, None)
    elif case == "zero":
        from zenyx_b200.models.llama import FlatBuffers
        from zenyx_b200.parallel.zero import ZeroAdamW

        flat = FlatBuffers([("w", (8192, 8192), True)], "cuda")
        opt = ZeroAdamW(flat, lr=1e-3)
        for _ in range(iters + 1):
            flat.grads.normal_()
            opt.step()
    else:
        raise SystemExit(f"unknown case {case!r}")
    _ext.check_status()
    torch.cuda.synchronize()
    print("done", case)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "attn_fwd")
