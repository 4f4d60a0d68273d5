"""bf16 GEMM on the tcgen05 kernel, plus the autograd `linear` built on it.

The reference reaches its matmuls through ``nn.Linear``/``F.linear`` (cuBLAS), e.g.
zenyx/distributed/tensor_parallel.py:48-50; here every projection of the hot path runs on
``csrc/gemm/gemm_bf16.cu``. On CPU tensors (unit tests, gloo ranks) the same functions fall back
to fp32 PyTorch math so that host-side logic is testable without a GPU.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import _ext


def gemm(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
         addend: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out = A @ B^T (+ addend)`` where logical A is [M, K] and logical B is [N, K].

    ``trans_a`` / ``trans_b`` say that the tensor passed is stored transposed ([K, M] / [K, N]).
    ``addend`` may alias ``out`` (gradient accumulation) and may be bf16 or fp32.
    """
    M = a.shape[1] if trans_a else a.shape[0]
    N = b.shape[1] if trans_b else b.shape[0]
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=out_dtype or a.dtype)
    if _ext.use_cuda_kernels(a) and a.dtype == torch.bfloat16:
        _ext.C().gemm(a, b, out, trans_a, trans_b, addend)
        return out
    af = (a.t() if trans_a else a).float()
    bf = (b if trans_b else b.t()).float()
    res = af @ bf
    if addend is not None:
        res = res + addend.float()
    out.copy_(res.to(out.dtype))
    return out


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        r2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
        y = gemm(x2, w, addend=r2)
        ctx.save_for_backward(x2, w)
        ctx.has_res = residual is not None
        ctx.in_shape = shape
        return y.reshape(*shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, w.shape[0]).contiguous()
        dx = gemm(dy2, w, trans_b=True) if ctx.needs_input_grad[0] else None          # dY [T,N] x W [N,K]
        dw = gemm(dy2, x2, trans_a=True, trans_b=True) if ctx.needs_input_grad[1] else None  # dY^T X
        dres = dy if ctx.has_res and ctx.needs_input_grad[2] else None
        return (dx.reshape(ctx.in_shape) if dx is not None else None), dw, dres


def linear(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T (+ residual)``; the residual add is fused into the GEMM epilogue."""
    return _LinearFn.apply(x, w, residual)


class Linear(nn.Module):
    """Bias-free linear layer running on the tcgen05 GEMM (bf16 on GPU)."""

    def __init__(self, in_features: int, out_features: int, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        nn.init.normal_(self.weight, std=in_features ** -0.5)

    def forward(self, x, residual=None):
        return linear(x, self.weight, residual)
