"""Bandwidth-bound operators (RMSNorm, RoPE, SwiGLU, embedding, cross-entropy, e4m3 KV quantisation,
AdamW, gradient norm) over ``csrc/fused/fused_ops.cu``, each with an fp32 PyTorch fallback for CPU
tensors. The reference has none of these as kernels: its models are ``nn.TransformerEncoderLayer``
stacks (README.md:64-77) and its optimizer is ``torch.optim.AdamW`` (zenyx/train/trainer.py:29).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _ext

# ------------------------------------------------------------------------------------------------
# RMSNorm
# ------------------------------------------------------------------------------------------------


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (y, rstd). x: [..., H]; rstd: [rows] fp32."""
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    if _ext.use_cuda_kernels(x) and x.dtype == torch.bfloat16:
        x2 = x2.contiguous()
        y = torch.empty_like(x2)
        rstd = torch.empty(x2.shape[0], device=x.device, dtype=torch.float32)
        _ext.C().rmsnorm_fwd(x2, w.contiguous(), y, rstd, eps)
        return y.view(x.shape), rstd
    xf = x2.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
    y = (xf * rstd[:, None] * w.float()).to(x.dtype)
    return y.view(x.shape), rstd


def rmsnorm_bwd(dy, x, w, rstd, dw_accum: torch.Tensor, dres: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Returns dx (+ dres, the gradient arriving through the residual branch); adds the weight
    gradient into the fp32 buffer `dw_accum` [H]."""
    H = x.shape[-1]
    if _ext.use_cuda_kernels(x) and x.dtype == torch.bfloat16:
        x2 = x.reshape(-1, H).contiguous()
        dy2 = dy.reshape(-1, H).contiguous()
        dx = torch.empty_like(x2)
        _ext.C().rmsnorm_bwd(dy2, x2, w.contiguous(), rstd, dx, dw_accum,
                             dres.reshape(-1, H).contiguous() if dres is not None else None)
        return dx.view(x.shape)
    xf, dyf, wf = x.reshape(-1, H).float(), dy.reshape(-1, H).float(), w.float()
    xh = xf * rstd[:, None]
    g = dyf * wf
    dx = rstd[:, None] * (g - xh * (g * xh).mean(-1, keepdim=True))
    dw_accum.add_((dyf * xh).sum(0))
    if dres is not None:
        dx = dx + dres.reshape(-1, H).float()
    return dx.to(x.dtype).view(x.shape)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        y, rstd = rmsnorm_fwd(x, w, eps)
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dw = torch.zeros(w.shape, device=w.device, dtype=torch.float32)
        dx = rmsnorm_bwd(dy, x, w, rstd, dw)
        return dx, dw.to(w.dtype), None


def rmsnorm(x, w, eps: float = 1e-5):
    return _RMSNormFn.apply(x, w, eps)


# ------------------------------------------------------------------------------------------------
# RoPE
# ------------------------------------------------------------------------------------------------


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables [len(positions), head_dim/2] (fp32) for arbitrary global positions."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=positions.device, dtype=torch.float64) / head_dim))
    ang = positions.to(torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


def rope_qkv_(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
              tokens_per_seq: int, *, inverse: bool = False, k_out: Optional[torch.Tensor] = None,
              v_out: Optional[torch.Tensor] = None) -> None:
    """Rotates the Q and K column blocks of a fused [tokens, (Hq+2Hkv)*D] projection in place
    (rotate-half pairing). With k_out / v_out the rotated K and the V block are written to those
    [tokens, Hkv, D] buffers instead (they may be peer-visible symmetric memory)."""
    if _ext.use_cuda_kernels(qkv) and qkv.dtype == torch.bfloat16:
        _ext.C().rope_qkv(qkv, cos, sin, k_out, v_out, n_heads, n_kv_heads, head_dim, tokens_per_seq, inverse)
        return
    T = qkv.shape[0]
    D, half = head_dim, head_dim // 2
    idx = torch.arange(T, device=qkv.device) % tokens_per_seq
    c, s = cos[idx][:, None, :], sin[idx][:, None, :]
    if inverse:
        s = -s

    def rot(x):
        x = x.float()
        x1, x2 = x[..., :half], x[..., half:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)

    q = qkv[:, : n_heads * D].view(T, n_heads, D)
    k = qkv[:, n_heads * D : (n_heads + n_kv_heads) * D].view(T, n_kv_heads, D)
    q.copy_(rot(q).to(qkv.dtype))
    kr = rot(k).to(qkv.dtype)
    if k_out is not None:
        k_out.view(T, n_kv_heads, D).copy_(kr)
    else:
        k.copy_(kr)
    if v_out is not None:
        v_out.view(T, n_kv_heads, D).copy_(qkv[:, (n_heads + n_kv_heads) * D :].view(T, n_kv_heads, D))


def rope_bwd_pack(dq: torch.Tensor, dk: torch.Tensor, dv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                  n_heads: int, n_kv_heads: int, head_dim: int, tokens_per_seq: int,
                  dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """fp32 dq [T,Hq,D] / dk, dv [T,Hkv,D] -> d(qkv) [T,(Hq+2Hkv)*D] in `dtype`, undoing the rotation on dq and dk."""
    T = dq.numel() // (n_heads * head_dim)
    out = torch.empty(T, (n_heads + 2 * n_kv_heads) * head_dim, device=dq.device, dtype=dtype)
    if _ext.use_cuda_kernels(dq) and dtype == torch.bfloat16:
        _ext.C().rope_bwd_pack(dq.contiguous(), dk.contiguous(), dv.contiguous(), cos, sin, out, n_heads, n_kv_heads,
                               head_dim, tokens_per_seq)
        return out
    D, half = head_dim, head_dim // 2
    idx = torch.arange(T, device=dq.device) % tokens_per_seq
    c, s = cos[idx][:, None, :], -sin[idx][:, None, :]

    def rot(x):
        x1, x2 = x[..., :half], x[..., half:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)

    out[:, : n_heads * D] = rot(dq.reshape(T, n_heads, D).float()).reshape(T, -1).to(dtype)
    out[:, n_heads * D : (n_heads + n_kv_heads) * D] = rot(dk.reshape(T, n_kv_heads, D).float()).reshape(T, -1).to(dtype)
    out[:, (n_heads + n_kv_heads) * D :] = dv.reshape(T, -1).to(dtype)
    return out


# ------------------------------------------------------------------------------------------------
# SwiGLU
# ------------------------------------------------------------------------------------------------


def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    """gu: [tokens, 2F] = gate | up  ->  silu(gate) * up  [tokens, F]."""
    F = gu.shape[-1] // 2
    if _ext.use_cuda_kernels(gu) and gu.dtype == torch.bfloat16:
        h = torch.empty(gu.shape[0], F, device=gu.device, dtype=gu.dtype)
        _ext.C().swiglu_fwd(gu, h)
        return h
    g, u = gu[:, :F].float(), gu[:, F:].float()
    return (torch.nn.functional.silu(g) * u).to(gu.dtype)


def swiglu_bwd(gu: torch.Tensor, dh: torch.Tensor) -> torch.Tensor:
    F = gu.shape[-1] // 2
    if _ext.use_cuda_kernels(gu) and gu.dtype == torch.bfloat16:
        dgu = torch.empty_like(gu)
        _ext.C().swiglu_bwd(gu, dh.contiguous(), dgu)
        return dgu
    g, u, d = gu[:, :F].float(), gu[:, F:].float(), dh.float()
    sg = torch.sigmoid(g)
    silu = g * sg
    return torch.cat([d * u * (sg + silu * (1 - sg)), d * silu], dim=-1).to(gu.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dh):
        (gu,) = ctx.saved_tensors
        return swiglu_bwd(gu, dh)


def swiglu(gu):
    shape = gu.shape
    return _SwiGLUFn.apply(gu.reshape(-1, shape[-1])).reshape(*shape[:-1], shape[-1] // 2)


# ------------------------------------------------------------------------------------------------
# Embedding
# ------------------------------------------------------------------------------------------------


def embedding_fwd(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    flat = ids.reshape(-1)
    if _ext.use_cuda_kernels(table) and table.dtype == torch.bfloat16:
        out = torch.empty(flat.numel(), table.shape[1], device=table.device, dtype=table.dtype)
        _ext.C().embedding_fwd(flat.contiguous(), table, out)
        return out
    return table[flat.clamp(0, table.shape[0] - 1)]


def embedding_bwd(ids: torch.Tensor, dout: torch.Tensor, dtable_accum: torch.Tensor) -> None:
    """Scatter-adds dout rows into the fp32 gradient table."""
    flat = ids.reshape(-1)
    if _ext.use_cuda_kernels(dout) and dout.dtype == torch.bfloat16:
        _ext.C().embedding_bwd(flat.contiguous(), dout.contiguous(), dtable_accum)
        return
    dtable_accum.index_add_(0, flat, dout.reshape(flat.numel(), -1).float())


# ------------------------------------------------------------------------------------------------
# Cross-entropy (forward + backward in one pass over a chunk of logits)
# ------------------------------------------------------------------------------------------------


def cross_entropy_fwd_bwd_(logits: torch.Tensor, targets: torch.Tensor, grad_scale: float,
                           ignore_index: int = -100) -> torch.Tensor:
    """Overwrites `logits` [rows, V] with grad_scale * d(sum of losses)/d(logits); returns the
    per-row losses (fp32)."""
    if _ext.use_cuda_kernels(logits) and logits.dtype == torch.bfloat16:
        loss = torch.empty(logits.shape[0], device=logits.device, dtype=torch.float32)
        _ext.C().ce_fwd_bwd(logits, targets.contiguous(), loss, grad_scale, ignore_index)
        return loss
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    valid = (targets != ignore_index) & (targets >= 0) & (targets < logits.shape[1])
    tsafe = targets.clamp(0, logits.shape[1] - 1)
    loss = torch.where(valid, lse - lf.gather(1, tsafe[:, None])[:, 0], torch.zeros_like(lse))
    p = torch.exp(lf - lse[:, None])
    p.scatter_add_(1, tsafe[:, None], -torch.ones_like(lse)[:, None])
    p = p * (valid.float() * grad_scale)[:, None]
    logits.copy_(p.to(logits.dtype))
    return loss


# ------------------------------------------------------------------------------------------------
# e4m3 KV quantisation (per head, per block of tokens)
# ------------------------------------------------------------------------------------------------

E4M3_MAX = 448.0


def kv_quantize_e4m3(x: torch.Tensor, block_tokens: int = 128, want_pow2: bool = False):
    """x [tokens, Hkv, D] -> (q float8_e4m3fn [tokens, Hkv, D], scales fp32 [blocks, Hkv][, pow2 scales])."""
    T, Hkv, D = x.shape
    blocks = (T + block_tokens - 1) // block_tokens
    if _ext.use_cuda_kernels(x) and x.dtype == torch.bfloat16:
        q = torch.empty(T, Hkv, D, device=x.device, dtype=torch.uint8)
        scales = torch.empty(blocks, Hkv, device=x.device, dtype=torch.float32)
        p2 = torch.empty_like(scales) if want_pow2 else None
        _ext.C().kv_quant_e4m3(x.contiguous(), q, scales, p2, block_tokens)
        q = q.view(torch.float8_e4m3fn)
        return (q, scales, p2) if want_pow2 else (q, scales)
    pad = blocks * block_tokens - T
    xf = torch.nn.functional.pad(x.float(), (0, 0, 0, 0, 0, pad)).view(blocks, block_tokens, Hkv, D)
    amax = xf.abs().amax(dim=(1, 3))
    scales = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (xf / scales[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).view(-1, Hkv, D)[:T].to(torch.float8_e4m3fn)
    if want_pow2:
        return q, scales, torch.exp2(torch.ceil(torch.log2(scales)))
    return q, scales


def kv_dequantize_e4m3(q: torch.Tensor, scales: torch.Tensor, block_tokens: int = 128,
                       dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    T, Hkv, D = q.shape
    if _ext.use_cuda_kernels(q) and dtype == torch.bfloat16:
        x = torch.empty(T, Hkv, D, device=q.device, dtype=dtype)
        _ext.C().kv_dequant_e4m3(q.view(torch.uint8).contiguous(), scales.contiguous(), x, block_tokens)
        return x
    idx = torch.arange(T, device=q.device) // block_tokens
    return (q.float() * scales[idx][:, :, None]).to(dtype)


# ------------------------------------------------------------------------------------------------
# AdamW with a split fp32 master weight, and gradient-norm helpers
# ------------------------------------------------------------------------------------------------


def split_master(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 -> (hi: bf16 = round-half-up of w, lo: int16 remainder); hi/lo reconstruct w exactly."""
    bits = w.contiguous().view(torch.int32)
    hi = ((bits + 0x8000) >> 16).to(torch.int16)
    lo = (bits - (hi.to(torch.int32) << 16)).to(torch.int16)
    return hi.view(torch.bfloat16), lo


def join_master(hi: torch.Tensor, lo: torch.Tensor) -> torch.Tensor:
    return ((hi.view(torch.int16).to(torch.int32) << 16) + lo.to(torch.int32)).view(torch.float32)


def adamw_step_(p_hi, p_lo, m, v, g, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
                grad_scale_tensor: Optional[torch.Tensor] = None) -> None:
    """One AdamW update of a flat shard (length a multiple of 4)."""
    if _ext.use_cuda_kernels(g):
        _ext.C().adamw(p_hi.view(torch.int16), p_lo, m, v, g, lr, beta1, beta2, eps, weight_decay, step, grad_scale,
                       grad_scale_tensor)
        return
    gs = grad_scale * (float(grad_scale_tensor.item()) if grad_scale_tensor is not None else 1.0)
    w = join_master(p_hi, p_lo)
    gg = g.float() * gs
    m.mul_(beta1).add_(gg, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gg, gg, value=1 - beta2)
    mhat = m / (1 - beta1 ** step)
    vhat = v / (1 - beta2 ** step)
    w = w * (1 - lr * weight_decay) - lr * mhat / (vhat.sqrt() + eps)
    hi, lo = split_master(w)
    p_hi.copy_(hi)
    p_lo.copy_(lo)


def sumsq_(g: torch.Tensor, out: torch.Tensor) -> None:
    """out[0] += sum(g^2) for a flat fp32 buffer (length a multiple of 4)."""
    if _ext.use_cuda_kernels(g):
        _ext.C().sumsq(g, out)
    else:
        out[0] += g.float().pow(2).sum()


def clip_coef_(sumsq: torch.Tensor, scale: float, max_norm: float, coef: torch.Tensor, norm_out: torch.Tensor) -> None:
    """coef = min(1, max_norm / (sqrt(sumsq) * scale + 1e-6)) computed on the device (no host sync)."""
    if _ext.use_cuda_kernels(sumsq):
        _ext.C().clip_coef(sumsq, scale, max_norm, coef, norm_out)
    else:
        norm = sumsq[0].sqrt() * scale
        norm_out.fill_(norm)
        coef.fill_(min(1.0, max_norm / (float(norm) + 1e-6)) if max_norm > 0 else 1.0)
