"""FP8 (e4m3) KV-cache quantisation with per-head dynamic scaling.

The reference documents ``FP8KVQuantizer`` / ``QuantizedRingAttention`` ("per-head dynamic scaling",
"2x memory compression", README.md:156-160,329,344); the module is not in its tree, and what it
ships under that label is a per-tensor int8 emulation (zenyx/streaming/precision.py:8-16). Here K
and V are stored as real e4m3 with one fp32 scale per (KV head, block of ``block_tokens`` tokens),
scale = absmax / 448, produced by one kernel pass (``kv_quant_e4m3`` in csrc/fused/fused_ops.cu).
Power-of-two (UE8M0-style) scales are emitted on request for block-scaled tensor-core formats.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn

from ..ops import fused
from ..ops.attention import MaskSpec, RingContext, ring_flash_attention


class FP8KVQuantizer:
    def __init__(self, num_kv_heads: int = 8, head_dim: int = 128, block_tokens: int = 128, fmt: str = "e4m3",
                 scale: str = "absmax"):
        if fmt != "e4m3":
            raise ValueError("only e4m3 is supported for KV storage")
        if scale != "absmax":
            raise ValueError("only absmax scaling is supported")
        self.num_kv_heads, self.head_dim, self.block_tokens = num_kv_heads, head_dim, block_tokens

    def quantize(self, x: torch.Tensor, want_pow2: bool = False):
        """x [B, S, Hkv, D] (or [S, Hkv, D]) -> (q float8_e4m3fn same shape, scales fp32 [B, S/block, Hkv])."""
        squeeze = x.dim() == 3
        xb = x.unsqueeze(0) if squeeze else x
        B, S, H, D = xb.shape
        if S % self.block_tokens != 0:
            raise ValueError("sequence length must be a multiple of block_tokens")
        out = fused.kv_quantize_e4m3(xb.reshape(B * S, H, D), self.block_tokens, want_pow2)
        q = out[0].view(B, S, H, D)
        scales = out[1].view(B, S // self.block_tokens, H)
        if squeeze:
            q, scales = q[0], scales[0]
        if want_pow2:
            p2 = out[2].view(B, S // self.block_tokens, H)
            return q, scales, (p2[0] if squeeze else p2)
        return q, scales

    def dequantize(self, q: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        squeeze = q.dim() == 3
        qb = q.unsqueeze(0) if squeeze else q
        B, S, H, D = qb.shape
        x = fused.kv_dequantize_e4m3(qb.reshape(B * S, H, D), scales.reshape(-1, H), self.block_tokens, dtype)
        x = x.view(B, S, H, D)
        return x[0] if squeeze else x

    def roundtrip(self, x: torch.Tensor) -> torch.Tensor:
        """What attention sees when the cache is held in e4m3."""
        q, s = self.quantize(x)
        return self.dequantize(q, s, x.dtype)

    @property
    def compression_ratio(self) -> float:
        """bf16 bytes / (e4m3 bytes + scales)."""
        per_block = self.block_tokens * self.head_dim
        return 2.0 * per_block / (per_block + 4.0)

    def relative_error(self, x: torch.Tensor) -> float:
        y = self.roundtrip(x)
        return float(((y.float() - x.float()).norm() / (x.float().norm() + 1e-12)).item())


class QuantizedRingAttention(nn.Module):
    """Ring attention whose K/V pass through the e4m3 cache format.

    K and V are quantised once per call (after RoPE); every ring step then works on the quantised
    values. When the ``RingContext`` carries peer buffers built with ``fp8_block_tokens``
    (``zenyx_b200.parallel.peer.RingBuffers``), the e4m3 codes and their scales are what sits in the
    peer-visible slots and what each ring step pulls over NVLink (half the bytes of bf16); the pulling
    rank expands them to bf16 right before its attention kernel. The tensor-core products themselves
    run in bf16: an e4m3 ``kind::f8f6f4`` MMA path is not built.
    """

    def __init__(self, num_heads: int, num_kv_heads: int, head_dim: int = 128, block_tokens: int = 128, group=None,
                 ring: Optional[RingContext] = None, causal: bool = True, sparse: Optional[MaskSpec] = None,
                 seq_len: Optional[int] = None):
        super().__init__()
        self.quantizer = FP8KVQuantizer(num_kv_heads, head_dim, block_tokens)
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.group, self.ring, self.causal, self.sparse, self.seq_len = group, ring, causal, sparse, seq_len
        self.scale = 1.0 / math.sqrt(head_dim)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        return ring_flash_attention(q, k, v, causal=self.causal, scale=self.scale, ring=self.ring, group=self.group,
                                    kv_fp8=self.quantizer, sparse=self.sparse, seq_len=self.seq_len)


__all__ = ["FP8KVQuantizer", "QuantizedRingAttention"]
