"""Block-sparse ring attention.

The reference documents ``SparseRingAttention`` / ``SparsePattern`` ("hardware-efficient sparse
patterns", "13.3x speedup with sliding window", README.md:168-172,331,346) without shipping the
module. ``SparsePattern`` is a 128x128-block mask: a causal sliding window of ``window_tokens`` plus
every ``global_every``-th key block visible to everyone. The attention kernels evaluate it per tile
from global token positions, so masked tiles are neither loaded nor multiplied, and ring steps in
which no tile survives are never launched nor pulled (``RingContext.active_steps``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..ops.attention import MaskSpec, RingContext, ring_flash_attention, shard_positions, step_has_work


@dataclass(frozen=True)
class SparsePattern:
    block: int = 128
    window_tokens: int = 4096
    global_every: int = 64
    causal: bool = True

    def __post_init__(self):
        if self.block != 128:
            raise ValueError("the kernels evaluate the mask at 128x128 granularity")
        if self.window_tokens % self.block != 0:
            raise ValueError("window_tokens must be a multiple of the block size")

    @property
    def window_blocks(self) -> int:
        return self.window_tokens // self.block

    def mask_spec(self) -> MaskSpec:
        return MaskSpec(causal=self.causal, window_blocks=self.window_blocks, global_every=self.global_every)

    def block_allowed(self, qb: int, kb: int) -> bool:
        return self.mask_spec().block_allowed(qb, kb)

    def tiles_for(self, q_range: Tuple[int, int], kv_range: Tuple[int, int]) -> List[Tuple[int, int]]:
        """Compressed tile list: (q block, kv block) pairs kept inside the two token ranges."""
        q0, q1 = q_range[0] // self.block, (q_range[1] - 1) // self.block
        k0, k1 = kv_range[0] // self.block, (kv_range[1] - 1) // self.block
        out = []
        for qb in range(q0, q1 + 1):
            lo = max(k0, qb - self.window_blocks + 1)
            hi = min(k1, qb if self.causal else qb + self.window_blocks - 1)
            kept = set(range(lo, hi + 1)) if lo <= hi else set()
            if self.global_every > 0:
                g = ((k0 + self.global_every - 1) // self.global_every) * self.global_every
                top = min(k1, qb) if self.causal else k1
                kept.update(range(g, top + 1, self.global_every))
            out.extend((qb, kb) for kb in sorted(kept))
        return out

    def step_is_empty(self, rank: int, step: int, degree: int, seq_len: int, layout: str = "zigzag") -> bool:
        """True when ring step `step` of `rank` (keys of rank - step) contains no kept tile."""
        owner = (rank - step) % degree
        local = seq_len // degree
        return not step_has_work(self.mask_spec(), shard_positions(rank, degree, seq_len, layout), local,
                                 shard_positions(owner, degree, seq_len, layout), local)

    def density(self, seq_len: int) -> float:
        """Fraction of the causal (or full) block matrix that is kept."""
        n = seq_len // self.block
        kept = 0
        for qb in range(n):
            w = min(self.window_blocks, qb + 1)
            g = 0
            if self.global_every > 0:
                first_window = qb - w + 1
                g = (first_window + self.global_every - 1) // self.global_every  # globals strictly below the window
            kept += w + max(0, g)
        total = n * (n + 1) // 2 if self.causal else n * n
        return kept / max(1, total)


class SparseRingAttention(nn.Module):
    """Attention module over a (possibly ring-sharded) sequence with a SparsePattern mask."""

    def __init__(self, pattern: SparsePattern, num_heads: int, num_kv_heads: int, head_dim: int = 128, group=None,
                 ring: Optional[RingContext] = None, seq_len: Optional[int] = None):
        super().__init__()
        if head_dim != 128:
            raise ValueError("the attention kernels are built for head_dim 128")
        self.pattern, self.num_heads, self.num_kv_heads, self.head_dim = pattern, num_heads, num_kv_heads, head_dim
        self.group, self.ring, self.seq_len = group, ring, seq_len
        self.scale = 1.0 / math.sqrt(head_dim)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        ring = self.ring
        if ring is not None and ring.mask != self.pattern.mask_spec():
            ring = RingContext(rank=ring.rank, degree=ring.degree, seq_len=ring.seq_len, layout=ring.layout,
                               group=ring.group, peer=ring.peer, mask=self.pattern.mask_spec())
        return ring_flash_attention(q, k, v, causal=self.pattern.causal, scale=self.scale, ring=ring, group=self.group,
                                    sparse=self.pattern.mask_spec(), seq_len=self.seq_len)


__all__ = ["SparsePattern", "SparseRingAttention"]
