"""Storage quantisation helpers with the reference's names (zenyx/streaming/precision.py:8-16).
The reference "emulates" FP8 with per-tensor int8; here the storage really is e4m3
(``torch.float8_e4m3fn``) with scale = absmax / 448. Per-head, per-block scaling for the KV cache is
``zenyx_b200.train.fp8_kv_quantization.FP8KVQuantizer``."""
from __future__ import annotations

from typing import Tuple

import torch

E4M3_MAX = 448.0


def quantize_to_fp8_storage(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    amax = x.detach().abs().amax().float()
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (x.float() / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q, scale


def dequantize_for_bf16_compute(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return (q.float() * scale).to(torch.bfloat16)
