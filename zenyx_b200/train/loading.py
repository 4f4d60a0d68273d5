"""Chunked state-dict loading (reference: zenyx/train/loading.py:11-30): a flat
``{parameter name: tensor}`` map is copied into a model a few tensors at a time through pinned
host memory. Unknown and shape-mismatched keys are reported instead of skipped silently."""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch
import torch.nn as nn


def load_state_dict_chunked(model: nn.Module, state_dict: Dict[str, torch.Tensor], chunk_size: int = 64,
                            strict: bool = False) -> Tuple[List[str], List[str]]:
    """Returns (missing keys, unexpected keys). ``strict`` raises when either is non-empty."""
    targets = dict(model.named_parameters())
    targets.update(dict(model.named_buffers()))
    if hasattr(model, "named_flat_parameters"):   # flat-buffer models expose dotted canonical names too
        targets.update(dict(model.named_flat_parameters()))
    keys = list(state_dict.keys())
    unexpected: List[str] = []
    loaded = set()
    with torch.no_grad():
        for i in range(0, len(keys), max(1, chunk_size)):
            staged = []
            for k in keys[i: i + chunk_size]:
                dst = targets.get(k)
                if dst is None:
                    unexpected.append(k)
                    continue
                src = state_dict[k]
                if tuple(src.shape) != tuple(dst.shape):
                    raise ValueError(f"shape mismatch for {k!r}: checkpoint {tuple(src.shape)} vs model {tuple(dst.shape)}")
                if dst.is_cuda and src.device.type == "cpu" and not src.is_pinned():
                    src = src.pin_memory()
                staged.append((dst, src, k))
            for dst, src, k in staged:
                dst.copy_(src, non_blocking=dst.is_cuda)
                loaded.add(k)
            if staged and staged[0][0].is_cuda:
                torch.cuda.current_stream().synchronize()  # pinned sources of this chunk may now be released
    canonical = set(dict(model.named_flat_parameters()).keys()) if hasattr(model, "named_flat_parameters") else \
        set(dict(model.named_parameters()).keys()) | set(dict(model.named_buffers()).keys())
    missing = sorted(canonical - loaded)
    if strict and (missing or unexpected):
        raise KeyError(f"missing keys {missing}, unexpected keys {unexpected}")
    return missing, unexpected
