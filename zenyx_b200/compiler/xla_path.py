"""``remat_or_checkpoint`` / ``maybe_offload_large_tensor`` keep the names of the reference's
zenyx/compiler/xla_path.py:15-38. There is no XLA here (nor in the reference file, which only calls
``torch.utils.checkpoint``); the JAX/TPU backend is intentionally not part of this framework."""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch.utils.checkpoint import checkpoint


@dataclass
class XLACheckpointPolicy:
    offload_threshold_bytes: int = 8 << 20


def remat_or_checkpoint(fn, *args, **kwargs):
    """Runs fn under activation checkpointing when a gradient may be needed, plainly otherwise.
    Errors raised by fn propagate (the reference swallows them and silently reruns fn)."""
    needs = torch.is_grad_enabled() and any(isinstance(a, torch.Tensor) and a.requires_grad for a in args)
    if not needs:
        return fn(*args, **kwargs)
    return checkpoint(fn, *args, use_reentrant=False, **kwargs)


def maybe_offload_large_tensor(tensor: torch.Tensor, policy: XLACheckpointPolicy | None = None) -> torch.Tensor:
    policy = policy or XLACheckpointPolicy()
    if tensor.numel() * tensor.element_size() < policy.offload_threshold_bytes or not tensor.is_cuda:
        return tensor
    host = torch.empty(tensor.shape, dtype=tensor.dtype, device="cpu", pin_memory=True)
    host.copy_(tensor.detach(), non_blocking=True)
    torch.cuda.current_stream().synchronize()
    return host
