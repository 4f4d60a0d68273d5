"""Activation / optimizer-state offload policy (reference: zenyx/compiler/offload_policy.py:18-148).
Unlike the reference, copies go through pinned host buffers on a side stream and return an event
to wait on, so an offload does not stall the compute stream."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch


@dataclass
class OffloadPolicy:
    offload_large_activations: int = 100 << 20   # byte threshold
    offload_optimizer_states: bool = True
    recompute_instead_of_offload: bool = True


def make_offload_policy(gpu_memory_gb: float = 180.0, batch_size: int = 1) -> OffloadPolicy:
    """Threshold = 10 % of device memory divided by the number of sequences kept in flight."""
    threshold = int(gpu_memory_gb * (1 << 30) * 0.10 / max(1, batch_size))
    return OffloadPolicy(offload_large_activations=threshold)


class OffloadManager:
    def __init__(self, policy: Optional[OffloadPolicy] = None):
        self.policy = policy or OffloadPolicy()
        self._stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self._events: Dict[int, "torch.cuda.Event"] = {}
        self.bytes_offloaded = 0

    def should_offload(self, tensor: torch.Tensor) -> bool:
        return tensor.is_cuda and tensor.numel() * tensor.element_size() >= self.policy.offload_large_activations

    def maybe_offload(self, tensor: torch.Tensor) -> torch.Tensor:
        """Returns a pinned host copy when the tensor is a large CUDA tensor, else the tensor itself."""
        if not self.should_offload(tensor):
            return tensor
        host = torch.empty(tensor.shape, dtype=tensor.dtype, device="cpu", pin_memory=True)
        self._stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._stream):
            host.copy_(tensor, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        tensor.record_stream(self._stream)
        self._events[id(host)] = ev
        self.bytes_offloaded += tensor.numel() * tensor.element_size()
        return host

    def maybe_load(self, tensor: torch.Tensor, device: torch.device) -> torch.Tensor:
        if tensor.device == device:
            return tensor
        ev = self._events.pop(id(tensor), None)
        if ev is not None:
            ev.synchronize()
        return tensor.to(device, non_blocking=tensor.is_pinned() if tensor.device.type == "cpu" else False)

    def estimate_offload_savings(self, activation_bytes: int, pcie_gbs: float = 50.0,
                                 step_seconds: float = 1.0) -> Tuple[float, float]:
        """(GB freed, fraction of a step spent on the round trip if nothing overlapped)."""
        gb = activation_bytes / 1e9
        return gb, min(1.0, 2 * gb / pcie_gbs / max(step_seconds, 1e-9))
