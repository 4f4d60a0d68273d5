"""Three-tier KV block store with the reference's interface (zenyx/streaming/kv_tiering.py:11-73):
``KVTierManager(t0_capacity, t1_capacity)`` with ``put`` / ``prefetch_to_t0`` / ``evict_from_t0``,
``KVBlockRef`` and ``build_ring_timeline``. Differences: T1 holds *pinned* host tensors and copies
run on a side stream (``cudaMemcpyAsync``), T0 eviction can follow a known future (``next_use``)
instead of LRU, and T2 is a real file tier when ``nvme_path`` is given (the reference's T2 is a
Python dict). The plan-driven manager for ring attention is
``zenyx_b200.train.belayd_kv_cache_tiering.BeladyKVCacheTieringManager``."""
from __future__ import annotations

import os
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional

import torch

from ..ops import _ext


@dataclass
class KVBlockRef:
    block_id: Hashable
    seq_start: int
    seq_end: int


def build_ring_timeline(num_blocks: int) -> Dict[str, List[int]]:
    """Forward visits blocks 0..n-1, backward visits them in reverse."""
    fwd = list(range(num_blocks))
    return {"forward": fwd, "backward": list(reversed(fwd))}


class KVTierManager:
    def __init__(self, t0_capacity: int = 2, t1_capacity: int = 32, device: Optional[torch.device] = None,
                 nvme_path: Optional[str] = None, block_bytes: Optional[int] = None, t2_slots: int = 1024):
        self.t0_capacity, self.t1_capacity = t0_capacity, t1_capacity
        self.device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.t0: "OrderedDict[Hashable, torch.Tensor]" = OrderedDict()
        self.t1: "OrderedDict[Hashable, torch.Tensor]" = OrderedDict()
        self.t2: Dict[Hashable, object] = {}
        self.next_use: Dict[Hashable, float] = {}
        self._stream = torch.cuda.Stream() if self.device.type == "cuda" else None
        self._file = None
        self._slots: Dict[Hashable, int] = {}
        self._meta: Dict[Hashable, tuple] = {}
        self.nvme_path = nvme_path
        if nvme_path is not None:
            if block_bytes is None:
                raise ValueError("a file tier needs block_bytes")
            os.makedirs(os.path.dirname(os.path.abspath(nvme_path)) or ".", exist_ok=True)
            self._file = _ext.host().FileTier(nvme_path, int(block_bytes), t2_slots, 2, False)
            self.block_bytes = int(block_bytes)

    # tier 2 ----------------------------------------------------------------------------------
    def _t2_store(self, block_id, host: torch.Tensor) -> None:
        if self._file is None:
            self.t2[block_id] = host
            return
        slot = self._slots.setdefault(block_id, len(self._slots))
        host = host.contiguous()
        nbytes = host.numel() * host.element_size()
        if self._file.wait(self._file.write_async(slot, host.data_ptr(), nbytes)) != 0:
            raise IOError(f"writing block {block_id!r} to {self.nvme_path} failed")
        self._meta[block_id] = (tuple(host.shape), host.dtype, nbytes)
        self.t2[block_id] = slot

    def _t2_load(self, block_id) -> torch.Tensor:
        if self._file is None:
            return self.t2[block_id]
        shape, dtype, nbytes = self._meta[block_id]
        host = torch.empty(shape, dtype=dtype)
        if self.device.type == "cuda":
            host = host.pin_memory()
        if self._file.wait(self._file.read_async(self._slots[block_id], host.data_ptr(), nbytes)) != 0:
            raise IOError(f"reading block {block_id!r} from {self.nvme_path} failed")
        return host

    # public API ------------------------------------------------------------------------------
    def put(self, block_id: Hashable, tensor: torch.Tensor) -> None:
        """New blocks enter at the bottom tier."""
        self._t2_store(block_id, tensor.detach().to("cpu"))

    def _to_t1(self, block_id, host: torch.Tensor) -> None:
        if self.device.type == "cuda" and not host.is_pinned():
            host = host.pin_memory()
        self.t1[block_id] = host
        self.t1.move_to_end(block_id)
        while len(self.t1) > self.t1_capacity:
            old_id, old = self.t1.popitem(last=False)
            if old_id not in self.t2:
                self._t2_store(old_id, old)

    def prefetch_to_t0(self, block_id: Hashable) -> torch.Tensor:
        if block_id in self.t0:
            self.t0.move_to_end(block_id)
            return self.t0[block_id]
        if block_id in self.t1:
            host = self.t1[block_id]
            self.t1.move_to_end(block_id)
        elif block_id in self.t2:
            host = self._t2_load(block_id)
            self._to_t1(block_id, host)
            host = self.t1[block_id]
        else:
            raise KeyError(block_id)
        while len(self.t0) >= self.t0_capacity:
            self.evict_from_t0(self._victim())
        if self._stream is not None:
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                dev = host.to(self.device, non_blocking=True)
            torch.cuda.current_stream().wait_stream(self._stream)
        else:
            dev = host.to(self.device)
        self.t0[block_id] = dev
        return dev

    def _victim(self) -> Hashable:
        if self.next_use:
            return max(self.t0, key=lambda b: self.next_use.get(b, float("inf")))
        return next(iter(self.t0))

    def evict_from_t0(self, block_id: Hashable) -> None:
        dev = self.t0.pop(block_id, None)
        if dev is None:
            return
        if block_id not in self.t1 and block_id not in self.t2:
            host = torch.empty(dev.shape, dtype=dev.dtype, pin_memory=self.device.type == "cuda")
            host.copy_(dev)
            self._to_t1(block_id, host)

    def location(self, block_id: Hashable) -> Optional[str]:
        return "t0" if block_id in self.t0 else "t1" if block_id in self.t1 else "t2" if block_id in self.t2 else None
