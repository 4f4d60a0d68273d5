"""Device-memory snapshots (reference: zenyx/memory/tracker.py:10-34). The history is a bounded
ring (the reference appends one snapshot per training step forever)."""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, Optional

import torch


@dataclass
class MemorySnapshot:
    allocated_bytes: int
    reserved_bytes: int
    peak_allocated_bytes: int = 0


class MemoryTracker:
    def __init__(self, history: int = 1024):
        self.snapshots: Deque[MemorySnapshot] = deque(maxlen=history)
        self._first: Optional[MemorySnapshot] = None

    def snapshot(self) -> MemorySnapshot:
        if torch.cuda.is_available():
            snap = MemorySnapshot(torch.cuda.memory_allocated(), torch.cuda.memory_reserved(),
                                  torch.cuda.max_memory_allocated())
        else:
            snap = MemorySnapshot(0, 0, 0)
        if self._first is None:
            self._first = snap
        self.snapshots.append(snap)
        return snap

    def possible_leak(self, threshold_bytes: int = 64 << 20) -> bool:
        """True when allocated memory grew by more than the threshold since the first snapshot."""
        if self._first is None or not self.snapshots:
            return False
        return self.snapshots[-1].allocated_bytes - self._first.allocated_bytes > threshold_bytes
