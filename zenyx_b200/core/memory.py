"""Memory budgeting for the three tiers (HBM / pinned DRAM / NVMe). The reference documents
``zenyx.core.memory`` ("memory management", a three-tier allocator, README.md:196,
ZENYX_2_0_PHASE_1_SUMMARY.md:49-52) without code."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from .hardware import HardwareDetector


@dataclass
class TierBudget:
    hbm_bytes: int
    dram_bytes: int
    nvme_bytes: int
    nvme_path: Optional[str]


def default_budget(hbm_fraction: float = 0.1, dram_fraction: float = 0.5, hbm_cap: int = 16 << 30) -> TierBudget:
    """KV budget defaults: min(16 GiB, 10 % of HBM), half of host DRAM, all free space of the file tier."""
    det = HardwareDetector()
    gpus = det.gpus()
    hbm = int(min(hbm_cap, hbm_fraction * gpus[0].hbm_bytes)) if gpus else hbm_cap
    path, free = det.nvme_candidate()
    return TierBudget(hbm, int(dram_fraction * det.host_dram_bytes()), int(free), path)


class PinnedPool:
    """Fixed-size pinned host blocks handed out and returned without re-pinning."""

    def __init__(self, block_bytes: int, num_blocks: int):
        self.block_bytes, self.num_blocks = block_bytes, num_blocks
        pin = torch.cuda.is_available()
        self._blocks = [torch.empty(block_bytes, dtype=torch.uint8, pin_memory=pin) for _ in range(num_blocks)]
        self._free = list(range(num_blocks))
        self._owner: Dict[int, int] = {}

    def acquire(self) -> Optional[torch.Tensor]:
        if not self._free:
            return None
        i = self._free.pop()
        t = self._blocks[i]
        self._owner[t.data_ptr()] = i
        return t

    def release(self, t: torch.Tensor) -> None:
        i = self._owner.pop(t.data_ptr())
        self._free.append(i)

    @property
    def free_blocks(self) -> int:
        return len(self._free)
