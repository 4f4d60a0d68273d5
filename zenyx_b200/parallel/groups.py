"""The DP x CP process mesh and its regrouping when the ring degree changes.

World ranks are laid out CP-fastest: rank = dp_index * cp + cp_index, so a ring is a block of
consecutive ranks (same NVSwitch domain, and what the curriculum needs: growing the ring merges
neighbouring blocks). Process groups for every ring degree a run may use are created once, up
front, because ``new_group`` is collective over the whole world. The reference has no mesh: its
only grouping is ``TopologyConfig(intra_node_ranks, inter_node_ranks)`` (zenyx/runtime/scheduler.py:19-22).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch.distributed as dist


@dataclass(frozen=True)
class ParallelLayout:
    """Degrees of one training phase. ``cp * dp * tp * pp == world``."""

    cp: int = 1
    dp: int = 1
    tp: int = 1
    pp: int = 1

    @property
    def world(self) -> int:
        return self.cp * self.dp * self.tp * self.pp

    def coords(self, rank: int) -> Dict[str, int]:
        return {"cp": rank % self.cp, "dp": (rank // self.cp) % self.dp}


def cp_group_ranks(world: int, cp: int) -> List[List[int]]:
    assert world % cp == 0, f"ring degree {cp} does not divide world size {world}"
    return [list(range(b * cp, (b + 1) * cp)) for b in range(world // cp)]


def dp_group_ranks(world: int, cp: int) -> List[List[int]]:
    return [list(range(i, world, cp)) for i in range(cp)]


class Mesh:
    """Holds the CP and DP process groups for a set of ring degrees."""

    def __init__(self, degrees: Sequence[int] = (1,), world: Optional[int] = None, rank: Optional[int] = None):
        self.initialized = dist.is_available() and dist.is_initialized()
        self.world = world if world is not None else (dist.get_world_size() if self.initialized else 1)
        self.rank = rank if rank is not None else (dist.get_rank() if self.initialized else 0)
        self._cp: Dict[int, object] = {}
        self._dp: Dict[int, object] = {}
        for d in sorted(set(int(x) for x in degrees)):
            if self.world % d != 0:
                raise ValueError(f"ring degree {d} does not divide world size {self.world}")
            if not self.initialized or self.world == 1:
                self._cp[d] = None
                self._dp[d] = None
                continue
            for ranks in cp_group_ranks(self.world, d):
                g = dist.new_group(ranks) if len(ranks) > 1 else None
                if self.rank in ranks:
                    self._cp[d] = g
            for ranks in dp_group_ranks(self.world, d):
                g = dist.new_group(ranks) if len(ranks) > 1 else None
                if self.rank in ranks:
                    self._dp[d] = g

    def layout(self, cp: int) -> ParallelLayout:
        return ParallelLayout(cp=cp, dp=self.world // cp)

    def cp_group(self, cp: int):
        return self._cp[cp]

    def dp_group(self, cp: int):
        return self._dp[cp]

    def cp_rank(self, cp: int) -> int:
        return self.rank % cp

    def dp_rank(self, cp: int) -> int:
        return self.rank // cp
