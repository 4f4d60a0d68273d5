"""``BeladyApproxCache`` with the reference's interface (zenyx/streaming/belady.py:8-58): the caller
feeds next-use steps, ``touch`` evicts the resident with the farthest next use when full. Capacity
may be counted in items (as in the reference) or in bytes (``size`` given to ``touch``). The
offline-optimal planner that knows the future by itself is
``zenyx_b200.train.belayd_kv_cache_tiering`` (C++: csrc/tier/belady_min.cpp)."""
from __future__ import annotations

import math
from typing import Dict, Hashable, List


class BeladyApproxCache:
    def __init__(self, capacity: int, unit: str = "items"):
        if unit not in ("items", "bytes"):
            raise ValueError("unit must be 'items' or 'bytes'")
        self.capacity, self.unit = capacity, unit
        self._next_use: Dict[Hashable, float] = {}
        self._resident: Dict[Hashable, int] = {}
        self.hits = 0
        self.misses = 0

    def update_future(self, item: Hashable, next_use_step: float) -> None:
        self._next_use[item] = next_use_step

    def __contains__(self, item: Hashable) -> bool:
        return item in self._resident

    @property
    def used(self) -> int:
        return sum(self._resident.values()) if self.unit == "bytes" else len(self._resident)

    def touch(self, item: Hashable, size: int = 1) -> List[Hashable]:
        """Marks `item` used now (inserting it if absent); returns what had to be evicted."""
        if item in self._resident:
            self.hits += 1
            return []
        self.misses += 1
        cost = size if self.unit == "bytes" else 1
        evicted: List[Hashable] = []
        while self._resident and self.used + cost > self.capacity:
            victim = max(self._resident, key=lambda k: self._next_use.get(k, math.inf))
            del self._resident[victim]
            evicted.append(victim)
        self._resident[item] = cost
        return evicted

    def evict(self, item: Hashable) -> None:
        self._resident.pop(item, None)

    def resident(self) -> List[Hashable]:
        return list(self._resident)
