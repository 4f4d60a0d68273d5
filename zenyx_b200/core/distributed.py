"""``DistributedTrainingManager`` and host-side failure detection.

The reference documents ``zenyx.core.distributed.DistributedTrainingManager`` ("distributed training
helpers", README.md:195,347) without code; its only failure handling is the 1800 s init timeout and
an async-to-sync retry (zenyx/distributed/communication.py:96-101,136-140). Here:

* ``DistributedTrainingManager`` = bootstrap + mesh + planner glue;
* ``Heartbeat`` = a per-rank watchdog over the process group's key-value store. Ranks publish the
  step they are about to start; a rank whose entry stops changing for ``timeout_s`` is reported
  dead, so the others can stop BEFORE their next launch instead of blocking in a collective. It is
  purely host-side: no kernel and no GPU wait is involved in detecting a failure.
* ``FaultInjector`` = host-side fault injection from ``ZX_FAULT_INJECT=step:rank:kind`` with kinds
  ``raise`` (exception), ``exit`` (process leaves between steps) and ``stall`` (stops beating).
  A device-side fault injector is deliberately not provided.
"""
from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch.distributed as dist

from ..parallel.communication import DistributedContext, init_distributed_from_env
from ..parallel.groups import Mesh


class RankFailure(RuntimeError):
    pass


class Heartbeat:
    def __init__(self, store=None, rank: int = 0, world_size: int = 1, timeout_s: float = 30.0, prefix: str = "zx_hb"):
        self.store, self.rank, self.world_size, self.timeout_s, self.prefix = store, rank, world_size, timeout_s, prefix
        self._seen: Dict[int, tuple] = {}
        self._stalled = False

    @classmethod
    def from_process_group(cls, timeout_s: float = 30.0) -> "Heartbeat":
        if not (dist.is_available() and dist.is_initialized()):
            return cls(None, 0, 1, timeout_s)
        store = dist.distributed_c10d._get_default_store()
        return cls(store, dist.get_rank(), dist.get_world_size(), timeout_s)

    def beat(self, step: int) -> None:
        if self.store is None or self._stalled:
            return
        self.store.set(f"{self.prefix}/{self.rank}", f"{step}:{time.time():.3f}")

    def stall(self) -> None:
        """Test hook: stop publishing beats (simulates a hung rank without hanging anything)."""
        self._stalled = True

    def dead_peers(self, now: Optional[float] = None) -> List[int]:
        """Ranks whose beat has not changed for longer than the timeout."""
        if self.store is None:
            return []
        now = time.time() if now is None else now
        dead = []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            key = f"{self.prefix}/{r}"
            try:
                val = self.store.get(key).decode() if self.store.check([key]) else None
            except Exception:  # noqa: BLE001
                val = None
            prev = self._seen.get(r)
            if val is None:
                first = prev[1] if prev else now
                self._seen[r] = (None, first)
                if now - first > self.timeout_s:
                    dead.append(r)
                continue
            if prev is None or prev[0] != val:
                self._seen[r] = (val, now)
            elif now - prev[1] > self.timeout_s:
                dead.append(r)
        return dead

    def check(self) -> None:
        dead = self.dead_peers()
        if dead:
            raise RankFailure(f"ranks {dead} have not reported for {self.timeout_s:.0f}s")


@dataclass
class FaultSpec:
    step: int
    rank: int
    kind: str


class FaultInjector:
    KINDS = ("raise", "exit", "stall")

    def __init__(self, spec: Optional[str] = None, rank: int = 0):
        spec = os.environ.get("ZX_FAULT_INJECT", "") if spec is None else spec
        self.rank = rank
        self.faults: List[FaultSpec] = []
        for item in filter(None, spec.split(",")):
            s, r, k = item.split(":")
            if k not in self.KINDS:
                raise ValueError(f"unknown fault kind {k!r}; expected one of {self.KINDS}")
            self.faults.append(FaultSpec(int(s), int(r), k))

    def maybe_fail(self, step: int, heartbeat: Optional[Heartbeat] = None) -> None:
        """Call between steps (no kernel or collective of this rank in flight)."""
        for f in self.faults:
            if f.step == step and f.rank == self.rank:
                if f.kind == "raise":
                    raise RankFailure(f"injected failure on rank {self.rank} at step {step}")
                if f.kind == "exit":
                    sys.stdout.flush()
                    os._exit(17)
                if f.kind == "stall" and heartbeat is not None:
                    heartbeat.stall()


class DistributedTrainingManager:
    """Bootstrap + mesh + plan for one training job."""

    def __init__(self, ring_degrees: Sequence[int] = (1,), heartbeat_timeout_s: float = 30.0):
        self.ctx: DistributedContext = init_distributed_from_env()
        self.mesh = Mesh(ring_degrees, world=self.ctx.world_size, rank=self.ctx.rank)
        self.heartbeat = Heartbeat.from_process_group(heartbeat_timeout_s)
        self.faults = FaultInjector(rank=self.ctx.rank)

    @property
    def rank(self) -> int:
        return self.ctx.rank

    @property
    def world_size(self) -> int:
        return self.ctx.world_size

    def plan(self, model_cfg, seq_len: int, global_batch: int, ring_degree: Optional[int] = None):
        from ..planner import plan

        return plan(model_cfg, seq_len, global_batch, self.ctx.world_size, ring_degree=ring_degree)

    def elastic_ring_degree(self, alive_ranks: int, preferred: int) -> int:
        """Largest prepared ring degree that still divides the surviving world (8 -> 4 ranks = ring 8 -> 4)."""
        for d in sorted(self.mesh._cp, reverse=True):
            if d <= preferred and alive_ranks % d == 0:
                return d
        return 1

    def before_step(self, step: int) -> None:
        self.heartbeat.beat(step)
        self.faults.maybe_fail(step, self.heartbeat)
        self.heartbeat.check()
