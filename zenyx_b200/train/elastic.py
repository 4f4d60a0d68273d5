"""Elastic recovery on the host: when a rank stops, the survivors agree on who is left, form a new
(smaller) process group, reload the last checkpoint and go on.

Everything here happens between steps and on the host: failures are noticed through the heartbeat in
the c10d store (``core/distributed.Heartbeat``) or through a collective that ran into its
process-group time-out; no kernel waits on a dead peer (every in-kernel wait is bounded anyway). The
sharded optimizer state re-shards on load (``train/checkpoint.load`` reads all shards of the saving
world), so a checkpoint written by W ranks resumes on any W' that divides the flat parameter space.

The reference has no failure handling beyond a rendezvous time-out and an async->sync retry
(zenyx/distributed/communication.py:96-101,123-140).

Limits: the rank that hosts the original TCP store (rank 0 of the first generation) must be among
the survivors for the roster exchange; later generations rendezvous through files in
``rendezvous_dir``, which must be visible to every rank (a node-local directory on one node).
"""
from __future__ import annotations

import datetime
import os
import time
from dataclasses import dataclass
from typing import Callable, Iterable, List, Optional, Tuple

import torch.distributed as dist

from ..core.distributed import Heartbeat, RankFailure
from ..utils.logging import get_logger


@dataclass
class ElasticConfig:
    rendezvous_dir: str
    backend: str = "gloo"
    heartbeat_timeout_s: float = 5.0
    settle_s: float = 1.0                 # time the survivors give each other to announce themselves
    group_timeout_s: float = 30.0         # process-group time-out of the re-formed group
    max_restarts: int = 3
    min_world: int = 1


class ElasticCoordinator:
    """Roster agreement and regrouping for one job. ``generation`` counts regroups."""

    def __init__(self, cfg: ElasticConfig):
        self.cfg = cfg
        self.generation = 0
        self.log = get_logger("zenyx_b200.elastic")
        os.makedirs(cfg.rendezvous_dir, exist_ok=True)

    # -- roster -------------------------------------------------------------------------------
    def survivors(self, dead: Iterable[int]) -> List[int]:
        """Every live rank announces itself under the next generation's prefix in the CURRENT store,
        waits ``settle_s``, then all read the same roster. Ranks in ``dead`` are not waited for."""
        store = dist.distributed_c10d._get_default_store()
        rank, world = dist.get_rank(), dist.get_world_size()
        gen = self.generation + 1
        store.set(f"zx_el/g{gen}/alive/{rank}", "1")
        deadline = time.time() + self.cfg.settle_s
        dead = set(dead)
        while time.time() < deadline:
            if all(store.check([f"zx_el/g{gen}/alive/{r}"]) for r in range(world) if r not in dead):
                break
            time.sleep(0.05)
        time.sleep(min(0.2, self.cfg.settle_s))   # let slower announcers land before everybody reads
        return [r for r in range(world) if store.check([f"zx_el/g{gen}/alive/{r}"])]

    # -- regroup ------------------------------------------------------------------------------
    def regroup(self, survivors: List[int]) -> Tuple[int, int]:
        """Leaves the current process group and joins the survivors' one. Returns (new rank, new world)."""
        old_rank = dist.get_rank()
        if old_rank not in survivors:
            raise RankFailure("this rank was declared dead by its peers")
        if len(survivors) < self.cfg.min_world:
            raise RankFailure(f"only {len(survivors)} ranks left, fewer than min_world={self.cfg.min_world}")
        self.generation += 1
        new_rank, new_world = survivors.index(old_rank), len(survivors)
        dist.destroy_process_group()
        path = os.path.join(self.cfg.rendezvous_dir, f"generation_{self.generation}")
        store = dist.FileStore(path, new_world)
        dist.init_process_group(self.cfg.backend, store=store, rank=new_rank, world_size=new_world,
                                timeout=datetime.timedelta(seconds=self.cfg.group_timeout_s))
        os.environ["RANK"], os.environ["WORLD_SIZE"] = str(new_rank), str(new_world)
        self.log.info("generation %d: rank %d -> %d of %d", self.generation, old_rank, new_rank, new_world)
        return new_rank, new_world


def run_elastic(make_trainer: Callable[[], "object"], make_data: Callable[[int, int], Iterable], loop_cfg,
                elastic_cfg: ElasticConfig, criterion=None, before_step: Optional[Callable[[int], None]] = None):
    """Runs ``train.loop.run`` and, when a peer stops, regroups the survivors and resumes from the last
    checkpoint until ``loop_cfg.steps`` optimizer steps are done.

    ``make_trainer()`` builds a fresh Trainer on the CURRENT default process group (it is called again
    after every regroup); ``make_data(rank, world)`` returns the batch iterator for that layout;
    ``loop_cfg`` needs a ``checkpoint_dir`` (and a ``checkpoint_every``) since resuming is how the
    survivors get back to a common state. ``before_step(step)`` is a hook for host-side fault injection.
    Returns (records of the last generation, coordinator).
    """
    from . import loop

    assert loop_cfg.checkpoint_dir, "elastic training resumes from checkpoints: set LoopConfig.checkpoint_dir"
    coord = ElasticCoordinator(elastic_cfg)
    log = coord.log
    while True:
        trainer = make_trainer()
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        hb = Heartbeat.from_process_group(elastic_cfg.heartbeat_timeout_s)
        hb.prefix = f"zx_hb_g{coord.generation}"

        def on_step(step, rec, _hook=before_step):
            if _hook is not None:
                _hook(step + 1)     # runs between steps: nothing of this rank is in flight

        try:
            records = loop.run(trainer, make_data(rank, world), criterion, loop_cfg, on_step=on_step, watchdog=hb)
            trainer.close()
            return records, coord
        except Exception as err:  # noqa: BLE001  (a dead peer shows up as a watchdog error or a failed collective)
            if world == 1 or coord.generation >= elastic_cfg.max_restarts:
                raise
            dead: List[int] = []
            deadline = time.time() + elastic_cfg.heartbeat_timeout_s + 2.0
            while time.time() < deadline and not dead:
                hb.beat(-1)                      # keep telling the others that this rank is alive
                dead = hb.dead_peers()
                if not dead:
                    time.sleep(0.1)
            if not dead:
                raise                            # everybody is alive: a genuine error, not a lost rank
            log.warning("ranks %s stopped (%s: %s); regrouping", dead, type(err).__name__, str(err)[:120])
            try:
                trainer.close()
            except Exception:  # noqa: BLE001
                pass
            left = coord.survivors(dead)
            coord.regroup(left)
