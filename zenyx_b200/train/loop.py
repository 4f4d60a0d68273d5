"""The training loop around ``Trainer``: logging, metrics JSONL, periodic checkpoints, resume,
host-side failure detection hooks (name from the reference's deleted ``zenyx/train/loop.py``,
ZENYX_2_0_DELIVERABLES.txt:190; its examples' loops write ``metrics.json``,
examples/03_expert_tpu_v5e8_training.py:220-228)."""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional

import torch

from ..utils import get_logger
from . import checkpoint as ckpt
from .trainer import Trainer


@dataclass
class LoopConfig:
    steps: int = 100
    log_every: int = 10
    checkpoint_every: int = 0          # 0: only at the end when checkpoint_dir is set
    checkpoint_dir: Optional[str] = None
    metrics_path: Optional[str] = None  # JSON-lines sink
    resume: bool = True
    tokens_per_step: Optional[int] = None


def run(trainer: Trainer, data_iter: Iterable, criterion=None, cfg: Optional[LoopConfig] = None,
        on_step: Optional[Callable[[int, Dict[str, Any]], None]] = None, watchdog=None) -> List[Dict[str, Any]]:
    """Runs ``cfg.steps`` optimizer steps; returns the per-step records.

    ``data_iter`` yields the batches of the WHOLE run from step 0; on resume from step ``s`` its first
    ``s`` batches are drawn and dropped, so the resumed run sees the batches an uninterrupted one would.

    ``watchdog`` is an optional ``zenyx_b200.core.distributed.Heartbeat``: it is beaten every step
    and, when it reports a dead peer, the loop stops before the next launch and raises.
    """
    cfg = cfg or LoopConfig()
    log = get_logger("zenyx_b200.train")
    rank = trainer.ctx.rank
    start = 0
    if cfg.resume and cfg.checkpoint_dir and ckpt.latest_step(cfg.checkpoint_dir) is not None:
        meta = ckpt.load(cfg.checkpoint_dir, trainer.model, trainer.optimizer)
        start = int(meta["step"])
        trainer.step = start
        cur = getattr(trainer.config, "curriculum", None)
        if cur is not None and meta.get("scheduler"):
            cur.load_state_dict(meta["scheduler"])
        log.info("resumed from step %d", start)
    records: List[Dict[str, Any]] = []
    sink = open(cfg.metrics_path, "a") if (cfg.metrics_path and rank == 0) else None
    it = iter(data_iter)
    for _ in range(start):      # a resumed run continues the batch stream where the checkpoint left it
        next(it)
    try:
        for step in range(start, cfg.steps):
            if watchdog is not None:
                watchdog.beat(step)
                dead = watchdog.dead_peers()
                if dead:
                    raise RuntimeError(f"ranks {dead} stopped responding before step {step}")
            batch, target = next(it)
            t0 = time.perf_counter()
            loss = trainer.train_step(batch, target, criterion)
            dt = time.perf_counter() - t0
            rec: Dict[str, Any] = {"step": step, "loss": loss, "step_s": dt}
            if cfg.tokens_per_step:
                rec["tokens_per_s"] = cfg.tokens_per_step / dt
                mcfg = getattr(trainer.model, "cfg", None)
                if trainer.engine is not None and mcfg is not None and hasattr(mcfg, "flops_per_token"):
                    from ..planner import HardwarePeaks   # model FLOPs utilisation against the measured sustained GEMM rate

                    peak = HardwarePeaks.load().bf16_tflops * 1e12 * trainer.ctx.world_size
                    rec["mfu"] = mcfg.flops_per_token(trainer.config.seq_len) * rec["tokens_per_s"] / peak
            if trainer.engine is not None:
                rec["ring_degree"] = trainer.engine.ring_degree
                rec["dp_degree"] = trainer.ctx.world_size // trainer.engine.ring_degree
            if torch.cuda.is_available():
                rec["peak_hbm_gb"] = torch.cuda.max_memory_allocated() / 1e9
            records.append(rec)
            if sink is not None:
                sink.write(json.dumps(rec) + "\n")
                sink.flush()
            if on_step is not None:
                on_step(step, rec)
            if rank == 0 and cfg.log_every and step % cfg.log_every == 0:
                log.info("step %d loss %.4f (%.2fs)", step, loss, dt)
            if cfg.checkpoint_dir and cfg.checkpoint_every and (step + 1) % cfg.checkpoint_every == 0:
                _save(trainer, cfg, step + 1, rec)
        if cfg.checkpoint_dir and records:
            _save(trainer, cfg, cfg.steps, records[-1])
    finally:
        if sink is not None:
            sink.close()
    return records


def _save(trainer: Trainer, cfg: LoopConfig, step: int, rec: Dict[str, Any]) -> None:
    cur = getattr(trainer.config, "curriculum", None)
    ckpt.save(cfg.checkpoint_dir, step, trainer.model, trainer.optimizer,
              scheduler_state=cur.state_dict() if cur is not None else None,
              config={"seq_len": trainer.config.seq_len, "global_batch": trainer.config.global_batch},
              metrics={k: v for k, v in rec.items() if isinstance(v, (int, float))})
