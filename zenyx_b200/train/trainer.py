"""``Trainer``: the public training entry point.

Two kinds of model are accepted:

* a ``LlamaConfig`` (or an existing ``LlamaModel``): the flagship path. The trainer builds the
  DP x CP mesh, ring buffers and the sharded fused optimizer (``LlamaEngine``);
  ``train_step(tokens, targets)`` takes the global batch [global_batch, seq_len] (host or device)
  and returns the global mean loss as a float.
* any other ``nn.Module``: the generic path with the reference's semantics
  (zenyx/train/trainer.py:16-57): ``train_step(batch, target, criterion)`` = forward, criterion,
  ``Scheduler.backward`` (bucketed data-parallel all-reduce, optimizer step at the accumulation
  boundary), mean of the loss over ranks.

Beyond the reference's four ``TrainerConfig`` fields (lr, accumulation_steps, overlap,
safety_barrier) the config carries what the reference's deleted training modules covered:
LR schedule, gradient clipping, mixed precision, checkpoint directory, ring curriculum.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Iterable, List, Optional, Sequence, Union

import torch
import torch.nn as nn

from ..memory import MemoryTracker
from ..models.llama import LlamaConfig, LlamaModel, RematPolicy
from ..parallel.communication import all_reduce, get_world_size, init_distributed_from_env
from ..runtime import Scheduler


@dataclass
class TrainerConfig:
    lr: float = 1e-3
    accumulation_steps: int = 1
    overlap: bool = True
    safety_barrier: bool = False
    # --- beyond the reference ---
    weight_decay: float = 0.01
    betas: tuple = (0.9, 0.95)
    max_grad_norm: Optional[float] = None
    lr_schedule: Optional[Callable[[int], float]] = None   # step -> learning rate
    precision: str = "fp32"                                # generic path: "fp32" | "bf16" | "fp16"
    # flagship path
    seq_len: int = 32768
    global_batch: int = 8
    ring_degree: int = 1
    ring_degrees: Sequence[int] = ()
    curriculum: Any = None                                 # a RingDegreeScheduler
    remat: Optional[RematPolicy] = None
    # storage of Adam's moments: "fp32", "bf16", or "auto" = the planner takes bf16 only where the memory it
    # frees buys at least 2 % of estimated step time (arithmetic and the master weights stay fp32 either way)
    optimizer_state_dtype: str = "auto"
    fused_peer: bool = True
    seed: int = 0


class Trainer:
    def __init__(self, model: Union[nn.Module, LlamaConfig], config: Optional[TrainerConfig] = None):
        self.config = config or TrainerConfig()
        self.ctx = init_distributed_from_env()
        self.memory = MemoryTracker()
        self.engine = None
        self.step = 0
        cfg = self.config
        if isinstance(model, LlamaConfig):
            from .engine import EngineConfig, LlamaEngine

            degrees = list(cfg.ring_degrees)
            if cfg.curriculum is not None:
                degrees += list(cfg.curriculum.degrees())
            self.engine = LlamaEngine(model, EngineConfig(
                seq_len=cfg.seq_len, global_batch=cfg.global_batch, ring_degree=cfg.ring_degree, ring_degrees=degrees,
                lr=cfg.lr, betas=cfg.betas, weight_decay=cfg.weight_decay, max_grad_norm=cfg.max_grad_norm,
                remat=cfg.remat, optimizer_state_dtype=cfg.optimizer_state_dtype, fused_peer=cfg.fused_peer,
                seed=cfg.seed), self.ctx)
            self.model = self.engine.model
            self.optimizer = self.engine.optimizer
            self.scheduler = None
            return
        self.model = model.to(self.ctx.device)
        self.optimizer = torch.optim.AdamW(self.model.parameters(), lr=cfg.lr, weight_decay=cfg.weight_decay)
        self.scheduler = Scheduler(accumulation_steps=cfg.accumulation_steps, enable_overlap=cfg.overlap)
        from .mixed_prec import MixedPrecision

        self.mixed = MixedPrecision(cfg.precision, self.ctx.device)

    # -------------------------------------------------------------------------------------------
    def _lr(self) -> float:
        return self.config.lr_schedule(self.step) if self.config.lr_schedule is not None else self.config.lr

    def train_step(self, batch: torch.Tensor, target: torch.Tensor, criterion: Optional[nn.Module] = None) -> float:
        if self.engine is not None:
            cur = self.config.curriculum
            if cur is not None:
                self.engine.set_ring_degree(cur.degree_at(self.step))
            local = self.engine.train_step(batch, target, lr=self._lr())
            loss = self.engine.global_loss(local)       # reads the loss back: the step's kernels have finished
            self._raise_on_kernel_error()
            if cur is not None:
                cur.step(loss)
            self.step += 1
            self.memory.snapshot()
            return loss
        if criterion is None:
            raise ValueError("the generic path needs a criterion: train_step(batch, target, criterion)")
        self.model.train()
        batch = batch.to(self.ctx.device, non_blocking=True)
        target = target.to(self.ctx.device, non_blocking=True)
        lr = self._lr()
        for g in self.optimizer.param_groups:
            g["lr"] = lr
        with self.mixed.autocast():
            output = self.scheduler.forward(self.model, batch)
            loss = criterion(output, target)
        if self.config.max_grad_norm is not None and self.scheduler._at_boundary():
            # clip between the gradient reduction and the optimizer step
            self.scheduler.backward(self.mixed.scale(loss), model=self.model, optimizer=None)
            self.mixed.unscale_(self.optimizer)
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.config.max_grad_norm)
            self.mixed.step(self.optimizer)
            self.optimizer.zero_grad(set_to_none=True)
            self.scheduler.step_count += 1
        elif self.mixed.uses_scaler:
            boundary = self.scheduler._at_boundary()
            self.scheduler.backward(self.mixed.scale(loss), model=self.model, optimizer=None)
            if boundary:
                self.mixed.step(self.optimizer)
                self.optimizer.zero_grad(set_to_none=True)
                self.scheduler.step_count += 1
        else:
            self.scheduler.backward(loss, model=self.model, optimizer=self.optimizer)
        reduced = all_reduce(loss.detach().clone().float(), op="sum", async_op=False,
                             safety_barrier=self.config.safety_barrier)
        self.step += 1
        self.memory.snapshot()
        return float(reduced.item() / get_world_size())

    def _raise_on_kernel_error(self) -> None:
        """Reads the device status word that the kernels' bounded waits write when they give up (a peer
        that never raised its flag, a barrier that ran out). Raises ``KernelError`` so that the caller, or
        ``train.elastic.run_elastic``, stops instead of training on from a half-reduced update. Called where
        the step has already synchronised, so it costs one 16-byte read."""
        if self.ctx.device.type != "cuda":
            return
        from ..ops import _ext

        _ext.check_status()

    def fit(self, data_iter: Iterable, criterion: Optional[nn.Module] = None, steps: int = 1) -> List[float]:
        losses: List[float] = []
        for i, (batch, target) in enumerate(data_iter):
            if i >= steps:
                break
            losses.append(self.train_step(batch, target, criterion))
        return losses

    def close(self) -> None:
        if self.engine is not None:
            self.engine.close()


__all__ = ["Trainer", "TrainerConfig"]
