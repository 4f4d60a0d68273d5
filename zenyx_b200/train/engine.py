"""Training engine of the Llama-shaped flagship: DP x CP mesh, ring buffers, sharded optimizer,
per-step orchestration. ``Trainer`` delegates to it when handed a ``LlamaModel`` configuration.

One optimizer step = ``global_batch`` sequences. Each data-parallel replica takes
``global_batch / dp`` of them, one sequence per micro-batch; inside a replica the sequence is
zigzag-sharded over the ``cp`` ring. Gradients accumulate in the model's flat fp32 buffer and are
reduced over ALL ranks (weights are replicated across both DP and CP) by the sharded optimizer.
The reference's counterpart is ``Trainer.train_step`` + ``Scheduler.backward``
(zenyx/train/trainer.py:36-49, zenyx/runtime/scheduler.py:135-163).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Sequence

import torch
import torch.distributed as dist

from ..models.llama import LlamaConfig, LlamaModel, RematPolicy
from ..ops.attention import MaskSpec, RingContext, shard_sequence
from ..parallel.communication import DistributedContext, init_distributed_from_env
from ..parallel.groups import Mesh
from ..parallel.zero import ZeroAdamW


@dataclass
class EngineConfig:
    seq_len: int = 32768
    global_batch: int = 8              # sequences per optimizer step
    ring_degree: int = 1               # context-parallel degree (cp); dp = world / cp
    ring_degrees: Sequence[int] = ()   # every degree a curriculum may switch to (groups/buffers built up front)
    lr: float = 3e-4
    betas: tuple = (0.9, 0.95)
    eps: float = 1e-8
    weight_decay: float = 0.1
    max_grad_norm: Optional[float] = 1.0
    remat: Optional[RematPolicy] = None    # None: ask the planner
    optimizer_state_dtype: str = "auto"    # "fp32" | "bf16" | "auto" (planner; fp32 when remat is given explicitly)
    fused_peer: bool = True                # False: NCCL reduce-scatter / all-gather baseline path
    layout: str = "zigzag"
    mask: MaskSpec = field(default_factory=MaskSpec)
    seed: int = 0
    barrier_timeout_ms: float = 60000.0


class LlamaEngine:
    def __init__(self, model_cfg: LlamaConfig, cfg: EngineConfig, ctx: Optional[DistributedContext] = None):
        self.ctx = ctx or init_distributed_from_env()
        self.cfg, self.model_cfg = cfg, model_cfg
        world, rank = self.ctx.world_size, self.ctx.rank
        degrees = sorted(set(list(cfg.ring_degrees) + [cfg.ring_degree]))
        self.mesh = Mesh(degrees, world=world, rank=rank)
        remat = cfg.remat
        state_dtype = cfg.optimizer_state_dtype
        if state_dtype not in ("auto", "fp32", "bf16"):
            raise ValueError("optimizer_state_dtype is 'auto', 'fp32' or 'bf16'")
        if remat is None:
            from ..planner import plan

            kw = {}
            if self.ctx.device.type == "cuda":   # size the plan for the memory this GPU really has
                kw = {"hbm_bytes": float(torch.cuda.mem_get_info(self.ctx.device)[1]), "memory_fraction": 0.93}
            # sized for the shortest ring among the prepared degrees: it holds the most tokens per rank
            chosen = plan(model_cfg, cfg.seq_len, cfg.global_batch, world, ring_degree=min(degrees),
                          optimizer_state_dtype=state_dtype, **kw)
            remat, state_dtype = chosen.remat, chosen.optimizer_state_dtype
        elif state_dtype == "auto":
            state_dtype = "fp32"
        self.optimizer_state_dtype = state_dtype
        dev = self.ctx.device
        sym_group = dist.group.WORLD if (world > 1 and dev.type == "cuda" and cfg.fused_peer) else None
        self.model = LlamaModel(model_cfg, device=dev, remat=remat, seed=cfg.seed, symmetric_group=sym_group,
                                world_size=world)
        self.optimizer = ZeroAdamW(self.model.flat, lr=cfg.lr, betas=cfg.betas, eps=cfg.eps,
                                   weight_decay=cfg.weight_decay, max_grad_norm=cfg.max_grad_norm,
                                   group=dist.group.WORLD if world > 1 else None, fused_peer=cfg.fused_peer,
                                   barrier_timeout_ms=cfg.barrier_timeout_ms,
                                   state_dtype=torch.bfloat16 if state_dtype == "bf16" else torch.float32)
        self._rings: Dict[int, RingContext] = {}
        for d in degrees:
            self._rings[d] = self._make_ring(d)
        self.ring_degree = cfg.ring_degree
        self.step_index = 0
        self._opt_events = None

    def _make_ring(self, degree: int) -> RingContext:
        cfg, mc = self.cfg, self.model_cfg
        peer = None
        if degree > 1 and self.ctx.device.type == "cuda":
            from ..parallel.peer import RingBuffers

            s_local = cfg.seq_len // degree
            peer = RingBuffers((1, s_local, mc.n_kv_heads, mc.head_dim), group=self.mesh.cp_group(degree),
                               timeout_ms=cfg.barrier_timeout_ms)
        return RingContext(rank=self.mesh.cp_rank(degree), degree=degree, seq_len=cfg.seq_len, layout=cfg.layout,
                           group=self.mesh.cp_group(degree), peer=peer, mask=cfg.mask)

    # ---------------------------------------------------------------------------------------
    def set_ring_degree(self, degree: int) -> None:
        """Switches the DP x CP split (the dynamic ring curriculum calls this between steps)."""
        if degree not in self._rings:
            raise ValueError(f"ring degree {degree} was not prepared; pass it in EngineConfig.ring_degrees")
        self.ring_degree = degree

    @property
    def ring(self) -> RingContext:
        return self._rings[self.ring_degree]

    def local_sequences(self) -> range:
        """Indices (into the global batch) of the sequences this rank's replica processes."""
        dp = self.ctx.world_size // self.ring_degree
        per = self.cfg.global_batch // dp
        r = self.mesh.dp_rank(self.ring_degree)
        return range(r * per, (r + 1) * per)

    def shard_batch(self, tokens: torch.Tensor) -> torch.Tensor:
        """[global_batch, seq_len] (host or device) -> this rank's [n_local, seq_len / cp] on the device."""
        idx = self.local_sequences()
        local = tokens[idx.start: idx.stop]
        ring = self.ring
        local = shard_sequence(local, ring.rank, ring.degree, ring.layout, dim=1)
        if local.device != self.ctx.device:
            if local.device.type == "cpu" and self.ctx.device.type == "cuda" and not local.is_pinned():
                local = local.contiguous().pin_memory()
            local = local.to(self.ctx.device, non_blocking=True)
        return local.contiguous()

    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor, lr: Optional[float] = None,
                   presharded: bool = False) -> torch.Tensor:
        """One optimizer step over the global batch. Returns this rank's share of the mean loss (a
        device scalar; summing it over ranks gives the global mean token loss)."""
        if not presharded:
            tokens, targets = self.shard_batch(tokens), self.shard_batch(targets)
        loss_weight = 1.0 / (self.cfg.global_batch * self.cfg.seq_len)
        ring = self.ring
        loss = torch.zeros((), device=self.ctx.device, dtype=torch.float32)
        for i in range(tokens.shape[0]):
            loss += self.model.forward_backward(tokens[i: i + 1], targets[i: i + 1], loss_weight, ring)
        timed = tokens.is_cuda
        if timed:   # two event records per step; read through optimizer_step_ms() once the step has finished
            if self._opt_events is None:
                self._opt_events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._opt_events[0].record()
        self.optimizer.step(lr=lr)
        if timed:
            self._opt_events[1].record()
        self.step_index += 1
        return loss

    def optimizer_step_ms(self) -> Optional[float]:
        """Device time of the last optimizer step (gradient reduction, clipping, update, parameter refresh; on
        several ranks it includes waiting for the slowest peer). None before the first GPU step has completed."""
        if self._opt_events is None or not self._opt_events[1].query():
            return None
        return self._opt_events[0].elapsed_time(self._opt_events[1])

    def global_loss(self, local_loss: torch.Tensor) -> float:
        t = local_loss.detach().clone()
        if self.ctx.world_size > 1:
            dist.all_reduce(t)
        return float(t.item())

    def close(self) -> None:
        self.optimizer.close()
        for r in self._rings.values():
            if r.peer is not None:
                r.peer.close()
        for sb in (self.model.flat.sym_params, self.model.flat.sym_grads):
            if sb is not None:
                sb.close()
