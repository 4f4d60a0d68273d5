"""Pipeline parallelism: multi-micro-batch GPipe and 1F1B over overlapped point-to-point.

Names follow the reference (zenyx/distributed/pipeline_parallel.py:18-218): ``PipelineStage``,
``DistributedPipelineEngine``, ``PipelineParallelModel``, ``create_pipeline_from_sequential``,
``SimpleGPipeSchedule``, ``Partial1F1BSchedule``. The reference's engine moves exactly one
micro-batch per step with blocking ``send``/``recv`` (bubble = (stages-1)/stages) and its two
schedule classes are single-process simulators. Here the engine runs ``num_microbatches`` per step
with either schedule, every boundary transfer is a non-blocking ``batch_isend_irecv`` whose receive
for the next micro-batch is posted before the current one computes, and gradients accumulate over
the micro-batches before one optimizer step. The single-process schedule classes are kept (they
are how the engine's arithmetic is tested without processes).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from . import communication as comm


class PipelineStage(nn.Module):
    def __init__(self, stage_id: int, num_stages: int, layers: Sequence[nn.Module],
                 input_shape: Optional[Tuple[int, ...]] = None, device=None):
        super().__init__()
        self.stage_id, self.num_stages, self.input_shape = stage_id, num_stages, input_shape
        self.layers = nn.ModuleList(layers)
        if device is not None:
            self.to(device)

    @property
    def is_first(self) -> bool:
        return self.stage_id == 0

    @property
    def is_last(self) -> bool:
        return self.stage_id == self.num_stages - 1

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return x


def split_layers(layers: Sequence[nn.Module], num_stages: int) -> List[List[nn.Module]]:
    """Contiguous split, as even as possible (earlier stages take the remainder)."""
    n = len(layers)
    base, extra = divmod(n, num_stages)
    out, i = [], 0
    for s in range(num_stages):
        k = base + (1 if s < extra else 0)
        out.append(list(layers[i: i + k]))
        i += k
    return out


def create_pipeline_from_sequential(model: nn.Sequential, num_stages: int, device=None) -> List[PipelineStage]:
    parts = split_layers(list(model.children()), num_stages)
    return [PipelineStage(i, num_stages, p, device=device) for i, p in enumerate(parts)]


class PipelineParallelModel(nn.Module):
    """Holds only the local stage of a model split over the pipeline group."""

    def __init__(self, model: nn.Module, num_stages: Optional[int] = None, stage_id: Optional[int] = None, group=None,
                 device=None):
        super().__init__()
        self.num_stages = num_stages if num_stages is not None else comm.get_world_size(group)
        self.stage_id = stage_id if stage_id is not None else comm.get_rank(group)
        parts = split_layers(list(model.children()), self.num_stages)
        self.stage = PipelineStage(self.stage_id, self.num_stages, parts[self.stage_id], device=device)

    def forward(self, x):
        return self.stage(x)


def one_f_one_b_order(stage: int, num_stages: int, num_microbatches: int) -> List[Tuple[str, int]]:
    """The (op, micro-batch) sequence stage `stage` executes under 1F1B."""
    warm = min(num_stages - 1 - stage, num_microbatches)
    order: List[Tuple[str, int]] = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < num_microbatches:
        order.append(("F", f))
        f += 1
        order.append(("B", b))
        b += 1
    while b < num_microbatches:
        order.append(("B", b))
        b += 1
    return order


def gpipe_order(num_microbatches: int) -> List[Tuple[str, int]]:
    return [("F", i) for i in range(num_microbatches)] + [("B", i) for i in reversed(range(num_microbatches))]


class DistributedPipelineEngine:
    """One pipeline stage per rank of `group`."""

    def __init__(self, stage: PipelineStage, optimizer: torch.optim.Optimizer, loss_fn: Optional[Callable] = None,
                 micro_batch_shape: Optional[Tuple[int, ...]] = None, dtype: torch.dtype = torch.float32,
                 num_microbatches: int = 1, schedule: str = "1f1b", group=None, device=None):
        if schedule not in ("1f1b", "gpipe"):
            raise ValueError("schedule must be '1f1b' or 'gpipe'")
        self.stage, self.optimizer, self.loss_fn = stage, optimizer, loss_fn
        self.micro_batch_shape, self.dtype = micro_batch_shape, dtype
        self.num_microbatches, self.schedule, self.group = num_microbatches, schedule, group
        self.device = device or next(stage.parameters()).device
        self.rank, self.world = comm.get_rank(group), comm.get_world_size(group)
        self._out_shape: Optional[Tuple[int, ...]] = None

    def _peer(self, stage_id: int) -> int:
        return dist.get_global_rank(self.group, stage_id) if self.group is not None else stage_id

    def _irecv(self, shape, src_stage: int):
        buf = torch.empty(shape, dtype=self.dtype, device=self.device)
        works = dist.batch_isend_irecv([dist.P2POp(dist.irecv, buf, self._peer(src_stage), self.group)])
        return buf, works

    def _isend(self, t: torch.Tensor, dst_stage: int):
        return dist.batch_isend_irecv([dist.P2POp(dist.isend, t.contiguous(), self._peer(dst_stage), self.group)])

    def run_step(self, inputs: Optional[torch.Tensor] = None, targets: Optional[torch.Tensor] = None) -> Optional[float]:
        """One optimizer step over ``num_microbatches`` micro-batches. The first stage passes
        ``inputs`` [num_microbatches * mb, ...]; the last stage passes ``targets``. Returns the mean
        loss on the last stage, None elsewhere."""
        st, M = self.stage, self.num_microbatches
        S, s = st.num_stages, st.stage_id
        order = gpipe_order(M) if self.schedule == "gpipe" else one_f_one_b_order(s, S, M)
        self.optimizer.zero_grad(set_to_none=True)
        in_chunks = list(inputs.to(self.device).chunk(M)) if (st.is_first and inputs is not None) else None
        tgt_chunks = list(targets.to(self.device).chunk(M)) if (st.is_last and targets is not None) else None
        acts_in: dict = {}
        acts_out: dict = {}
        pending_sends = []
        losses: List[torch.Tensor] = []
        # prefetch queues: the next forward input and the next backward gradient are received early
        fwd_ids = [i for op, i in order if op == "F"]
        bwd_ids = [i for op, i in order if op == "B"]
        recv_f, recv_b = {}, {}

        def post_fwd_recv(k: int) -> None:
            if not st.is_first and k < len(fwd_ids) and fwd_ids[k] not in recv_f:
                recv_f[fwd_ids[k]] = self._irecv(self.micro_batch_shape, s - 1)

        def post_bwd_recv(k: int) -> None:
            if not st.is_last and k < len(bwd_ids) and bwd_ids[k] not in recv_b and self._out_shape is not None:
                recv_b[bwd_ids[k]] = self._irecv(self._out_shape, s + 1)

        post_fwd_recv(0)
        fk = bk = 0
        for op, i in order:
            if op == "F":
                if st.is_first:
                    x = in_chunks[i]
                else:
                    buf, works = recv_f.pop(i)
                    for w in works:
                        w.wait()
                    x = buf.requires_grad_(True)
                fk += 1
                post_fwd_recv(fk)          # overlap the next activation transfer with this compute
                y = st(x)
                acts_in[i] = x
                if st.is_last:
                    loss = self.loss_fn(y, tgt_chunks[i]) / M
                    acts_out[i] = loss
                    losses.append(loss.detach())
                else:
                    acts_out[i] = y
                    if self._out_shape is None:
                        self._out_shape = tuple(y.shape)
                    pending_sends += self._isend(y.detach(), s + 1)
                    post_bwd_recv(bk)
            else:
                if st.is_last:
                    acts_out.pop(i).backward()
                else:
                    if i not in recv_b:
                        recv_b[i] = self._irecv(self._out_shape, s + 1)
                    buf, works = recv_b.pop(i)
                    for w in works:
                        w.wait()
                    bk += 1
                    post_bwd_recv(bk)
                    acts_out.pop(i).backward(buf)
                x = acts_in.pop(i)
                if not st.is_first:
                    pending_sends += self._isend(x.grad, s - 1)
                if st.is_last:
                    bk += 1
        for w in pending_sends:
            w.wait()
        self.optimizer.step()
        if st.is_last and losses:
            return float(torch.stack(losses).sum().item())
        return None


# ---------------------------------------------------------------------------------------------------
# Single-process schedules (all stages in one process): the arithmetic of the engine without ranks
# ---------------------------------------------------------------------------------------------------
class SimpleGPipeSchedule:
    def __init__(self, stages: Sequence[nn.Module], num_microbatches: int = 1):
        self.stages, self.num_microbatches = list(stages), num_microbatches

    def step(self, inputs: torch.Tensor, targets: torch.Tensor, loss_fn: Callable, optimizer=None) -> float:
        M = self.num_microbatches
        if optimizer is not None:
            optimizer.zero_grad(set_to_none=True)
        total = 0.0
        losses = []
        for x, t in zip(inputs.chunk(M), targets.chunk(M)):      # all forwards
            for st in self.stages:
                x = st(x)
            losses.append(loss_fn(x, t) / M)
        for l in reversed(losses):                                # then all backwards
            l.backward()
            total += float(l.detach())
        if optimizer is not None:
            optimizer.step()
        return total


class Partial1F1BSchedule:
    def __init__(self, stages: Sequence[nn.Module], num_microbatches: int = 1):
        self.stages, self.num_microbatches = list(stages), num_microbatches

    def step(self, inputs: torch.Tensor, targets: torch.Tensor, loss_fn: Callable, optimizer=None) -> float:
        """Runs the last stage's 1F1B order (warm-up forwards, then alternate) on one process."""
        M, S = self.num_microbatches, len(self.stages)
        if optimizer is not None:
            optimizer.zero_grad(set_to_none=True)
        xs, ts = list(inputs.chunk(M)), list(targets.chunk(M))
        live: dict = {}
        total = 0.0
        for op, i in one_f_one_b_order(0, S, M):
            if op == "F":
                x = xs[i]
                for st in self.stages:
                    x = st(x)
                live[i] = loss_fn(x, ts[i]) / M
            else:
                l = live.pop(i)
                l.backward()
                total += float(l.detach())
        if optimizer is not None:
            optimizer.step()
        return total
