"""Step scheduler for arbitrary ``nn.Module`` training: forward, backward, data-parallel gradient
reduction, optimizer step with gradient accumulation, optional walk over an ExecutionGraph.

Names follow the reference (zenyx/runtime/scheduler.py:19-294): ``TopologyConfig``,
``GradientBucketReducer``, ``Scheduler``, ``ExecutionPlan``. Behaviour that differs on purpose:

* gradients are reduced once per optimizer step, at the accumulation boundary (the reference
  reduces and re-divides on every micro-step, which mis-scales accumulated gradients);
* with ``enable_overlap`` buckets are launched from autograd hooks while backward is still
  running, on a side stream (the reference starts communication only after backward has ended);
* a non-contiguous gradient is reduced through a copy that is written back;
* ``backward(loss, optimizer)`` - the call form the reference's quick-start uses - is recognised
  instead of silently never stepping;
* the running loss is kept on the device; ``get_stats`` is the only place that reads it back.

The Llama flagship does not use this path: its gradients live in one flat buffer and are reduced
by the fused kernel of ``zenyx_b200.parallel.zero``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.nn as nn

from ..parallel import communication as comm
from .execution_graph import ExecutionGraph, OpNode, OpType


@dataclass
class TopologyConfig:
    intra_node_ranks: Sequence[int] = field(default_factory=list)
    inter_node_ranks: Sequence[int] = field(default_factory=list)


class _Bucket:
    def __init__(self, params: List[torch.nn.Parameter]):
        self.params = params
        self.pending = 0
        self.handle: Optional[comm.AsyncCollectiveHandle] = None
        self.flat: Optional[torch.Tensor] = None

    def launch(self, async_op: bool, stream, group) -> None:
        grads = [p.grad for p in self.params if p.grad is not None]
        if not grads:
            return
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                self.flat = torch.cat([g.reshape(-1) for g in grads])
                self.handle = comm.all_reduce(self.flat, op="avg", group=group, async_op=True)
        else:
            self.flat = torch.cat([g.reshape(-1) for g in grads])
            res = comm.all_reduce(self.flat, op="avg", group=group, async_op=async_op)
            self.handle = res if isinstance(res, comm.AsyncCollectiveHandle) else None

    def wait(self, stream) -> None:
        if self.flat is None:
            return
        if self.handle is not None:
            self.handle.wait()
        if stream is not None:
            torch.cuda.current_stream().wait_stream(stream)
        off = 0
        for p in self.params:
            if p.grad is None:
                continue
            n = p.grad.numel()
            p.grad.copy_(self.flat[off: off + n].view_as(p.grad))
            off += n
        self.flat, self.handle = None, None


class GradientBucketReducer:
    """Averages gradients over the data-parallel group in buckets of ``bucket_size_mb``."""

    def __init__(self, bucket_size_mb: float = 25.0, async_safe: bool = True, group=None):
        self.bucket_bytes = int(bucket_size_mb * 1024 * 1024)
        self.async_safe = async_safe
        self.group = group
        self._buckets: List[_Bucket] = []
        self._model_id: Optional[int] = None
        self._hooks: List[Any] = []
        self._armed = False
        self._stream = None

    def _build(self, model: nn.Module) -> None:
        params = [p for p in model.parameters() if p.requires_grad]
        self._buckets = []
        cur: List[torch.nn.Parameter] = []
        size = 0
        for p in reversed(params):  # gradients become ready roughly in reverse order
            nbytes = p.numel() * p.element_size()
            if cur and size + nbytes > self.bucket_bytes:
                self._buckets.append(_Bucket(cur))
                cur, size = [], 0
            cur.append(p)
            size += nbytes
        if cur:
            self._buckets.append(_Bucket(cur))
        self._model_id = id(model)

    def buckets_for(self, model: nn.Module) -> List[List[torch.nn.Parameter]]:
        if self._model_id != id(model):
            self._build(model)
        return [b.params for b in self._buckets]

    # overlap mode: arm before backward, buckets fire from hooks --------------------------------
    def arm(self, model: nn.Module, stream=None) -> None:
        if comm.get_world_size(self.group) == 1:
            return
        if self._model_id != id(model):
            self._build(model)
        self.disarm()
        self._stream = stream
        owner = {}
        for b in self._buckets:
            b.pending = len(b.params)
            for p in b.params:
                owner[p] = b

        def make_hook(bucket: _Bucket):
            def hook(_param):
                bucket.pending -= 1
                if bucket.pending == 0:
                    bucket.launch(True, self._stream, self.group)
            return hook

        for p, b in owner.items():
            self._hooks.append(p.register_post_accumulate_grad_hook(make_hook(b)))
        self._armed = True

    def disarm(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks.clear()
        self._armed = False

    def finish(self) -> None:
        """Waits for every bucket launched from hooks and launches the ones whose parameters got no gradient."""
        for b in self._buckets:
            if b.flat is None and b.pending not in (0, len(b.params)):
                b.launch(True, self._stream, self.group)
            b.wait(self._stream)
        self.disarm()

    # post-backward mode --------------------------------------------------------------------------
    def reduce(self, model: nn.Module) -> List[_Bucket]:
        if comm.get_world_size(self.group) == 1:
            return []
        if self._model_id != id(model):
            self._build(model)
        for b in self._buckets:
            b.launch(self.async_safe, None, self.group)
        return self._buckets


class Scheduler:
    def __init__(self, accumulation_steps: int = 1, enable_overlap: bool = True, bucket_size_mb: float = 25.0,
                 topology: Optional[TopologyConfig] = None, group=None):
        self.accumulation_steps = max(1, int(accumulation_steps))
        self.enable_overlap = bool(enable_overlap) and torch.cuda.is_available()
        self.bucket_size_mb = bucket_size_mb
        self.topology = topology
        self.group = group
        self.reducer = GradientBucketReducer(bucket_size_mb, async_safe=True, group=group)
        self.comm_stream = torch.cuda.Stream() if self.enable_overlap else None
        self.step_count = 0
        self.micro_step = 0
        self._loss_sum: Optional[torch.Tensor] = None
        self._pending: List[comm.AsyncCollectiveHandle] = []

    def forward(self, model: nn.Module, batch: Any) -> Any:
        return model(batch)

    def _at_boundary(self) -> bool:
        return (self.micro_step + 1) % self.accumulation_steps == 0

    def backward(self, loss: torch.Tensor, model: Optional[nn.Module] = None, optimizer=None,
                 execution_graph: Optional[ExecutionGraph] = None) -> None:
        if isinstance(model, torch.optim.Optimizer) and optimizer is None:
            model, optimizer = None, model  # backward(loss, optimizer)
        boundary = self._at_boundary()
        distributed = comm.get_world_size(self.group) > 1
        scaled = loss / self.accumulation_steps if self.accumulation_steps > 1 else loss
        overlap = boundary and distributed and model is not None and self.enable_overlap
        if overlap:
            self.reducer.arm(model, self.comm_stream)
        scaled.backward()
        if execution_graph is not None:
            self._execute_graph_nodes(execution_graph)
        if boundary and distributed and model is not None:
            if overlap:
                self.reducer.finish()
            else:
                for b in self.reducer.reduce(model):
                    b.wait(None)
        for h in self._pending:
            h.wait()
        self._pending.clear()
        d = loss.detach().float()
        self._loss_sum = d if self._loss_sum is None else self._loss_sum + d
        self.micro_step += 1
        if boundary and optimizer is not None:
            optimizer.step()
            optimizer.zero_grad(set_to_none=True)
            self.step_count += 1

    # graph walk ------------------------------------------------------------------------------
    def _priority(self, node: OpNode) -> int:
        if not node.is_comm_op():
            return 0
        if self.topology is not None and node.device_ids:
            intra = set(self.topology.intra_node_ranks)
            if intra and set(node.device_ids) <= intra:
                return 1
            return 2
        return 1

    def _select_next_ready_node(self, ready: List[str], graph: ExecutionGraph) -> str:
        """Compute first, then intra-node communication, then inter-node communication."""
        return min(ready, key=lambda n: (self._priority(graph.nodes[n]), n))

    def _execute_graph_nodes(self, graph: ExecutionGraph) -> List[str]:
        indeg = {n: len(d) for n, d in graph.dependencies.items()}
        ready = [n for n in graph.nodes if indeg[n] == 0]
        executed: List[str] = []
        while ready:
            name = self._select_next_ready_node(ready, graph)
            ready.remove(name)
            self._execute_node(graph.nodes[name])
            executed.append(name)
            for m in graph.dependents[name]:
                indeg[m] -= 1
                if indeg[m] == 0:
                    ready.append(m)
        if len(executed) != len(graph.nodes):
            raise RuntimeError("Deadlock/cycle detected while executing the graph")
        return executed

    def _tensors_of(self, node: OpNode) -> List[torch.Tensor]:
        if "tensor" not in node.metadata:
            raise ValueError(f"communication node {node.name!r} has no metadata['tensor']")
        t = node.metadata["tensor"]
        t = t() if callable(t) else t
        return [x for x in (t if isinstance(t, (list, tuple)) else [t]) if x is not None]

    def _execute_node(self, node: OpNode) -> None:
        if not node.is_comm_op():
            return  # compute and memory nodes are accounted for by autograd itself
        if node.op_type == OpType.ALLREDUCE:
            op = node.metadata.get("op", (node.comm_group or {}).get("op", "sum"))
            for t in self._tensors_of(node):
                self._launch(lambda x=t: comm.all_reduce(x, op=op, group=self.group, async_op=self.enable_overlap))
        elif node.op_type in (OpType.BROADCAST, OpType.SYNC_PARAMS):
            src = int(node.metadata.get("src", 0))
            for t in self._tensors_of(node):
                self._launch(lambda x=t: comm.broadcast(x, src=src, group=self.group, async_op=self.enable_overlap))

    def _launch(self, fn) -> None:
        if self.comm_stream is not None:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                res = fn()
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        else:
            res = fn()
        if isinstance(res, comm.AsyncCollectiveHandle):
            self._pending.append(res)

    def synchronize(self) -> None:
        for h in self._pending:
            h.wait()
        self._pending.clear()
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    @property
    def accumulated_loss(self) -> float:
        return float(self._loss_sum.item()) if self._loss_sum is not None else 0.0

    def get_stats(self) -> Dict[str, Any]:
        return {"step": self.step_count, "micro_step": self.micro_step, "accumulated_loss": self.accumulated_loss,
                "accumulation_steps": self.accumulation_steps, "overlap_enabled": self.enable_overlap,
                "bucket_size_mb": self.bucket_size_mb, "topology": self.topology}


@dataclass
class ExecutionPlan:
    num_forward_ops: int
    num_backward_ops: int
    total_compute_ms: float
    total_memory_mb: float

    def estimate_memory_gb(self) -> float:
        return self.total_memory_mb / 1024.0

    def estimate_time_seconds(self) -> float:
        return self.total_compute_ms / 1e3

    @classmethod
    def from_model(cls, model: nn.Module, batch_size: int = 1, seq_len: int = 1, tflops: float = 1400.0,
                   bytes_per_param_state: int = 16) -> "ExecutionPlan":
        """6 * params * tokens FLOPs at `tflops`; parameters, gradients and AdamW state at 16 B/param."""
        params = sum(p.numel() for p in model.parameters())
        n_ops = sum(1 for m in model.modules() if not list(m.children()))
        tokens = batch_size * seq_len
        compute_ms = 6.0 * params * tokens / (tflops * 1e12) * 1e3
        return cls(n_ops, n_ops, compute_ms, params * bytes_per_param_state / 1e6)
