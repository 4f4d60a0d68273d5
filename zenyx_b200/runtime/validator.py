"""Static checks of an ExecutionGraph before it is run (reference: zenyx/runtime/validator.py:15-112):
missing dependencies, a simulated execution that names the nodes blocked by a deadlock, ordering
violations, and communication-node metadata."""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import List

from .execution_graph import ExecutionGraph, OpType

_VALID_REDUCE = {"sum", "prod", "min", "max", "avg"}


class ValidationError(ValueError):
    pass


@dataclass
class ValidationResult:
    is_valid: bool
    errors: List[str] = field(default_factory=list)
    warnings: List[str] = field(default_factory=list)

    def raise_if_invalid(self) -> None:
        if not self.is_valid:
            raise ValidationError("; ".join(self.errors))


class GraphValidator:
    def __init__(self, graph: ExecutionGraph):
        self.graph = graph

    def validate(self) -> ValidationResult:
        errors: List[str] = []
        warnings: List[str] = []
        self._check_dependencies(errors)
        order = self._simulate(errors)
        self._check_order(order, errors)
        self._check_comm(errors, warnings)
        return ValidationResult(not errors, errors, warnings)

    def _check_dependencies(self, errors: List[str]) -> None:
        g = self.graph
        for n, deps in g.dependencies.items():
            for d in deps:
                if d not in g.nodes:
                    errors.append(f"node {n!r} depends on missing node {d!r}")

    def _simulate(self, errors: List[str]) -> List[str]:
        g = self.graph
        indeg = {n: sum(1 for d in deps if d in g.nodes) for n, deps in g.dependencies.items()}
        ready = deque(n for n in g.nodes if indeg[n] == 0)
        order: List[str] = []
        while ready:
            n = ready.popleft()
            order.append(n)
            for m in g.dependents.get(n, []):
                indeg[m] -= 1
                if indeg[m] == 0:
                    ready.append(m)
        if len(order) != len(g.nodes):
            blocked = sorted(n for n in g.nodes if n not in set(order))
            errors.append(f"deadlock: nodes never become ready: {blocked}")
        return order

    def _check_order(self, order: List[str], errors: List[str]) -> None:
        pos = {n: i for i, n in enumerate(order)}
        for n, deps in self.graph.dependencies.items():
            for d in deps:
                if n in pos and d in pos and pos[d] > pos[n]:
                    errors.append(f"order violation: {n!r} runs before its dependency {d!r}")

    def _check_comm(self, errors: List[str], warnings: List[str]) -> None:
        for n in self.graph.nodes.values():
            if not n.is_comm_op():
                continue
            if n.op_type in (OpType.ALLREDUCE, OpType.BROADCAST) and "tensor" not in n.metadata:
                errors.append(f"communication node {n.name!r} has no metadata['tensor']")
            if n.op_type == OpType.ALLREDUCE:
                op = n.metadata.get("op", (n.comm_group or {}).get("op", "sum"))
                if op not in _VALID_REDUCE:
                    errors.append(f"communication node {n.name!r} has an unknown reduce op {op!r}")
            if n.op_type == OpType.BROADCAST and "src" not in n.metadata:
                warnings.append(f"broadcast node {n.name!r} has no 'src'; rank 0 is assumed")
            if not n.device_ids:
                warnings.append(f"communication node {n.name!r} lists no device_ids")


def validate_graph(graph: ExecutionGraph) -> ValidationResult:
    return GraphValidator(graph).validate()
