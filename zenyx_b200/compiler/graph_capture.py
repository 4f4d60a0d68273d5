"""Analysis-flavoured view of the execution graph (reference: zenyx/compiler/graph_capture.py:17-204).
``ExecutionGraph`` here IS ``zenyx_b200.runtime.ExecutionGraph`` - one class for both uses;
``GraphNode`` is a light record of one captured module."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List

from ..runtime.execution_graph import ExecutionGraph, OpType


@dataclass
class GraphNode:
    name: str
    op: str
    inputs: List[str] = field(default_factory=list)
    outputs: List[str] = field(default_factory=list)
    params: int = 0
    flops: float = 0.0


def graph_nodes(graph: ExecutionGraph) -> List[GraphNode]:
    """The captured forward nodes as GraphNode records, in execution order."""
    out = []
    for n in graph.get_forward_execution_order():
        node = graph.nodes[n]
        out.append(GraphNode(name=node.name, op=node.module_name or "", inputs=graph.get_dependencies(n),
                             outputs=graph.get_dependents(n), params=node.params, flops=node.flops))
    return out


__all__ = ["ExecutionGraph", "GraphNode", "graph_nodes", "OpType"]
