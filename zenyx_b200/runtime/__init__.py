from .execution_graph import ExecutionGraph, ExecutionGraphBuilder, OpNode, OpType
from .scheduler import ExecutionPlan, GradientBucketReducer, Scheduler, TopologyConfig
from .validator import GraphValidator, ValidationError, ValidationResult, validate_graph

__all__ = [
    "ExecutionGraph", "ExecutionGraphBuilder", "OpNode", "OpType", "Scheduler", "ExecutionPlan", "TopologyConfig",
    "GradientBucketReducer", "GraphValidator", "validate_graph", "ValidationError", "ValidationResult",
]
