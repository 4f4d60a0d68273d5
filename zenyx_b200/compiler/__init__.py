from .graph_capture import ExecutionGraph, GraphNode, graph_nodes
from .offload_policy import OffloadManager, OffloadPolicy, make_offload_policy
from .xla_path import XLACheckpointPolicy, maybe_offload_large_tensor, remat_or_checkpoint

__all__ = ["ExecutionGraph", "GraphNode", "graph_nodes", "OffloadPolicy", "OffloadManager", "make_offload_policy",
           "XLACheckpointPolicy", "remat_or_checkpoint", "maybe_offload_large_tensor"]
