"""Parallelism layer: process bootstrap and collectives, peer (symmetric) memory, the DP x CP
mesh, sharded optimizer, tensor- and pipeline-parallel modules."""
from .communication import (AsyncCollectiveHandle, CollectiveGroup, CommunicationError, DistributedContext, all_gather,
                            all_reduce, barrier, broadcast, destroy_process_group, get_rank, get_world_size,
                            init_distributed_from_env, init_process_group, reduce_scatter)

__all__ = [
    "AsyncCollectiveHandle", "CollectiveGroup", "CommunicationError", "DistributedContext", "all_gather", "all_reduce",
    "barrier", "broadcast", "destroy_process_group", "get_rank", "get_world_size", "init_distributed_from_env",
    "init_process_group", "reduce_scatter",
]
