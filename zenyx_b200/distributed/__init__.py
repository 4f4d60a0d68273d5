"""``zenyx_b200.distributed``: the reference's import path for its communication, FSDP, tensor- and
pipeline-parallel layers (zenyx/distributed/__init__.py:35-59). The implementations live in
``zenyx_b200.parallel``; this package re-exports them under the names reference users import."""
from ..parallel.communication import (AsyncCollectiveHandle, CollectiveGroup, CommunicationError, DistributedContext,
                                      all_gather, all_reduce, barrier, broadcast, destroy_process_group, get_rank,
                                      get_world_size, init_distributed_from_env, init_process_group, reduce_scatter)
from ..parallel.fsdp_wrapper import FSDPWrapper
from ..parallel.groups import Mesh, ParallelLayout
from ..parallel.pipeline_parallel import (DistributedPipelineEngine, Partial1F1BSchedule, PipelineParallelModel,
                                          PipelineStage, SimpleGPipeSchedule, create_pipeline_from_sequential)
from ..parallel.tensor_parallel import (ColumnParallelLinear, RowParallelLinear, SequenceParallelColumnLinear,
                                        SequenceParallelRowLinear, TensorParallelEmbedding,
                                        make_tensor_parallel_model)
from ..parallel.zero import ZeroAdamW

__all__ = [
    "AsyncCollectiveHandle", "CollectiveGroup", "CommunicationError", "DistributedContext", "all_gather", "all_reduce",
    "barrier", "broadcast", "destroy_process_group", "get_rank", "get_world_size", "init_distributed_from_env",
    "init_process_group", "reduce_scatter", "FSDPWrapper", "Mesh", "ParallelLayout", "DistributedPipelineEngine",
    "Partial1F1BSchedule", "PipelineParallelModel", "PipelineStage", "SimpleGPipeSchedule",
    "create_pipeline_from_sequential", "ColumnParallelLinear", "RowParallelLinear", "TensorParallelEmbedding",
    "make_tensor_parallel_model", "ZeroAdamW", "SequenceParallelColumnLinear", "SequenceParallelRowLinear",
]
