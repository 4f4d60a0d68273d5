"""zenyx_b200 - a Blackwell-native long-context training runtime.

Public surface mirrors the reference package (zenyx/__init__.py:48-88) - every name in its
``__all__`` is importable from here, ``OpType`` included (the reference lists it but never imports
it) - and adds the components the reference only documents.
"""
from __future__ import annotations

import logging

__version__ = "0.1.0"

from .compiler import OffloadManager, OffloadPolicy, make_offload_policy
from .memory import ActivationManager, CheckpointPolicy, MemoryTracker
from .runtime import (ExecutionGraph, ExecutionGraphBuilder, ExecutionPlan, OpNode, OpType, Scheduler, TopologyConfig,
                      validate_graph)
from .utils import get_logger, set_log_level, setup_logging

logger = setup_logging(level=logging.WARNING)


def __getattr__(name):
    # heavier subsystems are imported on first use
    if name == "FSDPWrapper":
        from .parallel.fsdp_wrapper import FSDPWrapper

        return FSDPWrapper
    if name in ("Trainer", "TrainerConfig"):
        from . import train

        return getattr(train, name)
    raise AttributeError(f"module 'zenyx_b200' has no attribute {name!r}")


__all__ = [
    "__version__", "Scheduler", "ExecutionPlan", "ExecutionGraph", "ExecutionGraphBuilder", "OpNode", "OpType",
    "TopologyConfig", "validate_graph", "FSDPWrapper", "ActivationManager", "CheckpointPolicy", "MemoryTracker",
    "OffloadManager", "OffloadPolicy", "make_offload_policy", "setup_logging", "get_logger", "set_log_level",
    "Trainer", "TrainerConfig",
]
