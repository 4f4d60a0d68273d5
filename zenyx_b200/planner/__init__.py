"""Parallelism planner and the cost model behind it."""
from .cost_model import HardwarePeaks, StepEstimate, estimate
from .planner import ParallelPlan, plan

__all__ = ["plan", "ParallelPlan", "estimate", "StepEstimate", "HardwarePeaks"]
