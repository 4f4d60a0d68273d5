"""Lightweight tracing: NVTX ranges around the phases of a training step and CUDA-event phase timers.

Off by default (one attribute test per call). ``ZX_NVTX=1`` in the environment, or ``enable(True)``,
turns the ranges on, so that a timeline tool shows embedding / layer forward / head / layer backward /
optimizer per micro-batch. ``PhaseTimer`` collects device time per phase with CUDA events for use
without any external tool (``zenyx_b200/bench/step_breakdown.py`` brackets every kernel call the same way).
The reference has no tracing at all (only ``time.perf_counter`` around async launches,
zenyx/streaming/engine.py:75-81).
"""
from __future__ import annotations

import contextlib
import os
from collections import defaultdict
from typing import Dict, List, Tuple

import torch

_enabled = os.environ.get("ZX_NVTX", "0") not in ("", "0", "false", "False")


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


@contextlib.contextmanager
def trace_range(name: str):
    """NVTX range when tracing is on and a GPU is present; otherwise nothing."""
    if _enabled and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class PhaseTimer:
    """Device time per named phase: ``with timer.phase("forward"): ...``; ``summary()`` after a sync."""

    def __init__(self):
        self._events: Dict[str, List[Tuple["torch.cuda.Event", "torch.cuda.Event"]]] = defaultdict(list)
        self._cpu: Dict[str, float] = defaultdict(float)

    @contextlib.contextmanager
    def phase(self, name: str):
        if torch.cuda.is_available():
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            with trace_range(name):
                yield
            e1.record()
            self._events[name].append((e0, e1))
        else:
            import time

            t0 = time.perf_counter()
            yield
            self._cpu[name] += (time.perf_counter() - t0) * 1e3

    def summary(self) -> Dict[str, float]:
        """Milliseconds per phase (synchronises the device)."""
        out = dict(self._cpu)
        if self._events:
            torch.cuda.synchronize()
            for name, pairs in self._events.items():
                out[name] = out.get(name, 0.0) + sum(a.elapsed_time(b) for a, b in pairs)
        return out

    def reset(self) -> None:
        self._events.clear()
        self._cpu.clear()
