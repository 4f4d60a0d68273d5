"""Learning-rate schedules as plain ``step -> lr`` callables (name from the reference's deleted
``zenyx/train/lr_schedule.py``, ZENYX_2_0_DELIVERABLES.txt:189; its examples hand-roll warm-up +
cosine, examples/02_intermediate_finetuning.py:98-101)."""
from __future__ import annotations

import math
from typing import Callable


def constant(lr: float) -> Callable[[int], float]:
    return lambda step: lr


def warmup_cosine(peak_lr: float, warmup_steps: int, total_steps: int, min_lr: float = 0.0) -> Callable[[int], float]:
    def f(step: int) -> float:
        if warmup_steps > 0 and step < warmup_steps:
            return peak_lr * (step + 1) / warmup_steps
        if step >= total_steps:
            return min_lr
        t = (step - warmup_steps) / max(1, total_steps - warmup_steps)
        return min_lr + 0.5 * (peak_lr - min_lr) * (1.0 + math.cos(math.pi * t))
    return f


def warmup_linear(peak_lr: float, warmup_steps: int, total_steps: int, min_lr: float = 0.0) -> Callable[[int], float]:
    def f(step: int) -> float:
        if warmup_steps > 0 and step < warmup_steps:
            return peak_lr * (step + 1) / warmup_steps
        t = min(1.0, (step - warmup_steps) / max(1, total_steps - warmup_steps))
        return peak_lr + (min_lr - peak_lr) * t
    return f


def warmup_stable_decay(peak_lr: float, warmup_steps: int, stable_steps: int, decay_steps: int,
                        min_lr: float = 0.0) -> Callable[[int], float]:
    def f(step: int) -> float:
        if warmup_steps > 0 and step < warmup_steps:
            return peak_lr * (step + 1) / warmup_steps
        if step < warmup_steps + stable_steps:
            return peak_lr
        t = min(1.0, (step - warmup_steps - stable_steps) / max(1, decay_steps))
        return peak_lr + (min_lr - peak_lr) * t
    return f
