"""Dynamic ring-degree curriculum.

The reference documents ``RingDegreeScheduler`` and ``CurriculumPhase`` ("progressive ring degree
expansion", "adaptive scheduling based on loss landscape", README.md:162-166,330,345) but the module
``zenyx/train/dynamic_ring_curriculum.py`` is not in its tree. Here the ring (context-parallel)
degree grows in phases, by default 2 -> 4 -> 8 evenly over the first 200 steps; the data-parallel
degree is world / ring degree, so the global batch and the tokens per GPU per step stay constant.
``mode="loss_adaptive"`` additionally ends a phase early once the smoothed loss has stopped
improving (relative slope below ``plateau_tol`` over ``window`` steps).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

from ..parallel.groups import ParallelLayout


@dataclass
class CurriculumPhase:
    ring_degree: int
    num_steps: Optional[int] = None     # length of the phase; None = until the end of training
    until_step: Optional[int] = None    # alternative: absolute step at which the phase ends
    seq_len: Optional[int] = None       # optional sequence length of the phase


def default_phases(min_degree: int = 2, max_degree: int = 8, ramp_steps: int = 200) -> List[CurriculumPhase]:
    degrees = []
    d = max(1, min_degree)
    while d < max_degree:
        degrees.append(d)
        d *= 2
    degrees.append(max_degree)
    ramp = degrees[:-1]
    phases = []
    if ramp:
        base, extra = divmod(ramp_steps, len(ramp))
        for i, deg in enumerate(ramp):
            phases.append(CurriculumPhase(deg, num_steps=base + (1 if i < extra else 0)))
    phases.append(CurriculumPhase(degrees[-1], num_steps=None))
    return phases


class RingDegreeScheduler:
    def __init__(self, phases: Optional[Sequence[CurriculumPhase]] = None, *, min_degree: int = 2, max_degree: int = 8,
                 ramp_steps: int = 200, world_size: int = 8, mode: str = "step", window: int = 20,
                 plateau_tol: float = 1e-3, ema: float = 0.9):
        if mode not in ("step", "loss_adaptive"):
            raise ValueError("mode must be 'step' or 'loss_adaptive'")
        max_degree = min(max_degree, world_size)
        min_degree = min(min_degree, max_degree)
        self.phases = list(phases) if phases is not None else default_phases(min_degree, max_degree, ramp_steps)
        for p in self.phases:
            if world_size % p.ring_degree != 0:
                raise ValueError(f"ring degree {p.ring_degree} does not divide world size {world_size}")
        self.world_size, self.mode = world_size, mode
        self.window, self.plateau_tol, self.ema = window, plateau_tol, ema
        self._bounds = self._compute_bounds()
        self.current_step = 0
        self._shift = 0                 # steps skipped by early phase advances (loss-adaptive mode)
        self._smoothed: Optional[float] = None
        self._history: List[float] = []

    def _compute_bounds(self) -> List[Optional[int]]:
        bounds: List[Optional[int]] = []
        start = 0
        for p in self.phases:
            if p.until_step is not None:
                end: Optional[int] = p.until_step
            elif p.num_steps is not None:
                end = start + p.num_steps
            else:
                end = None
            bounds.append(end)
            if end is None:
                break
            start = end
        return bounds

    def degrees(self) -> List[int]:
        return sorted({p.ring_degree for p in self.phases})

    def phase_index_at(self, step: int) -> int:
        s = step + self._shift
        for i, end in enumerate(self._bounds):
            if end is None or s < end:
                return i
        return len(self._bounds) - 1

    def degree_at(self, step: int) -> int:
        return self.phases[self.phase_index_at(step)].ring_degree

    def layout_at(self, step: int) -> ParallelLayout:
        d = self.degree_at(step)
        return ParallelLayout(cp=d, dp=self.world_size // d)

    def interpolation(self, step: int) -> float:
        """Progress through the ramp in [0, 1]; 1 once the final degree is reached (usable to blend
        hyper-parameters smoothly across phases)."""
        last_end = [b for b in self._bounds if b is not None]
        if not last_end:
            return 1.0
        return min(1.0, (step + self._shift) / max(1, last_end[-1]))

    def step(self, loss: Optional[float] = None) -> ParallelLayout:
        """Advances one training step; returns the layout for the NEXT step."""
        if loss is not None:
            self._smoothed = loss if self._smoothed is None else self.ema * self._smoothed + (1 - self.ema) * loss
            self._history.append(self._smoothed)
            if self.mode == "loss_adaptive" and len(self._history) > self.window:
                old, new = self._history[-self.window - 1], self._history[-1]
                idx = self.phase_index_at(self.current_step)
                end = self._bounds[idx] if idx < len(self._bounds) else None
                if end is not None and abs(old - new) / max(abs(old), 1e-12) < self.plateau_tol:
                    self._shift += max(0, end - (self.current_step + 1 + self._shift))  # jump to the phase end
                    self._history.clear()
        self.current_step += 1
        return self.layout_at(self.current_step)

    def state_dict(self) -> Dict[str, object]:
        return {"current_step": self.current_step, "shift": self._shift, "smoothed": self._smoothed,
                "history": list(self._history)}

    def load_state_dict(self, sd: Dict[str, object]) -> None:
        self.current_step = int(sd["current_step"])
        self._shift = int(sd["shift"])
        self._smoothed = sd["smoothed"]  # type: ignore[assignment]
        self._history = list(sd["history"])  # type: ignore[arg-type]


__all__ = ["CurriculumPhase", "RingDegreeScheduler", "default_phases"]
