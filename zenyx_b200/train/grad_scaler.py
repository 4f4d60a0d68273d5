"""Dynamic loss scaling for fp16 training (name from the reference's deleted
``zenyx/train/grad_scaler.py``, ZENYX_2_0_DELIVERABLES.txt:189). Device-agnostic: works on CPU
tensors too, which ``torch.cuda.amp.GradScaler`` does not."""
from __future__ import annotations

import torch


class DynamicGradScaler:
    def __init__(self, init_scale: float = 2.0 ** 15, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 1000, min_scale: float = 1.0):
        self.scale_value = float(init_scale)
        self.growth_factor, self.backoff_factor = growth_factor, backoff_factor
        self.growth_interval, self.min_scale = growth_interval, min_scale
        self._good_steps = 0
        self._unscaled = False
        self.skipped_steps = 0

    def scale(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * self.scale_value

    def unscale_(self, optimizer) -> bool:
        """Divides gradients by the scale; returns True when every gradient is finite."""
        if self._unscaled:
            return self._finite
        inv = 1.0 / self.scale_value
        finite = True
        for group in optimizer.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                p.grad.mul_(inv)
                if not torch.isfinite(p.grad).all():
                    finite = False
        self._unscaled, self._finite = True, finite
        return finite

    def step(self, optimizer) -> bool:
        finite = self.unscale_(optimizer)
        self._unscaled = False
        if finite:
            optimizer.step()
            self._good_steps += 1
            if self._good_steps >= self.growth_interval:
                self.scale_value *= self.growth_factor
                self._good_steps = 0
            return True
        self.scale_value = max(self.min_scale, self.scale_value * self.backoff_factor)
        self._good_steps = 0
        self.skipped_steps += 1
        return False

    def state_dict(self):
        return {"scale": self.scale_value, "good_steps": self._good_steps, "skipped": self.skipped_steps}

    def load_state_dict(self, sd):
        self.scale_value, self._good_steps, self.skipped_steps = float(sd["scale"]), int(sd["good_steps"]), int(sd["skipped"])
