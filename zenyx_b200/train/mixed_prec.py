"""Mixed-precision policy and loss scaling for the generic ``nn.Module`` path. The reference lists
``mixed_prec.py`` and ``grad_scaler.py`` among its deleted training modules
(ZENYX_2_0_DELIVERABLES.txt:188-190); only their names survive. The Llama flagship needs neither:
its kernels are bf16 with fp32 accumulation and an fp32 master weight by construction."""
from __future__ import annotations

import contextlib

import torch

from .grad_scaler import DynamicGradScaler

_DTYPES = {"fp32": None, "no": None, "bf16": torch.bfloat16, "fp16": torch.float16}


class MixedPrecision:
    def __init__(self, precision: str = "fp32", device: torch.device | str = "cpu"):
        if precision not in _DTYPES:
            raise ValueError(f"precision must be one of {sorted(_DTYPES)}")
        self.precision = precision
        self.dtype = _DTYPES[precision]
        self.device_type = torch.device(device).type
        self.scaler = DynamicGradScaler() if precision == "fp16" else None

    @property
    def uses_scaler(self) -> bool:
        return self.scaler is not None

    def autocast(self):
        if self.dtype is None:
            return contextlib.nullcontext()
        return torch.autocast(device_type=self.device_type, dtype=self.dtype)

    def scale(self, loss: torch.Tensor) -> torch.Tensor:
        return self.scaler.scale(loss) if self.scaler is not None else loss

    def unscale_(self, optimizer) -> None:
        if self.scaler is not None:
            self.scaler.unscale_(optimizer)

    def step(self, optimizer) -> bool:
        """Runs optimizer.step() unless the scaler found an overflow; returns whether it stepped."""
        if self.scaler is None:
            optimizer.step()
            return True
        return self.scaler.step(optimizer)
