"""Activation checkpointing helpers (name from the reference's deleted
``zenyx/train/activation_checkpoint.py``, ZENYX_2_0_DELIVERABLES.txt:190). For arbitrary modules this
is a thin layer over ``ActivationManager``; for the Llama flagship it maps a policy name to the
model's explicit ``RematPolicy``."""
from __future__ import annotations

from typing import List

import torch.nn as nn

from ..memory import ActivationManager, CheckpointPolicy
from ..models.llama import RematPolicy


def apply_activation_checkpointing(model: nn.Module, attention: bool = False, ffn: bool = True,
                                   min_trainable_params: int = 50_000) -> List[str]:
    """Wraps the selected sub-modules; returns the wrapped module names."""
    mgr = ActivationManager(CheckpointPolicy(attention, ffn, min_trainable_params))
    return mgr.hook_into_model(model)


def remat_policy(name: str) -> RematPolicy:
    table = {"full": RematPolicy.full, "selective": RematPolicy.selective, "none": RematPolicy.none}
    if name not in table:
        raise ValueError(f"unknown rematerialisation policy {name!r}; expected one of {sorted(table)}")
    return table[name]()
