"""Selective rematerialisation for arbitrary ``nn.Module`` trees.

Same names as the reference (zenyx/memory/activation_manager.py:16-85): ``CheckpointPolicy`` and
``ActivationManager`` with ``should_checkpoint`` / ``checkpoint_module`` / ``hook_into_model`` /
``estimate_memory_saving``; plus the ``checkpoint_attention()`` / ``checkpoint_ffn()`` toggles the
reference's quick-start calls but never defined (ZENYX_2_0_QUICK_START.py:144-145), and
``unhook`` to restore the original forwards. The Llama flagship does not go through this class:
its per-activation policy is ``zenyx_b200.models.RematPolicy``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

_ATTENTION_KEYS = ("attention", "attn")
_FFN_KEYS = ("mlp", "ffn", "feed_forward", "feedforward")


@dataclass
class CheckpointPolicy:
    checkpoint_attention: bool = False
    checkpoint_ffn: bool = True
    min_trainable_params: int = 50_000


class ActivationManager:
    def __init__(self, policy: CheckpointPolicy | None = None):
        self.policy = policy or CheckpointPolicy()
        self._original: Dict[nn.Module, Callable] = {}
        self.wrapped_names: List[str] = []

    # toggles ---------------------------------------------------------------------------------
    def checkpoint_attention(self, enabled: bool = True) -> "ActivationManager":
        self.policy.checkpoint_attention = enabled
        return self

    def checkpoint_ffn(self, enabled: bool = True) -> "ActivationManager":
        self.policy.checkpoint_ffn = enabled
        return self

    # selection -------------------------------------------------------------------------------
    def should_checkpoint(self, name: str, module: nn.Module) -> bool:
        lname = name.lower()
        trainable = sum(p.numel() for p in module.parameters() if p.requires_grad)
        if trainable < self.policy.min_trainable_params:
            return False
        if self.policy.checkpoint_attention and any(k in lname for k in _ATTENTION_KEYS):
            return True
        if self.policy.checkpoint_ffn and any(k in lname for k in _FFN_KEYS):
            return True
        return False

    def checkpoint_module(self, module: nn.Module) -> Callable:
        """Returns a callable running `module` under activation checkpointing when a gradient is needed."""
        forward = module.forward

        def run(*args, **kwargs):
            needs_grad = torch.is_grad_enabled() and any(
                isinstance(a, torch.Tensor) and a.requires_grad for a in list(args) + list(kwargs.values()))
            needs_grad = needs_grad or (torch.is_grad_enabled() and any(p.requires_grad for p in module.parameters()))
            if not needs_grad:
                return forward(*args, **kwargs)
            return checkpoint(forward, *args, use_reentrant=False, **kwargs)

        return run

    def hook_into_model(self, model: nn.Module) -> List[str]:
        """Wraps every selected sub-module (outermost match only); returns their names."""
        chosen: List[str] = []
        for name, module in model.named_modules():
            if not name or module in self._original:
                continue
            if any(name.startswith(c + ".") for c in chosen):
                continue  # an ancestor is already checkpointed
            if self.should_checkpoint(name, module):
                self._original[module] = module.forward
                module.forward = self.checkpoint_module(module)  # type: ignore[method-assign]
                chosen.append(name)
        self.wrapped_names.extend(chosen)
        return chosen

    def unhook(self) -> None:
        for module, fwd in self._original.items():
            module.forward = fwd  # type: ignore[method-assign]
        self._original.clear()
        self.wrapped_names.clear()

    @staticmethod
    def estimate_memory_saving(num_layers: int, hidden_dim: int, seq_len: int, batch_size: int,
                               bytes_per_element: int = 2) -> Dict[str, float]:
        """bf16 bytes of B*S*H (attention) and B*S*4H (FFN) per layer, as the reference counts them."""
        attn = batch_size * seq_len * hidden_dim * bytes_per_element * num_layers
        ffn = batch_size * seq_len * 4 * hidden_dim * bytes_per_element * num_layers
        return {"attention_mb": attn / 1e6, "ffn_mb": ffn / 1e6, "total_gb": (attn + ffn) / 1e9}
