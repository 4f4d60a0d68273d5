"""Model loading: chunked ``state_dict`` loading (what the reference ships,
zenyx/train/loading.py:11-30), safetensors files and this package's checkpoint directories.
The reference's ``zenyx/loader`` package was removed from its tree (ZENYX_2_0_PHASE_1_SUMMARY.md:26-27);
the functions live in ``train/loading.py`` and ``train/checkpoint.py`` and are gathered here."""
from __future__ import annotations

from typing import Dict

import torch

from ..train.checkpoint import latest_step
from ..train.checkpoint import load as load_checkpoint
from ..train.checkpoint import save as save_checkpoint
from ..train.loading import load_state_dict_chunked


def load_safetensors(path: str, device: str = "cpu") -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return load_file(path, device=device)


def load_into(model: torch.nn.Module, path: str, chunk_size: int = 64, strict: bool = True):
    """Loads a ``.safetensors`` or ``torch.save`` file into ``model`` in chunks of ``chunk_size`` tensors,
    so that at most one chunk is converted / copied at a time. Returns (missing, unexpected) keys."""
    if path.endswith(".safetensors"):
        state = load_safetensors(path)
    else:
        state = torch.load(path, map_location="cpu", weights_only=True)
        if isinstance(state, dict) and "model" in state and isinstance(state["model"], dict):
            state = state["model"]
    return load_state_dict_chunked(model, state, chunk_size=chunk_size, strict=strict)


__all__ = ["load_state_dict_chunked", "load_safetensors", "load_into", "save_checkpoint", "load_checkpoint", "latest_step"]
