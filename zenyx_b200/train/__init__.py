"""Training API: ``Trainer`` / ``TrainerConfig`` / ``load_state_dict_chunked`` (the reference's
zenyx/train/__init__.py:1-4) plus the modules the reference documents but no longer ships."""
from .loading import load_state_dict_chunked
from .trainer import Trainer, TrainerConfig

__all__ = ["Trainer", "TrainerConfig", "load_state_dict_chunked"]
