from .activation_manager import ActivationManager, CheckpointPolicy
from .tracker import MemorySnapshot, MemoryTracker

__all__ = ["ActivationManager", "CheckpointPolicy", "MemoryTracker", "MemorySnapshot"]
