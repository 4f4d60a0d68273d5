from .distributed import DistributedTrainingManager, FaultInjector, Heartbeat, RankFailure
from .hardware import GPUInfo, HardwareDetector, HardwareInfo
from .memory import PinnedPool, TierBudget, default_budget

__all__ = ["DistributedTrainingManager", "Heartbeat", "FaultInjector", "RankFailure", "HardwareDetector",
           "HardwareInfo", "GPUInfo", "TierBudget", "default_budget", "PinnedPool"]
