"""``HardwareDetector``: what this process can see of the machine. The reference documents the name
under ``zenyx.core.hardware`` ("Hardware detection", README.md:197,348); the module is not in its
tree. Everything here only reads; no device setting is ever changed."""
from __future__ import annotations

import os
import shutil
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional

import torch


@dataclass
class GPUInfo:
    index: int
    name: str
    sm_arch: str
    sm_count: int
    hbm_bytes: int
    is_blackwell: bool


@dataclass
class HardwareInfo:
    gpus: List[GPUInfo] = field(default_factory=list)
    p2p_matrix: List[List[bool]] = field(default_factory=list)
    host_dram_bytes: int = 0
    cpu_count: int = 0
    nvme_path: Optional[str] = None
    nvme_free_bytes: int = 0
    native_extension: bool = False

    def as_dict(self) -> Dict:
        return asdict(self)


class HardwareDetector:
    def __init__(self, nvme_candidates=("/mnt/nvme", "/scratch", "/local", "/tmp")):
        self.nvme_candidates = nvme_candidates

    def gpu_count(self) -> int:
        return torch.cuda.device_count() if torch.cuda.is_available() else 0

    def gpus(self) -> List[GPUInfo]:
        out = []
        for i in range(self.gpu_count()):
            p = torch.cuda.get_device_properties(i)
            out.append(GPUInfo(i, p.name, f"sm_{p.major}{p.minor}", p.multi_processor_count, p.total_memory, p.major == 10))
        return out

    def p2p_matrix(self) -> List[List[bool]]:
        n = self.gpu_count()
        return [[i == j or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]

    def host_dram_bytes(self) -> int:
        try:
            import psutil

            return int(psutil.virtual_memory().total)
        except Exception:  # noqa: BLE001
            return os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES")

    def nvme_candidate(self):
        """First writable candidate directory with its free space (the file tier's default home)."""
        for p in self.nvme_candidates:
            if os.path.isdir(p) and os.access(p, os.W_OK):
                return p, shutil.disk_usage(p).free
        return None, 0

    def detect(self) -> HardwareInfo:
        from ..ops import _ext

        path, free = self.nvme_candidate()
        return HardwareInfo(gpus=self.gpus(), p2p_matrix=self.p2p_matrix(), host_dram_bytes=self.host_dram_bytes(),
                            cpu_count=os.cpu_count() or 1, nvme_path=path, nvme_free_bytes=free,
                            native_extension=_ext.have_cuda_ext())

    def supports_native_kernels(self) -> bool:
        g = self.gpus()
        return bool(g) and all(x.is_blackwell for x in g)
