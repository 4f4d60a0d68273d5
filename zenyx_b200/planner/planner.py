"""Parallelism planner: picks DP x CP degrees, the rematerialisation policy and the KV budget for a
model / sequence length / GPU count, sized for 180 GB of HBM per GPU and ring degrees 1/2/4/8.

The reference has no planner; its nearest relatives are ``ExecutionPlan.from_model``
(zenyx/runtime/scheduler.py:288-294), ``make_offload_policy`` (zenyx/compiler/offload_policy.py:33-58)
and ``estimate_memory_saving`` (zenyx/memory/activation_manager.py:74-85).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

from ..models.llama import LlamaConfig, RematPolicy
from .cost_model import HardwarePeaks, StepEstimate, estimate

# Host offload of the gate|up activation (RematPolicy.host_offload) is deliberately NOT on the ladder: on the
# B200 boxes this was measured on, the 120 GB per micro-batch it moves over PCIe ran at about 26 GB/s and
# made the 8B / 32K step 1.47x slower than recomputing the GEMM. It stays available as an explicit policy.
REMAT_LADDER = [RematPolicy.none(), RematPolicy(("x", "attn", "h1", "qkv")),
                RematPolicy(("x", "attn", "h1")), RematPolicy.selective(), RematPolicy.full()]


def host_memory_available_bytes() -> float:
    """MemAvailable of this machine (0 when it cannot be read)."""
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return float(line.split()[1]) * 1024.0
    except OSError:
        pass
    return 0.0


@dataclass
class ParallelPlan:
    dp: int
    cp: int
    tp: int = 1
    pp: int = 1
    micro_batch: int = 1
    micro_batches: int = 1
    remat: RematPolicy = field(default_factory=RematPolicy.selective)
    kv_budget_bytes: int = 16 << 30
    zero_stage: int = 1
    estimate: Optional[StepEstimate] = None
    notes: List[str] = field(default_factory=list)

    def describe(self) -> str:
        e = self.estimate
        mem = f"{e.total_bytes / 1e9:.0f} GB/GPU, ~{e.tokens_per_s:,.0f} tok/s" if e else ""
        return f"dp{self.dp} x cp{self.cp}, remat keeps {','.join(self.remat.saved)}, {mem}"


def plan(model_cfg: LlamaConfig, seq_len: int, global_batch: int, n_gpus: int, hbm_bytes: float = 180e9,
         nvlink_GBps: float = 770.0, ring_degree: Optional[int] = None, candidates: Sequence[int] = (1, 2, 4, 8),
         memory_fraction: float = 0.88, peaks: Optional[HardwarePeaks] = None,
         host_bytes: Optional[float] = None) -> ParallelPlan:
    """Returns the fastest plan whose estimated footprint fits in ``memory_fraction * hbm_bytes``.

    With ``ring_degree`` given only the rematerialisation policy is searched (the benchmark configs
    fix the ring degree). Otherwise every ring degree that divides ``n_gpus``, keeps at least one
    sequence per data-parallel replica and keeps every zigzag chunk a multiple of 128 tokens is tried.
    """
    peaks = peaks or HardwarePeaks.load()
    peaks.nvlink_gbs = nvlink_GBps
    peaks.hbm_bytes = hbm_bytes
    budget = hbm_bytes * memory_fraction
    degrees = [ring_degree] if ring_degree else [c for c in candidates if c <= n_gpus]
    best: Optional[ParallelPlan] = None
    for cp in degrees:
        if n_gpus % cp or global_batch % max(1, n_gpus // cp) or seq_len % (128 * (2 * cp if cp > 1 else 1)):
            continue
        dp = n_gpus // cp
        for remat in REMAT_LADDER:
            est = estimate(model_cfg, seq_len, global_batch, n_gpus, cp, remat, peaks)
            if est.total_bytes > budget:
                continue
            # pinned host memory for offloaded activations: every rank of the node needs its own, and half of
            # what the machine has free stays untouched
            need_host = remat.host_bytes_per_token_per_layer(model_cfg) * (seq_len // cp) * model_cfg.n_layers * n_gpus
            if need_host > 0.5 * (host_memory_available_bytes() if host_bytes is None else host_bytes):
                continue
            cand = ParallelPlan(dp=dp, cp=cp, micro_batch=1, micro_batches=global_batch // dp, remat=remat,
                                kv_budget_bytes=int(min(16 << 30, 0.1 * hbm_bytes)), estimate=est)
            if best is None or est.step_s < best.estimate.step_s:
                best = cand
            break  # the ladder is ordered from least to most recompute: first fit is the fastest for this cp
    if best is None:
        raise ValueError(
            f"no plan fits {model_cfg.num_params() / 1e9:.1f}B parameters at seq {seq_len} on {n_gpus} GPU(s) with "
            f"{hbm_bytes / 1e9:.0f} GB each; lower the sequence length or add GPUs")
    return best
