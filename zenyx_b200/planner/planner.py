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
    optimizer_state_dtype: str = "fp32"   # storage of Adam's moments: "fp32" or "bf16" (arithmetic and master stay fp32)
    estimate: Optional[StepEstimate] = None
    notes: List[str] = field(default_factory=list)

    def describe(self) -> str:
        e = self.estimate
        mem = f"{e.total_bytes / 1e9:.0f} GB/GPU, ~{e.tokens_per_s:,.0f} tok/s" if e else ""
        gu = f" (gate|up in {self.remat.gu_layers} layers)" if self.remat.gu_layers >= 0 and "gu" in self.remat.saved else ""
        return (f"dp{self.dp} x cp{self.cp}, remat keeps {','.join(self.remat.saved)}{gu}, "
                f"{self.optimizer_state_dtype} moments, {mem}")


def plan(model_cfg: LlamaConfig, seq_len: int, global_batch: int, n_gpus: int, hbm_bytes: float = 180e9,
         nvlink_GBps: float = 770.0, ring_degree: Optional[int] = None, candidates: Sequence[int] = (1, 2, 4, 8),
         memory_fraction: float = 0.88, peaks: Optional[HardwarePeaks] = None,
         host_bytes: Optional[float] = None, optimizer_state_dtype: str = "auto") -> ParallelPlan:
    """Returns the fastest plan whose estimated footprint fits in ``memory_fraction * hbm_bytes``.

    With ``ring_degree`` given only the rematerialisation policy is searched (the benchmark configs
    fix the ring degree). Otherwise every ring degree that divides ``n_gpus``, keeps at least one
    sequence per data-parallel replica and keeps every zigzag chunk a multiple of 128 tokens is tried.
    For each split the first rung of the rematerialisation ladder that fits is taken, and what memory is
    left then goes to the gate|up projection of as many layers as fit (``RematPolicy.gu_layers``).
    ``optimizer_state_dtype``: "fp32", "bf16", or "auto" = bf16 moments only where the memory they free buys
    at least 2 % of estimated step time (on one GPU at 32K context: 32 GB, i.e. 17 layers less recomputation).
    """
    if optimizer_state_dtype not in ("auto", "fp32", "bf16"):
        raise ValueError("optimizer_state_dtype is 'auto', 'fp32' or 'bf16'")
    peaks = peaks or HardwarePeaks.load()
    peaks.nvlink_gbs = nvlink_GBps
    peaks.hbm_bytes = hbm_bytes
    budget = hbm_bytes * memory_fraction
    degrees = [ring_degree] if ring_degree else [c for c in candidates if c <= n_gpus]
    host_free = host_memory_available_bytes() if host_bytes is None else host_bytes

    # A plan that departs from the plain choices (fp32 moments, a whole rung of the ladder) has to be worth it:
    # each departure must buy 2 % of estimated step time, so near-ties go to the plain, measured configurations.
    def score(pl: ParallelPlan) -> float:
        departures = (pl.optimizer_state_dtype != "fp32") + (pl.remat.gu_layers >= 0)
        return pl.estimate.step_s * (1.02 ** departures)

    def candidates_for(moment_bytes: int) -> List[ParallelPlan]:
        out: List[ParallelPlan] = []
        for cp in degrees:
            if n_gpus % cp or global_batch % max(1, n_gpus // cp) or seq_len % (128 * (2 * cp if cp > 1 else 1)):
                continue
            dp = n_gpus // cp

            def make(remat, est):
                return ParallelPlan(dp=dp, cp=cp, micro_batch=1, micro_batches=global_batch // dp, remat=remat,
                                    kv_budget_bytes=int(min(16 << 30, 0.1 * hbm_bytes)),
                                    optimizer_state_dtype="fp32" if moment_bytes == 4 else "bf16", estimate=est)

            for remat in REMAT_LADDER:
                est = estimate(model_cfg, seq_len, global_batch, n_gpus, cp, remat, peaks, moment_bytes=moment_bytes)
                if est.total_bytes > budget:
                    continue
                # pinned host memory for offloaded activations: every rank of the node needs its own, and half
                # of what the machine has free stays untouched
                need_host = (remat.host_bytes_per_token_per_layer(model_cfg) * (seq_len // cp) * model_cfg.n_layers *
                             n_gpus)
                if need_host > 0.5 * host_free:
                    continue
                out.append(make(remat, est))
                if "gu" not in remat.saved and "gu@host" not in remat.saved:
                    per_layer = 2 * 2 * model_cfg.ffn_dim * (seq_len // cp)
                    k = min(model_cfg.n_layers, int((budget - est.total_bytes) // per_layer))
                    if k >= 1:
                        partial = RematPolicy(tuple(remat.saved) + ("gu",), gu_layers=k)
                        out.append(make(partial, estimate(model_cfg, seq_len, global_batch, n_gpus, cp, partial, peaks,
                                                          moment_bytes=moment_bytes)))
                break  # the ladder is ordered from least to most recompute: first fit is the fastest for this cp
        return out

    pool: List[ParallelPlan] = []
    if optimizer_state_dtype in ("auto", "fp32"):
        pool += candidates_for(4)
    if optimizer_state_dtype in ("auto", "bf16"):
        pool += candidates_for(2)
    best = min(pool, key=score) if pool else None
    if best is None:
        raise ValueError(
            f"no plan fits {model_cfg.num_params() / 1e9:.1f}B parameters at seq {seq_len} on {n_gpus} GPU(s) with "
            f"{hbm_bytes / 1e9:.0f} GB each; lower the sequence length or add GPUs")
    return best
