"""Memory and time model of one training step of the Llama-shaped model on B200s.

Peaks come from ``MEASURED_PEAKS.json`` at the repository root when it exists (a copy benchmark
and a cuBLAS bf16 GEMM measured on the target GPUs), otherwise from an earlier measurement on the
same GPU model: 6.65 TB/s and 1.4 PFLOP/s sustained. NVLink is taken as 770 GB/s per direction per
GPU (measured peer copy). The reference's nearest relative is the four-line estimate in
``ExecutionPlan.from_model`` (zenyx/runtime/scheduler.py:288-294).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

from ..models.llama import LlamaConfig, RematPolicy


@dataclass
class HardwarePeaks:
    bf16_tflops: float = 1400.0      # sustained, per GPU
    hbm_gbs: float = 6650.0
    nvlink_gbs: float = 770.0        # per direction per GPU
    hbm_bytes: float = 180e9
    source: str = "fallback"

    @classmethod
    def load(cls, path: Optional[str] = None) -> "HardwarePeaks":
        p = Path(path) if path else Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
        if p.exists():
            d = json.loads(p.read_text())
            return cls(bf16_tflops=float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 1400.0))),
                       hbm_gbs=float(d.get("hbm_gbs", 6650.0)), source="measured")
        return cls()


@dataclass
class StepEstimate:
    state_bytes: float
    activation_bytes: float
    workspace_bytes: float
    total_bytes: float
    compute_s: float
    ring_s: float
    grad_sync_s: float
    step_s: float
    tokens_per_s: float


def estimate(cfg: LlamaConfig, seq_len: int, global_batch: int, n_gpus: int, cp: int, remat: RematPolicy,
             peaks: Optional[HardwarePeaks] = None, zero_shard: bool = True, kernel_efficiency: float = 0.69,
             moment_bytes: int = 4) -> StepEstimate:
    """``moment_bytes``: storage size of each of Adam's two moments (4 = fp32, 2 = bf16).
    ``kernel_efficiency``: achieved fraction of the GEMM peak over a whole step; 0.69 reproduces the measured
    8B / 32K runs on 1, 2, 4 and 8 B200s (12.3k, 24.9k, 50.1k and 97.1k tokens/s) within 3 %."""
    peaks = peaks or HardwarePeaks.load()
    P = cfg.num_params()
    dp = n_gpus // cp
    tokens_rank = seq_len // cp                      # one sequence per micro-batch
    micro_batches = max(1, global_batch // dp)
    # parameters bf16 + fp32 gradient buffer are replicated; master remainder + m + v are sharded
    state = P * (2 + 4) + P * (2 + 2 * moment_bytes) / (n_gpus if zero_shard else 1)
    if n_gpus > 1:
        state += P * 4 / n_gpus   # the reduced fp32 gradient shard kept between the norm pass and the update
    act = remat.bytes_per_token_per_layer(cfg) * tokens_rank * cfg.n_layers
    # live set of one layer's forward/backward (gate|up, its gradient, qkv, fp32 dq/dk/dv) + one logits chunk
    per_tok = 2 * (2 * 2 * cfg.ffn_dim + 2 * cfg.ffn_dim + 2 * cfg.qkv_dim + 4 * cfg.d_model) + 4 * cfg.qkv_dim
    work = per_tok * tokens_rank + 2 * 4096 * cfg.vocab_size * 2
    if "gu@host" in remat.saved:
        work += 2 * (2 * 2 * cfg.ffn_dim) * tokens_rank   # two device staging buffers for the host-resident gate|up
    flops_tok = cfg.flops_per_token(seq_len)
    recompute = 0.0
    per_layer_mm = 2.0 * (cfg.qkv_dim + cfg.n_heads * cfg.head_dim + 3 * cfg.ffn_dim) * cfg.d_model
    if "qkv" not in remat.saved:
        recompute += 2.0 * cfg.qkv_dim * cfg.d_model
    if "h1" not in remat.saved:
        recompute += 2.0 * cfg.n_heads * cfg.head_dim * cfg.d_model
    if "gu@host" not in remat.saved:   # the gate|up projection is recomputed in the layers that do not keep it
        recompute += 2.0 * 2 * cfg.ffn_dim * cfg.d_model * (1.0 - remat.gu_fraction(cfg))
    if "attn" not in remat.saved:
        recompute += 4.0 * seq_len * cfg.head_dim * cfg.n_heads * 0.5
    del per_layer_mm
    flops_tok += recompute * cfg.n_layers
    total_tokens = seq_len * global_batch
    compute_s = flops_tok * total_tokens / n_gpus / (peaks.bf16_tflops * 1e12 * kernel_efficiency)
    # Every extra ring step costs launches, two flag barriers per layer and shorter GEMM / attention
    # problems per rank. Measured on 8 GPUs at this shape: dp8 3.06 s, dp4 x cp2 3.14 s, cp8 3.68 s per step,
    # i.e. about 3 % per additional ring step.
    compute_s *= 1.0 + 0.03 * (cp - 1)
    kv_bytes_step = 2 * tokens_rank * cfg.n_kv_heads * cfg.head_dim * 2
    # forward pull + backward pull + fp32 dK/dV push, per layer per micro-batch, (cp-1) remote steps; overlapped
    ring_bytes = (2 * kv_bytes_step + 2 * kv_bytes_step) * (cp - 1) * cfg.n_layers * micro_batches
    ring_s = ring_bytes / (peaks.nvlink_gbs * 1e9)
    grad_sync_s = (P * 4 * (n_gpus - 1) / n_gpus + P * 2 * (n_gpus - 1) / n_gpus) / (peaks.nvlink_gbs * 1e9) if n_gpus > 1 else 0.0
    step_s = max(compute_s, ring_s) + grad_sync_s
    return StepEstimate(state, act, work, state + act + work, compute_s, ring_s, grad_sync_s, step_s,
                        total_tokens / step_s)
