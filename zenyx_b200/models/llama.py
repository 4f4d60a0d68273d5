"""Llama-3-shaped decoder built directly on the sm_100a kernels.

The reference has no model zoo: its examples stack ``nn.TransformerEncoderLayer``
(README.md:64-77, examples/03_expert_tpu_v5e8_training.py:31-78). This model is the flagship the
benchmarks run: RMSNorm, fused QKV projection, RoPE, GQA flash/ring attention, SwiGLU FFN, and a
chunked LM head whose cross-entropy never materialises the full logits.

Design points:

* every parameter is a view into ONE flat bf16 buffer, every gradient a view into ONE flat fp32
  buffer (weight gradients are accumulated there by the GEMM epilogue, so gradient accumulation over
  micro-batches costs no extra pass); the flat buffers are what the sharded optimizer
  (``zenyx_b200.parallel.zero``) reduces, updates and re-distributes;
* forward and backward of a layer are written out by hand (no autograd graph inside a layer) so
  the rematerialisation policy is explicit: ``RematPolicy.saved`` names exactly which activations
  are kept, everything else is recomputed in backward;
* the sequence may be sharded over a ring (context parallelism): positions come from the ring
  layout, K/V go to peer-visible slots and attention runs through ``ring_attn_forward/backward``.

Two entry points share that code: ``forward_backward`` (the training engine calls it once per
micro-batch) and ``loss`` (a normal autograd scalar, for ``loss.backward()`` style code).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import fused
from ..ops.attention import RingContext, ring_attn_backward, ring_attn_forward
from ..ops.gemm import gemm
from ..utils.tracing import trace_range


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    d_model: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn_dim: int = 14336
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    init_std: float = 0.02

    @classmethod
    def llama3_8b(cls) -> "LlamaConfig":
        return cls()

    @classmethod
    def tiny(cls, n_layers: int = 2, d_model: int = 256, n_heads: int = 2, n_kv_heads: int = 1, ffn_dim: int = 512,
             vocab_size: int = 1024) -> "LlamaConfig":
        return cls(vocab_size=vocab_size, d_model=d_model, n_layers=n_layers, n_heads=n_heads, n_kv_heads=n_kv_heads,
                   head_dim=128, ffn_dim=ffn_dim)

    @property
    def qkv_dim(self) -> int:
        return (self.n_heads + 2 * self.n_kv_heads) * self.head_dim

    def num_params(self) -> int:
        per_layer = (self.qkv_dim * self.d_model + self.n_heads * self.head_dim * self.d_model +
                     3 * self.ffn_dim * self.d_model + 2 * self.d_model)
        return 2 * self.vocab_size * self.d_model + self.n_layers * per_layer + self.d_model

    def flops_per_token(self, seq_len: int, causal: bool = True) -> float:
        """Training FLOPs per token: 6 x matmul parameters + attention (backward = 2.5 x forward)."""
        per_layer = (self.qkv_dim * self.d_model + self.n_heads * self.head_dim * self.d_model +
                     3 * self.ffn_dim * self.d_model)
        mm = 6.0 * (self.n_layers * per_layer + self.vocab_size * self.d_model)
        attn_fwd = 4.0 * seq_len * self.head_dim * self.n_heads * (0.5 if causal else 1.0)
        return mm + 3.5 * attn_fwd * self.n_layers


@dataclass
class RematPolicy:
    """Which per-layer activations are kept for backward; the rest is recomputed.

    Names: ``x`` (layer input, always kept), ``attn`` (attention output + log-sum-exp), ``qkv``
    (rotated Q/K/V), ``h1`` (post-attention residual stream), ``gu`` (gate|up projection),
    ``gu@host`` (gate|up projection kept in pinned host memory: copied out on a side stream while the
    layer's forward continues, prefetched one layer ahead during backward; costs no HBM beyond two
    staging buffers and replaces the largest recomputed GEMM of a layer by two PCIe copies).
    """

    saved: Tuple[str, ...] = ("x", "attn")
    # With "gu" in ``saved``: keep the gate|up projection (the largest activation, 4 * ffn_dim bytes per token)
    # only in the first ``gu_layers`` layers and recompute it in the others; -1 = in every layer. Lets the
    # planner spend whatever memory is left after the cheaper activations instead of all or nothing.
    gu_layers: int = -1

    @classmethod
    def full(cls) -> "RematPolicy":        # recompute everything, attention included
        return cls(("x",))

    @classmethod
    def selective(cls) -> "RematPolicy":   # keep attention results, recompute the projections
        return cls(("x", "attn"))

    @classmethod
    def none(cls) -> "RematPolicy":        # keep everything a GEMM or the attention produced
        return cls(("x", "attn", "qkv", "h1", "gu"))

    @classmethod
    def host_offload(cls) -> "RematPolicy":   # everything small in HBM, gate|up in pinned host memory
        return cls(("x", "attn", "qkv", "h1", "gu@host"))

    def host_bytes_per_token_per_layer(self, cfg: LlamaConfig) -> int:
        return 2 * 2 * cfg.ffn_dim if "gu@host" in self.saved else 0

    def keeps_gu(self, layer: int) -> bool:
        return "gu" in self.saved and (self.gu_layers < 0 or layer < self.gu_layers)

    def gu_fraction(self, cfg: LlamaConfig) -> float:
        """Share of the layers whose gate|up projection is kept."""
        if "gu" not in self.saved:
            return 0.0
        return 1.0 if self.gu_layers < 0 else min(self.gu_layers, cfg.n_layers) / max(1, cfg.n_layers)

    def bytes_per_token_per_layer(self, cfg: LlamaConfig) -> float:
        """Average over the layers (the gate|up projection may be kept in some of them only)."""
        sizes = {"x": cfg.d_model, "attn": cfg.n_heads * cfg.head_dim + 2 * cfg.n_heads, "qkv": cfg.qkv_dim,
                 "h1": cfg.d_model, "gu": 0, "gu@host": 0}
        return 2 * sum(sizes[n] for n in self.saved) + 2 * 2 * cfg.ffn_dim * self.gu_fraction(cfg)


class FlatBuffers:
    """The flat bf16 parameter buffer and the flat fp32 gradient buffer of a model.

    Parameters that take weight decay are laid out first; every tensor starts on a 256-byte
    boundary; the total is padded to a multiple of ``align * 840`` (840 = lcm(1..8)), which does NOT
    depend on the world size, so the same flat layout splits evenly into 4-aligned shards for any
    rank count that divides it (1-8, 10, 12, 14, 16, ...) and a checkpoint re-shards across world sizes.
    With ``symmetric_group`` the two buffers live in peer-visible memory (needed by the fused
    reduce-scatter / AdamW / all-gather kernel when there is more than one rank).
    """

    def __init__(self, specs: List[Tuple[str, Tuple[int, ...], bool]], device, align: int = 1024,
                 symmetric_group=None, world_size: int = 1, dtype: torch.dtype = torch.bfloat16):
        self.index: Dict[str, Tuple[int, Tuple[int, ...]]] = {}
        off = 0
        ordered = [s for s in specs if s[2]] + [s for s in specs if not s[2]]
        self.decay_end = 0
        for name, shape, decay in ordered:
            n = math.prod(shape)
            self.index[name] = (off, tuple(shape))
            off += (n + 127) // 128 * 128
            if decay:
                self.decay_end = off
        step = align * 840
        self.total = (off + step - 1) // step * step
        if self.total % (4 * max(world_size, 1)) != 0:
            raise ValueError(f"world size {world_size} does not divide the flat buffer into 4-aligned shards")
        self.sym_params = self.sym_grads = None
        dev = torch.device(device)
        if symmetric_group is not None and world_size > 1 and dev.type == "cuda":
            from ..parallel.peer import SymmetricBuffer

            self.sym_params = SymmetricBuffer(self.total * 2, symmetric_group)
            self.sym_grads = SymmetricBuffer(self.total * 4, symmetric_group)
            self.params = self.sym_params.tensor(None, 0, (self.total,), torch.bfloat16)
            self.grads = self.sym_grads.tensor(None, 0, (self.total,), torch.float32)
        else:
            self.params = torch.zeros(self.total, device=dev, dtype=dtype)
            self.grads = torch.zeros(self.total, device=dev, dtype=torch.float32)

    def param(self, name: str) -> torch.Tensor:
        off, shape = self.index[name]
        return self.params[off: off + math.prod(shape)].view(shape)

    def grad(self, name: str) -> torch.Tensor:
        off, shape = self.index[name]
        return self.grads[off: off + math.prod(shape)].view(shape)


class LlamaModel(nn.Module):
    def __init__(self, cfg: LlamaConfig, device="cpu", remat: Optional[RematPolicy] = None, seed: int = 0,
                 symmetric_group=None, world_size: int = 1, head_chunk_tokens: int = 4096,
                 dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        self.remat = remat or RematPolicy.selective()
        self.head_chunk_tokens = head_chunk_tokens
        H, F = cfg.d_model, cfg.ffn_dim
        specs: List[Tuple[str, Tuple[int, ...], bool]] = [("embed.weight", (cfg.vocab_size, H), True)]
        for l in range(cfg.n_layers):
            specs += [
                (f"layers.{l}.wqkv", (cfg.qkv_dim, H), True),
                (f"layers.{l}.wo", (H, cfg.n_heads * cfg.head_dim), True),
                (f"layers.{l}.wgu", (2 * F, H), True),
                (f"layers.{l}.wd", (H, F), True),
                (f"layers.{l}.norm1", (H,), False),
                (f"layers.{l}.norm2", (H,), False),
            ]
        specs += [("lm_head.weight", (cfg.vocab_size, H), True), ("final_norm", (H,), False)]
        self.flat = FlatBuffers(specs, device, symmetric_group=symmetric_group, world_size=world_size, dtype=dtype)
        self._names = [s[0] for s in specs]
        dev = self.flat.params.device
        gen = torch.Generator(device=dev).manual_seed(seed)
        for name, shape, _ in specs:
            p = self.flat.param(name)
            if len(shape) == 1:
                p.fill_(1.0)
            else:
                # generated on the target device, in row chunks so the fp32 temporary stays small
                rows = shape[0]
                step = max(1, (1 << 26) // shape[1])
                for r0 in range(0, rows, step):
                    r1 = min(rows, r0 + step)
                    p[r0:r1].copy_(
                        (torch.randn(r1 - r0, shape[1], generator=gen, device=dev) * cfg.init_std).to(p.dtype))
            param = nn.Parameter(p, requires_grad=True)
            param.main_grad = self.flat.grad(name)
            self.register_parameter(name.replace(".", "_"), param)
        self._rope_cache: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}
        # host offload of gate|up activations (RematPolicy name "gu@host")
        self._off_stream = None
        self._off_host: Dict[int, torch.Tensor] = {}
        self._off_stage: List[torch.Tensor] = []
        self._off_ready: Dict[int, "torch.cuda.Event"] = {}
        self._off_stage_free: List[Optional["torch.cuda.Event"]] = [None, None]

    # -------------------------------------------------------------------------------------------
    def w(self, name: str) -> torch.Tensor:
        return self.flat.param(name)

    def g(self, name: str) -> torch.Tensor:
        return self.flat.grad(name)

    def named_flat_parameters(self):
        for n in self._names:
            yield n, self.flat.param(n)

    def state_dict_flat(self) -> Dict[str, torch.Tensor]:
        return {n: self.flat.param(n) for n in self._names}

    def zero_grad(self, set_to_none: bool = False) -> None:  # noqa: ARG002
        self.flat.grads.zero_()

    # -------------------------------------------------------------------------------------------
    # gate|up activations in pinned host memory
    # -------------------------------------------------------------------------------------------
    def _offload_gu(self, l: int, gu: torch.Tensor) -> None:
        """Starts the device-to-host copy of layer l's gate|up activation on the side stream."""
        if self._off_stream is None:
            self._off_stream = torch.cuda.Stream()
        host = self._off_host.get(l)
        if host is None or host.shape != gu.shape:
            host = torch.empty(gu.shape, dtype=gu.dtype, pin_memory=True)
            self._off_host[l] = host
        main = torch.cuda.current_stream()
        self._off_stream.wait_stream(main)              # gu has been produced
        with torch.cuda.stream(self._off_stream):
            host.copy_(gu, non_blocking=True)
        gu.record_stream(self._off_stream)              # its memory is not reused before the copy has read it

    def _start_fetch_gu(self, l: int) -> None:
        """Starts the host-to-device copy of layer l's gate|up activation into a staging buffer."""
        if l < 0 or l in self._off_ready or l not in self._off_host:
            return
        host = self._off_host[l]
        slot = l % 2
        if len(self._off_stage) < 2:
            self._off_stage = [torch.empty(host.shape, dtype=host.dtype, device="cuda") for _ in range(2)]
        with torch.cuda.stream(self._off_stream):
            if self._off_stage_free[slot] is not None:
                self._off_stream.wait_event(self._off_stage_free[slot])   # the previous user of the slot is done
            self._off_stage[slot].view(-1)[: host.numel()].view(host.shape).copy_(host, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        self._off_ready[l] = ev

    def _fetch_gu(self, l: int) -> torch.Tensor:
        """Layer l's gate|up activation on the device; also starts the fetch for layer l - 1."""
        self._start_fetch_gu(l)
        torch.cuda.current_stream().wait_event(self._off_ready.pop(l))
        host = self._off_host[l]
        gu = self._off_stage[l % 2].view(-1)[: host.numel()].view(host.shape)
        self._start_fetch_gu(l - 1)
        return gu

    def _release_gu(self, l: int) -> None:
        ev = torch.cuda.Event()
        ev.record()
        self._off_stage_free[l % 2] = ev

    def _rope(self, ring: RingContext, s_local: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        key = (ring.rank, ring.degree, ring.seq_len, ring.layout, s_local, str(device))
        if key not in self._rope_cache:
            from ..ops.attention import _positions

            pos = _positions(ring.positions(), s_local, device)
            self._rope_cache = {key: fused.rope_tables(pos, self.cfg.head_dim, self.cfg.rope_theta)}
        return self._rope_cache[key]

    # -------------------------------------------------------------------------------------------
    # one layer
    # -------------------------------------------------------------------------------------------
    def _qkv(self, l: int, x, B: int, S: int, ring: RingContext):
        """norm1 -> QKV projection -> RoPE. Returns (q, k, v) as [B,S,H,D] views, and the norm output."""
        cfg = self.cfg
        D, Hq, Hkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
        xn, rstd1 = fused.rmsnorm_fwd(x, self.w(f"layers.{l}.norm1"), cfg.norm_eps)
        qkv = gemm(xn, self.w(f"layers.{l}.wqkv"))
        cos, sin = self._rope(ring, S, x.device)
        use_peer = ring.degree > 1 and x.is_cuda
        if use_peer:
            ks, vs = ring.peer.kv_views(ring.rank, l % 2, (B, S, Hkv, D))
            fused.rope_qkv_(qkv, cos, sin, Hq, Hkv, D, S, k_out=ks, v_out=vs)
            k, v = ks, vs
        else:
            fused.rope_qkv_(qkv, cos, sin, Hq, Hkv, D, S)
            k = qkv[:, Hq * D: (Hq + Hkv) * D].view(B, S, Hkv, D)
            v = qkv[:, (Hq + Hkv) * D:].view(B, S, Hkv, D)
        q = qkv[:, : Hq * D].view(B, S, Hq, D)
        return q, k, v, xn, rstd1, qkv

    def _layer_forward(self, l: int, x, B: int, S: int, ring: RingContext, keep: bool):
        cfg = self.cfg
        scale = 1.0 / math.sqrt(cfg.head_dim)
        q, k, v, xn, rstd1, qkv = self._qkv(l, x, B, S, ring)
        o, lse = ring_attn_forward(ring, q, k, v, scale, slot=l % 2)
        T = x.shape[0]
        h1 = gemm(o.view(T, -1), self.w(f"layers.{l}.wo"), addend=x)
        hn, rstd2 = fused.rmsnorm_fwd(h1, self.w(f"layers.{l}.norm2"), cfg.norm_eps)
        gu = gemm(hn, self.w(f"layers.{l}.wgu"))
        a = fused.swiglu_fwd(gu)
        out = gemm(a, self.w(f"layers.{l}.wd"), addend=h1)
        saved = None
        if keep:
            names = self.remat.saved
            saved = {"x": x}
            if "attn" in names:
                saved["o"], saved["lse"] = o, lse
            if "qkv" in names:
                saved["qkv"] = qkv
                if ring.degree > 1 and x.is_cuda:  # the peer slot is recycled two layers later
                    saved["k"], saved["v"] = k.clone(), v.clone()
            if "h1" in names:
                saved["h1"] = h1
            if self.remat.keeps_gu(l):
                saved["gu"] = gu
            elif "gu@host" in names and gu.is_cuda:
                self._offload_gu(l, gu)
                saved["gu_host"] = True
        return out, saved

    def _layer_backward(self, l: int, dout, saved, B: int, S: int, ring: RingContext):
        cfg = self.cfg
        D, Hq, Hkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
        scale = 1.0 / math.sqrt(D)
        x = saved["x"]
        T = x.shape[0]
        pre = f"layers.{l}."
        # ---- rematerialise what was not kept ----
        if "qkv" in saved:
            qkv = saved["qkv"]
            xn, rstd1 = fused.rmsnorm_fwd(x, self.w(pre + "norm1"), cfg.norm_eps)
            q = qkv[:, : Hq * D].view(B, S, Hq, D)
            if "k" in saved:
                k, v = ring.peer.kv_views(ring.rank, l % 2, (B, S, Hkv, D))
                k.copy_(saved["k"])
                v.copy_(saved["v"])
            else:
                k = qkv[:, Hq * D: (Hq + Hkv) * D].view(B, S, Hkv, D)
                v = qkv[:, (Hq + Hkv) * D:].view(B, S, Hkv, D)
        else:
            q, k, v, xn, rstd1, qkv = self._qkv(l, x, B, S, ring)
        if "o" in saved:
            o, lse = saved["o"], saved["lse"]
        else:
            o, lse = ring_attn_forward(ring, q, k, v, scale, slot=l % 2)
        h1 = saved["h1"] if "h1" in saved else gemm(o.view(T, -1), self.w(pre + "wo"), addend=x)
        hn, rstd2 = fused.rmsnorm_fwd(h1, self.w(pre + "norm2"), cfg.norm_eps)
        if "gu" in saved:
            gu = saved["gu"]
        elif "gu_host" in saved:
            gu = self._fetch_gu(l)
        else:
            gu = gemm(hn, self.w(pre + "wgu"))
        a = fused.swiglu_fwd(gu)
        # ---- FFN backward ----
        gwd, gwgu = self.g(pre + "wd"), self.g(pre + "wgu")
        da = gemm(dout, self.w(pre + "wd"), trans_b=True)
        gemm(dout, a, trans_a=True, trans_b=True, out=gwd, addend=gwd)
        del a
        dgu = fused.swiglu_bwd(gu, da)
        if "gu_host" in saved:
            self._release_gu(l)   # the staging slot may take the activation of layer l - 2 now
        del da, gu
        dhn = gemm(dgu, self.w(pre + "wgu"), trans_b=True)
        gemm(dgu, hn, trans_a=True, trans_b=True, out=gwgu, addend=gwgu)
        del dgu, hn
        dh1 = fused.rmsnorm_bwd(dhn, h1, self.w(pre + "norm2"), rstd2, self.g(pre + "norm2"), dres=dout)
        del dhn, h1
        # ---- attention backward ----
        gwo, gwqkv = self.g(pre + "wo"), self.g(pre + "wqkv")
        d_o = gemm(dh1, self.w(pre + "wo"), trans_b=True)
        gemm(dh1, o.view(T, -1), trans_a=True, trans_b=True, out=gwo, addend=gwo)
        dq, dk, dv = ring_attn_backward(ring, q, k, v, o, d_o.view(B, S, Hq, D), lse, scale, slot=l % 2)
        del d_o, o
        cos, sin = self._rope(ring, S, x.device)
        dqkv = fused.rope_bwd_pack(dq, dk, dv, cos, sin, Hq, Hkv, D, S, dtype=x.dtype)
        del dq, dk, dv, qkv
        dxn = gemm(dqkv, self.w(pre + "wqkv"), trans_b=True)
        gemm(dqkv, xn, trans_a=True, trans_b=True, out=gwqkv, addend=gwqkv)
        del dqkv, xn
        return fused.rmsnorm_bwd(dxn, x, self.w(pre + "norm1"), rstd1, self.g(pre + "norm1"), dres=dh1)

    # -------------------------------------------------------------------------------------------
    # LM head + loss, forward and backward in one sweep over token chunks
    # -------------------------------------------------------------------------------------------
    def _head_loss(self, h, targets, loss_weight: float, want_grad: bool):
        cfg = self.cfg
        T = h.shape[0]
        hn, rstd = fused.rmsnorm_fwd(h, self.w("final_norm"), cfg.norm_eps)
        W = self.w("lm_head.weight")
        gW = self.g("lm_head.weight")
        dhn = torch.empty_like(hn) if want_grad else None
        loss_sum = torch.zeros((), device=h.device, dtype=torch.float32)
        tflat = targets.reshape(-1)
        step = self.head_chunk_tokens
        for t0 in range(0, T, step):
            t1 = min(T, t0 + step)
            logits = gemm(hn[t0:t1], W)
            losses = fused.cross_entropy_fwd_bwd_(logits, tflat[t0:t1], loss_weight)
            loss_sum += losses.sum()
            if want_grad:
                gemm(logits, W, trans_b=True, out=dhn[t0:t1])
                gemm(logits, hn[t0:t1], trans_a=True, trans_b=True, out=gW, addend=gW)
            del logits
        loss = loss_sum * loss_weight
        if not want_grad:
            return loss, None
        dh = fused.rmsnorm_bwd(dhn, h, self.w("final_norm"), rstd, self.g("final_norm"))
        return loss, dh

    # -------------------------------------------------------------------------------------------
    # public entry points
    # -------------------------------------------------------------------------------------------
    def _ring(self, ring: Optional[RingContext], S: int) -> RingContext:
        return ring if ring is not None else RingContext(rank=0, degree=1, seq_len=S)

    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor, loss_weight: Optional[float] = None,
                         ring: Optional[RingContext] = None) -> torch.Tensor:
        """One micro-batch: forward, loss, backward; gradients are ADDED into the flat fp32 buffer.

        tokens/targets: [B, S_local] int64 (this rank's shard of the sequence). The returned scalar is
        ``loss_weight * sum(token losses)``; with ``loss_weight = 1 / (tokens in the global batch)``
        the per-micro-batch, per-rank values sum to the global mean loss and the accumulated
        gradient is its gradient.
        """
        B, S = tokens.shape
        ring = self._ring(ring, S)
        if loss_weight is None:
            loss_weight = 1.0 / (B * S * ring.degree)
        with torch.no_grad():
            with trace_range("embedding"):
                h = fused.embedding_fwd(tokens, self.w("embed.weight"))
            saved_all = []
            for l in range(self.cfg.n_layers):
                with trace_range(f"layer{l}.forward"):
                    h, saved = self._layer_forward(l, h, B, S, ring, keep=True)
                saved_all.append(saved)
            if "gu@host" in self.remat.saved and h.is_cuda:
                self._start_fetch_gu(self.cfg.n_layers - 1)   # under the LM head instead of in front of the last layer
            with trace_range("head+loss"):
                loss, dh = self._head_loss(h, targets, loss_weight, want_grad=True)
            del h
            for l in reversed(range(self.cfg.n_layers)):
                with trace_range(f"layer{l}.backward"):
                    dh = self._layer_backward(l, dh, saved_all.pop(), B, S, ring)
            with trace_range("embedding.backward"):
                fused.embedding_bwd(tokens, dh, self.g("embed.weight"))
        return loss

    def forward(self, tokens: torch.Tensor, ring: Optional[RingContext] = None) -> torch.Tensor:
        """Hidden states after the final norm, [B, S_local, d_model] (no gradient tracking)."""
        B, S = tokens.shape
        ring = self._ring(ring, S)
        with torch.no_grad():
            h = fused.embedding_fwd(tokens, self.w("embed.weight"))
            for l in range(self.cfg.n_layers):
                h, _ = self._layer_forward(l, h, B, S, ring, keep=False)
            hn, _ = fused.rmsnorm_fwd(h, self.w("final_norm"), self.cfg.norm_eps)
        return hn.view(B, S, -1)

    def logits(self, tokens: torch.Tensor, ring: Optional[RingContext] = None) -> torch.Tensor:
        hn = self.forward(tokens, ring)
        B, S, H = hn.shape
        return gemm(hn.view(B * S, H), self.w("lm_head.weight")).view(B, S, -1)

    def loss(self, tokens: torch.Tensor, targets: torch.Tensor, ring: Optional[RingContext] = None) -> torch.Tensor:
        """Mean token cross-entropy as an autograd scalar: ``model.loss(x, y).backward()`` adds the
        gradients into the flat fp32 buffer (``param.main_grad``) like forward_backward does."""
        anchor = next(self.parameters())
        return _LlamaLossFn.apply(anchor, self, tokens, targets, ring)


class _LlamaLossFn(torch.autograd.Function):
    """Whole-model autograd node: forward keeps the per-layer saved sets, backward replays them."""

    @staticmethod
    def forward(ctx, anchor, model: LlamaModel, tokens, targets, ring):  # noqa: ARG004
        B, S = tokens.shape
        ring = model._ring(ring, S)
        loss_weight = 1.0 / (B * S * ring.degree)
        h = fused.embedding_fwd(tokens, model.w("embed.weight"))
        saved_all = []
        for l in range(model.cfg.n_layers):
            h, saved = model._layer_forward(l, h, B, S, ring, keep=True)
            saved_all.append(saved)
        # the head computes its own backward in the same sweep; dh is scaled by grad_out in backward()
        loss, dh = model._head_loss(h, targets, loss_weight, want_grad=True)
        ctx.model, ctx.saved_all, ctx.dh, ctx.meta = model, saved_all, dh, (B, S, ring, tokens)
        return loss

    @staticmethod
    def backward(ctx, grad_out):
        model, saved_all, dh, (B, S, ring, tokens) = ctx.model, ctx.saved_all, ctx.dh, ctx.meta
        # The head's weight gradient was accumulated for grad_out == 1 during forward.
        dh = dh * grad_out.to(dh.dtype)
        for l in reversed(range(model.cfg.n_layers)):
            dh = model._layer_backward(l, dh, saved_all.pop(), B, S, ring)
        fused.embedding_bwd(tokens, dh, model.g("embed.weight"))
        return None, None, None, None, None
