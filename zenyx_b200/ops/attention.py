"""Flash attention and ring (context-parallel) flash attention.

The reference advertises ring attention (``zenyx/ops/attention``, ``ring_flash_cuda.py``,
``flash_cpu.py``; ZENYX_2_0_DELIVERABLES.txt:193-196) but ships no attention code; the only
surviving fragment is ``build_ring_timeline`` (zenyx/streaming/kv_tiering.py:69-73). This module is
the implementation of that story on B200:

* ``flash_attention``       - single-GPU autograd op on the tcgen05 kernels
  (``csrc/attn/attn_fwd.cu``, ``csrc/attn/attn_bwd.cu``),
* ``ring_flash_attention``  - the same kernels driven once per ring step. Each rank keeps its K/V in
  peer-visible memory; the kernel of step *s* pulls the K/V of step *s+1* from its owner with P2P
  loads while it computes, and the backward kernels add dK/dV straight into the owner's fp32
  accumulators with P2P reductions. No NCCL send/recv is involved on GPUs. On CPU tensors (gloo
  ranks in tests) the ring falls back to fp32 PyTorch math with an all-gather standing in for the
  peer reads, so the schedule, masks and merge logic stay testable without a GPU.

Token positions are explicit: a buffer of S tokens is a list of equal chunks with global start
positions (``chunk_pos``), which is what a zigzag shard looks like.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from . import _ext

# ------------------------------------------------------------------------------------------------
# Mask / layout descriptions
# ------------------------------------------------------------------------------------------------


@dataclass(frozen=True)
class MaskSpec:
    """Causal and/or block-sparse mask at 128x128 granularity (see SparsePattern)."""

    causal: bool = True
    window_blocks: int = 0   # > 0: keep kv blocks with |q_block - kv_block| < window_blocks ...
    global_every: int = 0    # ... plus kv blocks whose index is a multiple of this

    def block_allowed(self, q_block: int, kv_block: int) -> bool:
        if self.causal and kv_block > q_block:
            return False
        if self.window_blocks > 0:
            in_window = abs(q_block - kv_block) < self.window_blocks
            is_global = self.global_every > 0 and kv_block % self.global_every == 0
            return in_window or is_global
        return True


def zigzag_chunks(rank: int, degree: int) -> Tuple[int, int]:
    """The two chunk indices (out of 2*degree) held by `rank` under load-balanced zigzag sharding."""
    return rank, 2 * degree - 1 - rank


def shard_positions(rank: int, degree: int, seq_len: int, layout: str = "zigzag") -> List[int]:
    """Global start positions of the chunks held by `rank`."""
    if degree == 1:
        return [0]
    if layout == "zigzag":
        L = seq_len // (2 * degree)
        a, b = zigzag_chunks(rank, degree)
        return [a * L, b * L]
    L = seq_len // degree
    return [rank * L]


def shard_sequence(x: torch.Tensor, rank: int, degree: int, layout: str = "zigzag", dim: int = 1) -> torch.Tensor:
    """Slices the `dim` (sequence) axis of a full tensor down to what `rank` holds."""
    if degree == 1:
        return x
    S = x.shape[dim]
    if layout == "zigzag":
        L = S // (2 * degree)
        a, b = zigzag_chunks(rank, degree)
        return torch.cat([x.narrow(dim, a * L, L), x.narrow(dim, b * L, L)], dim=dim)
    L = S // degree
    return x.narrow(dim, rank * L, L)


def unshard_sequence(parts: Sequence[torch.Tensor], degree: int, layout: str = "zigzag", dim: int = 1) -> torch.Tensor:
    """Inverse of shard_sequence given every rank's shard in rank order."""
    if degree == 1:
        return parts[0]
    if layout != "zigzag":
        return torch.cat(list(parts), dim=dim)
    L = parts[0].shape[dim] // 2
    chunks: List[Optional[torch.Tensor]] = [None] * (2 * degree)
    for r, p in enumerate(parts):
        a, b = zigzag_chunks(r, degree)
        chunks[a] = p.narrow(dim, 0, L)
        chunks[b] = p.narrow(dim, L, L)
    return torch.cat(chunks, dim=dim)  # type: ignore[arg-type]


def _positions(chunk_pos: Sequence[int], S: int, device) -> torch.Tensor:
    n = len(chunk_pos)
    L = S // n
    return torch.cat([torch.arange(p, p + L, device=device) for p in chunk_pos])


def step_has_work(mask: MaskSpec, q_pos: Sequence[int], q_len: int, kv_pos: Sequence[int], kv_len: int) -> bool:
    """Host-side predicate: does any 128x128 tile of (q buffer x kv buffer) survive the mask?"""
    Lq, Lk = q_len // len(q_pos), kv_len // len(kv_pos)
    for qp in q_pos:
        for kp in kv_pos:
            if not mask.causal and mask.window_blocks == 0:
                return True
            q_lo, q_hi = qp // 128, (qp + Lq - 1) // 128
            k_lo, k_hi = kp // 128, (kp + Lk - 1) // 128
            if mask.window_blocks == 0:
                if k_lo <= q_hi:
                    return True
                continue
            if q_hi - q_lo > 4096 or k_hi - k_lo > 4096:  # large chunk: interval reasoning
                if mask.global_every > 0:
                    first_global = ((k_lo + mask.global_every - 1) // mask.global_every) * mask.global_every
                    if first_global <= k_hi and (not mask.causal or first_global <= q_hi):
                        return True
                lo = max(k_lo, q_lo - mask.window_blocks + 1)
                hi = min(k_hi, q_hi if mask.causal else q_hi + mask.window_blocks - 1)
                if lo <= hi:
                    return True
                continue
            for qb in range(q_lo, q_hi + 1):
                for kb in range(max(k_lo, 0), k_hi + 1):
                    if mask.block_allowed(qb, kb):
                        return True
    return False


# ------------------------------------------------------------------------------------------------
# Low-level forward / backward (GPU kernels, fp32 PyTorch on CPU)
# ------------------------------------------------------------------------------------------------


def _dense_mask(mask: MaskSpec, qpos: torch.Tensor, kpos: torch.Tensor) -> torch.Tensor:
    keep = torch.ones(qpos.numel(), kpos.numel(), dtype=torch.bool, device=qpos.device)
    if mask.causal:
        keep &= kpos[None, :] <= qpos[:, None]
    if mask.window_blocks > 0:
        qb, kb = (qpos // 128)[:, None], (kpos // 128)[None, :]
        k2 = (qb - kb).abs() < mask.window_blocks
        if mask.global_every > 0:
            k2 |= (kb % mask.global_every) == 0
        keep &= k2
    return keep


def _ref_scores(q, k, scale, mask, q_chunk_pos, kv_chunk_pos):
    B, Sq, Hq, D = q.shape
    Hkv = k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, dim=1)
    s = torch.einsum("bhqd,bhkd->bhqk", qf, kf) * scale
    keep = _dense_mask(mask, _positions(q_chunk_pos, Sq, q.device), _positions(kv_chunk_pos, k.shape[1], q.device))
    return s.masked_fill(~keep, float("-inf"))


def attn_forward(q, k, v, o, lse, scale: float, mask: MaskSpec, q_chunk_pos: Sequence[int],
                 kv_chunk_pos: Sequence[int], merge_prev: bool = False,
                 pull: Optional[Tuple[int, int, int]] = None) -> None:
    """Writes (or, with merge_prev, folds into) o [B,Sq,Hq,D] bf16 and lse [B,Hq,Sq] fp32.
    `pull` = (src_ptr, dst_ptr, nbytes): a peer copy fused into the kernel (GPU only)."""
    if _ext.use_cuda_kernels(q):
        ps, pd, pb = pull if pull is not None else (0, 0, 0)
        _ext.C().attn_fwd(q, k, v, o, lse, scale, mask.causal, mask.window_blocks, mask.global_every,
                          list(q_chunk_pos), list(kv_chunk_pos), merge_prev, ps, pd, pb)
        return
    s = _ref_scores(q, k, scale, mask, q_chunk_pos, kv_chunk_pos)
    Hq, Hkv = q.shape[2], k.shape[2]
    lse_cur = torch.logsumexp(s, dim=-1)
    p = torch.nan_to_num(torch.exp(s - lse_cur[..., None]), nan=0.0)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, dim=1)
    o_cur = torch.einsum("bhqk,bhkd->bhqd", p, vf).permute(0, 2, 1, 3)
    if merge_prev:
        lse_prev = lse.clone()
        lse_new = torch.logaddexp(lse_prev, lse_cur)
        w_prev = torch.nan_to_num(torch.exp(lse_prev - lse_new), nan=0.0).permute(0, 2, 1)[..., None]
        w_cur = torch.nan_to_num(torch.exp(lse_cur - lse_new), nan=0.0).permute(0, 2, 1)[..., None]
        o.copy_((o.float() * w_prev + o_cur * w_cur).to(o.dtype))
        lse.copy_(lse_new)
    else:
        o.copy_(o_cur.to(o.dtype))
        lse.copy_(lse_cur)


def attn_backward(q, k, v, o, d_o, lse, delta, dq, dk, dv, scale: float, mask: MaskSpec,
                  q_chunk_pos: Sequence[int], kv_chunk_pos: Sequence[int], compute_delta: bool = True,
                  dq_accumulate: bool = False, pull: Optional[Tuple[int, int, int]] = None) -> None:
    """dq (fp32) is written or accumulated; dk/dv (fp32) are always added to (zero them first).
    `lse` must be the final log-sum-exp over *all* keys the queries saw (all ring steps)."""
    if _ext.use_cuda_kernels(q):
        ps, pd, pb = pull if pull is not None else (0, 0, 0)
        _ext.C().attn_bwd(q, k, v, o, d_o, lse, delta, dq, dk, dv, scale, mask.causal, mask.window_blocks,
                          mask.global_every, list(q_chunk_pos), list(kv_chunk_pos), compute_delta, dq_accumulate,
                          ps, pd, pb)
        return
    Hq, Hkv = q.shape[2], k.shape[2]
    G = Hq // Hkv
    if compute_delta:
        delta.copy_((o.float() * d_o.float()).sum(-1).permute(0, 2, 1))
    s = _ref_scores(q, k, scale, mask, q_chunk_pos, kv_chunk_pos)
    p = torch.nan_to_num(torch.exp(s - lse[..., None]), nan=0.0)                    # [B,Hq,Sq,Skv]
    dof = d_o.float().permute(0, 2, 1, 3)                                          # [B,Hq,Sq,D]
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    qf = q.float().permute(0, 2, 1, 3)
    dp = torch.einsum("bhqd,bhkd->bhqk", dof, vf)
    ds = p * (dp - delta[..., None])
    dq_cur = (torch.einsum("bhqk,bhkd->bhqd", ds, kf) * scale).permute(0, 2, 1, 3)
    dk_cur = torch.einsum("bhqk,bhqd->bhkd", ds, qf) * scale
    dv_cur = torch.einsum("bhqk,bhqd->bhkd", p, dof)
    B, _, Skv, D = dk_cur.shape
    dk_cur = dk_cur.view(B, Hkv, G, Skv, D).sum(2).permute(0, 2, 1, 3)
    dv_cur = dv_cur.view(B, Hkv, G, Skv, D).sum(2).permute(0, 2, 1, 3)
    if dq_accumulate:
        dq.add_(dq_cur)
    else:
        dq.copy_(dq_cur)
    dk.add_(dk_cur)
    dv.add_(dv_cur)


# ------------------------------------------------------------------------------------------------
# Single-device autograd op
# ------------------------------------------------------------------------------------------------


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, mask, q_chunk_pos, kv_chunk_pos):
        o = torch.empty(q.shape, device=q.device, dtype=q.dtype)
        lse = torch.empty(q.shape[0], q.shape[2], q.shape[1], device=q.device, dtype=torch.float32)
        attn_forward(q, k, v, o, lse, scale, mask, q_chunk_pos, kv_chunk_pos)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.cfg = (scale, mask, tuple(q_chunk_pos), tuple(kv_chunk_pos))
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        scale, mask, qp, kp = ctx.cfg
        dq = torch.empty(q.shape, device=q.device, dtype=torch.float32)
        dk = torch.zeros(k.shape, device=q.device, dtype=torch.float32)
        dv = torch.zeros(v.shape, device=q.device, dtype=torch.float32)
        delta = torch.empty_like(lse)
        attn_backward(q, k, v, o, d_o.contiguous(), lse, delta, dq, dk, dv, scale, mask, qp, kp)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None, None, None


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = True,
                    scale: Optional[float] = None, sparse: Optional[MaskSpec] = None,
                    q_chunk_pos: Sequence[int] = (0,), kv_chunk_pos: Sequence[int] = (0,)) -> torch.Tensor:
    """q [B,S,Hq,128], k/v [B,S,Hkv,128] -> o [B,S,Hq,128]. Sequence lengths must be multiples of 128."""
    mask = sparse if sparse is not None else MaskSpec(causal=causal)
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _FlashAttnFn.apply(q, k, v, scale, mask, tuple(q_chunk_pos), tuple(kv_chunk_pos))


# ------------------------------------------------------------------------------------------------
# Ring attention
# ------------------------------------------------------------------------------------------------


@dataclass
class RingContext:
    """Everything one rank needs to run ring attention at a given degree.

    ``peer`` (GPU only) is a ``zenyx_b200.parallel.peer.RingBuffers`` holding this rank's
    peer-visible K/V slots, the staging buffers the kernels pull into, the fp32 dK/dV accumulators
    peers add into, and the flag barrier. ``group`` is only used on CPU (gloo) and for setup.
    """

    rank: int = 0
    degree: int = 1
    seq_len: int = 0
    layout: str = "zigzag"
    group: object = None
    peer: object = None
    mask: MaskSpec = field(default_factory=MaskSpec)

    def positions(self, owner: Optional[int] = None) -> List[int]:
        return shard_positions(self.rank if owner is None else owner, self.degree, self.seq_len, self.layout)

    def owner_at(self, step: int) -> int:
        return (self.rank - step) % self.degree

    def active_steps(self, q_len: int, kv_len: int) -> List[int]:
        """Ring steps that contain at least one unmasked tile (fully masked steps are never run)."""
        qp = self.positions()
        return [s for s in range(self.degree)
                if step_has_work(self.mask, qp, q_len, self.positions(self.owner_at(s)), kv_len)]


def _gather_kv_cpu(ctx: RingContext, k, v):
    import torch.distributed as dist

    ks = [torch.empty_like(k) for _ in range(ctx.degree)]
    vs = [torch.empty_like(v) for _ in range(ctx.degree)]
    dist.all_gather(ks, k.contiguous(), group=ctx.group)
    dist.all_gather(vs, v.contiguous(), group=ctx.group)
    return ks, vs


def ring_attn_forward(ctx: RingContext, q, k, v, scale: float, slot: int = 0):
    """Forward over all ring steps. On GPU, `k`/`v` must be this rank's views of peer slot `slot`
    (already written, e.g. by the RoPE kernel). Returns (o, lse)."""
    B, Sq, Hq, D = q.shape
    o = torch.empty(B, Sq, Hq, D, device=q.device, dtype=q.dtype)
    lse = torch.empty(B, Hq, Sq, device=q.device, dtype=torch.float32)
    if ctx.degree == 1:
        attn_forward(q, k, v, o, lse, scale, ctx.mask, ctx.positions(), ctx.positions())
        return o, lse
    steps = ctx.active_steps(Sq, k.shape[1])
    if not q.is_cuda:
        ks, vs = _gather_kv_cpu(ctx, k, v)
        for i, s in enumerate(steps):
            owner = ctx.owner_at(s)
            attn_forward(q, ks[owner], vs[owner], o, lse, scale, ctx.mask, ctx.positions(), ctx.positions(owner), i > 0)
        if not steps:
            o.zero_()
            lse.fill_(float("-inf"))
        return o, lse
    peer = ctx.peer
    fp8 = getattr(peer, "fp8_block_tokens", 0) > 0
    if fp8:   # e4m3 cache: this rank's K/V go into its slot as codes + scales; peers pull those (half the bytes)
        peer.quantize_into_slot(k, v, slot)
    peer.barrier()  # every rank's K/V slot is written and visible
    for i, s in enumerate(steps):
        owner = ctx.owner_at(s)
        if fp8:   # every step works on what the cache format can represent, the local one included
            kk, vv = peer.dequant_local(slot) if owner == ctx.rank else (None, None)
        else:
            kk, vv = (k, v) if owner == ctx.rank else peer.staged_kv(i % 2, k.shape)
        pull = None
        if i + 1 < len(steps):
            nxt = ctx.owner_at(steps[i + 1])
            pull = peer.pull_args(nxt, slot, (i + 1) % 2) if nxt != ctx.rank else None
        if i == 0 and owner != ctx.rank:
            peer.pull_now(owner, slot, 0)  # first active step is remote: nothing to overlap with yet
        if fp8 and owner != ctx.rank:
            kk, vv = peer.dequant_staged(i % 2)
        attn_forward(q, kk, vv, o, lse, scale, ctx.mask, ctx.positions(), ctx.positions(owner), i > 0, pull)
    if not steps:
        o.zero_()
        lse.fill_(float("-inf"))
    return o, lse


def ring_attn_backward(ctx: RingContext, q, k, v, o, d_o, lse, scale: float, slot: int = 0):
    """Backward over all ring steps. Returns (dq fp32, dk fp32, dv fp32) for this rank's tokens;
    on GPU dk/dv are views of this rank's peer-visible accumulators (valid until the slot is reused)."""
    B, Sq, Hq, D = q.shape
    dq = torch.empty(B, Sq, Hq, D, device=q.device, dtype=torch.float32)
    delta = torch.empty_like(lse)
    if ctx.degree == 1:
        dk = torch.zeros(k.shape, device=q.device, dtype=torch.float32)
        dv = torch.zeros(v.shape, device=q.device, dtype=torch.float32)
        attn_backward(q, k, v, o, d_o, lse, delta, dq, dk, dv, scale, ctx.mask, ctx.positions(), ctx.positions())
        return dq, dk, dv
    steps = ctx.active_steps(Sq, k.shape[1])
    if not q.is_cuda:
        import torch.distributed as dist

        ks, vs = _gather_kv_cpu(ctx, k, v)
        dks = [torch.zeros(k.shape, dtype=torch.float32) for _ in range(ctx.degree)]
        dvs = [torch.zeros(v.shape, dtype=torch.float32) for _ in range(ctx.degree)]
        for i, s in enumerate(steps):
            owner = ctx.owner_at(s)
            attn_backward(q, ks[owner], vs[owner], o, d_o, lse, delta, dq, dks[owner], dvs[owner], scale, ctx.mask,
                          ctx.positions(), ctx.positions(owner), i == 0, i > 0)
        if not steps:
            dq.zero_()
        dk_all, dv_all = torch.stack(dks), torch.stack(dvs)
        dist.all_reduce(dk_all, group=ctx.group)
        dist.all_reduce(dv_all, group=ctx.group)
        return dq, dk_all[ctx.rank], dv_all[ctx.rank]
    peer = ctx.peer
    fp8 = getattr(peer, "fp8_block_tokens", 0) > 0
    if fp8:   # the slot may have been reused since the forward: put this call's K/V back (same codes)
        peer.quantize_into_slot(k, v, slot)
    peer.zero_dkv(slot)
    peer.barrier()  # accumulators cleared everywhere, K/V slots still valid
    for i, s in enumerate(steps):
        owner = ctx.owner_at(s)
        if fp8:   # gradients are taken at the values the cache format holds (straight-through for K and V)
            kk, vv = peer.dequant_local(slot) if owner == ctx.rank else (None, None)
        else:
            kk, vv = (k, v) if owner == ctx.rank else peer.staged_kv(i % 2, k.shape)
        pull = None
        if i + 1 < len(steps):
            nxt = ctx.owner_at(steps[i + 1])
            pull = peer.pull_args(nxt, slot, (i + 1) % 2) if nxt != ctx.rank else None
        if i == 0 and owner != ctx.rank:
            peer.pull_now(owner, slot, 0)
        if fp8 and owner != ctx.rank:
            kk, vv = peer.dequant_staged(i % 2)
        dk_t, dv_t = peer.dkv_views(owner, slot, k.shape)
        attn_backward(q, kk, vv, o, d_o, lse, delta, dq, dk_t, dv_t, scale, ctx.mask, ctx.positions(),
                      ctx.positions(owner), i == 0, i > 0, pull)
    if not steps:
        dq.zero_()
    peer.barrier()  # every peer's contributions to my dK/dV have landed
    dk, dv = peer.dkv_views(ctx.rank, slot, k.shape)
    return dq, dk, dv


class _RingAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, ring):
        slots = ring.degree > 1 and q.is_cuda and getattr(ring.peer, "fp8_block_tokens", 0) == 0
        if slots:   # bf16 ring: K/V live in this rank's peer-visible slot (the e4m3 ring quantises into it itself)
            ks, vs = ring.peer.kv_views(ring.rank, 0, k.shape)
            ks.copy_(k)
            vs.copy_(v)
            k, v = ks, vs
        o, lse = ring_attn_forward(ring, q, k, v, scale, 0)
        ctx.save_for_backward(q, k.clone() if slots else k, v.clone() if slots else v, o, lse)
        ctx.cfg = (scale, ring)
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        scale, ring = ctx.cfg
        if ring.degree > 1 and q.is_cuda and getattr(ring.peer, "fp8_block_tokens", 0) == 0:
            ks, vs = ring.peer.kv_views(ring.rank, 0, k.shape)
            ks.copy_(k)
            vs.copy_(v)
            k, v = ks, vs
        dq, dk, dv = ring_attn_backward(ring, q, k, v, o, d_o.contiguous(), lse, scale, 0)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None


def ring_flash_attention(q, k, v, *, causal: bool = True, scale: Optional[float] = None, ring: Optional[RingContext] = None,
                         group=None, layout: str = "zigzag", kv_fp8=None, sparse: Optional[MaskSpec] = None,
                         seq_len: Optional[int] = None) -> torch.Tensor:
    """Context-parallel attention over this rank's sequence shard.

    q [B,S_local,Hq,128], k/v [B,S_local,Hkv,128] hold the tokens given by
    ``shard_positions(rank, degree, seq_len, layout)``. Pass a prepared ``RingContext`` (GPU ranks
    need its peer buffers), or a process ``group`` for the CPU/gloo fallback. ``kv_fp8`` is an
    optional ``FP8KVQuantizer``: the op then computes attention over the e4m3 cache (per-(head, block)
    scales). On GPU ranks whose ``RingContext.peer`` was built with ``fp8_block_tokens`` the codes and
    scales are what sits in the peer slots and crosses NVLink; otherwise K/V take a round trip through
    the format before the bf16 ring.
    """
    import torch.distributed as dist

    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if ring is None:
        degree = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        rank = dist.get_rank(group) if degree > 1 else 0
        ring = RingContext(rank=rank, degree=degree, seq_len=seq_len or q.shape[1] * degree, layout=layout, group=group,
                           mask=sparse if sparse is not None else MaskSpec(causal=causal))
    fp8_ring = ring.degree > 1 and q.is_cuda and getattr(ring.peer, "fp8_block_tokens", 0) > 0
    if kv_fp8 is not None and not fp8_ring:
        k, v = kv_fp8.roundtrip(k), kv_fp8.roundtrip(v)
    return _RingAttnFn.apply(q, k, v, scale, ring)
