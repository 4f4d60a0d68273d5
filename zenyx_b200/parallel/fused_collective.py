"""GEMMs fused with their collective over NVLink peer memory (sequence-parallel tensor parallelism).

Two operations, each ONE stream of tcgen05 GEMM launches whose communication rides inside the
kernels (``csrc/gemm/gemm_bf16.cu``), not a library collective next to them:

``allgather_gemm``       Y[R*m, N] = concat_r(X_r)[R*m, K] @ W[N, K]^T where rank r holds X_r.
                         R launches, one per shard, own shard first. While launch s multiplies shard
                         s out of LOCAL memory, the extra warp of every CTA copies a slice of shard
                         s+1 from its owner (plain 16-byte peer loads) into a local staging buffer, so
                         each remote byte crosses NVLink exactly once and underneath the math.
``gemm_reduce_scatter``  Y_r[m, N] = sum_q X_q[R*m, K_q] @ W_q[N, K_q]^T restricted to rank r's rows.
                         One GEMM launch whose epilogue stores every bf16 row block straight into the
                         receive slot its OWNER keeps for this rank (plain peer stores, tile by tile as
                         the accumulators drain), a flag barrier, and one small kernel that sums the
                         owner's slots in fp32. The wire carries (R-1)/R of one bf16 result per rank.

The reference does these with ``dist.all_gather`` / ``dist.all_reduce`` around ``F.linear``
(zenyx/distributed/tensor_parallel.py:48-50, 96-114). On CPU tensors (gloo ranks in the unit tests)
the same functions run exactly that, so the host-side logic is testable without a GPU.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _ext
from ..ops.gemm import gemm


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


class FusedCollectiveContext:
    """Peer-visible buffers for one (rows_per_rank, K, N) problem family.

    * ``shard``: this rank's [rows, K] bf16 operand, readable by every peer;
    * ``stage``: two local [rows, K] bf16 buffers the pull warps fill;
    * ``slots``: this rank's [world, rows, N] bf16 receive slots, one per source rank, writable by peers.
    """

    def __init__(self, rows_per_rank: int, k: int, n: int, group=None, timeout_ms: float = 20000.0):
        from .peer import PeerBarrier, SymmetricBuffer

        self.group = group
        self.world, self.rank = _world(group), _rank(group)
        self.rows, self.k, self.n = rows_per_rank, k, n
        self.shard = SymmetricBuffer(rows_per_rank * k * 2, group)
        self.slots = SymmetricBuffer(self.world * rows_per_rank * n * 2, group)
        self.stage = [torch.empty(rows_per_rank, k, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
        self.barrier = PeerBarrier(group, timeout_ms)

    def shard_view(self, rank: Optional[int], rows: int, k: int) -> torch.Tensor:
        return self.shard.tensor(rank, 0, (rows, k), torch.bfloat16)

    def slots_view(self, rows: int, n: int) -> torch.Tensor:
        return self.slots.tensor(None, 0, (self.world, rows, n), torch.bfloat16)

    def close(self) -> None:
        self.barrier.close()
        self.shard.close()
        self.slots.close()


# One pull warp per CTA keeps 16 loads of 16 bytes in flight per lane and a peer load takes about 2 us, so
# the 148 warps of a launch copy about 600 GB/s; the NVLink port itself gives 770 GB/s.
_PULL_BYTES_PER_S = 6.0e11
_GEMM_FLOPS_PER_S = 1.3e15


def _pull_hides_under_gemm(m: int, k: int, n: int) -> bool:
    """Whether copying one [m, k] bf16 shard fits underneath one [m, k] x [n, k]^T launch."""
    return 2.0 * m * k * n / _GEMM_FLOPS_PER_S >= 2.0 * m * k / _PULL_BYTES_PER_S


def allgather_gemm(x_local: torch.Tensor, w: torch.Tensor, ctx: Optional[FusedCollectiveContext] = None,
                   group=None, trans_b: bool = False, gathered: Optional[torch.Tensor] = None,
                   fused: Optional[bool] = None) -> torch.Tensor:
    """``concat over ranks of x_local`` times ``w^T`` (``w`` itself when ``trans_b``: w stored [K, N]).

    Returns [world * m, N] on every rank. ``gathered`` ([world * m, K]), when given, receives the
    gathered operand: the pull warps then copy each remote shard straight into its rows and the
    GEMMs read it from there, so the caller keeps it (for a weight gradient) at no extra traffic.
    ``fused``: None picks the fused path when one shard's copy fits under one launch's math (it does for
    n >= ~1100 output features per rank) and the NCCL all-gather + one GEMM otherwise.
    """
    world, rank = _world(group), _rank(group)
    m, k = x_local.shape
    if world == 1:
        if gathered is not None:
            gathered.copy_(x_local)
        return gemm(x_local, w, trans_b=trans_b)
    n_feat = w.shape[1] if trans_b else w.shape[0]
    if fused is None:
        fused = _pull_hides_under_gemm(m, k, n_feat)
    if not (_ext.use_cuda_kernels(x_local) and ctx is not None and fused):
        parts = [torch.empty_like(x_local) for _ in range(world)]
        dist.all_gather(parts, x_local.contiguous(), group=group)
        full = torch.cat(parts, dim=0)
        if gathered is not None:
            gathered.copy_(full)
        return gemm(full, w, trans_b=trans_b)
    assert m <= ctx.rows and k <= ctx.k and x_local.dtype == torch.bfloat16
    C = _ext.C()
    mine = ctx.shard_view(None, m, k)
    mine.copy_(x_local)
    ctx.barrier()                                   # every rank's shard is in place
    n_out = w.shape[1] if trans_b else w.shape[0]
    out = torch.empty(world * m, n_out, device=x_local.device, dtype=x_local.dtype)
    nbytes = m * k * 2
    if gathered is not None:
        gathered[rank * m: (rank + 1) * m].copy_(x_local)

    def landing(owner: int, s: int) -> torch.Tensor:  # local home of a remote shard
        if gathered is not None:
            return gathered[owner * m: (owner + 1) * m]
        return ctx.stage[s % 2].view(-1)[: m * k].view(m, k)

    a = mine
    for s in range(world):
        owner = (rank + s) % world
        pull_src = pull_dst = pull_bytes = 0
        nxt_a = None
        if s + 1 < world:                           # fetch the next shard underneath this launch
            nxt = (rank + s + 1) % world
            nxt_a = landing(nxt, s)
            pull_src, pull_dst, pull_bytes = ctx.shard.ptr(nxt), nxt_a.data_ptr(), nbytes
        C.gemm(a, w, out[owner * m: (owner + 1) * m], False, trans_b, None, pull_src, pull_dst, pull_bytes)
        a = nxt_a
    ctx.barrier()                                   # peers are done reading my shard
    return out


def gemm_reduce_scatter(x: torch.Tensor, w: torch.Tensor, ctx: Optional[FusedCollectiveContext] = None,
                        group=None, trans_b: bool = False, fused: Optional[bool] = None) -> torch.Tensor:
    """Rows ``[rank * m, (rank + 1) * m)`` of ``sum over ranks of x @ w^T`` (x: [world * m, K_local];
    ``w`` is [N, K_local], or [K_local, N] with ``trans_b``).

    ``fused``: None uses the scatter epilogue on 2 ranks (measured 1.05x over GEMM + NCCL) and GEMM + NCCL
    reduce-scatter beyond: the epilogue writes each thread's row in 16-byte pieces, which the local L2
    merges but NVLink carries one by one, and with 7/8 of the rows remote it measured 0.17x on 8 GPUs.
    A shared-memory-staged epilogue writing whole 128-byte row segments is what the fused path needs there.
    """
    world, rank = _world(group), _rank(group)
    M = x.shape[0]
    if world == 1:
        return gemm(x, w, trans_b=trans_b)
    assert M % world == 0, "rows must split evenly over the group"
    m, n = M // world, (w.shape[1] if trans_b else w.shape[0])
    if fused is None:
        fused = world == 2
    if not _ext.use_cuda_kernels(x):
        y = gemm(x, w, trans_b=trans_b, out_dtype=torch.float32)
        dist.all_reduce(y, group=group)             # gloo has no reduce_scatter
        return y[rank * m: (rank + 1) * m].to(x.dtype)
    if ctx is None or not fused:
        y = gemm(x, w, trans_b=trans_b)
        out = torch.empty(m, n, device=x.device, dtype=x.dtype)
        dist.reduce_scatter_tensor(out, y, group=group)
        return out
    assert m <= ctx.rows and n <= ctx.n and x.dtype == torch.bfloat16
    C = _ext.C()
    slots = ctx.slots_view(m, n)                    # [world, m, n]; slot q receives rank q's partial of my rows
    ptrs: List[int] = [ctx.slots.ptr(r) for r in range(world)]
    ctx.barrier()                                   # every rank has consumed its slots of the previous call
    C.gemm(x, w, slots[rank], False, trans_b, None, 0, 0, 0, ptrs, m, rank)
    ctx.barrier()                                   # every peer's partial rows have landed in my slots
    out = torch.empty(m, n, device=x.device, dtype=x.dtype)
    C.sum_slots_bf16(slots, world, out)
    return out


# ------------------------------------------------------------------------------------------------
# Autograd forms and the sequence-parallel linear layers built on them
# ------------------------------------------------------------------------------------------------
class _AllGatherLinearFn(torch.autograd.Function):
    """y_full = allgather(x_local) @ W_local^T; backward reduce-scatters dX through the GEMM epilogue."""

    @staticmethod
    def forward(ctx, x_local, w, fc, group):
        world = _world(group)
        gathered = torch.empty(world * x_local.shape[0], x_local.shape[1], device=x_local.device, dtype=x_local.dtype)
        y = allgather_gemm(x_local, w, fc, group, gathered=gathered)
        ctx.save_for_backward(gathered, w)
        ctx.cfg = (fc, group)
        return y

    @staticmethod
    def backward(ctx, dy):
        gathered, w = ctx.saved_tensors
        fc, group = ctx.cfg
        dy = dy.contiguous()
        dx_local = gemm_reduce_scatter(dy, w, fc, group, trans_b=True)      # dY [R m, N_l] x W [N_l, K]
        dw = gemm(dy, gathered, trans_a=True, trans_b=True)                 # dY^T X_full
        return dx_local, dw.to(w.dtype), None, None


class _LinearReduceScatterFn(torch.autograd.Function):
    """y_local = reduce_scatter(x @ W_local^T); backward all-gathers dY inside the dgrad GEMM."""

    @staticmethod
    def forward(ctx, x, w, fc, group):
        ctx.save_for_backward(x, w)
        ctx.cfg = (fc, group)
        return gemm_reduce_scatter(x, w, fc, group)

    @staticmethod
    def backward(ctx, dy_local):
        x, w = ctx.saved_tensors
        fc, group = ctx.cfg
        world = _world(group)
        dy_local = dy_local.contiguous()
        dy_full = torch.empty(world * dy_local.shape[0], dy_local.shape[1], device=dy_local.device, dtype=dy_local.dtype)
        dx = allgather_gemm(dy_local, w, fc, group, trans_b=True, gathered=dy_full)   # dY_full [R m, N] x W [N, K_l]
        dw = gemm(dy_full, x, trans_a=True, trans_b=True)
        return dx, dw.to(w.dtype), None, None


def allgather_linear(x_local, w, fc=None, group=None):
    return _AllGatherLinearFn.apply(x_local, w, fc, group)


def linear_reduce_scatter(x, w, fc=None, group=None):
    return _LinearReduceScatterFn.apply(x, w, fc, group)
