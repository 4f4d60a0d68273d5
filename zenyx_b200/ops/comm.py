"""Ring communication helpers on ``torch.distributed`` (NCCL on GPUs, gloo on CPU).

These are the library-collective forms of what the attention kernels do through peer memory:
``ring_exchange`` passes a tensor to the next rank and receives the previous rank's, and
``ring_all_gather`` builds every rank's shard by W-1 such hops. They serve the CPU paths, the
unit tests and the NCCL baseline of the ring-attention benchmark; the GPU hot path pulls K/V with
in-kernel P2P loads instead (``csrc/attn/attn_fwd.cu``, ``parallel/peer.py``). The reference only
names a ``zenyx/ops/comm`` directory (ZENYX_2_0_DELIVERABLES.txt:193-194); its transport is
``zenyx/distributed/communication.py:136-171``.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def _wr(group):
    if not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def ring_exchange(send: torch.Tensor, group=None, recv: Optional[torch.Tensor] = None, shift: int = 1) -> torch.Tensor:
    """Sends ``send`` to rank ``r + shift`` and returns what rank ``r - shift`` sent (one batched P2P pair)."""
    world, rank = _wr(group)
    if world == 1:
        return send if recv is None else recv.copy_(send)
    recv = torch.empty_like(send) if recv is None else recv
    dst = dist.get_global_rank(group, (rank + shift) % world) if group is not None else (rank + shift) % world
    src = dist.get_global_rank(group, (rank - shift) % world) if group is not None else (rank - shift) % world
    ops = [dist.P2POp(dist.isend, send.contiguous(), dst, group=group), dist.P2POp(dist.irecv, recv, src, group=group)]
    for req in dist.batch_isend_irecv(ops):
        req.wait()
    return recv


def ring_all_gather(x: torch.Tensor, group=None) -> List[torch.Tensor]:
    """Every rank's ``x``, indexed by owner rank, collected by passing blocks around the ring."""
    world, rank = _wr(group)
    out: List[Optional[torch.Tensor]] = [None] * world
    out[rank] = x
    cur = x
    for step in range(1, world):
        cur = ring_exchange(cur, group)
        out[(rank - step) % world] = cur
    return out  # type: ignore[return-value]


def ring_reduce_scatter(parts: List[torch.Tensor], group=None) -> torch.Tensor:
    """``parts[o]`` is this rank's contribution to owner ``o``; returns the sum of everyone's
    contribution to this rank, accumulated hop by hop (fp32 accumulation for half types)."""
    world, rank = _wr(group)
    if world == 1:
        return parts[0]
    acc_dtype = torch.float32 if parts[0].dtype in (torch.bfloat16, torch.float16) else parts[0].dtype
    # the block that ends at owner o starts at rank o + 1 and makes W - 1 forward hops; at hop s this rank
    # forwards the block of owner (rank - 1 - s) and adds its own share to the one it receives
    cur = parts[(rank - 1) % world].to(acc_dtype)
    for s in range(world - 1):
        got = ring_exchange(cur, group)
        cur = got + parts[(rank - 2 - s) % world].to(acc_dtype)
    return cur.to(parts[0].dtype)
