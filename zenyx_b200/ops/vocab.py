"""Vocabulary-parallel ops: cross-entropy over logits whose vocabulary dimension is split over a
group, without ever gathering the logits.

Each rank holds ``logits_local`` [T, V / W] for vocabulary slice ``[rank * V/W, (rank+1) * V/W)``.
The loss needs three scalars per token across the group (max, sum of exponentials, the target's
logit): two all-reduces of [T] floats instead of an all-gather of [T, V]. The backward is local:
``softmax - onehot`` on this rank's slice. The embedding counterpart is
``parallel/tensor_parallel.py::TensorParallelEmbedding``. The reference names a ``zenyx/ops/vocab``
directory without contents (ZENYX_2_0_DELIVERABLES.txt:193-194); its model head is a plain
``nn.Linear`` + ``F.cross_entropy`` (README.md:60-110). The single-GPU chunked head of the flagship
(``models/llama.py::_head_loss`` on ``csrc/fused/fused_ops.cu::ce_fwd_bwd_kernel``) is the fused form.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _wr(group):
    if not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits_local, targets, group):
        world, rank = _wr(group)
        T, Vl = logits_local.shape
        lf = logits_local.float()
        m = lf.max(dim=-1).values
        if world > 1:
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        e = torch.exp(lf - m[:, None])
        z = e.sum(dim=-1)
        lo = rank * Vl
        mine = (targets >= lo) & (targets < lo + Vl)
        idx = (targets - lo).clamp(0, Vl - 1)
        tgt_logit = torch.where(mine, lf.gather(1, idx[:, None]).squeeze(1), torch.zeros_like(m))
        if world > 1:
            pack = torch.stack([z, tgt_logit])
            dist.all_reduce(pack, group=group)
            z, tgt_logit = pack[0], pack[1]
        loss = torch.log(z) + m - tgt_logit
        ctx.save_for_backward(e / z[:, None], idx, mine)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        p, idx, mine = ctx.saved_tensors
        g = p.clone()
        rows = torch.nonzero(mine, as_tuple=False).squeeze(1)
        g[rows, idx[rows]] -= 1.0
        return (g * dloss[:, None]).to(p.dtype), None, None


def vocab_parallel_cross_entropy(logits_local: torch.Tensor, targets: torch.Tensor, group=None) -> torch.Tensor:
    """Per-token losses [T] (fp32) for vocabulary-sharded logits [T, V / W]; differentiable w.r.t. the logits."""
    return _VocabParallelCE.apply(logits_local, targets, group)
