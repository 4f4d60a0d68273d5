"""Tensor-parallel layers, autograd-correct.

Same names as the reference (zenyx/distributed/tensor_parallel.py:26-148): ``ColumnParallelLinear``,
``RowParallelLinear``, ``TensorParallelEmbedding``, ``make_tensor_parallel_model``. What differs:

* the collectives are autograd functions, so ``backward()`` works (the reference's column layer
  returns a tensor that does not require grad);
* ``RowParallelLinear`` adds its bias after the reduction on every rank (the reference adds it on
  rank 0 only, after the reduce, so ranks diverge);
* ``make_tensor_parallel_model`` alternates column / row layers so consecutive linears need one
  all-reduce per pair, and always copies (slices of) the original weights.

None of the benchmark configurations uses TP (degree 1 everywhere), so these run on NCCL/gloo
collectives plus the library-free GEMM op when the tensors are bf16 on a GPU.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from . import communication as comm


def _world(group) -> int:
    return comm.get_world_size(group)


def _rank(group) -> int:
    return comm.get_rank(group)


class _CopyToGroup(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        if _world(ctx.group) > 1:
            g = g.contiguous()
            dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromGroup(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        if _world(group) > 1:
            x = x.contiguous().clone()
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherLastDim(torch.autograd.Function):
    """All-gather along the last dim forward, take the local slice backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = _world(group)
        if w == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(w)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, g):
        w = _world(ctx.group)
        if w == 1:
            return g, None
        n = g.shape[-1] // w
        r = _rank(ctx.group)
        return g[..., r * n: (r + 1) * n].contiguous(), None


class _ScatterLastDim(torch.autograd.Function):
    """Take the local slice forward, all-gather backward (input split of a row-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = _world(group)
        if w == 1:
            return x
        n = x.shape[-1] // w
        r = _rank(group)
        return x[..., r * n: (r + 1) * n].contiguous()

    @staticmethod
    def backward(ctx, g):
        w = _world(ctx.group)
        if w == 1:
            return g, None
        parts = [torch.empty_like(g) for _ in range(w)]
        dist.all_gather(parts, g.contiguous(), group=ctx.group)
        return torch.cat(parts, dim=-1), None


class ColumnParallelLinear(nn.Module):
    """y = x W^T + b with the rows of W (output features) split over the group."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, gather_output: bool = True, group=None,
                 device=None, dtype=None):
        super().__init__()
        self.group, self.gather_output = group, gather_output
        w = _world(group)
        if out_features % w != 0:
            raise ValueError("out_features must be divisible by the tensor-parallel degree")
        self.in_features, self.out_features, self.local_out = in_features, out_features, out_features // w
        self.weight = nn.Parameter(torch.empty(self.local_out, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(self.local_out, device=device, dtype=dtype)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)

    def load_full(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        r = _rank(self.group)
        with torch.no_grad():
            self.weight.copy_(weight[r * self.local_out: (r + 1) * self.local_out])
            if bias is not None and self.bias is not None:
                self.bias.copy_(bias[r * self.local_out: (r + 1) * self.local_out])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = _CopyToGroup.apply(x, self.group)
        y = F.linear(x, self.weight, self.bias)
        return _GatherLastDim.apply(y, self.group) if self.gather_output else y


class RowParallelLinear(nn.Module):
    """y = x W^T + b with the columns of W (input features) split over the group."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, input_is_parallel: bool = False,
                 group=None, device=None, dtype=None):
        super().__init__()
        self.group, self.input_is_parallel = group, input_is_parallel
        w = _world(group)
        if in_features % w != 0:
            raise ValueError("in_features must be divisible by the tensor-parallel degree")
        self.in_features, self.out_features, self.local_in = in_features, out_features, in_features // w
        self.weight = nn.Parameter(torch.empty(out_features, self.local_in, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)

    def load_full(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        r = _rank(self.group)
        with torch.no_grad():
            self.weight.copy_(weight[:, r * self.local_in: (r + 1) * self.local_in])
            if bias is not None and self.bias is not None:
                self.bias.copy_(bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.input_is_parallel:
            x = _ScatterLastDim.apply(x, self.group)
        y = _ReduceFromGroup.apply(F.linear(x, self.weight), self.group)
        return y + self.bias if self.bias is not None else y


class SequenceParallelColumnLinear(nn.Module):
    """Column-parallel linear whose INPUT is split by rows (tokens) over the group: the all-gather of
    the tokens is fused into the GEMM (``parallel/fused_collective.py``); output [all tokens, local
    features]. No counterpart in the reference, whose column-parallel layer takes a replicated
    input (zenyx/distributed/tensor_parallel.py:29-58)."""

    def __init__(self, in_features: int, out_features: int, group=None, device=None, dtype=torch.bfloat16,
                 context=None):
        super().__init__()
        w = _world(group)
        if out_features % w != 0:
            raise ValueError("out_features must be divisible by the tensor-parallel degree")
        self.group, self.context, self.local_out = group, context, out_features // w
        self.weight = nn.Parameter(torch.empty(self.local_out, in_features, device=device, dtype=dtype))
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        from .fused_collective import allgather_linear

        return allgather_linear(x_local, self.weight, self.context, self.group)


class SequenceParallelRowLinear(nn.Module):
    """Row-parallel linear whose OUTPUT is split by rows (tokens): the partial products are
    reduce-scattered by the GEMM epilogue itself (peer ``red.add``), see
    ``parallel/fused_collective.py``. The reference's row-parallel layer all-reduces instead
    (zenyx/distributed/tensor_parallel.py:61-116)."""

    def __init__(self, in_features: int, out_features: int, group=None, device=None, dtype=torch.bfloat16,
                 context=None):
        super().__init__()
        w = _world(group)
        if in_features % w != 0:
            raise ValueError("in_features must be divisible by the tensor-parallel degree")
        self.group, self.context, self.local_in = group, context, in_features // w
        self.weight = nn.Parameter(torch.empty(out_features, self.local_in, device=device, dtype=dtype))
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .fused_collective import linear_reduce_scatter

        return linear_reduce_scatter(x, self.weight, self.context, self.group)


class TensorParallelEmbedding(nn.Module):
    """Vocabulary-sharded embedding: local lookup with out-of-range ids masked, then all-reduce."""

    def __init__(self, num_embeddings: int, embedding_dim: int, group=None, device=None, dtype=None):
        super().__init__()
        self.group = group
        w = _world(group)
        if num_embeddings % w != 0:
            raise ValueError("num_embeddings must be divisible by the tensor-parallel degree")
        self.num_embeddings, self.embedding_dim, self.local_vocab = num_embeddings, embedding_dim, num_embeddings // w
        self.vocab_start = _rank(group) * self.local_vocab
        self.weight = nn.Parameter(torch.empty(self.local_vocab, embedding_dim, device=device, dtype=dtype))
        nn.init.normal_(self.weight)

    def load_full(self, weight: torch.Tensor) -> None:
        with torch.no_grad():
            self.weight.copy_(weight[self.vocab_start: self.vocab_start + self.local_vocab])

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        local = ids - self.vocab_start
        mask = (local >= 0) & (local < self.local_vocab)
        out = F.embedding(local.clamp(0, self.local_vocab - 1), self.weight) * mask.unsqueeze(-1).to(self.weight.dtype)
        return _ReduceFromGroup.apply(out, self.group)


def make_tensor_parallel_model(model: nn.Module, group=None) -> nn.Module:
    """Replaces ``nn.Linear`` layers by parallel ones, in place, keeping the original weights.

    Inside every container, linears are paired in definition order: the first of a pair becomes
    column-parallel without gathering, the second row-parallel on the already split input (one
    all-reduce per pair, the Megatron MLP pattern), provided the shapes chain. A linear without a
    partner becomes column-parallel with a gathered output. ``nn.Embedding`` becomes vocabulary-sharded.
    """
    w = _world(group)

    def convert(parent: nn.Module) -> None:
        names = [n for n, _ in parent.named_children()]
        i = 0
        while i < len(names):
            child = getattr(parent, names[i])
            if isinstance(child, nn.Linear):
                nxt_idx = next((j for j in range(i + 1, len(names)) if isinstance(getattr(parent, names[j]), nn.Linear)), None)
                between_ok = nxt_idx is not None and all(
                    not list(getattr(parent, names[j]).parameters()) for j in range(i + 1, nxt_idx))
                nxt = getattr(parent, names[nxt_idx]) if nxt_idx is not None else None
                if (between_ok and nxt is not None and nxt.in_features == child.out_features
                        and child.out_features % w == 0):
                    col = ColumnParallelLinear(child.in_features, child.out_features, child.bias is not None, False, group,
                                               child.weight.device, child.weight.dtype)
                    col.load_full(child.weight.data, child.bias.data if child.bias is not None else None)
                    row = RowParallelLinear(nxt.in_features, nxt.out_features, nxt.bias is not None, True, group,
                                            nxt.weight.device, nxt.weight.dtype)
                    row.load_full(nxt.weight.data, nxt.bias.data if nxt.bias is not None else None)
                    setattr(parent, names[i], col)
                    setattr(parent, names[nxt_idx], row)
                    i = nxt_idx + 1
                    continue
                if child.out_features % w == 0:
                    col = ColumnParallelLinear(child.in_features, child.out_features, child.bias is not None, True, group,
                                               child.weight.device, child.weight.dtype)
                    col.load_full(child.weight.data, child.bias.data if child.bias is not None else None)
                    setattr(parent, names[i], col)
            elif isinstance(child, nn.Embedding) and child.num_embeddings % w == 0 and child.padding_idx is None:
                emb = TensorParallelEmbedding(child.num_embeddings, child.embedding_dim, group, child.weight.device,
                                              child.weight.dtype)
                emb.load_full(child.weight.data)
                setattr(parent, names[i], emb)
            else:
                convert(child)
            i += 1

    convert(model)
    return model
