"""Sharded AdamW over a model's flat buffers (ZeRO-style optimizer-state sharding).

Each rank owns 1/world of the flat parameter space: its slice of the fp32 master weights (stored
as the bf16 parameter plus an int16 remainder, so 4 bytes per parameter), and of Adam's m and v.
A step is: reduce-scatter of the fp32 gradients, scale/clip, AdamW on the shard, all-gather of
the new bf16 parameters. On GPUs all of that is ONE kernel (``csrc/optim/zero_adamw.cu``): the
reduce-scatter is done with P2P loads from every rank's gradient buffer, the all-gather with P2P
stores into every rank's parameter buffer. With gradient clipping the kernel runs twice (reduce +
norm, then update + push) around a scalar all-reduce. ``fused_peer=False`` selects the NCCL
baseline (reduce_scatter_tensor, local AdamW kernel, all_gather_into_tensor); gloo/CPU ranks use
all_reduce + all_gather with the same shard arithmetic.

This replaces the reference's post-backward bucketed all-reduce, divide-and-copy-back and
replicated ``torch.optim.AdamW`` (zenyx/runtime/scheduler.py:32-107,158-160, zenyx/train/trainer.py:29).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import _ext, fused


class ZeroAdamW:
    def __init__(self, flat, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1,
                 max_grad_norm: Optional[float] = None, group=None, fused_peer: bool = True,
                 barrier_timeout_ms: float = 60000.0, single_process: bool = False,
                 state_dtype: torch.dtype = torch.float32):
        """``state_dtype``: storage type of Adam's two moments, fp32 or bf16. bf16 halves their 8 bytes per
        parameter (32 GB for an 8B model on one GPU, which the planner spends on kept activations); the update
        arithmetic and the master weight stay fp32. The reference keeps parameters and both moments in bf16
        with no master copy at all (torch.optim.AdamW on a bf16 model, zenyx/train/trainer.py:29)."""
        assert state_dtype in (torch.float32, torch.bfloat16), "optimizer moments are kept in fp32 or bf16"
        self.state_dtype = state_dtype
        self.flat = flat
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.group = group
        multi = dist.is_initialized() and not single_process   # single_process: ignore the process group
        self.world = dist.get_world_size(group) if multi else 1
        self.rank = dist.get_rank(group) if multi else 0
        assert flat.total % (4 * self.world) == 0, "flat buffer must split into 4-aligned shards"
        self.n_shard = flat.total // self.world
        self.shard_begin = self.rank * self.n_shard
        dev = flat.params.device
        self.device = dev
        self.p_lo = torch.zeros(self.n_shard, device=dev, dtype=torch.int16)
        self.m = torch.zeros(self.n_shard, device=dev, dtype=state_dtype)
        self.v = torch.zeros(self.n_shard, device=dev, dtype=state_dtype)
        self.step_count = 0
        self.on_gpu = dev.type == "cuda"
        self.fused_peer = fused_peer and self.on_gpu and (self.world == 1 or flat.sym_grads is not None)
        # Clipping needs the global norm before the update. With several ranks the reduced shard is kept
        # between the two passes (re-reading every peer's gradients would double the NVLink traffic); on a
        # single GPU the second pass simply reads the gradient buffer again, which saves 4 bytes per
        # parameter (32 GB for the 8B model) for activations.
        self.rereduce = self.fused_peer and self.world == 1
        need_gshard = ((max_grad_norm is not None) and not self.rereduce) or not self.fused_peer
        self.g_shard = torch.zeros(self.n_shard, device=dev, dtype=torch.float32) if need_gshard else None
        self.sumsq = torch.zeros(1, device=dev, dtype=torch.float32)
        self.clip = torch.ones(1, device=dev, dtype=torch.float32)
        self.grad_norm = torch.zeros(1, device=dev, dtype=torch.float32)
        self.barrier = None
        if self.fused_peer and self.world > 1:
            from .peer import PeerBarrier

            self.barrier = PeerBarrier(group, barrier_timeout_ms)
            self.grad_ptrs, self.param_ptrs = list(flat.sym_grads.ptrs), list(flat.sym_params.ptrs)
        elif self.on_gpu:
            self.grad_ptrs, self.param_ptrs = [flat.grads.data_ptr()], [flat.params.data_ptr()]

    # ---------------------------------------------------------------------------------------
    def _local_slices(self):
        lo, hi = self.shard_begin, self.shard_begin + self.n_shard
        return lo, hi, min(max(self.flat.decay_end, lo), hi)

    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None) -> None:
        """Consumes the accumulated gradients (and clears them), updates parameters everywhere."""
        self.step_count += 1
        lr = self.lr if lr is None else lr
        b1, b2 = self.betas
        clipping = self.max_grad_norm is not None
        if self.fused_peer:
            C = _ext.C()
            rank_arg = self.rank if self.world > 1 else 0
            if self.barrier is not None:
                self.barrier()  # every rank's gradients are complete
            common = dict(grad_scale=grad_scale, lr=lr, beta1=b1, beta2=b2, eps=self.eps,
                          weight_decay=self.weight_decay, step=self.step_count)

            def launch(do_reduce, do_update, clip, zero_grads=None, want_norm=None):
                zero_grads = do_reduce if zero_grads is None else zero_grads
                want_norm = do_reduce if want_norm is None else want_norm
                C.zero_step(self.grad_ptrs, self.param_ptrs, rank_arg, self.shard_begin, self.n_shard,
                            self.flat.decay_end, self.g_shard, self.p_lo, self.m, self.v,
                            self.sumsq if want_norm else None, clip, do_reduce, do_update, zero_grads,
                            common["grad_scale"], common["lr"], common["beta1"], common["beta2"], common["eps"],
                            common["weight_decay"], common["step"])

            # With peers, the kernel does not clear the gradients it has read: clearing this rank's slice of every
            # peer's buffer means (world - 1) / world of the gradient bytes written across NVLink (28 GB of zeros per
            # rank for an 8B model on 8 GPUs). Each rank clears its own buffer after the closing barrier instead,
            # when every peer is done reading it: a local fill.
            local_clear = self.world > 1
            if clipping:
                self.sumsq.zero_()
                launch(True, False, None, zero_grads=not (self.rereduce or local_clear))
                if self.world > 1:
                    dist.all_reduce(self.sumsq, group=self.group)
                fused.clip_coef_(self.sumsq, 1.0, float(self.max_grad_norm), self.clip, self.grad_norm)
                if self.rereduce:
                    launch(True, True, self.clip, zero_grads=True, want_norm=False)
                else:
                    launch(False, True, self.clip)
            else:
                launch(True, True, None, zero_grads=not local_clear)
            if self.barrier is not None:
                self.barrier()  # every rank's parameter pushes have landed, and its reads of the gradients are done
            if local_clear:
                self.flat.grads.zero_()
            return
        # ---- NCCL / gloo path ----
        grads = self.flat.grads
        if self.world > 1:
            if self.on_gpu:
                dist.reduce_scatter_tensor(self.g_shard, grads, group=self.group)
            else:
                dist.all_reduce(grads, group=self.group)
                self.g_shard.copy_(grads[self.shard_begin: self.shard_begin + self.n_shard])
        else:
            self.g_shard.copy_(grads)
        coef = None
        if clipping:
            self.sumsq.zero_()
            fused.sumsq_(self.g_shard, self.sumsq)
            if self.world > 1:
                dist.all_reduce(self.sumsq, group=self.group)
            fused.clip_coef_(self.sumsq, grad_scale, float(self.max_grad_norm), self.clip, self.grad_norm)
            coef = self.clip
        lo, hi, mid = self._local_slices()
        p_shard = self.flat.params[lo:hi]
        # this path's update routine works on fp32 moments: widen bf16 ones for the call and round them back
        narrow = self.state_dtype != torch.float32
        m32, v32 = (self.m.float(), self.v.float()) if narrow else (self.m, self.v)
        for a, b, wd in ((0, mid - lo, self.weight_decay), (mid - lo, hi - lo, 0.0)):
            if b > a:
                fused.adamw_step_(p_shard[a:b], self.p_lo[a:b], m32[a:b], v32[a:b], self.g_shard[a:b], lr=lr,
                                  beta1=b1, beta2=b2, eps=self.eps, weight_decay=wd, step=self.step_count,
                                  grad_scale=grad_scale, grad_scale_tensor=coef)
        if narrow:
            self.m.copy_(m32)
            self.v.copy_(v32)
        if self.world > 1:
            dist.all_gather_into_tensor(self.flat.params, p_shard.clone(), group=self.group)
        grads.zero_()

    def zero_grad(self) -> None:
        self.flat.grads.zero_()

    # ---------------------------------------------------------------------------------------
    def state_dict(self) -> Dict[str, object]:
        return {"step": self.step_count, "rank": self.rank, "world": self.world, "shard_begin": self.shard_begin,
                "n_shard": self.n_shard, "p_lo": self.p_lo, "m": self.m, "v": self.v,
                "lr": self.lr, "betas": tuple(self.betas), "eps": self.eps, "weight_decay": self.weight_decay}

    def load_state_dict(self, sd: Dict[str, object]) -> None:
        assert int(sd["n_shard"]) == self.n_shard and int(sd["shard_begin"]) == self.shard_begin, \
            "optimizer shard layout differs; use load_full_state to re-partition"
        self.step_count = int(sd["step"])
        self.p_lo.copy_(sd["p_lo"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])

    def load_full_state(self, step: int, p_lo: torch.Tensor, m: torch.Tensor, v: torch.Tensor) -> None:
        """Loads from unsharded state vectors (used when the world size changed). A vector saved under an
        older layout may be shorter or longer than ``flat.total``: the difference is tail padding, which
        carries no parameter, so it is zero-filled or dropped."""
        lo, hi = self.shard_begin, self.shard_begin + self.n_shard
        self.step_count = int(step)
        for dst, src in ((self.p_lo, p_lo), (self.m, m), (self.v, v)):
            piece = src[lo: min(hi, src.numel())]
            dst[: piece.numel()].copy_(piece)
            if piece.numel() < dst.numel():
                dst[piece.numel():].zero_()

    def close(self) -> None:
        if self.barrier is not None:
            self.barrier.close()
            self.barrier = None
