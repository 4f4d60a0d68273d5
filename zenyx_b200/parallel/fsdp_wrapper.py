"""``FSDPWrapper``: the reference's ZeRO-3 façade (zenyx/distributed/fsdp_wrapper.py:24-175) with its
defects removed: ``backward_prefetch`` is the proper enum, ``cpu_offload`` is honoured, layers are
wrapped individually (size-based policy) so parameters are gathered and freed per layer instead of
for the whole model at once, and ``consolidate_state_dict`` really gathers a full state dict on
rank 0. On CPU-only processes (gloo ranks in tests) the wrapper degrades to replicated parameters
with an explicit gradient all-reduce in ``sync_gradients``. The Llama flagship uses the package's
own sharded optimizer (``zenyx_b200.parallel.zero``) instead of this wrapper.
"""
from __future__ import annotations

import functools
from typing import Dict, Optional

import torch
import torch.nn as nn

from . import communication as comm

_STRATEGIES = ("full_shard", "shard_grad_op", "no_shard")
_PRECISIONS = ("fp16", "bf16", "no")


class FSDPWrapper:
    def __init__(self, model: nn.Module, world_size: Optional[int] = None, rank: Optional[int] = None,
                 mixed_precision: str = "bf16", sharding_strategy: str = "full_shard", cpu_offload: bool = False,
                 min_wrap_params: int = 1_000_000, group=None):
        if sharding_strategy not in _STRATEGIES:
            raise ValueError(f"sharding_strategy must be one of {_STRATEGIES}")
        if mixed_precision not in _PRECISIONS:
            raise ValueError(f"mixed_precision must be one of {_PRECISIONS}")
        self.model = model
        self.world_size = world_size if world_size is not None else comm.get_world_size(group)
        self.rank = rank if rank is not None else comm.get_rank(group)
        self.mixed_precision, self.sharding_strategy, self.cpu_offload = mixed_precision, sharding_strategy, cpu_offload
        self.min_wrap_params, self.group = min_wrap_params, group
        self.wrapped: Optional[nn.Module] = None
        self.gradients_synced = False
        self._is_fsdp = False

    def _mp_policy(self):
        from torch.distributed.fsdp import MixedPrecision

        if self.mixed_precision == "no":
            return None
        dt = torch.float16 if self.mixed_precision == "fp16" else torch.bfloat16
        return MixedPrecision(param_dtype=dt, reduce_dtype=dt, buffer_dtype=dt)

    def wrap(self) -> nn.Module:
        if self.world_size == 1 or not comm.is_initialized():
            self.wrapped = self.model
            return self.model
        if not torch.cuda.is_available():
            # FSDP needs an accelerator; keep replicated parameters, reduce gradients explicitly
            for p in self.model.parameters():
                comm.broadcast(p.data, src=0, group=self.group)
            self.wrapped = self.model
            return self.model
        from torch.distributed.fsdp import BackwardPrefetch, CPUOffload, FullyShardedDataParallel as FSDP, ShardingStrategy
        from torch.distributed.fsdp.wrap import size_based_auto_wrap_policy

        strategy = {"full_shard": ShardingStrategy.FULL_SHARD, "shard_grad_op": ShardingStrategy.SHARD_GRAD_OP,
                    "no_shard": ShardingStrategy.NO_SHARD}[self.sharding_strategy]
        self.wrapped = FSDP(
            self.model, process_group=self.group, mixed_precision=self._mp_policy(), sharding_strategy=strategy,
            cpu_offload=CPUOffload(offload_params=True) if self.cpu_offload else None,
            auto_wrap_policy=functools.partial(size_based_auto_wrap_policy, min_num_params=self.min_wrap_params),
            backward_prefetch=BackwardPrefetch.BACKWARD_PRE, forward_prefetch=False,
            device_id=torch.cuda.current_device(), use_orig_params=True)
        self._is_fsdp = True
        return self.wrapped

    def sync_gradients(self) -> None:
        """FSDP reduces during backward; the replicated fallback averages gradients here."""
        if not self._is_fsdp and self.world_size > 1 and comm.is_initialized():
            for p in (self.wrapped or self.model).parameters():
                if p.grad is not None:
                    comm.all_reduce(p.grad, op="avg", group=self.group)
        self.gradients_synced = True

    def consolidate_state_dict(self) -> Dict[str, torch.Tensor]:
        """Full (unsharded) state dict; under FSDP it is materialised on rank 0 only, on the CPU."""
        m = self.wrapped or self.model
        if not self._is_fsdp:
            return m.state_dict()
        from torch.distributed.fsdp import FullStateDictConfig, FullyShardedDataParallel as FSDP, StateDictType

        with FSDP.state_dict_type(m, StateDictType.FULL_STATE_DICT, FullStateDictConfig(offload_to_cpu=True, rank0_only=True)):
            return m.state_dict()
