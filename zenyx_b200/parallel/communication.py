"""Process bootstrap and collective wrappers.

Same public surface as the reference's ``zenyx/distributed/communication.py`` (:214-227):
``init_process_group``, ``init_distributed_from_env``, ``destroy_process_group``, ``all_reduce``,
``broadcast``, ``barrier``, ``get_rank``, ``get_world_size``, ``AsyncCollectiveHandle``,
``CollectiveGroup``, ``DistributedContext``, ``CommunicationError``; plus ``reduce_scatter`` and
``all_gather`` which the reference never calls (:208). Behavioural differences, on purpose:

* a non-contiguous input to ``all_reduce`` / ``broadcast`` is reduced through a contiguous copy
  and copied back, so the caller's tensor is always updated (the reference silently drops the
  result, :61-64,87);
* a failed asynchronous collective raises ``CommunicationError`` instead of being retried as a
  blocking call on a communicator that has just failed (:96-100).
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


class CommunicationError(RuntimeError):
    pass


@dataclass
class DistributedContext:
    rank: int
    world_size: int
    local_rank: int
    device: torch.device


_OPS = {"sum": "SUM", "prod": "PRODUCT", "min": "MIN", "max": "MAX", "avg": "AVG"}


def _reduce_op(op: str):
    if op not in _OPS:
        raise ValueError(f"unknown reduce op {op!r}; expected one of {sorted(_OPS)}")
    return getattr(dist.ReduceOp, _OPS[op])


def is_initialized() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_world_size(group=None) -> int:
    return dist.get_world_size(group) if is_initialized() else 1


def get_rank(group=None) -> int:
    return dist.get_rank(group) if is_initialized() else 0


def init_process_group(backend: str = "nccl", timeout_seconds: int = 1800, **kwargs) -> None:
    if is_initialized():
        return
    dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_seconds), **kwargs)


def init_distributed_from_env(timeout_seconds: int = 1800) -> DistributedContext:
    """Reads WORLD_SIZE / RANK / LOCAL_RANK, binds the GPU, and starts NCCL (or gloo without CUDA)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local_rank % max(torch.cuda.device_count(), 1))
        device = torch.device("cuda", torch.cuda.current_device())
    else:
        device = torch.device("cpu")
    if world > 1 and not is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = {}
        if use_cuda:
            kwargs["device_id"] = device
        init_process_group("nccl" if use_cuda else "gloo", timeout_seconds, **kwargs)
    return DistributedContext(rank=rank, world_size=world, local_rank=local_rank, device=device)


def destroy_process_group() -> None:
    if is_initialized():
        dist.destroy_process_group()


class AsyncCollectiveHandle:
    """Completion handle of an asynchronous collective; ``wait()`` returns the result tensor."""

    def __init__(self, work, tensor: torch.Tensor, name: str = "collective", writeback: Optional[torch.Tensor] = None):
        self._work = work
        self._tensor = tensor
        self._writeback = writeback
        self.name = name
        self._done = work is None

    def wait(self) -> torch.Tensor:
        if not self._done:
            try:
                self._work.wait()
            except Exception as e:  # noqa: BLE001
                raise CommunicationError(f"{self.name} failed: {e}") from e
            self._done = True
        if self._writeback is not None:
            self._writeback.copy_(self._tensor)
            self._tensor, self._writeback = self._writeback, None
        return self._tensor

    def is_completed(self) -> bool:
        return self._done or bool(self._work.is_completed())


def _run(name, tensor, fn, async_op, group, safety_barrier):
    if not is_initialized() or get_world_size(group) == 1:
        return AsyncCollectiveHandle(None, tensor, name) if async_op else tensor
    work_tensor = tensor if tensor.is_contiguous() else tensor.contiguous()
    writeback = None if work_tensor is tensor else tensor
    try:
        if safety_barrier:
            dist.barrier(group=group)
        work = fn(work_tensor)
    except Exception as e:  # noqa: BLE001
        raise CommunicationError(f"{name} failed: {e}") from e
    if async_op:
        return AsyncCollectiveHandle(work, work_tensor, name, writeback)
    if writeback is not None:
        writeback.copy_(work_tensor)
    return tensor


def all_reduce(tensor: torch.Tensor, op: str = "sum", group=None, async_op: bool = False, safety_barrier: bool = False):
    rop = _reduce_op(op)
    return _run("all_reduce", tensor, lambda t: dist.all_reduce(t, op=rop, group=group, async_op=async_op), async_op,
                group, safety_barrier)


def broadcast(tensor: torch.Tensor, src: int = 0, group=None, async_op: bool = False, safety_barrier: bool = False):
    return _run("broadcast", tensor, lambda t: dist.broadcast(t, src=src, group=group, async_op=async_op), async_op,
                group, safety_barrier)


def reduce_scatter(output: torch.Tensor, input: torch.Tensor, op: str = "sum", group=None, async_op: bool = False):
    """output [n] = this rank's slice of the element-wise reduction of input [world * n]."""
    if not is_initialized() or get_world_size(group) == 1:
        output.copy_(input.view_as(output))
        return AsyncCollectiveHandle(None, output, "reduce_scatter") if async_op else output
    try:
        work = dist.reduce_scatter_tensor(output, input.contiguous(), op=_reduce_op(op), group=group, async_op=async_op)
    except Exception as e:  # noqa: BLE001
        raise CommunicationError(f"reduce_scatter failed: {e}") from e
    return AsyncCollectiveHandle(work, output, "reduce_scatter") if async_op else output


def all_gather(output: torch.Tensor, input: torch.Tensor, group=None, async_op: bool = False):
    """output [world * n] = concatenation of every rank's input [n]."""
    if not is_initialized() or get_world_size(group) == 1:
        output.copy_(input.view_as(output))
        return AsyncCollectiveHandle(None, output, "all_gather") if async_op else output
    try:
        work = dist.all_gather_into_tensor(output, input.contiguous(), group=group, async_op=async_op)
    except Exception as e:  # noqa: BLE001
        raise CommunicationError(f"all_gather failed: {e}") from e
    return AsyncCollectiveHandle(work, output, "all_gather") if async_op else output


def barrier(group=None) -> None:
    if is_initialized() and get_world_size(group) > 1:
        dist.barrier(group=group)


class CollectiveGroup:
    """Object façade binding one process group to the collective wrappers."""

    def __init__(self, group=None):
        self.group = group

    @property
    def world_size(self) -> int:
        return get_world_size(self.group)

    @property
    def rank(self) -> int:
        return get_rank(self.group)

    def all_reduce(self, tensor, op: str = "sum", async_op: bool = False, safety_barrier: bool = False):
        return all_reduce(tensor, op=op, group=self.group, async_op=async_op, safety_barrier=safety_barrier)

    def broadcast(self, tensor, src: int = 0, async_op: bool = False, safety_barrier: bool = False):
        return broadcast(tensor, src=src, group=self.group, async_op=async_op, safety_barrier=safety_barrier)

    def reduce_scatter(self, output, input, op: str = "sum", async_op: bool = False):
        return reduce_scatter(output, input, op=op, group=self.group, async_op=async_op)

    def all_gather(self, output, input, async_op: bool = False):
        return all_gather(output, input, group=self.group, async_op=async_op)

    def barrier(self) -> None:
        barrier(self.group)


__all__ = [
    "init_process_group", "init_distributed_from_env", "destroy_process_group", "all_reduce", "broadcast",
    "reduce_scatter", "all_gather", "barrier", "get_rank", "get_world_size", "is_initialized",
    "AsyncCollectiveHandle", "CollectiveGroup", "DistributedContext", "CommunicationError",
]
