"""Peer-visible (symmetric) GPU memory for one node, and the ring-attention buffers built on it.

Every rank allocates the same set of buffers with ``cudaMalloc`` (outside the PyTorch caching
allocator so the allocation can be exported), publishes the CUDA IPC handles through the process
group, and maps all peers' buffers. Kernels then read, write and reduce into peer memory directly
over NVLink. Pointers to peer memory are only ever handed to this package's own kernels.
The reference has no peer-memory layer (its transport is ``torch.distributed`` only,
zenyx/distributed/communication.py:136-171).
"""
from __future__ import annotations

import itertools
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..ops import _ext

_DTYPE_SIZE = {torch.bfloat16: 2, torch.float16: 2, torch.float32: 4, torch.uint8: 1, torch.int32: 4, torch.int16: 2,
               torch.float8_e4m3fn: 1}


class SymmetricBuffer:
    """`nbytes` of device memory on every rank of `group`, each mapped into every other rank."""

    def __init__(self, nbytes: int, group=None):
        self.C = _ext.C()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.local_ptr = self.C.peer_alloc(self.nbytes)
        self.ptrs: List[int] = [0] * self.world
        self.ptrs[self.rank] = self.local_ptr
        self._opened: List[int] = []
        if self.world > 1:
            handle = bytes(self.C.peer_export(self.local_ptr))
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, handle, group=group)
            for r, h in enumerate(handles):
                if r != self.rank:
                    p = self.C.peer_open(h)
                    self.ptrs[r] = p
                    self._opened.append(p)
            dist.barrier(group=group)

    def ptr(self, rank: Optional[int] = None, offset_bytes: int = 0) -> int:
        return self.ptrs[self.rank if rank is None else rank] + offset_bytes

    def tensor(self, rank: Optional[int], offset_bytes: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """A tensor view of (a slice of) rank's buffer; for a peer rank it aliases remote memory and
        must only be passed to this package's kernels."""
        n = 1
        for s in shape:
            n *= s
        assert offset_bytes + n * _DTYPE_SIZE[dtype] <= self.nbytes, "view exceeds the symmetric buffer"
        return self.C.tensor_from_ptr(self.ptr(rank, offset_bytes), list(shape), dtype)

    def close(self) -> None:
        if self.local_ptr == 0:
            return
        torch.cuda.synchronize()
        if self.world > 1 and dist.is_initialized():
            dist.barrier(group=self.group)  # nobody still reads my memory
        for p in self._opened:
            self.C.peer_close(p)
        self._opened.clear()
        self.C.peer_free(self.local_ptr)
        self.local_ptr = 0


class PeerBarrier:
    """Flag barrier over peer memory (bounded spin inside one small kernel per call)."""

    def __init__(self, group=None, timeout_ms: float = 20000.0):
        self.flags = SymmetricBuffer(256, group)
        self.epoch = 0
        self.timeout_ms = timeout_ms
        self.rank, self.world = self.flags.rank, self.flags.world

    def __call__(self) -> None:
        if self.world == 1:
            return
        self.epoch += 1
        self.flags.C.peer_barrier(self.flags.ptrs, self.rank, self.epoch, self.timeout_ms)

    def close(self) -> None:
        self.flags.close()


class RingBuffers:
    """Per-rank buffers of ring attention for a fixed local K/V shape [B, S_local, Hkv, D]:

    * ``kv``      2 slots x (K, V) bf16, peer-visible: what other ranks pull from,
    * ``staging`` 2 x (K, V) bf16, local: where the attention kernels drop the next step's K/V,
    * ``dkv``     2 slots x (dK, dV) fp32, peer-visible: where every rank adds its gradient share,
    * a flag barrier.
    Slots alternate between consecutive layers so one barrier per call is enough.

    With ``fp8_block_tokens > 0`` the K/V slots and the staging buffers hold the e4m3 cache format instead of
    bf16: per slot the K codes, the V codes (one byte per element) and their fp32 scales, one per (block of
    ``fp8_block_tokens`` tokens, KV head). That halves the peer-visible K/V memory and the bytes every ring
    step pulls over NVLink; the puller expands the staged codes to bf16 right before its attention kernel
    (``dequant_staged``), so the tensor-core path itself still runs in bf16.
    """

    def __init__(self, kv_shape: Sequence[int], group=None, timeout_ms: float = 20000.0, dtype=torch.bfloat16,
                 fp8_block_tokens: int = 0):
        self.kv_shape = tuple(kv_shape)
        n = 1
        for s in kv_shape:
            n *= s
        self.n = n
        self.fp8_block_tokens = int(fp8_block_tokens)
        self.dtype = dtype
        self.dkv_bytes = n * 4
        if self.fp8_block_tokens > 0:
            B, S, H, D = self.kv_shape
            assert S % self.fp8_block_tokens == 0, "local sequence length must be a multiple of the fp8 block"
            self.n_scales = B * (S // self.fp8_block_tokens) * H
            self.kv_bytes = n                                              # codes of one of K or V
            self.scale_bytes = (self.n_scales * 4 + 15) // 16 * 16         # scales of one of K or V
            self.slot_bytes = (2 * self.kv_bytes + 2 * self.scale_bytes + 255) // 256 * 256
            self.staging_raw = torch.empty(2, self.slot_bytes, device="cuda", dtype=torch.uint8)
            self.work = torch.empty(2, n, device="cuda", dtype=dtype)      # dequantised K, V of the current step
            self.staging = None
        else:
            self.esize = _DTYPE_SIZE[dtype]
            self.kv_bytes = n * self.esize        # one of K or V
            self.slot_bytes = 2 * self.kv_bytes
            self.staging = torch.empty(2, 2, n, device="cuda", dtype=dtype)
        self.kv = SymmetricBuffer(2 * self.slot_bytes, group)
        self.dkv = SymmetricBuffer(2 * 2 * self.dkv_bytes, group)
        self.barrier_obj = PeerBarrier(group, timeout_ms)
        self.rank, self.world = self.kv.rank, self.kv.world
        self.C = self.kv.C

    # e4m3 slots -----------------------------------------------------------------------------
    def _q_layout(self, base_tensor_fn):
        B, S, H, D = self.kv_shape
        nb = S // self.fp8_block_tokens
        kc = base_tensor_fn(0, (B * S, H, D), torch.uint8)
        vc = base_tensor_fn(self.kv_bytes, (B * S, H, D), torch.uint8)
        ks = base_tensor_fn(2 * self.kv_bytes, (B * nb, H), torch.float32)
        vs = base_tensor_fn(2 * self.kv_bytes + self.scale_bytes, (B * nb, H), torch.float32)
        return kc, vc, ks, vs

    def quantize_into_slot(self, k: torch.Tensor, v: torch.Tensor, slot: int) -> None:
        """Writes this rank's K and V (bf16 [B, S, Hkv, D]) into its slot as e4m3 codes + scales."""
        base = slot * self.slot_bytes
        kc, vc, ks, vs = self._q_layout(lambda off, shape, dt: self.kv.tensor(self.rank, base + off, shape, dt))
        B, S, H, D = self.kv_shape
        self.C.kv_quant_e4m3(k.reshape(B * S, H, D).contiguous(), kc, ks, None, self.fp8_block_tokens)
        self.C.kv_quant_e4m3(v.reshape(B * S, H, D).contiguous(), vc, vs, None, self.fp8_block_tokens)

    def _dequant(self, kc, vc, ks, vs) -> Tuple[torch.Tensor, torch.Tensor]:
        B, S, H, D = self.kv_shape
        kk, vv = self.work[0].view(B * S, H, D), self.work[1].view(B * S, H, D)
        self.C.kv_dequant_e4m3(kc, ks, kk, self.fp8_block_tokens)
        self.C.kv_dequant_e4m3(vc, vs, vv, self.fp8_block_tokens)
        return kk.view(self.kv_shape), vv.view(self.kv_shape)

    def dequant_local(self, slot: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """bf16 K, V as every rank sees this rank's slot (the values the cache format can represent)."""
        base = slot * self.slot_bytes
        return self._dequant(*self._q_layout(lambda off, shape, dt: self.kv.tensor(self.rank, base + off, shape, dt)))

    def dequant_staged(self, idx: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Expands the codes a previous kernel pulled into staging[idx] to bf16 K, V."""
        raw = self.staging_raw[idx]

        def view(off, shape, dt):
            nbytes = 1
            for d in shape:
                nbytes *= d
            nbytes *= _DTYPE_SIZE[dt]
            return raw[off: off + nbytes].view(dt).view(shape)

        return self._dequant(*self._q_layout(view))

    # K/V slot views -------------------------------------------------------------------------
    def kv_views(self, rank: int, slot: int, shape=None) -> Tuple[torch.Tensor, torch.Tensor]:
        assert self.fp8_block_tokens == 0, "e4m3 slots hold codes: use quantize_into_slot / dequant_*"
        shape = tuple(shape or self.kv_shape)
        base = slot * self.slot_bytes
        return (self.kv.tensor(rank, base, shape, self.dtype),
                self.kv.tensor(rank, base + self.kv_bytes, shape, self.dtype))

    def staged_kv(self, idx: int, shape=None) -> Tuple[torch.Tensor, torch.Tensor]:
        shape = tuple(shape or self.kv_shape)
        return self.staging[idx, 0].view(shape), self.staging[idx, 1].view(shape)

    def pull_args(self, owner: int, slot: int, stage: int) -> Tuple[int, int, int]:
        """(src, dst, nbytes) copying owner's slot (K and V, in e4m3 mode also their scales, are adjacent) into
        staging[stage]."""
        if self.fp8_block_tokens > 0:
            return (self.kv.ptr(owner, slot * self.slot_bytes), self.staging_raw[stage].data_ptr(),
                    2 * self.kv_bytes + 2 * self.scale_bytes)
        return (self.kv.ptr(owner, slot * self.slot_bytes), self.staging[stage].data_ptr(), 2 * self.kv_bytes)

    def pull_now(self, owner: int, slot: int, stage: int) -> None:
        src, dst, nbytes = self.pull_args(owner, slot, stage)
        self.C.peer_pull(src, dst, nbytes, 592)

    # dK/dV accumulators ---------------------------------------------------------------------
    def dkv_views(self, rank: int, slot: int, shape=None) -> Tuple[torch.Tensor, torch.Tensor]:
        shape = tuple(shape or self.kv_shape)
        base = slot * 2 * self.dkv_bytes
        return (self.dkv.tensor(rank, base, shape, torch.float32),
                self.dkv.tensor(rank, base + self.dkv_bytes, shape, torch.float32))

    def zero_dkv(self, slot: int) -> None:
        self.dkv.tensor(self.rank, slot * 2 * self.dkv_bytes, (2 * self.n,), torch.float32).zero_()

    def barrier(self) -> None:
        self.barrier_obj()

    def close(self) -> None:
        self.kv.close()
        self.dkv.close()
        self.barrier_obj.close()
