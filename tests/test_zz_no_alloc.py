"""The allocation-free attention backward (`zx_attn_bwd_noalloc`, csrc/noalloc/attn_bwd_static.h),
called through its exported C symbol exactly as a caller without an allocator would: raw device
pointers in, no scratch passed. Its results must match the regular entry point, which takes a
caller-allocated delta buffer. Two calls in a row share the library's built-in scratch array, so the
second call (different data) also checks that stale scratch contents do no harm. This file sorts
last on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes
import math
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import zenyx_b200
    from zenyx_b200.ops import _ext

    _ext.C()  # make sure torch's CUDA libraries and the extension are loaded
    lib = ctypes.CDLL(os.path.join(os.path.dirname(zenyx_b200.__file__), "_C.so"))
    fn = lib.zx_attn_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 9 + [ctypes.c_int] * 5 + [ctypes.c_longlong] * 3 + [ctypes.c_float, ctypes.c_int,
                                                                                            ctypes.c_void_p, ctypes.c_void_p,
                                                                                            ctypes.c_char_p, ctypes.c_int]
    return fn


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_noalloc_attn_bwd_matches_regular_entry_point_twice():
    from zenyx_b200.ops import _ext

    C = _ext.C()
    fn = _lib()
    D = 128
    scale = 1.0 / math.sqrt(D)
    for call, (B, S, Hq, Hkv, causal) in enumerate([(2, 512, 4, 2, True), (1, 768, 2, 1, False)]):
        torch.manual_seed(20 + call)
        q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
        k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
        v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
        do = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
        o = torch.empty_like(q)
        lse = torch.empty(B, Hq, S, device="cuda")
        C.attn_fwd(q, k, v, o, lse, scale, causal, 0, 0, [0], [0], False, 0, 0, 0)
        # regular entry point: caller allocates the delta scratch
        delta = torch.empty_like(lse)
        dq_r = torch.empty(B, S, Hq, D, device="cuda")
        dk_r = torch.zeros(B, S, Hkv, D, device="cuda")
        dv_r = torch.zeros(B, S, Hkv, D, device="cuda")
        C.attn_bwd(q, k, v, o, do, lse, delta, dq_r, dk_r, dv_r, scale, causal, 0, 0, [0], [0], True, False, 0, 0, 0)
        _ext.check_status()
        # allocation-free entry point: outputs deliberately pre-filled with garbage
        dq = torch.full((B, S, Hq, D), 7.0, device="cuda")
        dk = torch.full((B, S, Hkv, D), 7.0, device="cuda")
        dv = torch.full((B, S, Hkv, D), 7.0, device="cuda")
        status = torch.full((4,), 9, device="cuda", dtype=torch.int32)
        err = ctypes.create_string_buffer(256)
        stream = torch.cuda.current_stream().cuda_stream
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(), dq.data_ptr(),
                dk.data_ptr(), dv.data_ptr(), B, Hq, Hkv, S, S, q.stride(1), k.stride(1), v.stride(1), scale,
                int(causal), status.data_ptr(), stream, err, 256)
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0, 0, 0]
        # Same kernels, same inputs: dQ is computed without atomics and must match bit for bit; dK / dV are
        # accumulated with fp32 atomics whose order differs between launches.
        assert torch.equal(dq, dq_r)
        assert _rel(dk, dk_r) < 1e-5
        assert _rel(dv, dv_r) < 1e-5


def test_noalloc_attn_bwd_rejects_bad_shapes_before_touching_the_outputs():
    fn = _lib()
    err = ctypes.create_string_buffer(256)
    B, S, Hq, Hkv, D = 1, 200, 2, 1, 128       # 200 is not a multiple of 128
    x = torch.zeros(B, 256, Hq, D, device="cuda", dtype=torch.bfloat16)
    kv = torch.zeros(B, 256, Hkv, D, device="cuda", dtype=torch.bfloat16)
    lse = torch.zeros(B, Hq, 256, device="cuda")
    dq = torch.full((B, 256, Hq, D), 7.0, device="cuda")
    dk = torch.full((B, 256, Hkv, D), 7.0, device="cuda")
    dv = torch.full((B, 256, Hkv, D), 7.0, device="cuda")
    rc = fn(x.data_ptr(), kv.data_ptr(), kv.data_ptr(), x.data_ptr(), x.data_ptr(), lse.data_ptr(), dq.data_ptr(),
            dk.data_ptr(), dv.data_ptr(), B, Hq, Hkv, S, S, Hq * D, Hkv * D, Hkv * D, 0.1, 1, None, None, err, 256)
    torch.cuda.synchronize()
    assert rc == 1 and b"multiples of 128" in err.value
    assert float(dk.min()) == 7.0 and float(dv.min()) == 7.0 and float(dq.min()) == 7.0   # nothing was cleared


def test_noalloc_attn_bwd_rejects_oversized_problem():
    fn = _lib()
    err = ctypes.create_string_buffer(256)
    dummy = torch.zeros(16, device="cuda")
    p = dummy.data_ptr()
    # 64 heads x 32768 tokens = 2M rows > the 1M-row scratch: refused before anything is launched
    rc = fn(p, p, p, p, p, p, p, p, p, 1, 64, 8, 32768, 32768, 8192, 1024, 1024, 0.1, 1, None, None, err, 256)
    assert rc == 2
    assert b"exceeds the built-in scratch" in err.value
