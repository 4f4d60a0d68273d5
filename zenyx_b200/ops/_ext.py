"""Loader for the in-tree native extensions.

``C()`` returns the CUDA extension (``zenyx_b200/_C.so``: the sm_100a kernels); ``host()`` the
host-only C++ extension (``zenyx_b200/_host.so``). On a machine with a GPU a missing ``_C.so`` is
an error, never a silent fall back to eager PyTorch: build it with ``python -m zenyx_b200._build``.
The reference project has no native code, hence no counterpart of this module.
"""
from __future__ import annotations

import importlib.util
import os
import threading
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent.parent
_lock = threading.Lock()
_mods: dict = {}


class KernelError(RuntimeError):
    """A kernel reported a failure through the device status word (e.g. a bounded wait ran out)."""


def _load(name: str):
    with _lock:
        if name in _mods:
            return _mods[name]
        # ZENYX_B200_EXT_DIR: take the extensions from another directory (a build made with other
        # compile-time options, for A/B measurements); by default the in-tree build next to the package.
        path = Path(os.environ.get("ZENYX_B200_EXT_DIR", str(_PKG))) / f"{name}.so"
        if not path.exists():
            raise RuntimeError(
                f"zenyx_b200: native extension {path} is missing; run `python -m zenyx_b200._build` "
                "(needs nvcc for the CUDA part)"
            )
        spec = importlib.util.spec_from_file_location(f"zenyx_b200.{name}", str(path))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mods[name] = mod
        return mod


# Kernel launches issued per binding call (everything else launches exactly one kernel).
_LAUNCHES = {"attn_bwd": 3, "read_status": 0, "peer_alloc": 0, "peer_export": 0, "peer_open": 0, "peer_close": 0,
             "peer_free": 0, "tensor_from_ptr": 0}
launch_count = 0


class _CountingProxy:
    """Forwards to the extension module and counts the kernels it launches (for benchmark reports)."""

    def __init__(self, mod):
        self._mod = mod
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._mod, name)
            n = _LAUNCHES.get(name, 1)

            def fn(*args, __raw=raw, __n=n, **kwargs):
                global launch_count
                launch_count += __n
                return __raw(*args, **kwargs)

            self._cache[name] = fn
        return fn


_proxy = None


def C():
    global _proxy
    if _proxy is None:
        _proxy = _CountingProxy(_load("_C"))
    return _proxy


def host():
    return _load("_host")


def have_cuda_ext() -> bool:
    return torch.cuda.is_available() and (_PKG / "_C.so").exists()


def use_cuda_kernels(t: torch.Tensor) -> bool:
    """True when `t` lives on a GPU, in which case the native kernels are mandatory."""
    if not t.is_cuda:
        return False
    C()  # raises loudly if the extension was not built
    return True


_SITES = {
    1: "gemm: TMA producer", 2: "gemm: MMA issuer", 3: "gemm: epilogue",
    11: "attn_fwd: TMA producer", 12: "attn_fwd: MMA issuer", 13: "attn_fwd: softmax",
    21: "attn_bwd: TMA producer", 22: "attn_bwd: MMA issuer", 23: "attn_bwd: compute warps",
    31: "peer barrier", 41: "zero_adamw: peer flag",
    4: "gemm: reduce-scatter owner index", 14: "attn_fwd: output row", 15: "attn_fwd: batch index",
    24: "attn_bwd: dK/dV row", 25: "attn_bwd: dQ row",
}


def check_status(clear: bool = True) -> None:
    """Synchronise the current stream and raise if any kernel recorded an error."""
    code, site, block, info = C().read_status(clear)
    if code != 0:
        kinds = {1: "bounded wait timed out", 2: "bounds check failed", 3: "bad argument"}
        raise KernelError(
            f"kernel error: {kinds.get(code, code)} at {_SITES.get(site, site)} (block {block}, info {info})"
        )
