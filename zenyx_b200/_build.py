"""In-tree build of the native extensions.

Two shared objects are produced next to this file:

* ``_C.so``    - the sm_100a CUDA kernels plus their torch bindings (needs nvcc),
* ``_host.so`` - host-only C++ (Belady planner, tier engine, CPU reference math).

The reference project ships no native code at all (its ``pyproject.toml`` is a pure-Python
setuptools build), so this file has no counterpart there.

Sources are compiled one translation unit per nvcc/g++ process, in parallel, straight to
object files beside the sources; nothing is cached outside the repository.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
ROOT = PKG_DIR.parent
CSRC = ROOT / "csrc"
OBJ_DIR = CSRC / "_obj"

CUDA_SOURCES = [
    "gemm/gemm_bf16.cu",
    "attn/attn_fwd.cu",
    "attn/attn_bwd.cu",
    "fused/fused_ops.cu",
    "peer/peer_kernels.cu",
    "optim/zero_adamw.cu",
    "noalloc/attn_bwd_static.cu",
]
CUDA_CPP_SOURCES = ["bindings.cpp", "peer/ipc_memory.cpp"]
HOST_SOURCES = ["tier/belady_min.cpp", "tier/tier_engine.cpp", "cpu_ref/flash_cpu.cpp", "cpu_ref/quant_adamw_ref.cpp", "peer/barrier_model.cpp", "attn/tile_iter_host.cpp",
                "host_bindings.cpp"]

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    return str(Path(cuda_home) / "bin" / "nvcc")


def _torch_flags():
    import torch
    from torch.utils import cpp_extension as ce

    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc.append(f"-I{cuda_home}/include")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = [f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    libdirs = ce.library_paths()
    return inc, defs, libdirs, cuda_home


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(str(p).encode())
        h.update(Path(p).read_bytes())
    return h.hexdigest()


def _deps(src: Path):
    """The source plus every header under csrc/ (coarse but safe)."""
    return [src] + sorted(CSRC.rglob("*.h")) + sorted(CSRC.rglob("*.cuh")) + sorted(CSRC.rglob("*.inc"))


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr, flush=True)


def _compile_one(src: Path, obj: Path, cmd_prefix, verbose, extra_key=""):
    stamp = obj.with_suffix(".sha")
    key = _digest(_deps(src)) + extra_key
    if obj.exists() and stamp.exists() and stamp.read_text() == key:
        return False
    _run(cmd_prefix + ["-c", str(src), "-o", str(obj)], verbose)
    stamp.write_text(key)
    return True


def existing(sources):
    return [s for s in sources if (CSRC / s).exists()]


def build_cuda_extension(verbose: bool = False, checked: bool = False) -> Path:
    """Compile every CUDA kernel for sm_100a and link ``zenyx_b200/_C.so``. ``checked=True`` builds the same
    sources with ``-DZX_CHECKED`` (in-kernel index checks that record a bad index in the status word and skip the
    access) into ``zenyx_b200/_checked/_C.so``; load it with ``ZENYX_B200_EXT_DIR=<repo>/zenyx_b200/_checked``."""
    inc, defs, libdirs, cuda_home = _torch_flags()
    obj_dir = CSRC / ("_obj_checked" if checked else "_obj")
    obj_dir.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    nvcc_prefix = [nvcc, *ARCH_FLAGS, "-std=c++17", "-O3", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC",
                   f"-I{CSRC}"] + (["-DZX_CHECKED"] if checked else [])
    cxx_prefix = ["g++", "-std=c++17", "-O2", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", f"-I{CSRC}", *inc, *defs]
    jobs = []
    objs = []
    for s in existing(CUDA_SOURCES):
        obj = obj_dir / (s.replace("/", "_") + ".o")
        objs.append(obj)
        jobs.append((CSRC / s, obj, nvcc_prefix, "".join(nvcc_prefix)))
    for s in existing(CUDA_CPP_SOURCES):
        obj = obj_dir / (s.replace("/", "_") + ".o")
        objs.append(obj)
        jobs.append((CSRC / s, obj, cxx_prefix, "".join(cxx_prefix)))
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        changed = list(ex.map(lambda j: _compile_one(j[0], j[1], j[2], verbose, j[3]), jobs))
    out_dir = PKG_DIR / "_checked" if checked else PKG_DIR
    out_dir.mkdir(exist_ok=True)
    out = out_dir / "_C.so"
    if any(changed) or not out.exists():
        link = ["g++", "-shared", "-o", str(out), *map(str, objs)]
        for d in libdirs:
            link += [f"-L{d}", f"-Wl,-rpath,{d}"]
        link += ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
                 f"-L{cuda_home}/lib64", "-lcudart"]
        _run(link, verbose)
    return out


def build_host_extension(verbose: bool = False) -> Path:
    """Compile the host-only C++ (no CUDA, no torch) into ``zenyx_b200/_host.so`` via pybind11."""
    import pybind11

    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    inc = [f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{CSRC}"]
    prefix = ["g++", "-std=c++17", "-O3", "-fPIC", "-fopenmp", "-fvisibility=hidden", *inc]
    jobs, objs = [], []
    for s in existing(HOST_SOURCES):
        obj = OBJ_DIR / ("host_" + s.replace("/", "_") + ".o")
        objs.append(obj)
        jobs.append((CSRC / s, obj, prefix, "".join(prefix)))
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        changed = list(ex.map(lambda j: _compile_one(j[0], j[1], j[2], verbose, j[3]), jobs))
    out = PKG_DIR / "_host.so"
    if any(changed) or not out.exists():
        _run(["g++", "-shared", "-fopenmp", "-o", str(out), *map(str, objs), "-lpthread"], verbose)
    return out


def build_all(verbose: bool = False, checked: bool = False):
    outs = [build_host_extension(verbose)]
    if Path(_nvcc()).exists():
        outs.append(build_cuda_extension(verbose))
        if checked:
            import shutil

            outs.append(build_cuda_extension(verbose, checked=True))
            shutil.copy2(PKG_DIR / "_host.so", PKG_DIR / "_checked" / "_host.so")
    return outs


if __name__ == "__main__":
    for o in build_all(verbose="-v" in sys.argv, checked="--checked" in sys.argv):
        print("built", o)
