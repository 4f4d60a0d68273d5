"""Hardware microbenchmarks behind the attention kernels' design (``csrc/microbench/*.cu``): each is a
stand-alone CUDA program built on the same inline-PTX layer as the kernels (``csrc/common/ptx.cuh``),
every wait bounded.

    python -m zenyx_b200.bench.micro --build            # nvcc, sm_100a; binaries land in csrc/_obj/microbench/
    python -m zenyx_b200.bench.micro                    # run all on the current GPU
    python -m zenyx_b200.bench.micro softmax_body       # run one

* ``mma_rate``        clocks per ``tcgen05.mma`` by shape / operand source / majorness, branch-free issue loop
* ``mma_under_load``  the same while eight warps stream TMEM loads/stores and one thread streams bulk copies
* ``barrier_wake``    how late waiting warps see a ``tcgen05.commit`` arrive, by waiter count and wait length
* ``sync_op_cost``    cost of single synchronisation instructions in an otherwise idle CTA
* ``softmax_body``    clocks per 128x128 softmax tile per warp, variants of the row arithmetic, one or two warps
                      per scheduler, with and without polling neighbours

The reference ships no kernels and hence nothing comparable.
"""
from __future__ import annotations

import argparse
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
SRC = ROOT / "csrc" / "microbench"
OUT = ROOT / "csrc" / "_obj" / "microbench"
NAMES = ["mma_rate", "mma_under_load", "barrier_wake", "sync_op_cost", "softmax_body"]


def build(verbose: bool = False) -> None:
    from zenyx_b200._build import ARCH_FLAGS, _nvcc

    OUT.mkdir(parents=True, exist_ok=True)
    for n in NAMES:
        src, exe = SRC / f"{n}.cu", OUT / n
        if exe.exists() and exe.stat().st_mtime >= max(src.stat().st_mtime, (ROOT / "csrc/common/ptx.cuh").stat().st_mtime):
            continue
        cmd = [_nvcc(), *ARCH_FLAGS, "-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-o", str(exe), str(src)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"building {n} failed:\n{r.stderr}")
        if verbose:
            print("built", exe)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("names", nargs="*", default=NAMES)
    ap.add_argument("--build", action="store_true", help="only compile")
    args = ap.parse_args(argv)
    build(verbose=args.build)
    if args.build:
        return
    for n in args.names:
        print(f"== {n}", flush=True)
        r = subprocess.run([str(OUT / n)], capture_output=True, text=True, timeout=120)
        sys.stdout.write(r.stdout)
        if r.returncode != 0:
            sys.stdout.write(r.stderr)
            raise SystemExit(f"{n} exited with {r.returncode}")


if __name__ == "__main__":
    main()
