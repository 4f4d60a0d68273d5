"""Multi-GPU tests: fused ring attention (P2P pull / dK,dV push), fused sharded optimizer, GEMMs fused
with their all-gather / reduce-scatter, and a DP x CP training run. Each spawns one process per GPU on this node with torch.distributed.run."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(case, nproc):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29611", os.path.join(HERE, "_dist_gpu_worker.py"), case]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + "\n" + res.stderr[-3000:]
    return res.stdout


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("case", ["ring", "zero", "train", "tp"])
def test_two_gpus(case):
    out = _run(case, 2)
    assert f"{case} ok" in out


@pytest.mark.skipif(_ngpu() < 4, reason="needs at least 4 GPUs")
@pytest.mark.parametrize("case", ["ring", "train", "tp"])
def test_four_gpus(case):
    out = _run(case, 4)
    assert f"{case} ok" in out


@pytest.mark.skipif(_ngpu() < 8, reason="needs 8 GPUs")
@pytest.mark.parametrize("case", ["ring", "zero", "train", "tp"])
def test_eight_gpus(case):
    out = _run(case, 8)
    assert f"{case} ok" in out
