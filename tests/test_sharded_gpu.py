"""Sharded sample + gather + exchange on real GPUs: one process per GPU over NCCL, results
compared with the oracle's single-process gather from the concatenated table."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


def _run(world):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    if world == 1:
        cmd = [sys.executable, str(HERE / "sharded_gpu_worker.py")]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), str(HERE / "sharded_gpu_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert f"SHARDED_GPU_OK {world}" in out.stdout


def test_single_rank_direct_path():
    _run(1)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_over_nccl(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world)
