"""Tensor-parallel layer on real GPUs (skipped with fewer than two): the exchange fused into the
kernels over peer memory against NCCL and against the CPU oracle, one process per GPU.

NVLS is switched off for the child processes and the fused kernels use plain peer stores and loads
(no multimem), as is asked of tests in which a rank could leave early."""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _gpus() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_exchange_matches_nccl_and_the_oracle(world):
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29600 + world), str(ROOT / "tests" / "tp_fused_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=480)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert res.stdout.count("identical_across_ranks=True") == 7, res.stdout
