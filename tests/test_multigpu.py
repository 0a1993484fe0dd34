"""Real multi-GPU parity over NVLink symmetric memory (skipped where fewer than two GPUs are visible)."""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_agree_with_the_oracle(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), str(HERE / "mp_rowpar.py")]
    run = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert run.returncode == 0 and "MULTIGPU_OK" in run.stdout, run.stdout[-3000:] + run.stderr[-3000:]
