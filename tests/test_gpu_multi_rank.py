"""`run_sharded` on two GPUs of one box: one process per GPU over NCCL, output all-gathered.

Skipped where fewer than two GPUs are visible. The ranks run as child processes under torchrun
(`tests/multi_rank_worker.py`); the failure they provoke is a host-side exception on one rank
between launches, never a device fault.
"""

import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_two_ranks_reproduce_the_single_gpu_output_and_fail_together():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    result = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
         "--master-addr", "127.0.0.1", "--master-port", "29533", str(ROOT / "tests" / "multi_rank_worker.py")],
        capture_output=True, text=True, timeout=600, env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    assert result.returncode == 0, result.stdout[-2000:] + result.stderr[-4000:]
    assert "multi-rank sharding ok" in result.stdout
