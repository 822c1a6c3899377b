"""Expert parallelism over real GPUs: launches ``tests/multi_rank_worker.py`` with one process
per GPU (2, and 4 when available) and requires every rank to match the CPU oracle."""

import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("world", [2, 4])
def test_routed_experts_across_ranks(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29650 + world), str(ROOT / "tests" / "multi_rank_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0 and f"MULTI_RANK_OK {world}" in res.stdout, res.stdout[-3000:] + res.stderr[-6000:]
