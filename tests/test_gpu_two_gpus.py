"""The multi-GPU paths on two real GPUs (skipped where fewer are visible): one process per GPU, launched the
way the benchmark is (torch.distributed.run on 127.0.0.1). The checks live in tests/two_gpu_worker.py."""

import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]


def test_sharded_calls_and_sharded_chain_across_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", str(ROOT / "tests" / "two_gpu_worker.py")]
    done = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=900)
    tail = (done.stdout + done.stderr)[-4000:]
    assert done.returncode == 0, tail
    assert "TWO_GPU_WORKER_OK" in done.stdout, tail
