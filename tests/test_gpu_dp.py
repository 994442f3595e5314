"""Data parallelism on real GPUs (needs at least two): one process per GPU over NCCL, gradients all-reduced bucket by
bucket while the persistent kernels run, ordered only by device flags. Skipped on a single-GPU box."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_training_matches_global_batch_oracle():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", "29617",
           os.path.join(ROOT, "tests", "dp_parity_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0 and "DP_PARITY_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
