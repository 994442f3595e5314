"""Data parallelism on real GPUs (needs at least two): one process per GPU over NCCL, gradients all-reduced bucket by
bucket while the persistent kernels run, ordered only by device flags. Skipped on a single-GPU box."""
import os
import signal
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("side", ["torch", "native"])
def test_two_rank_training_matches_global_batch_oracle(side):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", "29617" if side == "torch" else "29618",
           os.path.join(ROOT, "tests", "dp_parity_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", DP_SIDE=side)
    p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env, start_new_session=True)
    try:
        out, err = p.communicate(timeout=240)
    except subprocess.TimeoutExpired:
        os.killpg(p.pid, signal.SIGKILL)          # the whole process group this test started, nothing else
        out, err = p.communicate()
        pytest.fail("data-parallel worker timed out\n" + out[-2000:] + err[-2000:])
    assert p.returncode == 0 and "DP_PARITY_OK" in out, out[-3000:] + err[-3000:]
