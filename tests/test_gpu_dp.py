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


def test_native_queue_on_one_rank(ofa, oracle):
    """The library's own communication side with a group of one (a single-rank NCCL communicator): the queue of stream waits,
    all-reduces and flag writes must let the kernel through, two launches in a row, and give exactly the weights of the same
    run whose all-reduce is done by torch.distributed's single-rank group; plus the argument checks of the entry points."""
    import ctypes as C
    import numpy as np
    import torch.distributed as dist
    ofa.dp.configure_env(8)                        # NCCL's blocks must fit beside the resident kernel (read when a communicator is created)
    ocfg = oracle.OracleConfig(V=1024, D=768, L=2, H=12, T=256, B=2, tied=False)
    flat0 = oracle.flatten(ocfg, oracle.init_weights(ocfg))
    tokens = oracle.synthetic_tokens(ocfg.V, 1 << 15, 3)
    starts = oracle.batch_starts(ocfg, 1 << 15, 6).astype(np.uint32)

    def make():
        cfg = ofa.default_config("gpt_s")
        cfg.vocab, cfg.valid_vocab, cfg.n_layer, cfg.ctx_len, cfg.batch = ocfg.V, ocfg.V, ocfg.L, ocfg.T, ocfg.B
        cfg.dp_world, cfg.grad_bf16, cfg.ext_sync, cfg.reserved_sms, cfg.bucket_bytes = 1, 1, 1, 8, 8 << 20
        mk = ofa.Megakernel(cfg)
        mk.load_weights(flat0); mk.set_tokens(tokens); mk.set_starts(starts)
        return mk

    mk = make()
    lib = mk.lib
    assert lib.ofa_dp_enqueue(mk.h, 1) == ofa.capi.BAD_ARGUMENT            # not initialised
    dp = ofa.dp.NativeDataParallel(mk, 0, 1, exchange=lambda ident: ident)
    assert lib.ofa_dp_init(mk.h, C.c_char_p(b"\0" * 128), 0, 1) == ofa.capi.BAD_ARGUMENT   # a second communicator for the same context
    assert lib.ofa_dp_enqueue(mk.h, 2) == ofa.capi.BAD_ARGUMENT            # nothing launched
    for n in (2, 4):
        mk.launch(n); dp.enqueue(n); dp.wait(60000, comm_timeout_s=30.0)
    losses, w = mk.losses().copy(), mk.read_weights()
    assert len(losses) == 6 and np.all(np.isfinite(losses))
    mk.close()

    if not dist.is_initialized():
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29633", rank=0, world_size=1)
    try:
        mk2 = make()
        dp2 = ofa.dp.DataParallel(mk2, dist)
        for n in (2, 4):
            mk2.launch(n); dp2.enqueue(n); dp2.wait(60000, comm_timeout_s=30.0)
        np.testing.assert_array_equal(losses, mk2.losses())
        np.testing.assert_array_equal(w, mk2.read_weights())
        mk2.close()
    finally:
        dist.destroy_process_group()
