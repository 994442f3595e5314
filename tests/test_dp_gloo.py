"""Data-parallel host logic on CPU: two gloo ranks. Each rank computes the oracle's gradients on its own micro-batch, the
buckets of a planning context are sum-all-reduced in schedule order, and 1/world is applied as AdamW will apply it; the
result must equal the oracle's gradient on the concatenated global batch (DP loss = mean of the per-rank mean losses)."""
import importlib
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from oracle import gpt_oracle as orc
    ofa = importlib.import_module("open-flapping-airplanes_b200")
    cfg = ofa.default_config("tiny")
    cfg.device, cfg.dp_world, cfg.ext_sync, cfg.bucket_bytes = -1, world, 1, 65536
    mk = ofa.Megakernel(cfg)
    buckets = mk.buckets()
    ocfg = orc.tiny_config(tied=False)
    w0 = orc.init_weights(ocfg)
    ntok = 1 << 13
    tokens = orc.synthetic_tokens(ocfg.V, ntok, 100 + rank)             # a distinct stream per rank
    starts = orc.batch_starts(ocfg, ntok, 1)
    r = orc.train(ocfg, w0, tokens, starts, 1, precision="fp32", grab_step0=True)
    flat = torch.from_numpy(orc.flatten(ocfg, r["grads0"]).copy())
    ofa.dp.allreduce_buckets_host(dist, flat, buckets)
    flat *= 1.0 / world
    loss = torch.tensor([r["losses"][0]], dtype=torch.float64); dist.all_reduce(loss); loss /= world
    if rank == 0:
        # global batch = both ranks' sequences in one batch of 2B
        gcfg = orc.OracleConfig(**{**orc.TINY, "B": 2 * orc.TINY["B"]}, tied=False, constant_lr=True, lr_max=3e-4, lr_min=3e-4)
        model = orc.GPTOracle(gcfg, w0, "fp32")
        xs, ys = [], []
        for rr in range(world):
            t = orc.synthetic_tokens(ocfg.V, ntok, 100 + rr)
            x, y = orc.get_batch(ocfg, t, starts[0]); xs.append(x); ys.append(y)
        gl = model(torch.cat(xs), torch.cat(ys)); gl.backward()
        gref = orc.flatten(gcfg, {n: p.grad for n, p in model.named_spec().items()})
        out.put((float(loss), float(gl.detach()), float(np.abs(flat.numpy() - gref).max() / np.abs(gref).max()), len(buckets),
                 ofa.dp.buckets_partition_params(buckets, mk.num_params)))
    mk.close()
    dist.barrier()
    dist.destroy_process_group()


def test_bucketed_allreduce_equals_global_batch_gradient():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    dp_loss, global_loss, gerr, nb, part = out.get()
    assert abs(dp_loss - global_loss) <= 1e-6 * global_loss
    assert gerr <= 1e-5 and nb >= 3 and part


def test_bucket_schedule_is_step_major(ofa=None):
    ofa = importlib.import_module("open-flapping-airplanes_b200")
    s = ofa.dp.bucket_schedule([(0, 4), (4, 4), (8, 2)], 2)
    assert s == [(0, 0), (0, 1), (0, 2), (1, 0), (1, 1), (1, 2)]


def _cancel_worker(rank, world, port, out):
    """Rank 1's "kernel" stops after the first of three steps (as a device-side bounded wait that expired would make it) and never
    raises the remaining ready flags; rank 0's runs all three. Nothing may block: rank 1 cancels its queue, the collectives
    complete on both ranks, and both learn that the launch is not valid."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ofa = importlib.import_module("open-flapping-airplanes_b200")
    cfg = ofa.default_config("tiny")
    cfg.device, cfg.dp_world, cfg.ext_sync, cfg.bucket_bytes = -1, world, 1, 65536
    mk = ofa.Megakernel(cfg)                           # planning context: bucket layout only
    grad = torch.ones(mk.num_params)
    q = ofa.dp.HostFlagQueue(grad, dist)
    dp = ofa.dp.DataParallel(mk, dist, queue=q)
    nb, nsteps = len(dp.buckets), 3
    dp.enqueue(nsteps, first_step=0)

    def fake_kernel():
        import time
        steps = nsteps if rank == 0 else 1
        for s in range(steps):
            for b in range(nb):
                q.flags[b] = s + 1                     # "grads ready"
            t0 = time.monotonic()
            while any(q.flags[32 + b] < s + 1 for b in range(nb)):   # "allreduce done", bounded like the device wait
                if time.monotonic() - t0 > 20:
                    raise ofa.OfaError(ofa.capi.DEVICE_ABORT, "external flag timeout")
                time.sleep(0.0005)
        if rank == 1:
            raise ofa.OfaError(ofa.capi.DEVICE_ABORT, "simulated: kernel stopped after step 1")

    res = "ok"
    try:
        dp.wait(comm_timeout_s=30.0, kernel_wait=fake_kernel)
    except ofa.dp.DataParallelAborted:
        res = "peer_aborted"
    except ofa.OfaError:
        res = "own_abort"
    out.put((rank, res, bool(q.drain(0.1)), [int(x) for x in q.flags[32:32 + nb]]))
    q.close(); mk.close()
    dist.barrier()
    dist.destroy_process_group()


def test_cancel_releases_queued_waits_and_all_ranks_learn_of_the_abort():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_cancel_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    got = dict((r, (res, drained, done)) for r, res, drained, done in [out.get(), out.get()])
    assert got[1][0] == "own_abort" and got[0][0] == "peer_aborted"
    assert got[0][1] and got[1][1]                                    # both queues drained
    assert all(d == 3 for d in got[0][2]) and all(d == 3 for d in got[1][2])   # every queued step's done flag was written


def test_finish_gives_up_after_its_timeout():
    """A queue whose wait is never satisfied: finish() returns False instead of blocking, cancel() then drains it."""
    ofa = importlib.import_module("open-flapping-airplanes_b200")

    class NoDist:
        def all_reduce(self, t, op=None):
            return None

    cfg = ofa.default_config("tiny")
    cfg.device, cfg.ext_sync, cfg.bucket_bytes = -1, 1, 65536
    mk = ofa.Megakernel(cfg)
    q = ofa.dp.HostFlagQueue(torch.zeros(mk.num_params), NoDist())
    dp = ofa.dp.DataParallel(mk, NoDist(), queue=q)
    dp.enqueue(2, first_step=5)
    assert dp.last_target == 7
    assert dp.finish(timeout_s=0.2) is False
    dp.cancel()
    assert dp.finish(timeout_s=10.0) is True
    assert all(int(q.flags[32 + b]) == 7 for b in range(len(dp.buckets)))
    q.close(); mk.close()
