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
