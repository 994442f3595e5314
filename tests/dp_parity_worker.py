"""Worker of tests/test_gpu_dp.py (one process per GPU, started by torch.distributed.run): trains a small bf16 model
data-parallel for a few steps through the device-flag all-reduce path and checks, on rank 0, that (a) every rank ends with
bitwise identical weights, (b) the mean of the per-rank losses follows the CPU oracle trained on the concatenated global
batch within 1e-2 relative. Prints DP_PARITY_OK on success."""
import importlib
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def log(msg):
    """progress lines (flushed) so that a run that is cut short still shows how far it got"""
    print(f"[rank {os.environ.get('RANK', '?')}] {msg}", flush=True)


def main():
    from oracle import gpt_oracle as orc
    ofa = importlib.import_module("open-flapping-airplanes_b200")
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    ofa.dp.configure_env(8)                        # before the first CUDA call
    torch.cuda.set_device(local)
    log("init_process_group")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    log("process group up")
    nsteps, V, L, T, B = 6, 1024, 2, 256, 2
    ocfg = orc.OracleConfig(V=V, D=768, L=L, H=12, T=T, B=B, tied=False)
    w0 = orc.init_weights(ocfg)
    ntok = 1 << 15
    tokens = orc.synthetic_tokens(V, ntok, 100 + rank)
    starts = orc.batch_starts(ocfg, ntok, nsteps)
    cfg = ofa.default_config("gpt_s")
    cfg.vocab, cfg.valid_vocab, cfg.n_layer, cfg.ctx_len, cfg.batch = V, V, L, T, B
    cfg.device, cfg.dp_world, cfg.grad_bf16, cfg.ext_sync, cfg.reserved_sms, cfg.bucket_bytes = local, world, 1, 1, 8, 8 << 20
    mk = ofa.Megakernel(cfg)
    mk.load_weights(orc.flatten(ocfg, w0)); mk.set_tokens(tokens); mk.set_starts(starts.astype(np.uint32))
    log("context created, buckets %s" % (mk.buckets(),))
    # DP_SIDE=native: the library's own C++ queue and communicator; otherwise the process group of this script
    dp = ofa.dp.NativeDataParallel(mk, rank, world) if os.environ.get("DP_SIDE") == "native" else ofa.dp.DataParallel(mk, dist)
    log("communication stream warmed up")
    for n in (2, nsteps - 2):                      # two launches: the flags restart, the optimizer state continues
        mk.launch(n); log(f"launched {n}"); dp.enqueue(n); log("enqueued"); dp.wait(60000, comm_timeout_s=60.0); log("kernel and communication done")
    losses = torch.tensor(mk.losses(), dtype=torch.float64, device="cuda")
    dist.all_reduce(losses); losses /= world
    w = torch.from_numpy(mk.read_weights()).cuda()
    wsum = [torch.zeros_like(w) for _ in range(world)]
    dist.all_gather(wsum, w)
    ok = True
    if rank == 0:
        same = all(torch.equal(wsum[0], x) for x in wsum[1:])
        gcfg = orc.OracleConfig(V=V, D=768, L=L, H=12, T=T, B=B * world, tied=False)
        model = orc.GPTOracle(gcfg, w0, "bf16_points"); opt = orc.make_optimizer(gcfg, model)
        ref = []
        toks = [orc.synthetic_tokens(V, ntok, 100 + r) for r in range(world)]
        for s in range(nsteps):
            for g in opt.param_groups:
                g["lr"] = orc.lr_at(gcfg, s)
            xs, ys = zip(*[orc.get_batch(ocfg, toks[r], starts[s]) for r in range(world)])
            loss = model(torch.cat(xs), torch.cat(ys)); loss.backward(); opt.step(); opt.zero_grad(set_to_none=True)
            ref.append(float(loss.detach()))
        ref = np.array(ref); got = losses.cpu().numpy()
        rel = np.abs(got - ref).max() / ref.max()
        print("dp losses", got, "oracle", ref, "rel", rel, "identical weights", same, flush=True)
        ok = same and rel <= 1e-2 and len(mk.buckets()) >= 3
    mk.close()
    dist.barrier(); dist.destroy_process_group()
    if rank == 0:
        print("DP_PARITY_OK" if ok else "DP_PARITY_FAIL", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
