"""Generates tests/golden/*.npz by IMPORTING the reference's own model file (llm/baseline/common.py) with its module
constants set to small configurations, and running its GPT class, init recipe, LR schedule, batch sampler and AdamW
parameter groups on the CPU. Run once in the build container (the reference checkout is not available elsewhere):

    python tests/golden/make_golden.py <path to a checkout of the reference>

The fixtures pin oracle/gpt_oracle.py (tests/test_oracle_golden.py). Stored: the initial weights' checksums and samples,
step-0 loss, every gradient tensor of step 0, weights after one and three AdamW steps (sampled), the loss of the first
steps, the LR schedule at probe steps, the sampler's first starts, and greedy continuations from the reference's
full-sequence forward.
"""
import importlib.util
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_common(ref_root):
    spec = importlib.util.spec_from_file_location("ofa_ref_common", os.path.join(ref_root, "llm", "baseline", "common.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def set_dims(c, V, D, L, H, T, B, steps=4000):
    c.V, c.D, c.L, c.H, c.T, c.B = V, D, L, H, T, B
    c.FFN, c.DH, c.STEPS = 4 * D, D // H, steps


def run_config(c, name, V, D, L, H, T, B, nsteps, ntok, constant_lr=None):
    set_dims(c, V, D, L, H, T, B)
    torch.manual_seed(0)
    tokens = np.random.default_rng(0).integers(0, V, size=ntok, dtype=np.uint32)
    starts = c.batch_starts(ntok, nsteps)
    w0 = c.init_weights()
    model = c.GPT()
    model.load_spec(w0)
    mats = [p for p in model.parameters() if p.dim() >= 2]
    vecs = [p for p in model.parameters() if p.dim() < 2]
    opt = torch.optim.AdamW([{"params": mats, "weight_decay": c.WD}, {"params": vecs, "weight_decay": 0.0}], lr=c.LR_MAX, betas=c.BETAS, eps=1e-8)
    out = {"dims": np.array([V, D, L, H, T, B]), "starts": starts, "ntok": np.array([ntok])}
    losses = []
    for s in range(nsteps):
        lr = c.lr_at(s) if constant_lr is None else constant_lr
        for g in opt.param_groups:
            g["lr"] = lr
        seq = np.stack([tokens[st:st + T + 1] for st in starts[s]]).astype(np.int64)
        x, y = torch.from_numpy(seq[:, :-1]).contiguous(), torch.from_numpy(seq[:, 1:]).contiguous()
        loss = model(x, y)
        loss.backward()
        if s == 0:
            for n, p in model.spec_tensors().items():
                out["g0_" + n] = c.spec_layout(n, p.grad).copy()
            with torch.no_grad():
                out["logits0_seq0"] = model(x)[0].float().numpy()[[0, T // 2, T - 1]]
        opt.step(); opt.zero_grad(set_to_none=True)
        losses.append(float(loss.detach()))
        if s in (0, nsteps - 1):
            for n, p in model.spec_tensors().items():
                out[f"w{s + 1}_" + n] = c.spec_layout(n, p).copy()   # copy: spec_layout may alias the live parameter
    for n, t in w0.items():
        out["w0_" + n] = t.numpy().copy()
    out["losses"] = np.array(losses)
    # greedy continuation with the reference model class (full-sequence forward each step), after training
    prompt = [int(t) for t in np.random.default_rng(7).integers(0, V, size=8)]
    ctx = list(prompt)
    with torch.no_grad():
        for _ in range(min(24, T - 8)):
            lg = model(torch.tensor([ctx]))[0, -1]
            ctx.append(int(torch.argmax(lg)))
    out["greedy_prompt"] = np.array(prompt); out["greedy_out"] = np.array(ctx[8:]); out["greedy_last_logits"] = lg.numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **{k: np.asarray(v) for k, v in out.items()})
    print(name, "losses", losses)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference>")
    ref_root = sys.argv[1]
    torch.set_num_threads(4)
    c = load_common(ref_root)
    # schedule probes at the reference's own constants
    probes = [0, 1, 50, 99, 100, 101, 2000, 3999, 4000]
    np.savez(os.path.join(HERE, "lr_schedule.npz"), steps=np.array(probes), lr=np.array([c.lr_at(s) for s in probes]),
             consts=np.array([c.LR_MAX, c.LR_MIN, c.WARMUP, c.STEPS, c.WD, c.BETAS[0], c.BETAS[1], c.SEED]))
    # the tiny fp32 preset's dims (tied, because the reference's class is tied) with the constant lr of that config
    run_config(c, "tiny_tied", 65, 64, 2, 4, 64, 16, nsteps=3, ntok=1 << 14, constant_lr=3e-4)
    # an odd small shape, reference LR schedule
    run_config(c, "small_tied", 96, 32, 3, 2, 24, 3, nsteps=3, ntok=1 << 12)


if __name__ == "__main__":
    main()
