"""File formats of the reference's megakernel program, so that its own tooling keeps working next to this library
(llm/b200/megakernel/ofa.cu): `--init` / `--dump-w` / `--dump-grads` are raw little-endian fp32 vectors of all parameters in
flat order (ofa.cu:489-507, 762-763; the order is that of make_init_flat.py:7-13, which for a tied head is this library's
order too), `--data` is raw uint32 token ids (ofa.cu:513-522), `--starts` raw uint32 [steps, batch] window starts
(ofa.cu:523-528), `--loss-out` one "step loss" line per step with six decimals (ofa.cu:730), `--text-out` token ids separated
by blanks (ofa.cu:753-754). The reference has no optimizer-state file; a checkpoint here is a directory of three such fp32
vectors (weights, first and second moments) plus meta.json, and resuming from it continues bit-for-bit."""
import json
import os

import numpy as np


def read_flat_f32(path, expect=None):
    a = np.fromfile(path, dtype="<f4")
    if expect is not None and a.size != expect:
        raise ValueError(f"{path}: {a.size} fp32 values, expected {expect}")
    return a


def write_flat_f32(path, values):
    np.ascontiguousarray(values, dtype="<f4").tofile(path)


def read_tokens_u32(path):
    return np.fromfile(path, dtype="<u4")


def read_starts_u32(path, batch):
    s = np.fromfile(path, dtype="<u4")
    if s.size % batch:
        raise ValueError(f"{path}: {s.size} values are not a whole number of batches of {batch}")
    return s.reshape(-1, batch)


def write_starts_u32(path, starts):
    np.ascontiguousarray(starts, dtype="<u4").tofile(path)


def write_loss_log(path, losses, first_step=0):
    with open(path, "w") as f:
        for i, v in enumerate(losses):
            f.write("%d %.6f\n" % (first_step + i, float(v)))


def read_loss_log(path):
    steps, losses = [], []
    with open(path) as f:
        for line in f:
            a, b = line.split()
            steps.append(int(a)); losses.append(float(b))
    return np.asarray(steps), np.asarray(losses, dtype=np.float64)


def write_token_ids(path, ids):
    with open(path, "w") as f:
        for t in ids:
            f.write("%d " % int(t))


def save_checkpoint(mk, directory):
    """weights.f32, adam_m.f32, adam_v.f32 (flat fp32, the library's parameter order) and meta.json of a context at rest."""
    os.makedirs(directory, exist_ok=True)
    m, v = mk.read_adam()
    write_flat_f32(os.path.join(directory, "weights.f32"), mk.read_weights())
    write_flat_f32(os.path.join(directory, "adam_m.f32"), m)
    write_flat_f32(os.path.join(directory, "adam_v.f32"), v)
    c = mk.cfg
    meta = {"steps_done": int(mk.steps_done), "num_params": int(mk.num_params),
            "config": {k: int(getattr(c, k)) for k in ("vocab", "d_model", "n_layer", "n_head", "ctx_len", "batch", "tied_head", "dtype")}}
    with open(os.path.join(directory, "meta.json"), "w") as f:
        json.dump(meta, f)
    return meta


def load_checkpoint(mk, directory):
    """Loads a checkpoint written by save_checkpoint into a fresh context of the same configuration; the next launch continues
    the learning-rate schedule, the AdamW step count and the data windows where the saved run stopped."""
    with open(os.path.join(directory, "meta.json")) as f:
        meta = json.load(f)
    c = mk.cfg
    for k, want in meta["config"].items():
        if int(getattr(c, k)) != want:
            raise ValueError(f"checkpoint was written with {k}={want}, this context has {int(getattr(c, k))}")
    n = meta["num_params"]
    mk.load_weights(read_flat_f32(os.path.join(directory, "weights.f32"), n))
    mk.load_adam_state(read_flat_f32(os.path.join(directory, "adam_m.f32"), n), read_flat_f32(os.path.join(directory, "adam_v.f32"), n),
                       meta["steps_done"])
    return meta
