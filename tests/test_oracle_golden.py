"""Pins the CPU oracle (oracle/gpt_oracle.py) against fixtures generated from the reference's own PyTorch model
(tests/golden/make_golden.py imports llm/baseline/common.py). fp32 on both sides: agreement is to rounding."""
import os

import numpy as np
import pytest
import torch


def _cfg(oracle, g, **kw):
    V, D, L, H, T, B = [int(x) for x in g["dims"]]
    return oracle.OracleConfig(V=V, D=D, L=L, H=H, T=T, B=B, tied=True, **kw)


@pytest.mark.parametrize("name,kw", [("tiny_tied", dict(constant_lr=True, lr_max=3e-4, lr_min=3e-4)), ("small_tied", dict())])
def test_training_matches_reference_model(oracle, golden_dir, name, kw):
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    cfg = _cfg(oracle, g, **kw)
    torch.set_num_threads(4)
    w0 = oracle.init_weights(cfg)
    for n in oracle.param_names(cfg):
        np.testing.assert_array_equal(w0[n].numpy(), g["w0_" + n], err_msg=f"init {n}")     # same generator, same draw order
    ntok = int(g["ntok"][0])
    tokens = oracle.synthetic_tokens(cfg.V, ntok, 0)
    starts = oracle.batch_starts(cfg, ntok, 3)
    np.testing.assert_array_equal(starts, g["starts"])
    r = oracle.train(cfg, w0, tokens, starts, 3, precision="fp32", grab_step0=True)
    np.testing.assert_allclose(r["losses"], g["losses"], rtol=2e-6)
    for n in oracle.param_names(cfg):
        ref = g["g0_" + n]
        np.testing.assert_allclose(r["grads0"][n].numpy(), ref, rtol=2e-4, atol=2e-6 * max(1e-30, np.abs(ref).max()) + 1e-9, err_msg=f"grad {n}")
        np.testing.assert_allclose(r["weights"][n].numpy(), g["w3_" + n], rtol=1e-5, atol=2e-7, err_msg=f"weights after 3 steps {n}")
    # one-step weights: rerun a single step
    r1 = oracle.train(cfg, w0, tokens, starts, 1, precision="fp32")
    for n in oracle.param_names(cfg):
        np.testing.assert_allclose(r1["weights"][n].numpy(), g["w1_" + n], rtol=1e-5, atol=2e-7, err_msg=f"weights after 1 step {n}")


@pytest.mark.parametrize("name,kw", [("tiny_tied", dict(constant_lr=True, lr_max=3e-4, lr_min=3e-4)), ("small_tied", dict())])
def test_logits_and_greedy_decode_match_reference_model(oracle, golden_dir, name, kw):
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    cfg = _cfg(oracle, g, **kw)
    w0 = oracle.init_weights(cfg)
    ntok = int(g["ntok"][0])
    tokens = oracle.synthetic_tokens(cfg.V, ntok, 0)
    x, _ = oracle.get_batch(cfg, tokens, g["starts"][0])
    with torch.no_grad():
        lg = oracle.GPTOracle(cfg, w0, "fp32").logits(x)[0].numpy()
    np.testing.assert_allclose(lg[[0, cfg.T // 2, cfg.T - 1]], g["logits0_seq0"], rtol=1e-4, atol=1e-6)
    # greedy continuation from the weights after 3 steps
    w3 = {n: torch.from_numpy(g["w3_" + n]) for n in oracle.param_names(cfg)}
    out, last = oracle.greedy_decode(cfg, w3, [int(t) for t in g["greedy_prompt"]], len(g["greedy_out"]))
    assert out == [int(t) for t in g["greedy_out"]]
    np.testing.assert_allclose(last, g["greedy_last_logits"], rtol=1e-4, atol=1e-6)


def test_lr_schedule_matches_reference(oracle, golden_dir):
    g = np.load(os.path.join(golden_dir, "lr_schedule.npz"))
    lr_max, lr_min, warm, steps, wd, b1, b2, seed = g["consts"]
    cfg = oracle.gpt_s_config()
    assert (cfg.lr_max, cfg.lr_min, cfg.warmup, cfg.sched_steps, cfg.wd, cfg.betas[0], cfg.betas[1], cfg.seed) == (lr_max, lr_min, warm, steps, wd, b1, b2, seed)
    for s, lr in zip(g["steps"], g["lr"]):
        if s < 4000:   # the reference never asks for s = STEPS; the oracle clamps the cosine there
            assert abs(oracle.lr_at(cfg, int(s)) - lr) <= 1e-12 * abs(lr) + 1e-18, s


def test_untied_head_changes_only_the_head(oracle):
    """The untied variant (the GPT-S and tiny presets of this library) draws lm_head right after wpe and leaves every other tensor's recipe alone."""
    c_t = oracle.tiny_config(tied=True); c_u = oracle.tiny_config(tied=False)
    wt, wu = oracle.init_weights(c_t), oracle.init_weights(c_u)
    np.testing.assert_array_equal(wt["wte"].numpy(), wu["wte"].numpy())
    np.testing.assert_array_equal(wt["wpe"].numpy(), wu["wpe"].numpy())
    assert wu["lm_head"].shape == (65, 64) and not np.array_equal(wu["lm_head"].numpy(), wu["wte"].numpy())
    assert oracle.flatten(c_u, wu).size == oracle.flatten(c_t, wt).size + 65 * 64
    back = oracle.unflatten(c_u, oracle.flatten(c_u, wu))
    for n in oracle.param_names(c_u):
        np.testing.assert_array_equal(back[n].numpy(), wu[n].numpy())


def test_bf16_points_oracle_is_close_to_fp32(oracle):
    cfg = oracle.tiny_config(tied=False)
    w0 = oracle.init_weights(cfg)
    tokens = oracle.synthetic_tokens(cfg.V, 1 << 13, 0)
    starts = oracle.batch_starts(cfg, 1 << 13, 1)
    a = oracle.train(cfg, w0, tokens, starts, 1, precision="fp32")["losses"][0]
    b = oracle.train(cfg, w0, tokens, starts, 1, precision="bf16_points")["losses"][0]
    c = oracle.train(cfg, w0, tokens, starts, 1, precision="bf16_autocast")["losses"][0]
    assert abs(a - b) / a < 5e-3 and abs(a - c) / a < 5e-3
