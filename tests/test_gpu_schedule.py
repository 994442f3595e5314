"""Properties of the scheduler itself, on the GPU through the C ABI.

1. Order independence. The reference pulls the tasks of its libraries in shuffled orders and requires the same bits
   (llm/gemm/test_gemm.cu:20-49,238-278, llm/attention/test_attention.cu:45-77). Here the test hook
   ofa_debug_set_task_shuffle makes every phase hand out its tasks in a permuted order; GEMM, attention, LayerNorm,
   cross-entropy and embedding-backward outputs, and a whole training step, must not change by one bit.
2. Bounded waits. Every device-side wait gives up after a deadline and the kernel RETURNS with a status; nothing here
   faults or hangs a GPU: an external flag that nobody raises makes the wait run out (ST_EXTERNAL_TIMEOUT), ofa_abort
   stops a long launch, ofa_wait with a short timeout reports OFA_TIMEOUT and a later wait succeeds."""
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DIMS = dict(vocab=1024, d_model=768, n_layer=1, n_head=12, ctx_len=256, batch=2)


def bfr(t):
    return t.bfloat16().float()


def _task_chain(ofa):
    """one launch exercising every task kind whose result could depend on the order tasks are pulled in; returns output buffers"""
    K = ofa.capi
    V, D, T, B = DIMS["vocab"], DIMS["d_model"], DIMS["ctx_len"], DIMS["batch"]
    N = B * T
    g = torch.Generator().manual_seed(42)
    dev = lambda t, dt="bf16": ofa.DeviceBuffer.from_host(t.numpy(), dt)
    x = bfr(torch.randn(N, D, generator=g)); gamma = bfr(1 + 0.1 * torch.randn(D, generator=g))
    Wqkv = bfr(torch.randn(D, 3 * D, generator=g) * 0.05); Wh = bfr(torch.randn(V, D, generator=g) * 0.05)
    dO = bfr(torch.randn(N, D, generator=g)); tok = torch.randint(0, V, (N,), generator=g, dtype=torch.int32); tok[:40] = 3
    d_x, d_g, d_W, d_Wh, d_dO = dev(x), dev(gamma), dev(Wqkv), dev(Wh), dev(dO)
    d_tok = ofa.DeviceBuffer.from_host(tok.numpy(), np.int32)
    y = ofa.DeviceBuffer((N, D), "bf16"); mean = ofa.DeviceBuffer((N,), np.float32); rstd = ofa.DeviceBuffer((N,), np.float32)
    qkv = ofa.DeviceBuffer((N, 3 * D), "bf16"); o = ofa.DeviceBuffer((N, D), "bf16"); lse = ofa.DeviceBuffer((B, 12, T), np.float32)
    Dr = ofa.DeviceBuffer((B, 12, T), np.float32); dqkv = ofa.DeviceBuffer((N, 3 * D), "bf16")
    logits = ofa.DeviceBuffer((N, V), "bf16"); loss = ofa.DeviceBuffer((N,), np.float32)
    dW = ofa.DeviceBuffer((D, 3 * D), np.float32); dx = ofa.DeviceBuffer((N, D), "bf16"); part = ofa.DeviceBuffer(((N + 15) // 16, D), np.float32)
    dwte = ofa.DeviceBuffer((V, D), np.float32)
    phases = [
        ofa.phase(K.TK_LN_FWD, [y, mean, rstd, d_x, d_g]),
        ofa.gemm_phase(0, 0, N, 3 * D, D, y, D, d_W, 3 * D, qkv, 3 * D, nsub=2),
        ofa.phase(K.TK_ATT_FWD, [qkv, o, lse]),
        ofa.phase(K.TK_ATT_PREP, [o, d_dO, Dr]),
        ofa.phase(K.TK_ATT_BWD, [qkv, d_dO, lse, Dr, dqkv, o]),
        ofa.gemm_phase(2, 4, D, 3 * D, N, y, D, dqkv, 3 * D, dW, 3 * D),
        ofa.gemm_phase(1, 0, N, V, D, o, D, d_Wh, D, logits, V),
        ofa.phase(K.TK_CE, [logits, d_tok, loss]),
        ofa.phase(K.TK_LN_BWD, [dx, part, d_dO, d_x, mean, rstd, d_g, None]),
        ofa.phase(K.TK_EMB_WTE, [dwte, dx, d_tok], i0=0),
    ]
    ofa.run_phases(K.DTYPE_BF16, DIMS, phases)
    keep = [d_x, d_g, d_W, d_Wh, d_dO, d_tok]
    outs = {"y": y, "qkv": qkv, "o": o, "lse": lse, "dqkv": dqkv, "dW": dW, "dlogits": logits, "loss": loss, "dx": dx, "part": part, "dwte": dwte}
    return {k: (v.download().view(np.uint32) if v.dtype != "bf16" else v.download()).copy() for k, v in outs.items()}, keep


def test_task_order_does_not_change_any_bit(ofa):
    lib = ofa.capi.load()
    base, _ = _task_chain(ofa)
    assert np.isfinite(base["loss"].view(np.float32)).all()
    try:
        for seed in (1, 2024, 987654321):
            lib.ofa_debug_set_task_shuffle(seed)
            got, _ = _task_chain(ofa)
            for k in base:
                assert np.array_equal(got[k], base[k]), (seed, k)
    finally:
        lib.ofa_debug_set_task_shuffle(0)


def _small_training(ofa, oracle, nsteps=3):
    ocfg = oracle.OracleConfig(V=1024, D=768, L=2, H=12, T=256, B=2, tied=False)
    w0 = oracle.init_weights(ocfg)
    tokens = oracle.synthetic_tokens(ocfg.V, 1 << 15, 0)
    cfg = ofa.default_config("gpt_s")
    cfg.vocab, cfg.valid_vocab, cfg.n_layer, cfg.ctx_len, cfg.batch = ocfg.V, ocfg.V, ocfg.L, ocfg.T, ocfg.B
    return ocfg, w0, tokens, cfg


def test_training_steps_are_bitwise_identical_under_a_permuted_task_order(ofa, oracle):
    """also covers the hashed window starts (no starts table), which is what the benchmark uses"""
    lib = ofa.capi.load()
    ocfg, w0, tokens, cfg = _small_training(ofa, oracle)
    res = []
    try:
        for seed in (0, 31337):
            lib.ofa_debug_set_task_shuffle(seed)
            mk = ofa.Megakernel(cfg)
            mk.load_weights(oracle.flatten(ocfg, w0)); mk.set_tokens(tokens)
            mk.run(3, timeout_ms=120000)
            res.append((mk.losses().copy(), mk.read_weights().copy()))
            mk.close()
    finally:
        lib.ofa_debug_set_task_shuffle(0)
    assert np.array_equal(res[0][0].view(np.uint32), res[1][0].view(np.uint32))
    assert np.array_equal(res[0][1].view(np.uint32), res[1][1].view(np.uint32))
    # hashed starts: the first step's loss equals the oracle's on the windows the documented hash selects
    def splitmix64(z):
        m = (1 << 64) - 1
        z = (z + 0x9E3779B97F4A7C15) & m
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        return z ^ (z >> 31)
    starts0 = np.array([[splitmix64(0 ^ (0 * ocfg.B + b)) % (len(tokens) - ocfg.T - 1) for b in range(ocfg.B)]], dtype=np.int64)
    ref = oracle.train(ocfg, w0, tokens, starts0, 1, precision="bf16_points")
    assert abs(res[0][0][0] - ref["losses"][0]) <= 1e-2 * ref["losses"][0]


def test_external_flag_that_nobody_raises_makes_the_wait_run_out(ofa, oracle):
    """ext_sync without a communication side: the graph raises "grads ready" and waits (bounded, 0.2 s here) for "allreduce done",
    which never comes. The kernel must RETURN with ST_EXTERNAL_TIMEOUT; the context can be destroyed and a fresh one trains."""
    ocfg, w0, tokens, cfg = _small_training(ofa, oracle)
    cfg.ext_sync, cfg.grad_bf16, cfg.timeout_s = 1, 1, 0.2
    mk = ofa.Megakernel(cfg)
    mk.load_weights(oracle.flatten(ocfg, w0)); mk.set_tokens(tokens)
    assert len(mk.buckets()) >= 2
    mk.launch(2)
    t0 = time.monotonic()
    with pytest.raises(ofa.OfaError) as e:
        mk.wait(20000)
    assert time.monotonic() - t0 < 10.0
    assert e.value.code == ofa.capi.DEVICE_ABORT and e.value.status.dev_code == 6        # ST_EXTERNAL_TIMEOUT
    name = mk.phases()[e.value.status.phase]["name"]
    assert name.startswith("allreduce done"), name
    assert mk.steps_done == 0
    mk.close()
    cfg.ext_sync, cfg.grad_bf16, cfg.timeout_s = 0, 0, 0.0
    ok = ofa.Megakernel(cfg)
    ok.load_weights(oracle.flatten(ocfg, w0)); ok.set_tokens(tokens)
    ok.run(2, timeout_ms=60000)
    assert np.all(np.isfinite(ok.losses())) and ok.steps_done == 2
    ok.close()


def test_abort_and_wait_timeout(ofa, oracle):
    ocfg, w0, tokens, cfg = _small_training(ofa, oracle)
    mk = ofa.Megakernel(cfg)
    mk.load_weights(oracle.flatten(ocfg, w0)); mk.set_tokens(tokens)
    mk.launch(20000)                                   # several seconds of work
    with pytest.raises(ofa.OfaError) as e:
        mk.wait(1)                                     # 1 ms: still running
    assert e.value.code == ofa.capi.TIMEOUT
    live = mk.live()
    assert mk.abort() == ofa.capi.OK
    t0 = time.monotonic()
    with pytest.raises(ofa.OfaError) as e:
        mk.wait(10000)
    assert time.monotonic() - t0 < 1.5, "the kernel did not return within a second of the abort request"
    assert e.value.code == ofa.capi.DEVICE_ABORT and e.value.status.dev_code == 0        # host-requested: no device-side failure recorded
    assert mk.abort() == ofa.capi.NOT_LAUNCHED
    # the context is still usable: an aborted launch does not count its steps, the next one runs to the end
    done_before = mk.steps_done
    mk.launch(300)
    with pytest.raises(ofa.OfaError) as e:
        mk.wait(0)
    assert e.value.code == ofa.capi.TIMEOUT
    mk.wait(60000)                                     # a later wait on the same launch succeeds
    assert mk.steps_done == done_before + 300
    assert live["steps"] >= 0
    mk.close()
