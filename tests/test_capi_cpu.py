"""CPU-side checks of the boundary: the shared library builds for sm_100a, loads without a GPU, exports every symbol the
header declares, and fails loudly (no fallback) when there is no device. No compute calls here."""
import ctypes as C
import os
import re

import numpy as np
import pytest


def _declared_symbols(root):
    src = open(os.path.join(root, "include", "ofa_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(ofa_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol(ofa):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib = ofa.capi.load()
    names = _declared_symbols(root)
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ofa_b200.h but not exported"
        assert n in ofa.capi.PROTOTYPES, f"{n} has no ctypes prototype"
    assert sorted(ofa.capi.PROTOTYPES) == names


def test_presets(ofa):
    t = ofa.default_config("tiny")
    assert (t.vocab, t.d_model, t.n_layer, t.n_head, t.ctx_len, t.batch) == (65, 64, 2, 4, 64, 16)
    assert t.dtype == ofa.capi.DTYPE_F32 and t.constant_lr == 1 and abs(t.lr_max - 3e-4) < 1e-9 and t.n_prompt == 8 and t.answer_len == 64
    s = ofa.default_config("gpt_s")
    assert (s.vocab, s.d_model, s.n_layer, s.n_head, s.ctx_len, s.batch) == (50304, 768, 12, 12, 1024, 4)
    assert s.dtype == ofa.capi.DTYPE_BF16 and s.warmup == 100 and s.sched_steps == 4000 and s.tied_head == 0
    assert abs(s.beta2 - 0.95) < 1e-7 and abs(s.weight_decay - 0.1) < 1e-7 and s.answer_len == 256 and s.n_prompt == 6
    with pytest.raises(ofa.OfaError):
        ofa.default_config("nope")


def test_no_gpu_means_error_not_fallback(ofa):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(ofa.OfaError) as e:
        ofa.Megakernel(ofa.default_config("tiny"))
    assert e.value.code == ofa.capi.CUDA_ERROR
    with pytest.raises(ofa.OfaError):
        ofa.DeviceBuffer((16,), np.float32)


def test_bad_config_is_rejected_before_touching_the_device(ofa):
    cfg = ofa.default_config("gpt_s")
    cfg.d_model = 512
    with pytest.raises(ofa.OfaError) as e:
        ofa.Megakernel(cfg)
    assert e.value.code == ofa.capi.BAD_CONFIG
    cfg = ofa.default_config("tiny")
    cfg.ctx_len = 512
    with pytest.raises(ofa.OfaError) as e:
        ofa.Megakernel(cfg)
    assert e.value.code == ofa.capi.BAD_CONFIG


def test_bf16_bit_conversion_matches_torch(ofa):
    import torch
    rng = np.random.default_rng(0)
    a = np.concatenate([rng.standard_normal(10000).astype(np.float32) * 10.0 ** rng.integers(-20, 20, 10000), np.array([0.0, -0.0, np.inf, -np.inf, 1.0, 3.3895314e38], np.float32)])
    ours = ofa.to_bf16_bits(a)
    ref = torch.from_numpy(a).bfloat16().view(torch.int16).numpy().view(np.uint16)
    np.testing.assert_array_equal(ours, ref)
    np.testing.assert_array_equal(ofa.from_bf16_bits(ours), torch.from_numpy(a).bfloat16().float().numpy())


def test_flat_layout_order(ofa, oracle):
    cfg = oracle.tiny_config(tied=False)
    w = oracle.init_weights(cfg)
    flat = ofa.flat_from_named({k: v.numpy() for k, v in w.items()}, cfg.L, tied=False)
    np.testing.assert_array_equal(flat, oracle.flatten(cfg, w))
    assert flat.size == 2 * 65 * 64 + 64 * 64 + 2 * (2 * 64 + 12 * 64 * 64) + 64


def test_oversize_shared_memory_needs_are_refused_on_the_host(ofa):
    """Tasks whose shared-memory need grows with the batch or the context are checked against the block's task area before
    anything is built: a planning context (device < 0) is enough to see the refusal, nothing runs on a GPU."""
    ok = ofa.default_config("gpt_s"); ok.device = -1
    ofa.Megakernel(ok).close()
    big = ofa.default_config("gpt_s"); big.device, big.batch = -1, 32                 # 32,768 tokens: the embedding-backward token list
    with pytest.raises(ofa.OfaError) as e:
        ofa.Megakernel(big)
    assert e.value.code == ofa.capi.BAD_CONFIG and "embedding-backward" in str(e.value)
    fwd = ofa.default_config("gpt_s"); fwd.device, fwd.batch, fwd.mode = -1, 32, ofa.capi.MODE_FORWARD
    ofa.Megakernel(fwd).close()                                                        # no backward pass, no such task
    dec = ofa.default_config("gpt_s"); dec.device, dec.ctx_len, dec.batch, dec.use_decode = -1, 2048, 2, 1
    with pytest.raises(ofa.OfaError) as e:
        ofa.Megakernel(dec)
    assert e.value.code == ofa.capi.BAD_CONFIG and "serving tasks" in str(e.value)
    dec.use_decode = 0
    ofa.Megakernel(dec).close()                                                        # the same context without the serving job fits
    # task level: refused before the device is looked at
    K = ofa.capi
    dims = dict(vocab=1024, d_model=768, n_layer=1, n_head=12, ctx_len=1024, batch=32)
    with pytest.raises(ofa.OfaError) as e:
        ofa.run_phases(K.DTYPE_BF16, dims, [ofa.phase(K.TK_EMB_WTE, [1 << 20, 1 << 21, 1 << 22])])
    assert e.value.code == K.BAD_CONFIG
