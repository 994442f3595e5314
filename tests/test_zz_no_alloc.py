"""The allocation-free LayerNorm-backward entry point (ofa_ln_bwd_noalloc) against the scheduler path it mirrors.

Some hosts of this library cannot call cudaMalloc where they need LayerNorm backward: their device memory is owned by
another allocator's pool, or they run next to a resident persistent kernel that a device-wide allocation sync would
stall. For them the entry point keeps its only scratch (the dgamma partials) in a fixed device array. This test drives it
through the C ABI twice in a row - the second call with a smaller batch and the accumulate flag, so stale partials of the
first call would show - and compares with the existing TK_LN_BWD + TK_LN_DG phases (caller-allocated partials), bit for bit
(both run the same device function), and with autograd through F.layer_norm at the gradient tolerances the other GPU tests use. The file name sorts last on purpose: a run that stops at the first failure
has then already executed every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

D = 768


def relmax(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)


def _inputs(ofa, N, seed):
    g = torch.Generator().manual_seed(seed)
    bf = lambda t: t.bfloat16().float()
    x = bf(torch.randn(N, D, generator=g) * 2 + 0.5); gamma = bf(torch.randn(D, generator=g) * 0.2 + 1.0)
    dy = bf(torch.randn(N, D, generator=g)); dres = bf(torch.randn(N, D, generator=g))
    mean = x.mean(1); rstd = torch.rsqrt(x.var(1, unbiased=False) + 1e-5)
    dev = {k: ofa.DeviceBuffer.from_host(v.numpy(), "bf16") for k, v in dict(x=x, gamma=gamma, dy=dy, dres=dres).items()}
    dev["mean"] = ofa.DeviceBuffer.from_host(mean.numpy().astype(np.float32)); dev["rstd"] = ofa.DeviceBuffer.from_host(rstd.numpy().astype(np.float32))
    return dev


def _existing(ofa, dev, N, dg0, accumulate, use_dres):
    K = ofa.capi
    dims = dict(vocab=1024, d_model=D, n_layer=1, n_head=12, ctx_len=N, batch=1)
    dx = ofa.DeviceBuffer((N, D), "bf16"); part = ofa.DeviceBuffer(((N + 15) // 16, D), np.float32); dg = ofa.DeviceBuffer.from_host(dg0)
    ofa.run_phases(K.DTYPE_BF16, dims, [ofa.phase(K.TK_LN_BWD, [dx, part, dev["dy"], dev["x"], dev["mean"], dev["rstd"], dev["gamma"], dev["dres"] if use_dres else None]),
                                       ofa.phase(K.TK_LN_DG, [dg, part], i0=accumulate)])
    return dx.download(), dg.download()


def _noalloc(ofa, dev, N, dg0, accumulate, use_dres):
    lib = ofa.capi.load()
    dx = ofa.DeviceBuffer((N, D), "bf16"); dg = ofa.DeviceBuffer.from_host(dg0)
    rc = lib.ofa_ln_bwd_noalloc(dx.ptr, dg.ptr, dev["dy"].ptr, dev["x"].ptr, dev["mean"].ptr, dev["rstd"].ptr, dev["gamma"].ptr,
                                dev["dres"].ptr if use_dres else None, N, D, accumulate, None)
    assert rc == ofa.capi.OK, lib.ofa_noalloc_last_error().decode()
    return dx.download(), dg.download()


def test_noalloc_ln_backward_matches_scheduler_path_twice_in_a_row(ofa):
    import torch.nn.functional as F
    for call, (N, accumulate, use_dres, seed) in enumerate([(4096, 0, False, 11), (528, 1, True, 12)]):
        dev = _inputs(ofa, N, seed)
        dg0 = np.full(D, 3.0, np.float32)
        dx_ref, dg_ref = _existing(ofa, dev, N, dg0, accumulate, use_dres)
        dx_new, dg_new = _noalloc(ofa, dev, N, dg0, accumulate, use_dres)
        # both paths run the same device function on the same rows in the same order: identical bits, not merely close
        np.testing.assert_array_equal(dx_new, dx_ref, err_msg=f"call {call}: dx")
        np.testing.assert_array_equal(dg_new.view(np.uint32), dg_ref.view(np.uint32), err_msg=f"call {call}: dgamma")
        # and both against autograd through F.layer_norm on the same (bf16-valued) inputs, at the tolerances of the other GPU tests
        x = torch.from_numpy(dev["x"].download()).requires_grad_(); gm = torch.from_numpy(dev["gamma"].download()).requires_grad_()
        F.layer_norm(x, (D,), gm, None, 1e-5).backward(torch.from_numpy(dev["dy"].download()))
        want_dx = x.grad + (torch.from_numpy(dev["dres"].download()) if use_dres else 0)
        want_dg = gm.grad + (torch.from_numpy(dg0) if accumulate else 0)
        assert relmax(dx_new, want_dx.numpy()) <= 5e-2, f"call {call}: dx vs autograd"
        assert relmax(dg_new, want_dg.numpy()) <= 5e-3, f"call {call}: dgamma vs autograd"
        assert np.all(np.isfinite(dx_new)) and np.all(np.isfinite(dg_new))


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch(ofa):
    lib = ofa.capi.load()
    assert lib.ofa_noalloc_max_rows() == 32768
    d = ofa.DeviceBuffer((16,), np.float32)
    rc = lib.ofa_ln_bwd_noalloc(d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, None, lib.ofa_noalloc_max_rows() + 1, D, 0, None)
    assert rc == ofa.capi.BAD_ARGUMENT and b"exceeds" in lib.ofa_noalloc_last_error()
    assert lib.ofa_ln_bwd_noalloc(d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, None, 16, 512, 0, None) == ofa.capi.BAD_ARGUMENT
