"""File formats shared with the reference's megakernel program (llm/b200/megakernel/ofa.cu:489-528, 730, 753-763) and the
checkpoint directory built from them. No GPU needed."""
import importlib

import numpy as np
import pytest


@pytest.fixture(scope="module")
def files():
    return importlib.import_module("open-flapping-airplanes_b200.files")


def test_flat_f32_round_trip_and_size_check(files, tmp_path):
    a = np.random.default_rng(0).standard_normal(1000).astype(np.float32)
    p = tmp_path / "w.f32"
    files.write_flat_f32(p, a)
    assert p.stat().st_size == 4000                                   # raw fp32, no header (ofa.cu:762-763 fwrite of NP floats)
    np.testing.assert_array_equal(files.read_flat_f32(p, expect=1000), a)
    with pytest.raises(ValueError):
        files.read_flat_f32(p, expect=999)


def test_loss_log_is_the_reference_text_format(files, tmp_path):
    p = tmp_path / "loss.txt"
    files.write_loss_log(p, [10.9648123, 10.5, 2.15749999])
    assert p.read_text() == "0 10.964812\n1 10.500000\n2 2.157500\n"   # fprintf(f, "%d %.6f\n", s, loss[s]) (ofa.cu:730)
    steps, losses = files.read_loss_log(p)
    np.testing.assert_array_equal(steps, [0, 1, 2])
    np.testing.assert_allclose(losses, [10.964812, 10.5, 2.1575], atol=1e-6)


def test_tokens_and_starts(files, tmp_path):
    tok = np.arange(50, dtype=np.uint32); st = np.arange(12, dtype=np.uint32).reshape(3, 4)
    tok.tofile(tmp_path / "t.u32"); files.write_starts_u32(tmp_path / "s.u32", st)
    np.testing.assert_array_equal(files.read_tokens_u32(tmp_path / "t.u32"), tok)
    np.testing.assert_array_equal(files.read_starts_u32(tmp_path / "s.u32", 4), st)
    with pytest.raises(ValueError):
        files.read_starts_u32(tmp_path / "s.u32", 5)
    files.write_token_ids(tmp_path / "o.txt", [3, 1, 4])
    assert (tmp_path / "o.txt").read_text() == "3 1 4 "               # "%d " per token (ofa.cu:754)


def test_flat_order_of_a_tied_model_is_the_reference_init_file_order(oracle):
    """make_init_flat.py:7-13 writes wte, wpe, then per layer gamma1, Wqkv, Wo, gamma2, Wup, Wdown, then gamma_f: with a tied head the
    library's flat vector is that file."""
    ofa = importlib.import_module("open-flapping-airplanes_b200")
    ocfg = oracle.tiny_config(tied=True)
    w = oracle.init_weights(ocfg)
    flat = oracle.flatten(ocfg, w)
    order = ["wte", "wpe"] + [f"L{l:02d}_{n}" for l in range(ocfg.L) for n in ("gamma1", "Wqkv", "Wo", "gamma2", "Wup", "Wdown")] + ["gamma_f"]
    ref = np.concatenate([np.asarray(w[k], dtype=np.float32).reshape(-1) for k in order])
    np.testing.assert_array_equal(flat, ref)
    np.testing.assert_array_equal(ofa.flat_from_named(w, ocfg.L, True), ref)
