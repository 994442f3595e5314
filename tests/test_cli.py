"""The command-line host (csrc/ofa_cli.cpp): the reference program's flags and files over the C ABI
(llm/b200/megakernel/ofa.cu:394-431 flags, :722-763 report and dumps)."""
import importlib
import subprocess

import numpy as np
import pytest


@pytest.fixture(scope="module")
def cli():
    return importlib.import_module("open-flapping-airplanes_b200.build").build_cli()


def test_cli_builds_and_knows_the_reference_flags(cli):
    r = subprocess.run([cli, "--help"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0
    for flag in ("--steps", "--sched-steps", "--split", "--infer-sms", "--doom-sms", "--train-sms", "--data", "--starts", "--init", "--prompt",
                 "--answer-len", "--temp", "--no-opt", "--loss-out", "--text-out", "--dump-w", "--dump-grads"):
        assert flag in r.stdout
    bad = subprocess.run([cli, "--no-such-flag"], capture_output=True, text=True, timeout=60)
    assert bad.returncode == 2 and "unknown" in bad.stderr


@pytest.mark.gpu
def test_cli_run_equals_the_python_host_on_the_same_files(cli, ofa, oracle, tmp_path):
    """Tiny fp32 model, 3 steps from files (init, tokens, starts): the loss log and the dumped weights of the C++ host equal what the
    ctypes host gets from the same library on the same inputs, bit for bit; --no-opt dumps the step-0 gradients."""
    ocfg = oracle.tiny_config(tied=False)
    w0 = oracle.flatten(ocfg, oracle.init_weights(ocfg))
    ntok = 1 << 14
    tokens = oracle.synthetic_tokens(ocfg.V, ntok, 0)
    starts = oracle.batch_starts(ocfg, ntok, 3).astype(np.uint32)
    ofa.files.write_flat_f32(tmp_path / "init.f32", w0)
    np.ascontiguousarray(tokens, dtype=np.uint32).tofile(tmp_path / "tok.u32")
    ofa.files.write_starts_u32(tmp_path / "starts.u32", starts)
    common = [cli, "--preset", "tiny", "--init", str(tmp_path / "init.f32"), "--data", str(tmp_path / "tok.u32"), "--starts", str(tmp_path / "starts.u32")]
    r = subprocess.run(common + ["--steps", "3", "--loss-out", str(tmp_path / "loss.txt"), "--dump-w", str(tmp_path / "w.f32")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "loss: step0" in r.stdout and "busy time by phase kind" in r.stdout
    cfg = ofa.default_config("tiny")
    mk = ofa.Megakernel(cfg)
    mk.load_weights(w0); mk.set_tokens(tokens); mk.set_starts(starts)
    mk.run(3)
    steps, losses = ofa.files.read_loss_log(tmp_path / "loss.txt")
    np.testing.assert_array_equal(steps, [0, 1, 2])
    np.testing.assert_allclose(losses, mk.losses(), atol=5e-7)                 # six decimals in the log
    np.testing.assert_array_equal(ofa.files.read_flat_f32(tmp_path / "w.f32", mk.num_params), mk.read_weights())
    mk.close()
    g = subprocess.run(common + ["--steps", "1", "--no-opt", "--dump-grads", str(tmp_path / "g.f32")], capture_output=True, text=True, timeout=300)
    assert g.returncode == 0, g.stdout + g.stderr
    cfg = ofa.default_config("tiny"); cfg.mode = 2
    mk = ofa.Megakernel(cfg)
    mk.load_weights(w0); mk.set_tokens(tokens); mk.set_starts(starts)
    mk.run(1)
    np.testing.assert_array_equal(ofa.files.read_flat_f32(tmp_path / "g.f32", mk.num_params), mk.read_grads())
    mk.close()
