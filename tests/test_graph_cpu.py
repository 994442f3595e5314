"""Host logic without a GPU: planning contexts (device < 0) build the flat layout, the gradient buckets and the training /
serving phase graphs exactly as a real context does; these tests check their structure."""
import numpy as np
import pytest


def plan(ofa, preset, **kw):
    cfg = ofa.default_config(preset)
    cfg.device = -1
    for k, v in kw.items():
        setattr(cfg, k, v)
    return ofa.Megakernel(cfg)


@pytest.mark.parametrize("preset,kw", [("gpt_s", {}), ("gpt_s", dict(tied_head=1)), ("gpt_s", dict(mode=1)), ("gpt_s", dict(mode=2)),
                                       ("gpt_s", dict(dp_world=8, grad_bf16=1, ext_sync=1)), ("gpt_s", dict(adam_interleave=1, head_dx_splitk=1)), ("gpt_s", dict(adam_interleave=12)), ("tiny", {}), ("tiny", dict(tied_head=1)), ("tiny", dict(mode=2))])
def test_training_graph_is_topologically_ordered(ofa, preset, kw):
    mk = plan(ofa, preset, **kw)
    ph = mk.phases()
    names = [p["name"] for p in ph]
    assert len(set(names)) == len(names) and names[0] == "data" and names[-1] == "step barrier"
    reached_from_prev_step = 0
    for i, p in enumerate(ph):
        assert p["ntasks"] > 0
        deps = mk.phase_deps(i)
        for d, delta in deps:
            assert 0 <= d < len(ph) and delta in (0, -1)
            if delta == 0:
                assert d < i, f"{p['name']} depends on later phase {names[d]} of the same step"   # => every dependency is a lower ticket
            else:
                reached_from_prev_step += 1
        if i > 0 and p["name"] != "data":
            assert any(delta == 0 for _, delta in deps), f"{p['name']} has no producer in its own step"
    assert reached_from_prev_step >= 1                     # steps are chained
    mode = kw.get("mode", 0)
    if mode == 0:
        L = mk.cfg.n_layer
        for l in range(L):                                 # next step's forward of layer l waits for this step's AdamW of layer l
            i = names.index(f"L{l} ln1")
            assert (names.index(f"adamw L{l}"), -1) in mk.phase_deps(i)
        head = "adamw wte" if kw.get("tied_head") else "adamw head"
        assert (names.index(head), -1) in mk.phase_deps(names.index("logits"))
        assert (names.index("head dW"), -1) in mk.phase_deps(names.index("lnf"))
        seen, todo = set(), [names.index(head)]            # same-step ancestors of the head's AdamW (direct, or through an all-reduce gate)
        while todo:
            for d, delta in mk.phase_deps(todo.pop()):
                if delta == 0 and d not in seen:
                    seen.add(d); todo.append(d)
        assert names.index("head dX") in seen              # the head may not be updated while dX still reads it
    mk.close()


def test_gpt_s_task_counts_and_layout(ofa):
    mk = plan(ofa, "gpt_s", adam_interleave=1, head_dx_splitk=1)
    assert mk.num_params == 163007232
    ph = {p["name"]: p for p in mk.phases()}
    assert ph["embed"]["ntasks"] == 256 and ph["L0 ln1"]["ntasks"] == 256 and ph["cross-entropy"]["ntasks"] == 1024
    assert ph["L3 attn"]["ntasks"] == 4 * 12 * 8 and ph["L3 attn bwd"]["ntasks"] == 2 * 4 * 12 * 8
    assert (32 * 18) % ph["L0 qkv"]["ntasks"] == 0 and ph["L0 dWo"]["ntasks"] == 36 and ph["embed bwd wte"]["ntasks"] == 393   # GEMM tasks are strips of whole tiles
    # head dX is cut along K into partial products that a reduce phase sums; its name stays the dependency target
    names = list(ph)
    parts = [n for n in names if n.startswith("head dX k")]
    assert len(parts) in (2, 3, 4) and all(names.index(p) < names.index("head dX") for p in parts)
    # a layer's AdamW sits inside the backward pass, below the layer it updates
    assert names.index("adamw L11") < names.index("L10 dln2") and names.index("adamw L0") > names.index("L0 ln1 bwd")
    assert ph["adamw L5"]["ntasks"] == 109 and ph["adamw head"]["ntasks"] == 590 and ph["adamw wpe"]["ntasks"] == 12
    assert 32 * 393 // 8 <= ph["logits"]["ntasks"] <= 32 * 393
    order = ["wte", "wpe", "lm_head"] + [f"L{l}.{t}" for l in range(12) for t in ("g1", "Wqkv", "Wo", "g2", "Wup", "Wdn")] + ["gf"]
    pos = 0
    for n in order:
        off, cnt = mk.param_span(n)
        assert off == pos and off % 64 == 0
        pos += cnt
    assert pos == mk.num_params
    mk.close()


def test_serving_graph_is_a_chain(ofa):
    mk = plan(ofa, "gpt_s", use_decode=1, infer_sms=24, reserved_sms=8, train_sms=116)
    n = 3 * 12 + 2
    for i in range(n):
        deps = mk.phase_deps(i, job=1)
        assert ((i - 1, 0) in deps) if i > 0 else deps == [(n - 1, -1)]
    mk.close()


@pytest.mark.parametrize("preset,kw", [("gpt_s", dict(dp_world=8, grad_bf16=1, ext_sync=1)), ("gpt_s", dict(dp_world=2, grad_bf16=1, ext_sync=1, tied_head=1)),
                                       ("tiny", dict(dp_world=2, ext_sync=1, bucket_bytes=65536))])
def test_gradient_buckets_partition_the_parameters(ofa, preset, kw):
    mk = plan(ofa, preset, **kw)
    b = mk.buckets()
    assert len(b) >= 3 and ofa.dp.buckets_partition_params(b, mk.num_params)
    names = [p["name"] for p in mk.phases()]
    for i in range(len(b)):
        r, w = names.index(f"grads ready {i}"), names.index(f"allreduce done {i}")
        assert mk.phase_deps(w) == [(r, 0)]
    # every AdamW phase is gated by exactly one all-reduce
    for i, nm in enumerate(names):
        if nm.startswith("adamw"):
            deps = mk.phase_deps(i)
            assert len(deps) == 1 and names[deps[0][0]].startswith("allreduce done")
    mk.close()


def test_planning_context_cannot_touch_a_device(ofa):
    mk = plan(ofa, "tiny")
    with pytest.raises(ofa.OfaError):
        mk.launch(1)
    with pytest.raises(ofa.OfaError):
        mk.load_weights(np.zeros(mk.num_params, np.float32))
    mk.close()


def test_trickled_adamw_covers_every_parameter_once(ofa):
    """cfg.adam_interleave = n >= 2 cuts the optimizer phases into chunks spread through the backward pass: the chunks of a group
    must add up to the group's tasks, and the group's usual name must wait for all of them."""
    base = plan(ofa, "gpt_s"); tr = plan(ofa, "gpt_s", adam_interleave=12)
    pb, pt = base.phases(), tr.phases()
    K_ADAMW = 13
    count = lambda ph: sum(p["ntasks"] for p in ph if p["kind"] == K_ADAMW)
    assert count(pb) == count(pt)
    names = [p["name"] for p in pt]
    for group in ["adamw head"] + [f"adamw L{l}" for l in range(1, 12)]:
        parts = [i for i, n in enumerate(names) if n.startswith(group + " .")]
        assert len(parts) >= 2
        whole = next(p["ntasks"] for p in pb if p["name"] == group)
        assert sum(pt[i]["ntasks"] for i in parts) == whole
        deps = {d for d, delta in tr.phase_deps(names.index(group)) if delta == 0}
        assert deps == set(parts)                                          # the join phase waits for every chunk
        ready = names.index(group + " ready")
        for i in parts:
            assert tr.phase_deps(i) == [(ready, 0)]
    assert "adamw L0 .0" not in names and "adamw L0" in names             # nothing left to spread the last group into
    base.close(); tr.close()


def test_row_block_dependencies_follow_the_layer_chain(ofa):
    """On the tensor-core path the layer chain waits per 128-token row block: LayerNorm -> GEMM -> attention -> GEMM ... Every such
    edge must join two phases whose tasks map to row blocks, stay inside one step, and the producers must have a whole number of
    tasks per row block; reductions over all tokens (weight-gradient GEMMs, dgamma, embedding backward, AdamW) keep the phase grain.
    The fp32 preset (row counts that are not multiples of 128) keeps the phase grain everywhere."""
    mk = plan(ofa, "gpt_s")
    ph = mk.phases(); names = [p["name"] for p in ph]
    nrb = 4 * 1024 // 128
    fine = {}
    for i, p in enumerate(ph):
        rb_map, grain = mk.phase_dep_grain(i)
        deps = mk.phase_deps(i)
        for (d, delta), g in zip(deps, grain):
            if g:
                assert delta == 0 and rb_map != 0 and mk.phase_dep_grain(d)[0] != 0
                assert ph[d]["ntasks"] % nrb == 0, names[d]
                fine[(names[d], p["name"])] = True
    for l in (0, 5, 11):
        for a, b in [("ln1", "qkv"), ("qkv", "attn"), ("attn", "wo+res"), ("wo+res", "ln2"), ("ln2", "up+gelu"), ("up+gelu", "down+res"),
                     ("dpre", "dln2"), ("dln2", "ln2 bwd"), ("ln2 bwd", "dO"), ("dO", "attn bwd"), ("attn bwd", "dln1"), ("dln1", "ln1 bwd")]:
            assert (f"L{l} {a}", f"L{l} {b}") in fine, (l, a, b)
    for a, b in [("embed", "L0 ln1"), ("L3 down+res", "L4 ln1"), ("L11 down+res", "lnf"), ("lnf", "logits"), ("logits", "cross-entropy"),
                 ("cross-entropy", "head dX"), ("head dX", "lnf bwd"), ("lnf bwd", "L11 dpre"), ("L4 ln1 bwd", "L3 dpre")]:
        assert (a, b) in fine, (a, b)
    coarse = lambda name: all(g == 0 for g in mk.phase_dep_grain(names.index(name))[1])
    for name in ["head dW", "L7 dWdown", "L7 dWup", "L7 dWo", "L7 dWqkv", "L7 dgamma1", "L7 dgamma2", "embed bwd wte", "embed bwd wpe", "adamw L7", "adamw head", "loss mean", "step barrier"]:
        assert coarse(name), name
    mk.close()
    tiny = plan(ofa, "tiny")
    assert all(not any(tiny.phase_dep_grain(i)[1]) for i in range(len(tiny.phases())))
    tiny.close()
