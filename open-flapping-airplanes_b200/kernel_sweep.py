#!/usr/bin/env python
"""Standalone kernel sweep on one B200: every task kind of the megakernel run alone as a one-kind job on
the persistent scheduler, at the GPT-S shapes, timed with CUDA events and reported against the measured roofline.

  python open-flapping-airplanes_b200/kernel_sweep.py [--only NAME[,NAME..]] [--repeats R] [--list]

Each case rotates over enough independent buffer sets to exceed the 126 MB L2 between reuses (so DRAM numbers mean something),
runs `repeats` passes over all sets in ONE launch, and prints one JSON line: time per pass, TFLOP/s or GB/s from the
algorithmic work, and the fraction of the measured peak (MEASURED_PEAKS.json when present, else the pool's fallback figures).
Inputs are N(0, 0.02) bf16 from a seeded generator. This is also the command the ncu captures under profiles/ were made with
(`--only <case> --repeats 1`).
"""
import argparse
import importlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

M = 4096
D, FF, V, H, T, B = 768, 3072, 50304, 12, 1024, 4
L2_BYTES = 126 << 20
DIMS = dict(vocab=V, d_model=D, n_layer=1, n_head=H, ctx_len=T, batch=B)

# name: (layout, epi, M, N, K)   layouts 0 NN, 1 NT, 2 TN; epilogues 0 store, 1 +res, 2 gelu, 3 dgelu, 4 f32
GEMMS = {
    "gemm_qkv": (0, 0, M, 3 * D, D), "gemm_proj": (0, 1, M, D, D), "gemm_up_gelu": (0, 2, M, FF, D), "gemm_down": (0, 1, M, D, FF),
    "gemm_logits": (1, 0, M, V, D), "gemm_dpre_dgelu": (1, 3, M, FF, D), "gemm_dln2": (1, 0, M, D, FF), "gemm_dO": (1, 0, M, D, D),
    "gemm_dln1": (1, 0, M, D, 3 * D), "gemm_head_dX": (0, 0, M, D, V), "gemm_dWqkv": (2, 4, D, 3 * D, M), "gemm_dWo": (2, 4, D, D, M),
    "gemm_dWup": (2, 4, D, FF, M), "gemm_dWdown": (2, 4, FF, D, M), "gemm_head_dW": (2, 4, V, D, M),
}
OTHERS = ["attn_fwd", "attn_bwd", "adamw", "cross_entropy", "ln_fwd", "ln_bwd", "embed_bwd_wte", "decode_148sm", "decode_24sm", "decode_attn", "sched_empty", "head_fused"]


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))); return p["hbm_gbs"], p["bf16_tflops"], "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def rand_bf16(ofa, rng, shape, scale=0.02):
    return ofa.DeviceBuffer.from_host(rng.standard_normal(shape, dtype=np.float32) * scale, "bf16")


def run_gemm(ofa, name, repeats, nsub):
    K = ofa.capi
    layout, epi, Mm, Nn, Kk = GEMMS[name]
    if name == "gemm_head_dW" and nsub == 0:
        nsub = 4001                      # 128 x 256 tiles, one per task, tasks ordered along N first: as the training graph runs this one shape
    rng = np.random.default_rng(0)
    ashape = (Mm, Kk) if layout != 2 else (Kk, Mm)
    bshape = (Kk, Nn) if layout != 1 else (Nn, Kk)
    out_b = 4 if epi == 4 else 2
    bytes_set = 2 * (Mm * Kk + Kk * Nn) + out_b * Mm * Nn + (2 * Mm * Nn if epi in (1, 2, 3) else 0)
    nsets = max(1, min(16, -(-2 * L2_BYTES // bytes_set)))
    if REF_METHOD:
        nsets = 1
    keep, phases = [], []
    for _ in range(nsets):
        A = rand_bf16(ofa, rng, ashape); Bm = rand_bf16(ofa, rng, bshape)
        C = ofa.DeviceBuffer((Mm, Nn), np.float32 if epi == 4 else "bf16")
        aux = rand_bf16(ofa, rng, (Mm, Nn), 1.0) if epi in (1, 3) else (ofa.DeviceBuffer((Mm, Nn), "bf16") if epi == 2 else None)
        keep += [A, Bm, C, aux]
        phases.append(ofa.gemm_phase(layout, epi, Mm, Nn, Kk, A, ashape[1], Bm, bshape[1], C, Nn, aux, Nn if aux is not None else 0, nsub=nsub))
    flop = 2.0 * Mm * Nn * Kk
    if REF_METHOD:      # the reference test's method (llm/gemm/test_gemm.cu:179-190,284): same operands, 20 (5 for the largest) back-to-back passes, best of 6
        it = 5 if flop > 5e11 else 20
        ofa.run_phases(K.DTYPE_BF16, DIMS, phases, repeats=2)
        ms = min(ofa.run_phases(K.DTYPE_BF16, DIMS, phases, repeats=it) / it for _ in range(6))
    else:
        ms = ofa.run_phases(K.DTYPE_BF16, DIMS, phases, repeats=repeats) / (repeats * nsets)
    return {"kernel": name, "shape": [Mm, Nn, Kk], "ms": ms, "tflops": flop / ms / 1e9, "bound": "tensor", "algorithmic_bytes": bytes_set, "buffer_sets": nsets,
            "timing": "same operands, best of 6 x back-to-back passes in one launch" if REF_METHOD else "operands rotated beyond L2"}


REF_METHOD = False   # --ref-method: time GEMMs the way the reference's test program does (warm operands, best of several)


def run_attn(ofa, which, repeats):
    K = ofa.capi
    rng = np.random.default_rng(1)
    N = B * T
    nsets = 6
    keep, phases = [], []
    for _ in range(nsets):
        qkv = rand_bf16(ofa, rng, (N, 3 * D), 1.0); dO = rand_bf16(ofa, rng, (N, D), 1.0)
        o = ofa.DeviceBuffer((N, D), "bf16"); lse = ofa.DeviceBuffer((B, H, T), np.float32); Dr = ofa.DeviceBuffer((B, H, T), np.float32); dqkv = ofa.DeviceBuffer((N, 3 * D), "bf16")
        keep += [qkv, dO, o, lse, Dr, dqkv]
        if which == "attn_fwd":
            phases.append(ofa.phase(K.TK_ATT_FWD, [qkv, o, lse]))
        else:
            ofa.run_phases(K.DTYPE_BF16, DIMS, [ofa.phase(K.TK_ATT_FWD, [qkv, o, lse])])
            phases += [ofa.phase(K.TK_ATT_PREP, [o, dO, Dr]), ofa.phase(K.TK_ATT_BWD, [qkv, dO, lse, Dr, dqkv, o])]
    ms = ofa.run_phases(K.DTYPE_BF16, DIMS, phases, repeats=repeats) / (repeats * nsets)
    fwd_flop = 4.0 * B * H * T * T * 64 / 2
    flop = fwd_flop if which == "attn_fwd" else 2.5 * fwd_flop
    return {"kernel": which, "shape": [B, H, T, 64], "ms": ms, "tflops": flop / ms / 1e9, "bound": "tensor", "buffer_sets": nsets}


def run_adamw(ofa, repeats):
    K = ofa.capi
    n = 163007232
    rng = np.random.default_rng(2)
    W = ofa.DeviceBuffer.from_host(rng.standard_normal(n, dtype=np.float32) * 0.02); G = ofa.DeviceBuffer.from_host(rng.standard_normal(n, dtype=np.float32) * 0.01)
    Mb = ofa.DeviceBuffer((n,), np.float32); Vb = ofa.DeviceBuffer((n,), np.float32); Wa = ofa.DeviceBuffer((n,), "bf16"); nd = ofa.DeviceBuffer.from_host(np.array([[0, 768]], np.int32))
    ms = ofa.run_phases(K.DTYPE_BF16, DIMS, [ofa.phase(K.TK_ADAMW, [W, G, Mb, Vb, Wa, nd], n=n, i0=1)], repeats=repeats, adam=[6e-4, 0.9, 0.95, 1e-8, 0.1, 1.0]) / repeats
    by = 30.0 * n
    return {"kernel": "adamw", "shape": [n], "ms": ms, "gbs": by / ms / 1e6, "bound": "hbm", "algorithmic_bytes": by, "bytes_per_param": 30}


def run_ce(ofa, repeats):
    K = ofa.capi
    rng = np.random.default_rng(3)
    N = B * T
    lg = ofa.DeviceBuffer.from_host(rng.standard_normal((N, V), dtype=np.float32) * 0.5, "bf16")
    tg = ofa.DeviceBuffer.from_host(rng.integers(0, V, N).astype(np.int32)); loss = ofa.DeviceBuffer((N,), np.float32)
    ms = ofa.run_phases(K.DTYPE_BF16, DIMS, [ofa.phase(K.TK_CE, [lg, tg, loss])], repeats=repeats) / repeats
    by = 2.0 * N * V * 2
    return {"kernel": "cross_entropy", "shape": [N, V], "ms": ms, "gbs": by / ms / 1e6, "bound": "hbm", "algorithmic_bytes": by}


def run_head_fused(ofa, repeats):
    """The fused LM head: the logits GEMM whose epilogue leaves per-tile softmax partials, then cross-entropy streaming the logits
    once. Two records: the GEMM (tensor bound) and the cross-entropy task (HBM bound: reads and rewrites the bf16 logits). The
    cross-entropy launch is timed on its own, after one launch has produced logits and partials; repeats work in place on what
    the pass before left (the arithmetic is the same, the values are not meaningful)."""
    K = ofa.capi
    rng = np.random.default_rng(7)
    N = B * T
    x = rand_bf16(ofa, rng, (N, D), 1.0); W = rand_bf16(ofa, rng, (V, D), 0.05)
    lg = ofa.DeviceBuffer((N, V), "bf16"); part = ofa.DeviceBuffer((N, V // 128, 2), np.float32)
    tg = ofa.DeviceBuffer.from_host(rng.integers(0, V, N).astype(np.int32)); loss = ofa.DeviceBuffer((N,), np.float32)
    ph = ofa.gemm_phase(1, K.EPI_LSE, N, V, D, x, D, W, D, lg, V)
    ph.p[4] = part.ptr
    ofa.run_phases(K.DTYPE_BF16, DIMS, [ph])
    ms_g = ofa.run_phases(K.DTYPE_BF16, DIMS, [ph], repeats=repeats) / repeats
    ms_c = ofa.run_phases(K.DTYPE_BF16, DIMS, [ofa.phase(K.TK_CE, [lg, tg, loss, part])], repeats=repeats) / repeats
    flop = 2.0 * N * V * D
    by = 2.0 * N * V * 2
    return [{"kernel": "gemm_logits_lse", "shape": [N, V, D], "ms": ms_g, "tflops": flop / ms_g / 1e9, "bound": "tensor"},
            {"kernel": "cross_entropy_stream", "shape": [N, V], "ms": ms_c, "gbs": by / ms_c / 1e6, "bound": "hbm", "algorithmic_bytes": by}]


def run_ln(ofa, which, repeats):
    K = ofa.capi
    rng = np.random.default_rng(4)
    N = B * T
    nsets = 24
    keep, phases = [], []
    gamma = rand_bf16(ofa, rng, (D,), 1.0)
    for _ in range(nsets):
        x = rand_bf16(ofa, rng, (N, D), 1.0); y = ofa.DeviceBuffer((N, D), "bf16"); mean = ofa.DeviceBuffer((N,), np.float32); rstd = ofa.DeviceBuffer((N,), np.float32)
        keep += [x, y, mean, rstd]
        if which == "ln_fwd":
            phases.append(ofa.phase(K.TK_LN_FWD, [y, mean, rstd, x, gamma]))
        else:
            dy = rand_bf16(ofa, rng, (N, D), 1.0); dx = ofa.DeviceBuffer((N, D), "bf16"); part = ofa.DeviceBuffer((N // 16, D), np.float32)
            keep += [dy, dx, part]
            ofa.run_phases(K.DTYPE_BF16, DIMS, [ofa.phase(K.TK_LN_FWD, [y, mean, rstd, x, gamma])])
            phases.append(ofa.phase(K.TK_LN_BWD, [dx, part, dy, x, mean, rstd, gamma, None]))
    ms = ofa.run_phases(K.DTYPE_BF16, DIMS, phases, repeats=repeats) / (repeats * nsets)
    by = (2.0 if which == "ln_fwd" else 3.0) * N * D * 2
    return {"kernel": which, "shape": [N, D], "ms": ms, "gbs": by / ms / 1e6, "bound": "hbm", "algorithmic_bytes": by, "buffer_sets": nsets}


def run_embed_bwd(ofa, repeats):
    K = ofa.capi
    rng = np.random.default_rng(5)
    N = B * T
    tok = ofa.DeviceBuffer.from_host(rng.integers(0, V, N).astype(np.int32)); dx = rand_bf16(ofa, rng, (N, D), 1.0); dw = ofa.DeviceBuffer((V, D), np.float32)
    ms = ofa.run_phases(K.DTYPE_BF16, DIMS, [ofa.phase(K.TK_EMB_WTE, [dw, dx, tok])], repeats=repeats) / repeats
    by = V * D * 4.0 + N * D * 2.0
    return {"kernel": "embed_bwd_wte", "shape": [V, D, N], "ms": ms, "gbs": by / ms / 1e6, "bound": "hbm", "algorithmic_bytes": by}


def run_decode(ofa, sms, ntok):
    cfg = ofa.default_config("gpt_s")
    cfg.mode, cfg.use_decode, cfg.infer_sms, cfg.reserved_sms = ofa.capi.MODE_DECODE_ONLY, 1, sms, 0
    for i, t in enumerate(np.random.default_rng(1234).integers(0, V, 6)):
        cfg.prompt[i] = int(t)
    cfg.n_prompt, cfg.answer_len = 6, 256
    mk = ofa.Megakernel(cfg)
    rng = np.random.default_rng(6)
    mk.load_weights(rng.standard_normal(mk.num_params, dtype=np.float32) * np.float32(0.02))
    mk.run(64)
    ms = mk.run(ntok)
    if os.environ.get("OFA_SWEEP_VERBOSE"):
        bb = mk.block_busy_ns()[:, 1]
        act = bb[bb > 0]
        smid, role = mk.block_info()
        print("  blocks per role (1 serve, 2 reserved, 3 train, 4 idle):", {int(r): int((role == r).sum()) for r in np.unique(role)}, file=sys.stderr)
        print("  serve blocks: ids", np.nonzero(role == 1)[0].tolist(), "smids", smid[role == 1].tolist(), file=sys.stderr)
        cnt = np.bincount(smid, minlength=160)
        print("  smids with 3 blocks:", np.nonzero(cnt == 3)[0].tolist(), file=sys.stderr)
        print("  smid of blocks 272..295:", smid[272:].tolist(), "roles", role[272:].tolist(), file=sys.stderr)
        print("  smid of blocks 148..171:", smid[148:172].tolist(), file=sys.stderr)
        print("  smid of blocks 0..23:", smid[0:24].tolist(), file=sys.stderr)
        print("  blocks per smid histogram:", np.bincount(np.bincount(smid, minlength=160)).tolist(), " max smid", int(smid.max()), file=sys.stderr)
        print(f"  serving blocks that ran tasks: {act.size}, mean busy {act.mean() / 1e6:.2f} ms of {ms:.2f} ms, min {act.min() / 1e6:.2f} max {act.max() / 1e6:.2f}", file=sys.stderr)
        tr = mk.decode_trace().astype(np.int64)
        print("  qkv task stages (us): issue+prefetch %.2f, LN prologue %.2f, gemv %.2f, store %.2f | scheduler view: start->task %.2f, task end->signal %.2f" % (
            (tr[1] - tr[0]) / 1e3, (tr[2] - tr[1]) / 1e3, (tr[3] - tr[2]) / 1e3, (tr[4] - tr[3]) / 1e3, (tr[0] - tr[16]) / 1e3, (tr[17] - tr[4]) / 1e3), file=sys.stderr)
        print("  up+down task stages (us): issue+prefetch %.2f, LN prologue %.2f, up gemv %.2f, gelu+down %.2f | start->task %.2f, end->signal %.2f" % (
            (tr[9] - tr[8]) / 1e3, (tr[10] - tr[9]) / 1e3, (tr[11] - tr[10]) / 1e3, (tr[12] - tr[11]) / 1e3, (tr[8] - tr[18]) / 1e3, (tr[19] - tr[12]) / 1e3), file=sys.stderr)
        for p in mk.decode_phases()[:3] + mk.decode_phases()[-2:]:
            print(f"  {p['name']:20s} tasks {p['ntasks']:4d}  mean task {p['busy_ns'] / 1e3 / max(1, p['ntasks']) / ntok:7.2f} us", file=sys.stderr)
    mk.close()
    by = 2.0 * (12 * 12 * D * D + V * D) + 36864.0 * 131      # weights + KV at the mean position of a 261-step answer cycle
    return {"kernel": f"decode_{sms}sm", "shape": [sms], "ms": ms / ntok, "tok_s": ntok / ms * 1e3, "gbs": by / (ms / ntok) / 1e6, "bound": "hbm", "algorithmic_bytes": by}


def run_sched_empty(ofa, repeats):
    """What one task costs the scheduler when it does nothing: phases of empty tasks (64 per resident block and phase, two phases
    chained) through the persistent kernel; time per task per block = claim + hand-off to the block + completion signal."""
    K = ofa.capi
    per_block, nblocks = 64, 296
    phases = [ofa.phase(K.TK_BARRIER, n=per_block * nblocks), ofa.phase(K.TK_BARRIER, n=per_block * nblocks)]
    ofa.run_phases(K.DTYPE_BF16, DIMS, phases, repeats=2)
    ms = min(ofa.run_phases(K.DTYPE_BF16, DIMS, phases, repeats=max(5, repeats)) for _ in range(3)) / max(5, repeats)
    us = ms * 1e3 / (2 * per_block)
    return {"kernel": "sched_empty", "shape": [2, per_block * nblocks], "ms": ms, "us_per_task_per_block": us, "gbs": 0.0, "bound": "hbm", "note": "empty tasks: scheduler cost only"}


def run_decode_attn(ofa, sms=148):
    """The serving job's attention task (one head's softmax attention over the KV cache + its slice of Wo; the reference's task_attwo,
    llm/b200/megakernel/decode_wide.cuh:321-428) at KV lengths 128 ... 1024: a decode-only context walks one context from position 0
    to 1023 in launches of 128 tokens, and after each launch the summed task time of the 12 "att+wo" phases gives the mean time of
    one task at the KV lengths of that window. Bytes per task: K and V rows of one head up to the position (2 * len * 64 * 2 B)
    plus the task's Wo slice (64 x 256 x 2 B). Returns one record per window."""
    cfg = ofa.default_config("gpt_s")
    cfg.mode, cfg.use_decode, cfg.infer_sms, cfg.reserved_sms = ofa.capi.MODE_DECODE_ONLY, 1, sms, 0
    cfg.n_prompt, cfg.answer_len = 1, 0                      # no answer mode: the context simply grows to 1024 positions
    cfg.prompt[0] = 11
    mk = ofa.Megakernel(cfg)
    rng = np.random.default_rng(6)
    mk.load_weights(rng.standard_normal(mk.num_params, dtype=np.float32) * np.float32(0.02))
    out = []
    for w in range(T // 128):
        ms = mk.run(128)
        ph = [p for p in mk.decode_phases() if p["name"].endswith("att+wo")]
        ntasks = sum(p["ntasks"] for p in ph) * 128
        us = sum(p["busy_ns"] for p in ph) / 1e3 / ntasks
        mean_len = w * 128 + 64.5
        by = 2.0 * mean_len * 64 * 2 + 64 * 256 * 2
        out.append({"kernel": f"decode_attn_kv{(w + 1) * 128}", "shape": [int(w * 128 + 1), int((w + 1) * 128)], "us_per_task": us, "ms": us / 1e3,
                    "tok_s": 128 / ms * 1e3, "gbs_per_block": by / us / 1e3, "gbs": by / us / 1e3 * 2 * sms, "bound": "hbm", "algorithmic_bytes": by,
                    "note": "gbs = per-task rate x the 2 x %d resident serving blocks (the rate if every block ran such tasks back to back)" % sms})
    mk.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--nsub", type=int, default=0)
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--ref-method", action="store_true", help="GEMM cases: the reference test program's timing method (same operands repeated, best of 6)")
    ap.add_argument("--ref-vocab", action="store_true", help="GEMM cases with a vocabulary dimension use the reference's 100352 instead of 50304")
    a = ap.parse_args()
    global REF_METHOD
    REF_METHOD = a.ref_method
    if a.ref_vocab:
        for k, (l, e, m, n, kk) in list(GEMMS.items()):
            GEMMS[k] = (l, e, 100352 if m == V else m, 100352 if n == V else n, 100352 if kk == V else kk)
    names = list(GEMMS) + OTHERS
    if a.list:
        print("\n".join(names)); return
    sel = [n for n in a.only.split(",") if n] or names
    ofa = importlib.import_module("open-flapping-airplanes_b200")
    hbm, tf, how = peaks()
    # one small launch first: loading the kernel image at the first launch takes milliseconds and would otherwise be counted
    # in the first case timed (cases that work in place cannot warm themselves up)
    rng = np.random.default_rng(99)
    wx = rand_bf16(ofa, rng, (B * T, D), 1.0); wy = ofa.DeviceBuffer((B * T, D), "bf16")
    wm = ofa.DeviceBuffer((B * T,), np.float32); wr = ofa.DeviceBuffer((B * T,), np.float32); wg = rand_bf16(ofa, rng, (D,), 1.0)
    ofa.run_phases(ofa.capi.DTYPE_BF16, DIMS, [ofa.phase(ofa.capi.TK_LN_FWD, [wy, wm, wr, wx, wg])])
    for n in sel:
        if n in GEMMS: r = run_gemm(ofa, n, a.repeats, a.nsub)
        elif n in ("attn_fwd", "attn_bwd"): r = run_attn(ofa, n, a.repeats)
        elif n == "adamw": r = run_adamw(ofa, a.repeats)
        elif n == "cross_entropy": r = run_ce(ofa, a.repeats)
        elif n in ("ln_fwd", "ln_bwd"): r = run_ln(ofa, n, a.repeats)
        elif n == "embed_bwd_wte": r = run_embed_bwd(ofa, a.repeats)
        elif n == "decode_148sm": r = run_decode(ofa, 148, 261 * max(1, a.repeats))
        elif n == "decode_24sm": r = run_decode(ofa, 24, 261 * max(1, a.repeats))
        elif n == "decode_attn": r = run_decode_attn(ofa)
        elif n == "sched_empty": r = run_sched_empty(ofa, a.repeats)
        elif n == "head_fused": r = run_head_fused(ofa, a.repeats)
        else: raise SystemExit(f"unknown case {n}")
        for rec in (r if isinstance(r, list) else [r]):
            rec["frac"] = (rec["tflops"] / tf) if rec["bound"] == "tensor" else (rec["gbs"] / hbm)
            rec["peak"] = f"{how}: {tf if rec['bound'] == 'tensor' else hbm} {'TFLOP/s (burst)' if rec['bound'] == 'tensor' else 'GB/s'}"
            print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
