#!/usr/bin/env python
"""Benchmark of the hot path: GPT-S (162M class, V=50304 untied, T=1024, B=4 => 4,096 tokens/step) trained by the
persistent megakernel, with the live-weight decoder running concurrently on its own SM partition (116 train / 24 serve /
8 reserved SMs). One "step" = one optimizer step. Prints ONE JSON line.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload split|train_only]

Timing: W warm-up steps run in a first persistent launch; K timed steps are ONE further persistent launch bracketed by CUDA
events on the launching stream (and a barrier + synchronize on both sides), max over ranks; that K-step launch is repeated
(at least 5 times, more than a second in total) and the median launch is reported with the spread. `value` counts the
tokens all ranks trained on. The working set of a step (326 MB of bf16 weights + GBs of activations) exceeds the 126 MB L2,
so no explicit flush is needed. `e2e` repeats the K steps through the public API with host buffers: token upload, launch,
wait and loss read-back inside a host-timed region.

--impl reference: the CPU implementation of the same step (the oracle port of the reference's PyTorch model, batch 4 x 1024,
forward + backward + AdamW) on all host cores; it runs as many of the requested steps as fit in about two minutes and prints
how many it ran.
"""
import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

V, D, L, H, T, B = 50304, 768, 12, 12, 1024, 4
TOKENS_PER_STEP = B * T
P_MM = L * 12 * D * D + V * D                                   # matmul parameters
FLOP_PER_STEP = 6 * TOKENS_PER_STEP * P_MM + L * 3.5 * (4 * B * H * T * T * (D // H) / 2)   # 3.307e12, causal attention counted once
# dram__bytes_read.sum + dram__bytes_write.sum of the megakernel per step, split workload on one GPU: a constant taken from ONE ncu
# capture of a 2-step launch (concurrent decoder included), not measured by this program. profiles/ofa_kernel_bench_split_dram_traffic.md
# holds the command, the raw figures, the date and the commit of the capture; it has to be re-captured when the training graph changes.
SPLIT_DRAM_BYTES_PER_STEP = 18.0e9


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clocks/throttle reasons sampled every 200 ms while the timed region runs."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True); self.th.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # the load raises the clock: take the median of the upper half of the samples as "under load"
        sm_sorted = sorted(sm)
        under = sm_sorted[len(sm_sorted) // 2:] if sm_sorted else []
        return {"sm_mhz": float(np.median(under)) if under else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def init_flat(mk, seed=1234):
    """N(0, 0.02) weights with the reference's scaling (Wo/Wdown by 1/sqrt(2L), gammas 1), from numpy for speed."""
    rng = np.random.default_rng(seed)
    flat = rng.standard_normal(mk.num_params, dtype=np.float32) * np.float32(0.02)
    sc = np.float32(1 / np.sqrt(2.0 * L))
    for l in range(L):
        for g in ("g1", "g2"):
            off, cnt = mk.param_span(f"L{l}.{g}"); flat[off:off + cnt] = 1.0
        for t in ("Wo", "Wdn"):
            off, cnt = mk.param_span(f"L{l}.{t}"); flat[off:off + cnt] *= sc
    off, cnt = mk.param_span("gf"); flat[off:off + cnt] = 1.0
    return flat


def cpu_steps(warmup, steps, max_seconds):
    """The oracle's training step - the reference's PyTorch model and recipe, fp32, all host threads - on the SAME step the GPU arm
    runs: batch 4 x 1024 tokens of the same synthetic stream, forward + backward + one AdamW update of the full 163M-parameter
    model per step. Runs `warmup` untimed and up to `steps` timed steps, stopping early when `max_seconds` of timed work are used
    up. Returns (tokens/s, cores, warm-ups run, steps timed, seconds per step list)."""
    import torch
    from oracle import gpt_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = orc.gpt_s_config()
    w0 = orc.init_weights(cfg)
    model = orc.GPTOracle(cfg, w0, "fp32")
    opt = orc.make_optimizer(cfg, model)
    ntok = 1 << 20
    tokens = orc.synthetic_tokens(V, ntok, 1000)
    starts = orc.batch_starts(cfg, ntok, warmup + steps)
    def one(i):
        for g in opt.param_groups:
            g["lr"] = orc.lr_at(cfg, i)
        x, y = orc.get_batch(cfg, tokens, starts[i])
        t0 = time.perf_counter()
        loss = model(x, y); loss.backward(); opt.step(); opt.zero_grad(set_to_none=True)
        return time.perf_counter() - t0

    times, w_done, i = [], 0, 0
    for _ in range(warmup):
        dt = one(i); i += 1; w_done += 1
        if dt > max_seconds / 3:                       # a host this slow gets one warm-up only
            break
    for _ in range(steps):
        dt = one(i); i += 1
        times.append(dt)
        if sum(times) + dt > max_seconds:
            break
    total = sum(times)
    return TOKENS_PER_STEP * len(times) / total, cores, w_done, len(times), times


def run_reference(args, rank, world):
    if rank != 0:
        return
    tps, cores, w_done, k_done, times = cpu_steps(max(1, min(args.warmup, 2)), max(1, args.steps), max_seconds=120.0)
    sample = (f"{k_done} timed step(s) after {w_done} warm-up step(s), each the full step: batch {B} x {T} tokens, fp32 forward + backward + AdamW of the "
              f"163M-parameter model; {sum(times):.1f} s of timed work")
    line = {"impl": "reference", "metric": "GPT-S 162M train tokens/s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": k_done,
            "warmup": w_done, "steps_requested": args.steps, "ms_per_step": TOKENS_PER_STEP / tps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "gpt_s V=50304 untied D=768 L=12 H=12 T=1024 B=4 (4096 tok/step), CPU oracle port of the reference PyTorch model, training only"},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="split", choices=["split", "train_only", "ref_split", "ref_train_only"],
                    help="ref_*: the same two workloads at the shapes the reference program is compiled for (vocab 100352 tied, context 512, batch 8), for a like-for-like line beside its own binary")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--repeats", type=int, default=0, help="timed K-step launches (0 = enough for more than a second of timed work, at least 5)")
    ap.add_argument("--dp-side", choices=["native", "torch"], default="native", help="N > 1: gradient all-reduce queued by the library's C++ side (its own NCCL communicator) or through torch.distributed")
    ap.add_argument("--phase-table", action="store_true", help="also print the per-phase busy table to stderr")
    ap.add_argument("--cfg", action="append", default=[], metavar="FIELD=INT", help="override an integer field of ofa_config (experiments, e.g. gemm_nsub=2, head_dx_splitk=1); the run is then not the headline configuration")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank, world)

    ofa = importlib.import_module("open-flapping-airplanes_b200")
    if world > 1:
        ofa.dp.configure_env(8)                        # before the first CUDA call of the process
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the megakernel")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    W, K = max(3, args.warmup), args.steps
    split = args.workload in ("split", "ref_split")
    ref_shapes = args.workload.startswith("ref_")
    global V, T, B, TOKENS_PER_STEP, FLOP_PER_STEP
    if ref_shapes:                                      # llm/b200/megakernel/ofa.cu:71
        V, T, B = 100352, 512, 8
        TOKENS_PER_STEP = B * T
        FLOP_PER_STEP = 6 * TOKENS_PER_STEP * (L * 12 * D * D + V * D) + L * 3.5 * (4 * B * H * T * T * (D // H) / 2)

    cfg = ofa.default_config("gpt_s")
    if ref_shapes:
        cfg.vocab, cfg.valid_vocab, cfg.tied_head, cfg.ctx_len, cfg.batch = V, 100277, 1, T, B
    cfg.device = local_rank
    cfg.data_seed = rank
    if split:
        cfg.infer_sms, cfg.reserved_sms, cfg.train_sms = 24, 8, 116
        cfg.use_decode = 1 if rank == 0 else 0
        if rank != 0:
            cfg.reserved_sms = 32                      # other ranks leave the serving partition idle so that all ranks train on 116 SMs
        prompt = np.random.default_rng(1234).integers(0, min(V, 100277), size=6)
        for i, t in enumerate(prompt):
            cfg.prompt[i] = int(t)
        cfg.n_prompt, cfg.answer_len, cfg.temperature = 6, 256, 0.0
        cfg.decode_out_cap = 1 << 20
    elif world > 1:
        cfg.reserved_sms = 8
    dp = None
    dp_side = args.dp_side
    if world > 1:
        cfg.dp_world, cfg.grad_bf16, cfg.ext_sync = world, 1, 1
    cfg.sched_profile = 1 if args.phase_table else 0    # the in-kernel time tables are only read by --phase-table
    for kv in args.cfg:
        k, v = kv.split("=")
        if k not in [f[0] for f in cfg._fields_]:
            raise SystemExit(f"--cfg: ofa_config has no field {k!r}")
        setattr(cfg, k, int(v))
    mk = ofa.Megakernel(cfg)
    mk.load_weights(init_flat(mk))
    ntok = 1 << 22
    tokens = np.random.default_rng(1000 + rank).integers(0, V, size=ntok, dtype=np.uint32)     # uniform ids, a distinct seed per rank
    mk.set_tokens(tokens)
    if world > 1:
        # NCCL gradient all-reduce ordered by device flags
        if dp_side == "native":
            try:
                dp = ofa.dp.NativeDataParallel(mk, rank, world)
            except Exception as e:                         # e.g. no NCCL library found by the C++ side: every rank takes the same branch below
                print(f"[rank {rank}] the library's own communication side is unavailable ({e}); using torch.distributed", file=sys.stderr)
                dp = None
            ok_all = torch.tensor([1 if dp is not None else 0], device="cuda", dtype=torch.int32)
            dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)
            if int(ok_all.item()) == 0:
                if dp is not None:
                    dp.close()
                dp, dp_side = None, "torch"
        if dp is None:
            dp = ofa.dp.DataParallel(mk, dist)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def run(n):
        mk.launch(n)
        if dp is not None:
            dp.enqueue(n)                              # after the launch: a stream wait must never sit in front of the kernel that satisfies it
            dp.wait(600000)                            # kernel + communication queue; a rank that stopped early makes every rank raise
        else:
            mk.wait(600000)
        return mk.last_launch_ms

    run(W)
    barrier()
    # The K-step launch is repeated so that the timed work exceeds a second (one launch of 20 steps is 0.18 s: too few clock samples
    # and no spread); every launch is K steps bracketed by its own CUDA events, the reported time is the median launch.
    est = run(K)
    barrier()
    reps = int(min(25, max(5, np.ceil(1200.0 / max(est, 1e-3))))) if args.repeats <= 0 else args.repeats
    dec0 = mk.decode_steps
    sampler = ClockSampler(local_rank); sampler.start()
    time.sleep(0.25)
    all_ms = []
    for _ in range(reps):
        m = run(K)
        barrier()
        if dist is not None:
            t = torch.tensor([m], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            m = float(t.item())
        all_ms.append(m)
    clocks = sampler.stop()
    dec_steps = mk.decode_steps - dec0
    ms = float(np.median(all_ms))
    losses = mk.losses()

    # ---- end to end through the public API with host buffers (rank-local; inputs uploaded and results read inside the timed region)
    window = tokens[: min(ntok, max(1 << 16, K * B * (T + 1) * 2))]
    starts = np.random.default_rng(7).integers(0, window.size - T - 1, size=(K, B)).astype(np.uint32)
    barrier()
    t0 = time.perf_counter()
    mk.set_tokens(window)
    mk.set_starts(starts)
    run(K)
    e2e_losses = mk.losses()[-K:]
    t1 = time.perf_counter()
    e2e_s = t1 - t0
    if dist is not None:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    assert np.all(np.isfinite(e2e_losses))

    if rank == 0:
        peaks, how = measured_peaks()
        sms_used = cfg.train_sms if split else 148 - (cfg.reserved_sms if world > 1 else 0)
        peak_tf = peaks["bf16_tflops_sustained"] * sms_used / 148.0
        achieved_tf = FLOP_PER_STEP * K / (ms * 1e-3) / 1e12
        value = world * TOKENS_PER_STEP * K / (ms * 1e-3)
        # sampled decode tokens: of every 261 decode steps (5 forced + 256 sampled) 256 are counted, as the reference counts (ofa.cu:747-752)
        dec_tok_s = (dec_steps * 256.0 / 261.0) / (sum(all_ms) * 1e-3) if split else None
        line = {
            "metric": "GPT-S 162M train tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "timed_launches": {"n": reps, "steps_each": K, "ms_per_step_median": ms / K, "ms_per_step_min": min(all_ms) / K, "ms_per_step_max": max(all_ms) / K},
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": ((f"gpt_s at the reference program's shapes V={V} tied D=768 L=12 H=12 T={T} B={B} (4096 tok/step/GPU), " if ref_shapes else "gpt_s V=50304 untied D=768 L=12 H=12 T=1024 B=4 (4096 tok/step/GPU), ") +
                                    ("116 train / 24 serve / 8 reserved SMs with concurrent batch-1 greedy decode (6-token prompt, 256 generated, repeating)" if split else "training only on all SMs")),
                       "parallelism": f"dp{world}" + (", ranks > 0 train on 116 SMs and leave the 24 serving SMs idle (one serving replica, on rank 0)" if (world > 1 and split) else ""), "l2": "working set per step (>2 GB) exceeds the 126 MB L2; no flush needed",
                       "projected_4000_steps_s": ms / K * 4000 / 1e3, **({"allreduce_queue": ("library (C++, own NCCL communicator)" if dp_side == "native" else "torch.distributed")} if world > 1 else {}), **({"overrides": args.cfg} if args.cfg else {})},
            "decode_tok_s": dec_tok_s, "final_loss": float(losses[-1]), "first_loss": float(losses[0]),
            "e2e": {"value": world * TOKENS_PER_STEP * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": int(window.nbytes / K + starts.nbytes / K), "d2h_bytes_per_step": 4},
            "gpu_launches": 2 if split else 1,   # the persistent kernel, and with the decoder its one-block residual rebuild before it
            "roofline": {"bound": "tensor", "achieved": achieved_tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved_tf / peak_tf,
                         "traffic": SPLIT_DRAM_BYTES_PER_STEP if (args.workload == "split" and world == 1 and not args.cfg) else None, "peak_source": f"{how} bf16_tflops_sustained x {sms_used}/148 SMs", "flop_per_step": FLOP_PER_STEP},
            "clocks": clocks,
        }
        if args.phase_table:
            bb = mk.block_busy_ns()
            bw = mk.block_wait_ns()
            act = bb[:, 0] > 0
            print(f"  per training block, ms/step: dependency wait {bw[0][act].mean() / 1e6 / K:.3f}, claim {bw[1][act].mean() / 1e6 / K:.3f}, hand-off {bw[2][act].mean() / 1e6 / K:.3f}, signalling {bw[3][act].mean() / 1e6 / K:.3f}; tasks per step {sum(p['ntasks'] for p in mk.phases())}", file=sys.stderr)
            print(f"  blocks that ran training tasks: {(bb[:, 0] > 0).sum()}, serving tasks: {(bb[:, 1] > 0).sum()}; mean training-block busy {bb[:, 0][bb[:, 0] > 0].mean() / 1e6 / K:.3f} ms/step", file=sys.stderr)
            tot = sum(p["busy_ns"] for p in mk.phases()) or 1
            import re
            cat = {}
            for p in mk.phases():
                key = re.sub(r"^L\d+ ", "L* ", p["name"]); key = re.sub(r"adamw L\d+", "adamw L*", key)
                c = cat.setdefault(key, [0, 0, 0]); c[0] += p["busy_ns"]; c[1] += p["ntasks"]; c[2] += p["wait_ns"]
            print("  per category (block-ms per step, share of busy, mean us per task, block-ms per step waiting for its dependencies):", file=sys.stderr)
            for k, (b, n, w) in sorted(cat.items(), key=lambda kv: -kv[1][0]):
                print(f"    {k:22s} {b / 1e6 / K:8.3f}  {100.0 * b / tot:5.1f} %  {b / 1e3 / K / max(1, n):8.2f} us/task  ({n} tasks)  wait {w / 1e6 / K:8.3f}", file=sys.stderr)
            win = mk.phase_windows(); names = [p["name"] for p in mk.phases()]
            valid = [(a, b, n) for (a, b), n in zip(win, names) if a != 0xFFFFFFFFFFFFFFFF and b]
            if valid:
                t0 = min(a for a, _, _ in valid)
                print("  phase windows in the last step (first task start -> last task end, ms from the step's first task):", file=sys.stderr)
                for a, b, n in valid:
                    if n.startswith("L") and not (n.startswith("L0 ") or n.startswith("L11 ") or n.startswith("L5 ")):
                        continue
                    print(f"    {n:22s} {(a - t0) / 1e6:8.3f} -> {(b - t0) / 1e6:8.3f}  ({(b - a) / 1e3:7.1f} us)", file=sys.stderr)
            for p in sorted(mk.phases(), key=lambda p: -p["busy_ns"])[:40]:
                print(f"  {p['name']:24s} tasks {p['ntasks']:6d}  busy {p['busy_ns'] / 1e6 / K:8.3f} ms/step  {100.0 * p['busy_ns'] / tot:5.1f} %", file=sys.stderr)
        if world == 1 and not args.no_cpu_baseline and not ref_shapes:
            tps, cores, w_done, k_done, times = cpu_steps(1, 3, max_seconds=25.0)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                                    "sample": f"{k_done} timed step(s) after {w_done} warm-up, each the full step (batch {B} x {T} tokens, fp32 forward + backward + AdamW, training only), {sum(times):.1f} s"}
        print(json.dumps(line), flush=True)
    mk.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
