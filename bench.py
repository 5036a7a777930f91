#!/usr/bin/env python
"""Benchmark of the Heron forward + next-token CE hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # CPU arm (oracle port on the host cores)

Workload (default): Heron D=512 / L=12 / T=2048 / vocab 8192, 64 sequences
of seeded Zipf(1.1) token ids, random-init weights from a seeded v2 checkpoint -
forward + streamed CE, no backward.  Sequences are independent, so ranks take
disjoint contiguous blocks of the 64 sequences (strong scaling: rank r of W
owns sequences [r*64/W, (r+1)*64/W)) and only {loss_sum, n_valid} is
all-reduced over NCCL, on the device.  `--scaling weak` keeps `--batch`
sequences on every GPU instead.

A "step" is one forward+CE over the rank's sequences.  `value` times K steps
with the token ids already resident in HBM (CUDA events on the backend's
stream, max over ranks, no per-kernel instrumentation); `e2e` times the public
C-ABI call with pinned HOST buffers, copies and the loss read-back inside the
timed region.  The per-kernel table comes from a separate pass with an event
behind every launch.  One JSON line is printed by rank 0; at one GPU its
`extra` object adds the other configurations of the same path (one sequence of
the default and of the small model, the LayerNorm-gain-one weight variant, the
three packed-linear shapes).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "heron_forward_ce_tokens_per_s"
UNIT = "tokens/s"
# algorithmic bytes of the ROSA 1-bit forward per (sequence, step, channel):
# 3 FP16 activations in, 1 idx byte + 1 FP16 activation out
ROSA_BYTES_PER_UNIT = 9.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["cuda", "reference"], default="cuda")
    ap.add_argument("--model", default="default", help="checkpoint shape: default (D512 L12 T2048), small, tiny")
    ap.add_argument("--batch", type=int, default=64,
                    help="sequences: in the whole job with --scaling strong (the default), per GPU with --scaling weak")
    ap.add_argument("--scaling", choices=["strong", "weak"], default="strong")
    ap.add_argument("--ln-gain-one", action="store_true",
                    help="LayerNorm weights 1 + N(0, 0.02) instead of N(0, 0.02): no constant channels, every stream "
                         "reaches the automaton")
    ap.add_argument("--no-extras", action="store_true", help="skip the `extra` measurements of the one-GPU line")
    ap.add_argument("--time", type=int, default=0, help="steps per sequence (0 = the model's context length)")
    ap.add_argument("--mode", choices=["fast", "exact"], default="fast")
    ap.add_argument("--sam", choices=["euler", "eager"], default="euler")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-run", action="store_true",
                    help="short run for a profiler: warm-up count as given, no end-to-end leg, no CPU baseline")
    ap.add_argument("--workload", choices=["heron", "rosa", "linear", "generate", "train", "pushers"], default="heron",
                    help="heron = the benchmark; rosa / linear = single-op loops; generate = incremental decoding; "
                         "pushers = RosaSam::push for many streams at a late position")
    ap.add_argument("--rosa-variant", choices=["iid", "periodic"], default="iid")
    ap.add_argument("--channels", type=int, default=512)
    ap.add_argument("--linear-shape", default="2048x512x512", help="MxKxN of the packed linear loop")
    return ap.parse_args()


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback"


def profiled_traffic(kernel: str):
    """DRAM bytes per launch of `kernel` from the committed ncu summary, if any."""
    try:
        with open(os.path.join(ROOT, "profiles", "roofline_traffic.json")) as f:
            return json.load(f).get(kernel)
    except Exception:  # noqa: BLE001
        return None


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []
        self.proc = None
        self.thread = None
        self.first_of_region = 0

    def mark_region(self, wait_s: float = 3.0):
        """The timed region starts now.  nvidia-smi needs a moment before its first line, and the region can be
        shorter than that: wait (bounded) until the sampler is delivering, and remember where the region begins."""
        t0 = time.perf_counter()
        while self.proc is not None and not self.samples and time.perf_counter() - t0 < wait_s:
            time.sleep(0.01)
        self.first_of_region = len(self.samples)

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:  # noqa: BLE001
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        if self.thread:
            self.thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        # the samples of the timed region; should it have been too short for one, those of the warm-up steps right
        # before it (the same kernels on the same device) stand in, and the line says so
        window = self.samples[self.first_of_region:]
        during = "timed region"
        if not window:
            window, during = self.samples, "warm-up steps before the timed region (it was shorter than a sampling interval)"
        for s in window:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, flag in zip(names, s[2:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "sampled_during": during}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def sequence_tokens(model_vocab: int, first_seq: int, n_seq: int, time_: int) -> np.ndarray:
    from ullis_b200 import synth
    return np.concatenate([synth.zipf_tokens(11 + first_seq + b, time_, model_vocab) for b in range(n_seq)])


def cpu_baseline_sample(data: bytes, vocab: int, time_: int, threads: int = 0):
    """Oracle port on the host cores (all of them unless `threads` says otherwise) over ONE sequence of the workload."""
    from oracle import oracle as O
    threads = threads or O.max_threads()
    O.set_threads(threads)
    m = O.HeronOracle(data)
    tokens = sequence_tokens(vocab, 0, 1, time_)
    t0 = time.perf_counter()
    mean, n_valid, _, _ = m.forward_ce(tokens, tokens, O.CE_NO_IGNORE, 1, time_)
    dt = time.perf_counter() - t0
    return {"value": time_ / dt, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"1 sequence (B=1, T={time_}) of the workload, full depth, {dt:.1f} s, mean CE {mean:.4f}"}, mean


def run_reference(args):
    """CPU arm: the oracle port (the reference crate is Rust; no rustc here) on
    every host core, one sequence of the workload per step."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from oracle import oracle as O
    from ullis_b200 import synth
    shape = synth.CONFIGS[args.model]
    time_ = args.time or shape[3]
    data = synth.heron_checkpoint(args.model, batch_size=max(args.batch, 1), ln_gain_one=args.ln_gain_one)
    threads = O.max_threads()
    O.set_threads(threads)
    m = O.HeronOracle(data)
    steps_tokens = [sequence_tokens(shape[2], s, 1, time_) for s in range(args.steps + args.warmup)]
    for s in range(args.warmup):
        m.forward_ce(steps_tokens[s], steps_tokens[s], O.CE_NO_IGNORE, 1, time_)
    t0 = time.perf_counter()
    for s in range(args.steps):
        tk = steps_tokens[args.warmup + s]
        m.forward_ce(tk, tk, O.CE_NO_IGNORE, 1, time_)
    dt = time.perf_counter() - t0
    value = args.steps * time_ / dt
    sample = f"each step = 1 sequence (B=1, T={time_}) of the workload through the oracle port, {threads} threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / max(args.steps, 1), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, shape, time_, world),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def rank_sequences(args, rank, world):
    """[lo, hi) of the job's sequences that `rank` owns."""
    from ullis_b200 import dp
    if args.scaling == "weak":
        return rank * args.batch, (rank + 1) * args.batch
    return dp.shard_range(args.batch, rank, world)


def workload_config(args, shape, time_, world):
    d, layers, vocab, ctx, ffn = shape
    total = args.batch * world if args.scaling == "weak" else args.batch
    per_gpu = [hi - lo for lo, hi in (rank_sequences(args, r, world) for r in range(world))]
    return {"workload": f"Heron D={d} L={layers} T={time_} vocab={vocab} forward + next-token CE, "
                        f"{total} sequences (Zipf(1.1) ids) over {world} GPU(s)",
            "d_model": d, "n_layers": layers, "seq_len": time_, "vocab": vocab, "dim_ffn": ffn,
            "global_sequences": total, "sequences_per_gpu": per_gpu,
            "parallelism": f"dp{world} over independent sequences (contiguous blocks), 16-byte loss all-reduce on the device",
            "weights": "LayerNorm gain 1 + N(0, 0.02)" if args.ln_gain_one else "LayerNorm gain N(0, 0.02) (the literal reading of the configuration)",
            "mode": args.mode, "sam": args.sam,
            "l2": f"no flush: a step moves at least {min(per_gpu) * time_ * d * 4 * 8 * layers / 1e9:.1f} GB of activations per GPU "
                  "(8 f32-row-equivalents per layer), beyond the 126 MB L2"}


def device_steps_ms(model, rt, stream, torch, B, time_, steps, warm, reduce_loss=None):
    """ms per forward+CE step with the ids already uploaded: `warm` untimed steps, then `steps` steps between
    two CUDA events on the backend's stream.  Every step reads its loss back (the step's result)."""
    from ullis_b200 import cuda
    last = None
    for _ in range(warm):
        model.enqueue_forward_ce(cuda.CE_NO_IGNORE, B, time_)
        last = reduce_loss() if reduce_loss else model.read_loss()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(steps):
        model.enqueue_forward_ce(cuda.CE_NO_IGNORE, B, time_)
        last = reduce_loss() if reduce_loss else model.read_loss()
    ev1.record(stream)
    torch.cuda.synchronize()
    return ev0.elapsed_time(ev1) / max(steps, 1), last


def extra_measurements(args, rt, stream, torch, peaks):
    """The other configurations of the same path, one GPU: a single sequence of the default and of the small
    model (latency: a step is as long as the 2048-step serial chain of one stream per layer), the
    LayerNorm-gain-one weight variant of the benchmark (no constant channels), and the packed-linear shapes."""
    from ullis_b200 import cuda, synth
    out = {}

    def one(model_name, B, gain_one, steps, warm, with_kernels=False):
        d, layers, vocab, ctx, ffn = synth.CONFIGS[model_name]
        data = synth.heron_checkpoint(model_name, batch_size=B, ln_gain_one=gain_one)
        model = cuda.CudaHeron(rt, data)
        tokens = sequence_tokens(vocab, 0, B, ctx)
        model.upload_tokens(tokens, tokens, B, ctx)
        ms, last = device_steps_ms(model, rt, stream, torch, B, ctx, steps, warm)
        counts = rt.sam_counts()
        res = {"model": f"D={d} L={layers} T={ctx} vocab={vocab}", "sequences": B,
               "weights": "ln gain 1 + N(0,0.02)" if gain_one else "ln gain N(0,0.02)",
               "ms_per_forward": ms, "tokens_per_s": B * ctx / (ms * 1e-3), "mean_ce": last[0],
               "automaton_streams_last_layer": counts["automaton"], "constant_q_streams_last_layer": counts["constant_q"],
               "streams_per_layer": counts["total"]}
        if with_kernels:
            # one more forward with an event behind every launch, itself between two events: what share of that
            # forward no kernel accounts for (launch gaps: at one sequence a kernel is often shorter than a launch)
            rt.kernel_timing(True)
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(stream)
            model.enqueue_forward_ce(cuda.CE_NO_IGNORE, B, ctx)
            a1.record(stream)
            model.read_loss()
            km = rt.kernel_times()
            rt.kernel_timing(False)
            inst_ms = a0.elapsed_time(a1)
            busy = sum(t for k, (t, _) in km.items() if not k.startswith("(") and k != "rosa_constq")   # side stream: overlaps
            res["instrumented_forward_ms"] = inst_ms
            res["kernel_ms_sum_instrumented"] = busy
            res["launches"] = int(sum(n for k, (_, n) in km.items() if not k.startswith("(")))
            res["launch_gap_share"] = max(0.0, 1.0 - busy / inst_ms) if inst_ms > 0 else None
            top = sorted(((k, t) for k, (t, _) in km.items() if not k.startswith("(")), key=lambda kv: -kv[1])[:4]
            res["top_kernels_ms"] = {k: round(t, 3) for k, t in top}
        model.close()
        return res, data

    out["config3_default_batch1"], data3 = one("default", 1, args.ln_gain_one, 10, 3, with_kernels=True)
    out["config0_small_batch1"], data0 = one("small", 1, args.ln_gain_one, 20, 3, with_kernels=True)
    out["config4_ln_gain_one" if not args.ln_gain_one else "config4_literal_weights"], _ = one(
        "default", args.batch, not args.ln_gain_one, 3, 2)
    if not args.no_cpu_baseline:
        from oracle import oracle as O
        for key, data, name in (("config0_small_batch1", data0, "small"),):
            d, layers, vocab, ctx, ffn = synth.CONFIGS[name]
            for threads in (O.max_threads(), 1):
                base, _ = cpu_baseline_sample(data, vocab, ctx, threads)
                out[key][f"oracle_{threads}_threads_tokens_per_s" if threads > 1 else "oracle_1_thread_tokens_per_s"] = base["value"]
    # BASELINE configuration 1: the three packed-linear shapes at M = 2048 and at the benchmark's row count
    linear = {}
    sustained = float(peaks.get("bf16_tflops_sustained", 1400.0))
    for M in (2048, 131072):
        for K, N in ((512, 512), (512, 2048), (512, 8192)):
            x, bits, scale, bias = synth.packed_linear_case(3, M, K, N)
            reps = 3 if M * N > (1 << 28) else 10
            for _ in range(2):
                rt.binary_linear(x, bits, scale, bias, M, K, N)
            rt.kernel_timing(True)
            for _ in range(reps):
                rt.binary_linear(x, bits, scale, bias, M, K, N)
            km = rt.kernel_times()
            rt.kernel_timing(False)
            gemm_ms = sum(t for name, (t, _) in km.items() if name.startswith("gemm_")) / reps
            tf = 2.0 * M * K * N / (gemm_ms * 1e-3) / 1e12 if gemm_ms else None
            linear[f"M{M}_{K}x{N}"] = {"gemm_ms": gemm_ms, "tflops": tf,
                                       "frac_of_sustained_peak": tf / sustained if tf else None}
            del x
    out["linear_f32_out"] = linear
    return out


def run_cuda(args):
    import torch
    import torch.distributed as dist

    from ullis_b200 import cuda, synth

    rank, world, local = dist_env()
    if world != args.gpus and world > 1:
        args.gpus = world
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    rt = cuda.CudaRuntime(local)
    rt.set_mode(cuda.MODE_EXACT if args.mode == "exact" else cuda.MODE_FAST)
    rt.set_sam(cuda.SAM_EAGER if args.sam == "eager" else cuda.SAM_EULER)
    stream = torch.cuda.ExternalStream(rt.stream, device=torch.device("cuda", local))

    if args.workload != "heron":
        return run_op_loop(args, rt, stream, torch)

    shape = synth.CONFIGS[args.model]
    d, layers, vocab, ctx, ffn = shape
    time_ = args.time or ctx
    lo, hi = rank_sequences(args, rank, world)
    B = hi - lo                                  # this rank's sequences
    total_seqs = args.batch * world if args.scaling == "weak" else args.batch
    if B == 0:
        raise SystemExit("more ranks than sequences")
    data = synth.heron_checkpoint(args.model, batch_size=max(B, 1), ln_gain_one=args.ln_gain_one)
    model = cuda.CudaHeron(rt, data)
    tokens = sequence_tokens(vocab, lo, B, time_)
    labels = tokens
    rows = B * time_
    total_rows = total_seqs * time_

    if world > 1:
        uid = [cuda.CudaRuntime.dp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        rt.dp_init(rank, world, uid[0])

    # the step's result: the mean over every rank's valid positions, summed on the device at N > 1
    reduce_loss = model.read_loss_global if world > 1 else None

    # ---------------- device-resident timing (`value`), no per-kernel instrumentation
    model.upload_tokens(tokens, labels, B, time_)
    n_warm = args.warmup if args.profile_run else max(args.warmup, 3)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()   # before the warm-up: the sampler is then already running when the timed region starts
    device_steps_ms(model, rt, stream, torch, B, time_, 0, n_warm, reduce_loss)
    if rank == 0:
        sampler.mark_region()
    barrier()
    launches0 = rt.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        model.enqueue_forward_ce(cuda.CE_NO_IGNORE, B, time_)
        mean, total_sum, total_n = reduce_loss() if reduce_loss else model.read_loss()
    ev1.record(stream)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    launches = rt.launch_count - launches0
    ms_total = ev0.elapsed_time(ev1)
    t = torch.tensor([ms_total], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    value = total_rows * args.steps / (ms_total / 1e3)

    # ---------------- per-kernel table and phases: a separate pass with an event behind every launch
    model.set_profile(True)
    rt.kernel_timing(True)
    n_table = min(args.steps, 3)
    for _ in range(n_table):
        model.enqueue_forward_ce(cuda.CE_NO_IGNORE, B, time_)
        reduce_loss() if reduce_loss else model.read_loss()
    phases = model.phase_ms()  # of the last instrumented step
    kernel_ms = rt.kernel_times()  # over the instrumented steps: {name: (total ms, launches)}
    sam_counts = rt.sam_counts()
    rt.kernel_timing(False)
    model.set_profile(False)

    if args.profile_run:
        if rank == 0:
            top = sorted(((k, v) for k, v in kernel_ms.items() if not k.startswith("(")), key=lambda kv: -kv[1][0])[:8]
            print(json.dumps({"profile_run": True, "ms_per_step": ms_total / args.steps, "phases_ms": phases,
                              "gpu_launches": int(launches),
                              "kernel_ms_per_launch": {k: round(t / max(c, 1), 4) for k, (t, c) in top}}), flush=True)
        if world > 1:
            rt.dp_finalize()
            dist.destroy_process_group()
        model.close()
        rt.close()
        return

    # ---------------- end-to-end timing through the public call, pinned host buffers
    pin_tok = torch.from_numpy(tokens.astype(np.int64)).to(torch.int32).pin_memory()
    pin_lab = pin_tok.clone().pin_memory()
    tok_np = pin_tok.numpy().view(np.uint32)
    lab_np = pin_lab.numpy().view(np.uint32)

    def e2e_step():
        if world > 1:   # ids in, forward, loss summed over the ranks on the device, one read-back
            model.upload_tokens(tok_np, lab_np, B, time_)
            model.enqueue_forward_ce(cuda.CE_NO_IGNORE, B, time_)
            return model.read_loss_global()
        return model.forward_ce(tok_np, lab_np, cuda.CE_NO_IGNORE, B, time_)

    for _ in range(2):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        e2e_step()
    e1.record(stream)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = total_rows * args.steps / (float(t.item()) / 1e3)

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except Exception:  # noqa: BLE001
            pass
        # dominant kernel = the one with the largest share of device time in the instrumented pass
        kernel_ms = {k: v for k, v in kernel_ms.items() if not k.startswith("(")}   # drop the between-steps bracket
        top = sorted(kernel_ms.items(), key=lambda kv: -kv[1][0])
        # (on every supported shape that is one of the suffix-automaton kernels; should a GEMM
        # ever lead, the line still reports the leading automaton kernel and names the leader)
        leader = top[0][0]
        dominant, (dom_total, dom_launches) = next((kv for kv in top if kv[0].startswith("rosa_")), top[0])
        dom_ms = dom_total / max(dom_launches, 1)
        # Algorithmic bytes of the ROSA match per launch: 9 B per (sequence, step, channel)
        # (three FP16 inputs, one idx byte, one FP16 output), one launch per layer.
        alg_bytes = ROSA_BYTES_PER_UNIT * B * time_ * d
        achieved = alg_bytes / (dom_ms * 1e-3) / 1e9 if dom_ms > 0 else 0.0
        # kernels on a side stream run beside the others: they are listed, but add no time to a layer
        rosa_ms = sum(t for name, (t, _) in kernel_ms.items()
                      if name.startswith("rosa_") and name != "rosa_constq") / (n_table * layers)
        shares = {name: {"ms_per_step": t / n_table, "launches_per_step": n / n_table,
                         "share": t / sum(v[0] for v in kernel_ms.values())} for name, (t, n) in top[:12]}
        flops_per_token = layers * (4 * 2 * d * d + 2 * d * ffn + 2 * ffn * d) + 2 * d * vocab
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": n_warm, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f32" if args.mode == "exact" else "fp16 tensor-core operands, f32 accumulate; u16 automaton state",
            "data": "synthetic", "config": workload_config(args, shape, time_, world),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(2 * rows * 4),
                    "d2h_bytes_per_step": 16 if world > 1 else 32},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"kernel": dominant, "bound": "hbm", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "traffic": profiled_traffic(dominant),
                         "peak_source": peak_kind, "launch_ms": dom_ms, "leading_kernel": leader,
                         "algorithmic_bytes_per_launch": alg_bytes,
                         "rosa_kernels_ms_per_layer": rosa_ms,
                         "achieved_all_rosa_kernels": alg_bytes / (rosa_ms * 1e-3) / 1e9 if rosa_ms > 0 else 0.0},
            "tensor_core": {"flop_per_token": flops_per_token, "tflops_whole_step": flops_per_token * value / world / 1e12,
                            "frac_of_sustained_peak": flops_per_token * value / world / 1e12 /
                            float(peaks.get("bf16_tflops_sustained", 1421.6))},
            "kernels": shares,
            "kernels_note": f"per-kernel times from a separate pass of {n_table} step(s) with an event behind every launch; "
                            "`value` and `e2e` are timed without it",
            "phases_ms_last_step": phases,
            "automaton_streams_last_layer": sam_counts,
            "mean_ce": total_sum / total_n if total_n else 0.0,
        }
        if world == 1 and not args.no_extras:
            line["extra"] = extra_measurements(args, rt, stream, torch, peaks)
        if not args.no_cpu_baseline:
            base, cpu_mean = cpu_baseline_sample(data, vocab, time_)
            line["cpu_baseline"] = base
            if world == 1:
                one, _ = cpu_baseline_sample(data, vocab, time_, threads=1)
                base["one_thread"] = {"value": one["value"], "unit": UNIT, "cores": 1, "sample": one["sample"],
                                      "note": "the reference's own scheduling of this path is single-threaded"}
        print(json.dumps(line), flush=True)
    if world > 1:
        rt.dp_finalize()
        dist.destroy_process_group()
    model.close()
    rt.close()


def run_op_loop(args, rt, stream, torch):
    """Single-op loops through the op-level ABI (host buffers in and out).  The
    host-timed figure is dominated by the copies, so the line also carries the
    device time of every kernel of the op (events behind each launch): these are
    the per-shape microbenchmarks, not the headline."""
    from ullis_b200 import synth
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:  # noqa: BLE001
        pass

    def timed(call):
        for _ in range(max(args.warmup, 1)):
            call()
        rt.kernel_timing(True)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            call()
        dt = (time.perf_counter() - t0) / args.steps
        per_kernel = {k: t / args.steps for k, (t, _) in rt.kernel_times().items() if not k.startswith("(")}
        rt.kernel_timing(False)
        return dt, per_kernel

    if args.workload == "generate":
        # incremental decoding: `steps` tokens for each of `batch` sequences, logits back on the host every step
        from ullis_b200 import cuda
        d, layers, vocab, ctx, ffn = synth.CONFIGS[args.model]
        B = args.batch
        data = synth.heron_checkpoint(args.model, batch_size=max(B, 1))
        model = cuda.CudaHeron(rt, data)
        state = model.generate_state(B)
        tokens = sequence_tokens(vocab, 0, B, ctx).reshape(B, ctx)
        n_prof = min(16, ctx - args.warmup)          # a few plain-launch steps for the per-kernel times
        n_tok = min(args.steps, ctx - args.warmup - n_prof)
        for t in range(args.warmup):
            model.generate_step(state, tokens[:, t])
        t0 = time.perf_counter()
        for t in range(args.warmup, args.warmup + n_tok):   # the step replayed as a CUDA graph
            model.generate_step(state, tokens[:, t])
        dt = (time.perf_counter() - t0) / n_tok
        rt.kernel_timing(True)                                # timing needs the launches one by one
        for t in range(args.warmup + n_tok, args.warmup + n_tok + n_prof):
            model.generate_step(state, tokens[:, t])
        per_kernel = {k: round(v[0] / n_prof, 4) for k, v in rt.kernel_times().items() if not k.startswith("(")}
        launches = sum(v[1] for k, v in rt.kernel_times().items() if not k.startswith("(")) / n_prof
        rt.kernel_timing(False)
        line = {"workload": "generate", "model": args.model, "batch": B, "steps": n_tok,
                "context_position": args.warmup + n_tok, "ms_per_step_host_timed": dt * 1e3,
                "tokens_per_s": B / dt, "plain_launch_device_ms_per_step": sum(per_kernel.values()),
                "launches_per_step": launches, "kernels_ms": per_kernel}
        if not args.no_cpu_baseline:
            # the oracle's generate_step (one sequence, the same first tokens) on the host
            from oracle import oracle as O
            O.set_threads(O.max_threads())
            ref = O.HeronOracle(data)
            ref_state = ref.generate_state()
            n_ref = min(32, ctx)
            t0 = time.perf_counter()
            for t in range(n_ref):
                ref.generate_step(ref_state, int(tokens[0, t]))
            ref_dt = (time.perf_counter() - t0) / n_ref
            line["cpu_baseline"] = {"value": 1.0 / ref_dt, "unit": "tokens/s", "cores": O.max_threads(), "kind": "port",
                                    "sample": f"oracle generate_step, 1 sequence, first {n_ref} tokens"}
        print(json.dumps(line))
        state.close()
        model.close()
        rt.close()
        return
    if args.workload == "train":
        # one optimiser step per step: tokens from the host, forward with the tape, backward, updates on the device
        from ullis_b200 import cuda
        d, layers, vocab, ctx, ffn = synth.CONFIGS[args.model]
        B = args.batch
        data = synth.heron_checkpoint(args.model, batch_size=max(B, 1))
        model = cuda.CudaHeron(rt, data)
        state = model.train_state()
        tokens = sequence_tokens(vocab, 0, B, ctx)
        lr = 0.005
        losses = []

        def step():
            losses.append(state.train_step(tokens, tokens, cuda.CE_NO_IGNORE, B, ctx, lr)["loss"])

        dt, per_kernel = timed(step)
        top = dict(sorted(per_kernel.items(), key=lambda kv: -kv[1])[:12])
        line = {"workload": "train", "model": args.model, "batch": B, "time": ctx, "steps": args.steps,
                "learning_rate": lr, "ms_per_step_host_timed": dt * 1e3, "tokens_per_s": B * ctx / dt,
                "device_ms_per_step": sum(per_kernel.values()), "loss_first": losses[0], "loss_last": losses[-1],
                "kernels_ms": {k: round(v, 3) for k, v in top.items()}}
        if not args.no_cpu_baseline:
            # the restated CPU step on one sequence of the same tokens
            from oracle import oracle as O
            from oracle import train as OT
            O.set_threads(O.max_threads())
            ref = OT.HeronTrainer(synth.heron_checkpoint(args.model, batch_size=1))
            t0 = time.perf_counter()
            ref.train_step(tokens[:ctx], tokens[:ctx], O.CE_NO_IGNORE, 1, ctx, lr)
            ref_dt = time.perf_counter() - t0
            line["cpu_baseline"] = {"value": ctx / ref_dt, "unit": "tokens/s", "cores": O.max_threads(), "kind": "port",
                                    "sample": f"restated CPU step (C forward, numpy gradients), 1 sequence of T={ctx}"}
        print(json.dumps(line))
        state.close()
        model.close()
        rt.close()
        return
    if args.workload == "pushers":
        # RosaSam::push at op level: batch x channels streams with the benchmark's kind of bias (a flip every ~50
        # steps on a third of the streams, i.i.d. bits on the rest), pushed up to position T - steps untimed,
        # then `steps` pushes timed: what a step of incremental decoding pays per layer late in the context.
        from ullis_b200 import cuda
        import numpy as np
        B, T, C = args.batch, args.time or 2048, args.channels
        n, steps = B * C, min(args.steps, (args.time or 2048) // 2)
        rng = np.random.default_rng(33)
        pr = rng.choice([0.02, 0.5, 0.98], (1, n))
        q, k, v = ((rng.random((T, n)) < pr).astype(np.uint8) for _ in range(3))
        pushers = cuda.CudaRosaPushers(rt, n, T)
        pushers.push(q[:T - steps], k[:T - steps], v[:T - steps])
        rt.kernel_timing(True)
        t0 = time.perf_counter()
        pushers.push(q[T - steps:], k[T - steps:], v[T - steps:])
        dt = time.perf_counter() - t0
        ms, launches = rt.kernel_times().get("gen_push", (0.0, 0))
        rt.kernel_timing(False)
        print(json.dumps({"workload": "pushers", "streams": n, "position": T - steps, "pushes_timed": steps,
                          "gen_push_ms_per_push": ms / max(launches, 1), "launches": launches,
                          "stream_pushes_per_s": n * launches / (ms * 1e-3) if ms else None,
                          "ms_per_call_host_timed": dt * 1e3}))
        pushers.close()
    elif args.workload == "rosa":
        B, T, C = args.batch, args.time or 8192, args.channels
        gen = synth.rosa_bits_iid if args.rosa_variant == "iid" else synth.rosa_bits_periodic
        q, k, v = gen(21, B, T, C)
        e = synth.f16_bits(0.02 * synth.normal(5, C))
        dt, per_kernel = timed(lambda: rt.rosa_qkv_1bit_fwd(q, k, v, e, B, T, C))
        sam_ms = sum(t for name, t in per_kernel.items() if name.startswith("rosa_") and name != "rosa_emit")
        units = B * T * C
        hbm = float(peaks.get("hbm_gbs", 6650.0))
        print(json.dumps({"workload": "rosa", "variant": args.rosa_variant, "B": B, "T": T, "C": C,
                          "ms_per_call_host_timed": dt * 1e3, "kernels_ms": per_kernel,
                          "automaton_ms": sam_ms, "stream_steps_per_s": units / (sam_ms * 1e-3),
                          "ns_per_stream_step": sam_ms * 1e6 / units,
                          "algorithmic_GBps": ROSA_BYTES_PER_UNIT * units / (sam_ms * 1e-3) / 1e9,
                          "frac_of_hbm_peak": ROSA_BYTES_PER_UNIT * units / (sam_ms * 1e-3) / 1e9 / hbm}))
    else:
        M, K, N = (int(x) for x in args.linear_shape.lower().split("x"))
        x, bits, scale, bias = synth.packed_linear_case(3, M, K, N)
        dt, per_kernel = timed(lambda: rt.binary_linear(x, bits, scale, bias, M, K, N))
        gemm_ms = sum(t for name, t in per_kernel.items() if name.startswith("gemm_") or name == "binary_linear_exact")
        flops = 2.0 * M * K * N
        peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
        print(json.dumps({"workload": "linear", "M": M, "K": K, "N": N, "ms_per_call_host_timed": dt * 1e3,
                          "kernels_ms": per_kernel, "gemm_ms": gemm_ms,
                          "tflops": flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms else None,
                          "frac_of_sustained_peak": flops / (gemm_ms * 1e-3) / 1e12 / peak if gemm_ms else None,
                          "frac_of_burst_peak": flops / (gemm_ms * 1e-3) / 1e12 / float(peaks.get("bf16_tflops", 1590.0))
                          if gemm_ms else None}))
    rt.close()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
