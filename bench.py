#!/usr/bin/env python
"""Benchmark of the attention path on B200: one JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A *step* is one forward + backward pass of packed-varlen causal GQA attention over ONE synthetic
batch (8 sequences, lengths U[512,4096] rescaled to T = 16384, 32 query / 8 key-value heads,
D = 128, bf16 inputs, f32 accumulation), through the C ABI.  ``value`` is the whole-job TFLOP/s
with inputs resident in HBM, counted as algorithmic work: forward 4 D Hq pairs, backward
10 D Hq pairs (five products; what a deterministic backward recomputes is not counted).

With N > 1 (launched under torch.distributed.run) that one batch is cut across the ranks as
``dashmag_b200.sharding.training_plan`` says - whole key-value heads first, read in place through
the tensors' strides; bins of sequences once the heads run out - with no collective on the data
path, and ``value`` is the one workload's FLOPs over the slowest rank's time: strong scaling.

The same line carries, as extra keys: the other benchmark configurations (the windowed packed batch
of T = 65536, the single causal sequence of T = 131072, the small f32 case beside the CPU path, the
reference's own D = 256 shape), the decoding step against a bf16 key-value cache (batch 64, lengths
U[1024,32768], 32 / 8 heads, D = 128) as GB/s of cache read and its host overhead on a short cache,
the rotation and the sampler either side of it, the optional all-gather of the output's head shards
(N > 1), each pass's roofline fraction against MEASURED_PEAKS.json, the end-to-end number with host
buffers, and the CPU oracle timed on the host cores beside it.

``--impl reference`` times the CPU port of the reference's own CPU path (oracle/, f32, every host
thread) on a bounded sample of the same workload; the reference itself is a Rust workspace over
un-vendored crates and cannot be built here.
"""
from __future__ import annotations

import argparse
import ctypes
import dataclasses
import json
import os
import pathlib
import re
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

TRAIN = dict(seqs=8, lo=512, hi=4096, total=16384, hq=32, hkv=8, d=128, window=None, seed=0)      # BASELINE configs[1]
WINDOWED = dict(seqs=16, lo=1024, hi=8192, total=65536, hq=16, hkv=4, d=128, window=4096, seed=4)  # configs[3]
LONG = dict(seqs=1, lo=131072, hi=131072, total=131072, hq=64, hkv=8, d=128, window=None, seed=5)  # configs[4]
SMALL_F32 = dict(lengths=[128, 256], hq=4, hkv=4, d=64)                                            # configs[0]
HEADLINE_256 = dict(seqs=1, lo=6144, hi=6144, total=6144, hq=8, hkv=2, d=256, window=None, seed=6)  # the reference's own benchmark shape
DECODE = dict(b=64, lo=1024, hi=32768, s=32768, hq=32, hkv=8, d=128)                                # configs[2]
DECODE_SHORT = dict(b=8, s=6144, hq=8, hkv=2, d=256, calls=24)   # the reference's host-overhead case


def seq_lengths(n, lo, hi, total, seed):
    """n integers uniform in [lo, hi], rescaled to sum to `total` (floor, then +1 to the first few)."""
    rng = np.random.default_rng(seed)
    raw = rng.integers(lo, hi + 1, size=n).astype(np.float64)
    lens = np.floor(raw * total / raw.sum()).astype(np.int64)
    lens[: total - lens.sum()] += 1
    return lens


def visible_pairs(lens, window=None) -> int:
    """(query, key) pairs a causal packed batch sees, with an optional window of `window` keys back."""
    total = 0
    for n in (int(x) for x in lens):
        if window is None or n <= window + 1:
            total += n * (n + 1) // 2
        else:
            total += (window + 1) * (window + 2) // 2 + (n - window - 1) * (window + 1)
    return total


causal_pairs = visible_pairs


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        m = json.loads(path.read_text())
        return dict(hbm=m["hbm_gbs"], tensor_burst=m["bf16_tflops"], tensor_sustained=m["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, tensor_burst=1590.0, tensor_sustained=1400.0, source="fallback")


def dram_traffic():
    """Bytes of DRAM traffic per launch, per kernel, from the committed table of profiler captures:
    rows `| kernel | workload | bytes | ... |`."""
    table = {}
    path = ROOT / "profiles" / "dram_traffic.md"
    if path.exists():
        for line in path.read_text().splitlines():
            cells = [c.strip() for c in line.strip().strip("|").split("|")]
            if len(cells) >= 3 and re.fullmatch(r"[0-9.]+e?[0-9+]*", cells[2] or "x"):
                table[cells[0].strip("`")] = float(cells[2])
    return table


class ClockSampler:
    """Samples nvidia-smi during the timed region (SM clock, throttle reasons)."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        sm, mx, power, reasons = [], [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # "under load": samples that drew more than half of the largest power seen
        loaded = [s for s, p in zip(sm, power) if power and p >= 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(loaded) if loaded else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_under_load": len(loaded),
                "power_w_max": max(power) if power else None}


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's CPU path
# ---------------------------------------------------------------------------------------------

def bf16_round(x):
    return (x.astype(np.float32).view(np.uint32) + 0x8000 & 0xFFFF0000).view(np.float32)


def cpu_inputs(t, hq, hkv, d, seed, rounded=True):
    rng = np.random.default_rng(seed)
    r = bf16_round if rounded else (lambda x: x.astype(np.float32))
    return (r(rng.standard_normal((1, t, hq, d))), r(rng.standard_normal((1, t, hkv, d))),
            r(rng.standard_normal((1, t, hkv, d))), r(rng.standard_normal((1, t, hq, d))))


def cpu_threads():
    """Every host core this process may run on: launchers such as torch.distributed.run set
    OMP_NUM_THREADS=1, which would time the CPU arm on one thread."""
    from oracle import attention_oracle as oracle
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    oracle.set_threads(n)
    return oracle.threads()


def cpu_step(inputs, **mask):
    from oracle import attention_oracle as oracle
    q, k, v, g = inputs
    o, lse = oracle.forward(q, k, v, causal=True, precise=False, **mask)
    oracle.backward(q, k, v, o, lse, g, causal=True, precise=False, **mask)


def train_lengths(cfg=TRAIN):
    return seq_lengths(cfg["seqs"], cfg["lo"], cfg["hi"], cfg["total"], cfg["seed"])


def cpu_sample():
    """The bounded sample of the training workload the reference arm repeats: the batch's sequence
    of median length, alone, with the batch's heads."""
    lens = train_lengths()
    n = int(sorted(lens)[len(lens) // 2])
    flops = 14 * TRAIN["d"] * TRAIN["hq"] * (n * (n + 1) // 2)
    text = (f"one sequence of the batch (its median length, {n} tokens), {TRAIN['hq']} query / {TRAIN['hkv']} kv heads, "
            f"D {TRAIN['d']}, causal, fwd+bwd, f32 arithmetic on bf16-rounded inputs")
    return cpu_inputs(n, TRAIN["hq"], TRAIN["hkv"], TRAIN["d"], 0), flops, text


def cpu_baseline():
    """The CPU port on the benchmark's own batch IN FULL, sequence by sequence (the eight sequences
    are independent; the port materialises one sequence's scores at a time), once; and the small f32
    configuration in full, 20 runs."""
    from oracle import attention_oracle as oracle
    cores = cpu_threads()
    lens = train_lengths()
    cpu_step(cpu_inputs(256, TRAIN["hq"], TRAIN["hkv"], TRAIN["d"], 1))   # warm the threads
    seconds = 0.0
    for i, n in enumerate(int(x) for x in lens):
        inputs = cpu_inputs(n, TRAIN["hq"], TRAIN["hkv"], TRAIN["d"], 10 + i)
        t0 = time.perf_counter()
        cpu_step(inputs)
        seconds += time.perf_counter() - t0
        del inputs
    flops = 14 * TRAIN["d"] * TRAIN["hq"] * visible_pairs(lens)
    small = cpu_small_f32(runs=20)
    return {"value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"the whole batch of the workload once, its {len(lens)} sequences one after another "
                      f"(lengths {[int(x) for x in lens]}), f32 arithmetic on bf16-rounded inputs",
            "seconds_per_sample": seconds, "small_f32": small}


def small_f32_inputs():
    c = SMALL_F32
    t = sum(c["lengths"])
    cu = np.concatenate([[0], np.cumsum(c["lengths"])]).astype(np.int64)
    return cpu_inputs(t, c["hq"], c["hkv"], c["d"], 3, rounded=False), cu, 14 * c["d"] * c["hq"] * visible_pairs(c["lengths"])


def cpu_small_f32(runs=20):
    inputs, cu, flops = small_f32_inputs()
    cpu_step(inputs, cu_q=cu, cu_k=cu)
    times = []
    for _ in range(runs):
        t0 = time.perf_counter()
        cpu_step(inputs, cu_q=cu, cu_k=cu)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"workload": "two packed causal sequences of 128 and 256 tokens, 4 / 4 heads, D 64, f32, fwd+bwd (BASELINE configs[0]), in full",
            "runs": runs, "ms_median": med * 1e3, "ms_min": min(times) * 1e3, "ms_max": max(times) * 1e3,
            "tflops": flops / med / 1e12}


def workload_config(n, plan_text=None):
    lens = [int(x) for x in train_lengths()]
    return {"workload": "packed-varlen causal GQA attention fwd+bwd, bf16 in / f32 accumulate: 8 sequences, lengths "
                        f"U[512,4096] rescaled to T=16384 ({lens}), Hq 32 / Hkv 8, D 128 (BASELINE configs[1]), "
                        "one batch whatever the number of GPUs",
            "l2": "inputs larger than L2 (a step touches 700 MB; the decode leg 4.5 GB)",
            "parallelism": plan_text or (f"the batch's {TRAIN['hkv']} key-value heads (with their query heads) dealt over {n} GPU(s), "
                                         "every rank all sequences; no collective on the data path"),
            "cpu_sample": cpu_sample()[2] + " (what --impl reference repeats per step; cpu_baseline runs the batch in full)"}


def run_reference(args, rank):
    if rank != 0:
        return
    from oracle import attention_oracle as oracle
    inputs, flops, sample = cpu_sample()
    cores = cpu_threads()
    for _ in range(args.warmup):
        cpu_step(inputs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(inputs)
    dt = (time.perf_counter() - t0) / args.steps
    value = flops / dt / 1e12
    line = {
        "impl": "reference", "metric": "attention_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-decode", action="store_true", help="leave the decode leg out (profiling captures)")
    ap.add_argument("--skip-cpu", action="store_true", help="leave the CPU baseline out (profiling captures)")
    ap.add_argument("--skip-extra", action="store_true", help="leave the other configurations out (profiling captures)")
    ap.add_argument("--no-soak", action="store_true", help="leave the half-second soak out (profiling captures)")
    ap.add_argument("--decode-batch", type=int, default=DECODE["b"], help="decode batch (smaller for captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist

    from dashmag_b200 import _lib, sharding
    from dashmag_b200 import attention as A
    from dashmag_b200.contract import AttentionMask, AttentionOptions
    from dashmag_b200.rope import Rope
    from dashmag_b200.sample import SampleOptions, sample

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the attention path has no CPU fallback")
    lib = _lib.lib()  # fail loudly here if the library is not built
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL prints its version banner to stdout when the communicator comes up: that goes to stderr,
        # so that stdout carries the one JSON line and nothing else.
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier(device_ids=[local_rank])
            torch.cuda.synchronize()
        finally:
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def over_ranks(x: float, op) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=op)
        return float(t.item())

    max_over_ranks = lambda x: over_ranks(x, dist.ReduceOp.MAX)
    sum_over_ranks = lambda x: over_ranks(x, dist.ReduceOp.SUM)
    pk = peaks()
    traffic = dram_traffic()
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def normal(shape, seed, dtype=torch.bfloat16):
        g = torch.Generator(device=dev).manual_seed(seed)
        return torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(dtype)

    class Pass:
        """A forward + backward over fixed buffers, called straight through the C ABI: parameters,
        outputs and workspace are made once, so a step is two library calls and nothing else on the
        host (at eight GPUs a rank's share of the batch is a quarter of a millisecond of kernels)."""

        def __init__(self, q, k, v, g, mask, options):
            self.t = (q, k, v, g)
            self.o = torch.empty(q.shape, dtype=q.dtype, device=dev)
            self.lse = torch.empty(q.shape[:3], dtype=torch.float32, device=dev)
            self.dq, self.dk, self.dv = torch.empty_like(self.o), torch.empty(k.shape, dtype=k.dtype, device=dev), torch.empty(v.shape, dtype=v.dtype, device=dev)
            self.p, self.keep = A.make_params("attention", q, k, v, mask, options, self.o, g)
            need = max(lib.dash_attn_forward_workspace(ctypes.byref(self.p)), lib.dash_attn_backward_workspace(ctypes.byref(self.p)), 256)
            self.ws = torch.empty(need, dtype=torch.uint8, device=dev)
            self.empty = q.numel() == 0

        def forward(self):
            if self.empty:
                return
            q, k, v, g = self.t
            rc = lib.dash_attn_forward(ctypes.byref(self.p), q.data_ptr(), k.data_ptr(), v.data_ptr(), self.o.data_ptr(),
                                       self.lse.data_ptr(), self.ws.data_ptr(), self.ws.numel(), stream())
            if rc != _lib.OK:
                raise RuntimeError(_lib.last_error())

        def backward(self):
            if self.empty:
                return
            q, k, v, g = self.t
            rc = lib.dash_attn_backward(ctypes.byref(self.p), q.data_ptr(), k.data_ptr(), v.data_ptr(), self.o.data_ptr(),
                                        self.lse.data_ptr(), g.data_ptr(), self.dq.data_ptr(), self.dk.data_ptr(), self.dv.data_ptr(),
                                        self.ws.data_ptr(), self.ws.numel(), stream())
            if rc != _lib.OK:
                raise RuntimeError(_lib.last_error())

    def spread(ms):
        return {"min": min(ms), "median": statistics.median(ms), "max": max(ms)}

    def time_passes(work: Pass, steps, warmup):
        """`steps` timed steps after `warmup`: total (start to end, max over ranks) and, per pass,
        the mean and the spread of the per-step event times of this rank."""
        for _ in range(warmup):
            work.forward()
            work.backward()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3 * steps)]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for i in range(steps):
            ev[3 * i].record()
            work.forward()
            ev[3 * i + 1].record()
            work.backward()
            ev[3 * i + 2].record()
        end.record()
        barrier()
        fwd = [ev[3 * i].elapsed_time(ev[3 * i + 1]) for i in range(steps)]
        bwd = [ev[3 * i + 1].elapsed_time(ev[3 * i + 2]) for i in range(steps)]
        step_ms = max_over_ranks(start.elapsed_time(end) / steps)
        return {"ms_per_step": step_ms, "fwd_ms": max_over_ranks(statistics.mean(fwd)), "bwd_ms": max_over_ranks(statistics.mean(bwd)),
                "step_spread_ms": spread([a + b for a, b in zip(fwd, bwd)]), "fwd_spread_ms": spread(fwd), "bwd_spread_ms": spread(bwd)}

    def packed_workload(cfg, deterministic=True):
        """The whole batch of a configuration on this rank's GPU (one seed: the same on every rank)
        and this rank's share of it under the training plan."""
        lens = train_lengths(cfg)
        t, hq, hkv, d = cfg["total"], cfg["hq"], cfg["hkv"], cfg["d"]
        base = 1000 + 10 * cfg["seed"]
        q, k, v, g = normal((1, t, hq, d), base), normal((1, t, hkv, d), base + 1), normal((1, t, hkv, d), base + 2), normal((1, t, hq, d), base + 3)
        plan = sharding.training_plan(lens, hkv, hq // hkv, world, cfg["window"])
        mine, qr, kr, vr, gr = sharding.training_share(plan[rank], lens, q, k, v, g)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(mine)]) if mine else [0], dtype=torch.int32, device=dev)
        options = AttentionOptions.causal_().with_deterministic(deterministic)
        if cfg["window"] is not None:
            options = options.with_window(cfg["window"], 0)
        mask = AttentionMask.packed(cu, cu) if cfg["seqs"] > 1 else AttentionMask.none()
        pairs = visible_pairs(lens, cfg["window"])
        bins = any(list(s) != list(range(len(lens))) for s, _, _ in plan)
        text = (f"{hkv} key-value heads over {world} GPU(s)" + (f", {world // hkv} ranks per head each with a bin of the sequences "
                "(balanced by visible pairs, gathered into packed tensors of their own)" if bins else
                ", head slices read in place through strides") + "; no collective on the data path")
        return dict(full=(q, k, v, g), share=(qr, kr, vr, gr), mask=mask, options=options, lens=lens, pairs=pairs,
                    fwd_flops=4 * d * hq * pairs, bwd_flops=10 * d * hq * pairs, plan=plan, plan_text=text, cu=cu)

    def tensor_roofline(tflops, kernel, traffic_key, note=None):
        out = {"bound": "tensor", "achieved": tflops, "peak": pk["tensor_burst"], "unit": "TFLOP/s",
               "frac": tflops / pk["tensor_burst"], "frac_of_nominal_2250": tflops / 2250.0,
               "frac_of_sustained_peak": tflops / pk["tensor_sustained"],
               "peak_source": pk["source"] + " burst (kernel timed alone)",
               "traffic": traffic.get(traffic_key), "traffic_unit": "DRAM bytes per launch, from the profiler capture of this workload",
               "kernel": kernel}
        if note:
            out["note"] = note
        return out

    def extra_leg(cfg, name, steps, warmup, deterministic=True):
        """Another configuration, cut over the ranks the same way: per-pass times and fractions."""
        w = packed_workload(cfg, deterministic)
        r = time_passes(Pass(*w["share"], w["mask"], w["options"]), steps, warmup)
        fwd_tf = w["fwd_flops"] / (r["fwd_ms"] * 1e-3) / 1e12
        bwd_tf = w["bwd_flops"] / (r["bwd_ms"] * 1e-3) / 1e12
        per_gpu = 1.0 / world
        return {"workload": name, "parallelism": w["plan_text"], "steps": steps, "warmup": warmup, "scaling": "strong",
                "value": (w["fwd_flops"] + w["bwd_flops"]) / (r["ms_per_step"] * 1e-3) / 1e12, "unit": "TFLOP/s",
                "ms_per_step": r["ms_per_step"], "step_spread_ms": r["step_spread_ms"],
                "fwd": {"ms": r["fwd_ms"], "tflops": fwd_tf, "flops": w["fwd_flops"], "frac_of_measured_peak_per_gpu": fwd_tf * per_gpu / pk["tensor_burst"],
                        "frac_of_sustained_peak_per_gpu": fwd_tf * per_gpu / pk["tensor_sustained"]},
                "bwd": {"ms": r["bwd_ms"], "tflops": bwd_tf, "flops": w["bwd_flops"], "frac_of_measured_peak_per_gpu": bwd_tf * per_gpu / pk["tensor_burst"],
                        "frac_of_sustained_peak_per_gpu": bwd_tf * per_gpu / pk["tensor_sustained"]}}

    # ---- the training workload: one batch, this rank's share ----
    c = TRAIN
    w = packed_workload(c)
    work = Pass(*w["share"], w["mask"], w["options"])
    sampler = ClockSampler(local_rank)
    for _ in range(args.warmup):
        work.forward()
        work.backward()
    barrier()
    if rank == 0:
        sampler.start()
    launches0 = _lib.probe("kernel_launches")
    r = time_passes(work, args.steps, 0)
    launches = sum_over_ranks(_lib.probe("kernel_launches") - launches0)
    step_ms, fwd_ms, bwd_ms = r["ms_per_step"], r["fwd_ms"], r["bwd_ms"]
    total_flops = w["fwd_flops"] + w["bwd_flops"]
    value = total_flops / (step_ms * 1e-3) / 1e12
    # The same step back to back for at least half a second: long enough for the clock sampler to see
    # the GPU under this load, and for the power cap to bite if it is going to.
    soak_steps = args.steps if args.no_soak else max(args.steps, int(0.6 / (step_ms * 1e-3)) + 1)
    soak = time_passes(work, soak_steps, 0)
    clocks = sampler.stop() if rank == 0 else None
    soak_leg = {"steps": soak_steps, "ms_per_step": soak["ms_per_step"], "value": total_flops / (soak["ms_per_step"] * 1e-3) / 1e12,
                "unit": "TFLOP/s", "step_spread_ms": soak["step_spread_ms"], "fwd_ms": soak["fwd_ms"], "bwd_ms": soak["bwd_ms"]}

    # ---- the other way of summing the query gradient (deterministic = false) ----
    atomic_leg = None
    a0 = _lib.probe("atomic_runs")
    wa = Pass(*w["share"], w["mask"], w["options"].with_deterministic(False))
    ra = time_passes(wa, max(args.steps, 10), 3)
    if _lib.probe("atomic_runs") > a0:
        atf = w["bwd_flops"] / (ra["bwd_ms"] * 1e-3) / 1e12
        atomic_leg = {"ms": ra["bwd_ms"], "tflops": atf, "spread_ms": ra["bwd_spread_ms"],
                      "roofline": tensor_roofline(atf / world, "backward pass with the query gradient added by atomics: five products", "bwd_atomic")}
    del wa

    # ---- end to end through the public API: host buffers in, results back to the host, every step ----
    # Each rank holds ITS share of the batch in pinned host memory (head slices made contiguous: what a
    # rank that owns those heads holds) and copies that in and its results out.  The three legs run on
    # three streams over two sets of device inputs, so that the copy-in of step i + 1 and the copy-out
    # of step i - 1 overlap the kernels of step i (PCIe is full duplex).
    names = ("q", "k", "v", "do")
    host = {n: t.contiguous().cpu().pin_memory() for n, t in zip(names, w["share"])}
    host_out = {n: torch.empty_like(host[s]).pin_memory() for n, s in (("o", "q"), ("dq", "q"), ("dk", "k"), ("dv", "v"))}
    host_lse = torch.empty(host["q"].shape[:3], dtype=torch.float32).pin_memory()
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dev_in = [{n: torch.empty_like(host[n], device=dev) for n in names} for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    mask, options = w["mask"], w["options"]

    def train_step_e2e(i):
        cur = torch.cuda.current_stream(dev)
        buf = dev_in[i % 2]
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[i % 2])          # the kernels of step i - 2 have read this set
            for n in names:
                buf[n].copy_(host[n], non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(s_in)
        cur.wait_event(ready)
        if buf["q"].numel():
            o, lse = A.attention_with_lse(buf["q"], buf["k"], buf["v"], mask, options)
            gq, gk, gv = A.attention_backward(buf["q"], buf["k"], buf["v"], o, lse, buf["do"], mask, options)
        else:
            o, lse, gq, gk, gv = buf["q"], host_lse.to(dev), buf["q"], buf["k"], buf["v"]
        in_free[i % 2].record(cur)
        done = torch.cuda.Event()
        done.record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            for dst, src in ((host_out["o"], o), (host_lse, lse), (host_out["dq"], gq), (host_out["dk"], gk), (host_out["dv"], gv)):
                dst.copy_(src, non_blocking=True)
                src.record_stream(s_out)

    for i in range(2):
        train_step_e2e(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        train_step_e2e(i)
    torch.cuda.current_stream(dev).wait_stream(s_out)
    torch.cuda.current_stream(dev).wait_stream(s_in)
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    h2d = sum_over_ranks(sum(host[n].numel() * 2 for n in names))
    d2h = sum_over_ranks(sum(t.numel() * 2 for t in host_out.values()) + host_lse.numel() * 4)
    del host_out, dev_in, host

    # ---- the one optional collective: the output's head shards gathered onto every rank ----
    gather_leg = None
    if world > 1 and all(list(s) == list(range(len(w["lens"]))) for s, _, _ in w["plan"]):
        work.forward()
        group = c["hq"] // c["hkv"]
        whole = sharding.all_gather_heads(work.o, c["hq"], group)
        full = Pass(*w["full"], w["mask"], w["options"])
        full.forward()
        torch.cuda.synchronize(dev)
        same = bool(torch.equal(whole, full.o))
        del full
        for _ in range(3):
            sharding.all_gather_heads(work.o, c["hq"], group)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(10):
            sharding.all_gather_heads(work.o, c["hq"], group)
        g1.record()
        barrier()
        g_ms = max_over_ranks(g0.elapsed_time(g1) / 10)
        out_bytes = whole.numel() * 2
        gather_leg = {"what": "all_gather_heads of the forward's output [1, T, Hq, D] (one all_gather_into_tensor over NCCL, plus the "
                              "copies that pad and reassemble the shards), only for callers that want the whole output on every rank",
                      "ms": g_ms, "bytes_gathered": out_bytes, "bus_gbs": out_bytes * (world - 1) / world / (g_ms * 1e-3) / 1e9,
                      "share_of_a_step": g_ms / step_ms, "bit_equal_to_the_unsharded_forward": same}
        del whole

    # ---- the other configurations ----
    extra = {}
    if not args.skip_extra:
        extra["windowed_t65536"] = extra_leg(WINDOWED, "packed causal, window 4096: 16 sequences, lengths U[1024,8192] rescaled to T=65536, "
                                             "Hq 16 / Hkv 4, D 128, bf16 (BASELINE configs[3]); pairs counted inside the window", max(args.steps // 2, 5), 3)
        extra["long_t131072"] = extra_leg(LONG, "one causal sequence of T=131072, Hq 64 / Hkv 8, D 128, bf16 (BASELINE configs[4]), cut by key-value head", 2, 1)
        if world == 1:
            extra["d256_t6144"] = extra_leg(HEADLINE_256, "one causal sequence of T=6144, Hq 8 / Hkv 2, D 256, bf16: the shape of the reference's own published "
                                            "numbers (crates/dash-ops/src/attention.rs:111-117: backward 6.70 ms on an RTX 5070 Ti)", 10, 3)
            # the small f32 configuration on the generic (IEEE f32) kernels, beside the CPU port's time for it
            (q32, k32, v32, g32), cu32, flops32 = small_f32_inputs()
            t32 = [torch.from_numpy(x).to(dev) for x in (q32, k32, v32, g32)]
            cu_t = torch.tensor(cu32, dtype=torch.int32, device=dev)
            small = Pass(*t32, AttentionMask.packed(cu_t, cu_t), AttentionOptions.causal_())
            rs = time_passes(small, 50, 5)
            extra["small_f32"] = {"workload": "two packed causal sequences of 128 and 256 tokens, 4 / 4 heads, D 64, f32, fwd+bwd (BASELINE configs[0]) "
                                              "on the f32 kernels", "ms_per_step": rs["ms_per_step"], "step_spread_ms": rs["step_spread_ms"],
                                  "tflops": flops32 / (rs["ms_per_step"] * 1e-3) / 1e12, "note": "launch-bound: five kernels of a few microseconds"}
            del small, t32

    # ---- rotation of the step's query and key (the prologue in front of the attention call) ----
    q, k = w["share"][0], w["share"][1]
    rope_leg = None
    if q.numel():
        qc, kc_ = q.contiguous(), k.contiguous()
        rope = Rope(c["d"], 10000.0, int(max(w["lens"])), torch.bfloat16, device=dev)
        for _ in range(3):
            rope.apply_packed(qc, w["cu"], other=kc_)
        barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        rope_reps = max(args.steps, 10)
        rl0 = _lib.probe("kernel_launches")
        r0.record()
        for _ in range(rope_reps):
            rope.apply_packed(qc, w["cu"], other=kc_)
        r1.record()
        barrier()
        rope_launches = _lib.probe("kernel_launches") - rl0
        rope_ms = max_over_ranks(r0.elapsed_time(r1) / rope_reps)
        rope_bytes = sum_over_ranks(2 * 2 * (qc.numel() + kc_.numel()))   # each read once and written once
        rope_gbs = rope_bytes / (rope_ms * 1e-3) / 1e9
        rope_leg = {
            "metric": "rope_qk_bytes_moved", "value": rope_gbs, "unit": "GB/s", "ms_per_step": rope_ms,
            "bytes_per_step": rope_bytes, "gpu_launches_per_step": rope_launches / rope_reps,
            "roofline": {"bound": "hbm", "achieved": rope_gbs / world, "peak": pk["hbm"], "unit": "GB/s",
                         "frac": rope_gbs / world / pk["hbm"], "traffic": traffic.get("rope_kernel"),
                         "traffic_unit": "DRAM bytes per launch at one GPU, from the profiler capture of this workload",
                         "kernel": "rope_kernel (1 launch rotates Q and K)"},
        }
        del qc, kc_
    del work, w, q, k

    # ---- decoding leg: the batch dealt over the ranks by cache length ----
    decode = None
    dec_ms = None
    if not args.skip_decode:
        dcfg = dict(DECODE, b=args.decode_batch)
        dl_all = np.random.default_rng(77).integers(dcfg["lo"], dcfg["hi"] + 1, size=dcfg["b"])
        mine = sharding.decode_plan(dl_all, world)[rank]
        dl = dl_all[mine]
        nb = len(mine)
        lengths = torch.tensor(dl, dtype=torch.int32, device=dev)
        g2 = torch.Generator(device=dev).manual_seed(2000 + rank)
        shape = (nb, dcfg["s"], dcfg["hkv"], dcfg["d"])
        kc = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        vc = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        for t in (kc, vc):  # filled in slices: no f32 temporary of the whole cache
            for b0 in range(0, nb, 8):
                t[b0:b0 + 8] = torch.randn((min(8, nb - b0),) + shape[1:], generator=g2, device=dev, dtype=torch.float32).to(torch.bfloat16)
        qd_host = torch.randn((nb, dcfg["hq"], dcfg["d"]), dtype=torch.float32).to(torch.bfloat16).pin_memory()
        qd = qd_host.to(dev)
        out_host = torch.empty_like(qd_host).pin_memory()
        dec_bytes = sum_over_ranks(int(dl.sum()) * dcfg["hkv"] * dcfg["d"] * 2 * 2)
        dec_options = AttentionOptions()
        # Between passes the cache itself evicts L2 (a pass reads tens of times its 126 MB).
        for _ in range(max(args.warmup, 3)):
            A.attention_decode(qd, kc, vc, lengths, dec_options)
        barrier()
        reps = max(args.steps, 10)
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dl0 = _lib.probe("kernel_launches")
        d0.record()
        for _ in range(reps):
            A.attention_decode(qd, kc, vc, lengths, dec_options)
        d1.record()
        barrier()
        dec_launches = _lib.probe("kernel_launches") - dl0
        dec_ms = max_over_ranks(d0.elapsed_time(d1) / reps)
        # end to end: the cache is resident state of the decoder; the step's inputs are the queries
        d0.record()
        for _ in range(reps):
            out = A.attention_decode(qd_host.to(dev, non_blocking=True), kc, vc, lengths, dec_options)
            out_host.copy_(out, non_blocking=True)
        d1.record()
        barrier()
        dec_e2e_ms = max_over_ranks(d0.elapsed_time(d1) / reps)
        gbs = dec_bytes / (dec_ms * 1e-3) / 1e9
        scale = traffic.get("decode_traffic_over_algorithmic", None)
        decode = {
            "metric": "decode_cache_read", "value": gbs, "unit": "GB/s", "ms_per_step": dec_ms, "scaling": "strong",
            "parallelism": f"the batch's {dcfg['b']} sequences dealt over {world} GPU(s), balanced by cache length; no collective",
            "bytes_per_step": dec_bytes, "gpu_launches_per_step": dec_launches / reps,
            "e2e": {"value": dec_bytes / (dec_e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": sum_over_ranks(qd_host.numel() * 2), "d2h_bytes_per_step": sum_over_ranks(out_host.numel() * 2)},
            "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": pk["hbm"], "unit": "GB/s",
                         "frac": gbs / world / pk["hbm"], "frac_of_nominal_8TBs": gbs / world / 8000.0,
                         "traffic": None if scale is None else dec_bytes / world * scale,
                         "traffic_unit": "DRAM bytes per pass: the profiler's ratio of traffic to algorithmic bytes at batch 8, times this pass's bytes",
                         "kernels": "decode_split_mma_kernel + decode_merge_kernel (pass-level)"},
        }
        del kc, vc
        # Host overhead of a short decoding step (crates/dash-ops/src/attention.rs:123-127,
        # examples/attention_bench.rs:58-73): wall clock over back-to-back calls beside the device's time.
        if rank == 0:
            sc = DECODE_SHORT
            qs, ks, vs = normal((sc["b"], sc["hq"], sc["d"]), 31), normal((sc["b"], sc["s"], sc["hkv"], sc["d"]), 32), normal((sc["b"], sc["s"], sc["hkv"], sc["d"]), 33)
            for _ in range(5):
                A.attention_decode(qs, ks, vs, None, dec_options)
            torch.cuda.synchronize(dev)
            h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            enc0 = _lib.probe("tensor_map_encodes")
            t0 = time.perf_counter()
            h0.record()
            for _ in range(sc["calls"]):
                A.attention_decode(qs, ks, vs, None, dec_options)
            t_issue = time.perf_counter() - t0
            h1.record()
            torch.cuda.synchronize(dev)
            wall = time.perf_counter() - t0
            decode["host_overhead"] = {"workload": f"B {sc['b']}, S {sc['s']}, Hq {sc['hq']} / Hkv {sc['hkv']}, D {sc['d']}, bf16, {sc['calls']} calls back to back "
                                                   "through the Python entry point (allocation of the output and the workspace included)",
                                       "wall_us_per_call": wall / sc["calls"] * 1e6, "host_issue_us_per_call": t_issue / sc["calls"] * 1e6,
                                       "device_us_per_call": h0.elapsed_time(h1) / sc["calls"] * 1e3,
                                       "tensor_maps_encoded": _lib.probe("tensor_map_encodes") - enc0}
            del qs, ks, vs
        barrier()

    # ---- sampling the next token from the decoding step's logits ----
    scfg = dict(b=max(DECODE["b"] // world, 1), v=151936)
    zl = (torch.randn((scfg["b"], scfg["v"]), generator=torch.Generator(device=dev).manual_seed(3000 + rank), device=dev) * 3).to(torch.bfloat16)
    sample_leg = {"workload": f"logits [{scfg['b']} per GPU, {scfg['v']}] bf16, N(0, 3): every token within reach of the draw (the worst case)",
                  "bound": "instruction issue (a quarter of a Philox call and up to three logarithms per kept token); the logits come from L2 after the first pass"}
    for name, so in (("plain", SampleOptions(seed=1)), ("t0.7_k50_p0.9", SampleOptions(temperature=0.7, top_k=50, top_p=0.9, seed=1))):
        for _ in range(3):
            sample(zl, so)
        barrier()
        q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sreps = max(args.steps, 10)
        sl0 = _lib.probe("kernel_launches")
        q0.record()
        for i in range(sreps):
            sample(zl, dataclasses.replace(so, offset=i))
        q1.record()
        barrier()
        s_ms = max_over_ranks(q0.elapsed_time(q1) / sreps)
        sample_leg[name] = {"ms_per_step": s_ms, "tokens_per_s": sum_over_ranks(scfg["b"]) / (s_ms * 1e-3),
                            "gpu_launches_per_step": (_lib.probe("kernel_launches") - sl0) / sreps,
                            "ns_per_logit": s_ms * 1e6 / (scfg["b"] * scfg["v"]),
                            "share_of_the_decoding_step_it_follows": None if dec_ms is None else s_ms / dec_ms}
    del zl

    if rank == 0:
        fwd_tf = total_flops * 4 / 14 / (fwd_ms * 1e-3) / 1e12
        bwd_tf = total_flops * 10 / 14 / (bwd_ms * 1e-3) / 1e12
        line = {
            "metric": "attention_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world),
            "step_spread_ms": r["step_spread_ms"],
            "fwd": {"ms": fwd_ms, "tflops": fwd_tf, "flops": total_flops * 4 // 14, "spread_ms": r["fwd_spread_ms"]},
            "bwd": {"ms": bwd_ms, "tflops": bwd_tf, "flops": total_flops * 10 // 14, "spread_ms": r["bwd_spread_ms"], "deterministic": True},
            "bwd_atomic": atomic_leg,
            "soak": soak_leg,
            "e2e": {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "what": "attention_with_lse + attention_backward on each rank's share, inputs from and results to pinned host memory every step"},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": tensor_roofline(fwd_tf / world, "fwd2_sm100_kernel (1 launch per pass)", "fwd2_sm100_kernel"),
            "roofline_backward": tensor_roofline(bwd_tf / world, "backward pass: delta_rows + bwd_dq_sm100 + bwd_plan + bwd_dkdv_sm100", "bwd_pass"),
            "gather": gather_leg,
            "configs": extra,
            "rope": rope_leg,
            "sample": sample_leg,
            "decode": decode,
            "cpu_baseline": None if (args.skip_cpu or world > 1) else cpu_baseline(),
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
