#!/usr/bin/env python
"""Benchmark of the attention path on B200: one JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A *step* is one forward + backward pass of packed-varlen causal GQA attention over one synthetic
batch (8 sequences, lengths U[512,4096] rescaled to T = 16384, 32 query / 8 key-value heads,
D = 128, bf16 inputs, f32 accumulation), through the C ABI.  ``value`` is the whole-job
TFLOP/s with inputs resident in HBM, counted as algorithmic work: forward 4 D Hq pairs, backward
10 D Hq pairs (five products; what a deterministic backward recomputes is not counted).  The same
line carries the decoding step against a bf16 key-value cache (batch 64, lengths U[1024,32768],
32 / 8 heads, D = 128) as GB/s of cache read, the rotation of the step's query and key in front of
the attention call as GB/s moved, each pass's roofline fraction against
MEASURED_PEAKS.json, the end-to-end number with host buffers, and the CPU oracle timed on the host
cores beside it.

With N > 1 (launched under torch.distributed.run) every rank runs its own batch - the path's units
(sequence x head, batch x kv-head) are independent, so there is no data-path collective - and the
reported time is the maximum over ranks: weak scaling.

``--impl reference`` times the CPU port of the reference's own CPU path (oracle/, f32, every host
thread) on a bounded sample of the same workload; the reference itself is a Rust workspace over
un-vendored crates and cannot be built here.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

TRAIN = dict(seqs=8, lo=512, hi=4096, total=16384, hq=32, hkv=8, d=128)
ROPE_TRAFFIC = 291.1e6  # dram read + write of one rope_kernel launch on config 2 (profiles/rope_kernel_config2.md)
DECODE = dict(b=64, lo=1024, hi=32768, s=32768, hq=32, hkv=8, d=128)


def seq_lengths(n, lo, hi, total, seed):
    """n integers uniform in [lo, hi], rescaled to sum to `total` (floor, then +1 to the first few)."""
    rng = np.random.default_rng(seed)
    raw = rng.integers(lo, hi + 1, size=n).astype(np.float64)
    lens = np.floor(raw * total / raw.sum()).astype(np.int64)
    lens[: total - lens.sum()] += 1
    return lens


def causal_pairs(lens) -> int:
    return int(sum(int(l) * (int(l) + 1) // 2 for l in lens))


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        m = json.loads(path.read_text())
        return dict(hbm=m["hbm_gbs"], tensor_burst=m["bf16_tflops"], tensor_sustained=m["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, tensor_burst=1590.0, tensor_sustained=1400.0, source="fallback")


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
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
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
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's CPU path on a bounded sample of the workload
# ---------------------------------------------------------------------------------------------

def cpu_sample_inputs(seed=0):
    """One sequence of 4096 tokens with the training batch's heads (32 query / 8 key-value, D 128)."""
    t, hq, hkv, d = 4096, TRAIN["hq"], TRAIN["hkv"], TRAIN["d"]
    rng = np.random.default_rng(seed)
    bf16 = lambda x: (x.astype(np.float32).view(np.uint32) + 0x8000 & 0xFFFF0000).view(np.float32)
    q, g = bf16(rng.standard_normal((1, t, hq, d))), bf16(rng.standard_normal((1, t, hq, d)))
    k, v = bf16(rng.standard_normal((1, t, hkv, d))), bf16(rng.standard_normal((1, t, hkv, d)))
    flops = 14 * d * hq * (t * (t + 1) // 2)
    return (q, k, v, g), flops, f"1 sequence of {t} tokens, {hq} query / {hkv} kv heads, D {d}, causal, fwd+bwd, f32"


def cpu_threads():
    """Every host core this process may run on: launchers such as torch.distributed.run set
    OMP_NUM_THREADS=1, which would time the CPU arm on one thread."""
    from oracle import attention_oracle as oracle
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    oracle.set_threads(n)
    return oracle.threads()


def cpu_step(inputs):
    from oracle import attention_oracle as oracle
    q, k, v, g = inputs
    o, lse = oracle.forward(q, k, v, causal=True, precise=False)
    oracle.backward(q, k, v, o, lse, g, causal=True, precise=False)


def cpu_baseline(reps=2):
    from oracle import attention_oracle as oracle
    inputs, flops, sample = cpu_sample_inputs()
    cpu_threads()
    cpu_step(inputs)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        cpu_step(inputs)
        times.append(time.perf_counter() - t0)
    best = statistics.median(times)
    return {"value": flops / best / 1e12, "unit": "TFLOP/s", "cores": oracle.threads(), "kind": "port",
            "sample": sample, "seconds_per_sample": best}


def run_reference(args, rank):
    if rank != 0:
        return
    from oracle import attention_oracle as oracle
    inputs, flops, sample = cpu_sample_inputs()
    cpu_threads()
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
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": oracle.threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(n):
    return {"workload": "packed-varlen causal GQA attention fwd+bwd, bf16 in / f32 accumulate: 8 sequences, lengths "
                        "U[512,4096] rescaled to T=16384, Hq 32 / Hkv 8, D 128 (BASELINE configs[1]); decode leg: "
                        "B 64, cache lengths U[1024,32768], Hq 32 / Hkv 8, D 128, bf16 cache (configs[2])",
            "l2": "inputs larger than L2 (train step touches 700 MB, decode 4.5 GB)",
            "parallelism": f"{n} independent batches, one per GPU, no collective"}


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-decode", action="store_true", help="leave the decode leg out (profiling captures)")
    ap.add_argument("--skip-cpu", action="store_true", help="leave the CPU baseline out (profiling captures)")
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

    from dashmag_b200 import _lib
    from dashmag_b200 import attention as A
    from dashmag_b200.contract import AttentionMask, AttentionOptions
    from dashmag_b200.rope import Rope
    from dashmag_b200.sample import SampleOptions, sample

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the attention path has no CPU fallback")
    _lib.lib()  # fail loudly here if the library is not built
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

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    pk = peaks()
    # ---- training workload (this rank's batch) ----
    c = TRAIN
    lens = seq_lengths(c["seqs"], c["lo"], c["hi"], c["total"], seed=rank)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=dev)
    pairs = causal_pairs(lens)
    fwd_flops = 4 * c["d"] * c["hq"] * pairs
    bwd_flops = 10 * c["d"] * c["hq"] * pairs
    gen = torch.Generator(device="cpu").manual_seed(1000 + rank)
    host = {}
    for name, heads in (("q", c["hq"]), ("k", c["hkv"]), ("v", c["hkv"]), ("do", c["hq"])):
        host[name] = torch.randn((1, c["total"], heads, c["d"]), generator=gen, dtype=torch.float32).to(torch.bfloat16).pin_memory()
    q, k, v, g = (host[n].to(dev) for n in ("q", "k", "v", "do"))
    mask = AttentionMask.packed(cu, cu)
    options = AttentionOptions.causal_()
    host_out = {n: torch.empty_like(host[s]).pin_memory() for n, s in (("o", "q"), ("dq", "q"), ("dk", "k"), ("dv", "v"))}
    host_lse = torch.empty((1, c["total"], c["hq"]), dtype=torch.float32).pin_memory()

    def train_step():
        o, lse = A.attention_with_lse(q, k, v, mask, options)
        return (o, lse) + tuple(A.attention_backward(q, k, v, o, lse, g, mask, options))

    # End to end: every step copies its inputs from pinned host memory and its results back.  The
    # three legs run on three streams over two sets of device input buffers, so that the copy-in of
    # step i + 1 and the copy-out of step i - 1 overlap the kernels of step i (PCIe is full duplex).
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dev_in = [{n: torch.empty_like(host[n], device=dev) for n in ("q", "k", "v", "do")} for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]

    def train_step_e2e(i):
        cur = torch.cuda.current_stream(dev)
        buf = dev_in[i % 2]
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[i % 2])          # the kernels of step i - 2 have read this set
            for n in ("q", "k", "v", "do"):
                buf[n].copy_(host[n], non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(s_in)
        cur.wait_event(ready)
        o, lse = A.attention_with_lse(buf["q"], buf["k"], buf["v"], mask, options)
        gq, gk, gv = A.attention_backward(buf["q"], buf["k"], buf["v"], o, lse, buf["do"], mask, options)
        in_free[i % 2].record(cur)
        done = torch.cuda.Event()
        done.record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            for dst, src in ((host_out["o"], o), (host_lse, lse), (host_out["dq"], gq), (host_out["dk"], gk), (host_out["dv"], gv)):
                dst.copy_(src, non_blocking=True)
                src.record_stream(s_out)

    for _ in range(args.warmup):
        train_step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.probe("kernel_launches")
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3 * args.steps)]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for i in range(args.steps):
        ev[3 * i].record()
        o, lse = A.attention_with_lse(q, k, v, mask, options)
        ev[3 * i + 1].record()
        A.attention_backward(q, k, v, o, lse, g, mask, options)
        ev[3 * i + 2].record()
    end.record()
    barrier()
    launches = _lib.probe("kernel_launches") - launches0
    clocks = sampler.stop() if rank == 0 else None
    step_ms = max_over_ranks(start.elapsed_time(end) / args.steps)
    fwd_ms = statistics.mean(ev[3 * i].elapsed_time(ev[3 * i + 1]) for i in range(args.steps))
    bwd_ms = statistics.mean(ev[3 * i + 1].elapsed_time(ev[3 * i + 2]) for i in range(args.steps))
    total_flops = sum_over_ranks(fwd_flops + bwd_flops)
    value = total_flops / (step_ms * 1e-3) / 1e12

    # end to end: host buffers in, results back to the host, every step
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
    h2d = sum(host[n].numel() * 2 for n in ("q", "k", "v", "do"))
    d2h = sum(t.numel() * 2 for t in host_out.values()) + host_lse.numel() * 4
    del host_out, dev_in

    # ---- rotation of the step's query and key (the prologue in front of the attention call) ----
    rope = Rope(c["d"], 10000.0, int(max(lens)), torch.bfloat16, device=dev)
    for _ in range(3):
        rope.apply_packed(q, cu, other=k)
    barrier()
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    rope_reps = max(args.steps, 10)
    rl0 = _lib.probe("kernel_launches")
    r0.record()
    for _ in range(rope_reps):
        rope.apply_packed(q, cu, other=k)
    r1.record()
    barrier()
    rope_launches = _lib.probe("kernel_launches") - rl0
    rope_ms = max_over_ranks(r0.elapsed_time(r1) / rope_reps)
    rope_bytes = 2 * 2 * (q.numel() + k.numel())   # each read once and written once
    rope_gbs = sum_over_ranks(rope_bytes) / (rope_ms * 1e-3) / 1e9
    rope_leg = {
        "metric": "rope_qk_bytes_moved", "value": rope_gbs, "unit": "GB/s", "ms_per_step": rope_ms,
        "bytes_per_step": rope_bytes, "gpu_launches_per_step": rope_launches / rope_reps,
        "roofline": {"bound": "hbm", "achieved": rope_gbs / world, "peak": pk["hbm"], "unit": "GB/s",
                     "frac": rope_gbs / world / pk["hbm"],
                     # dram read + write of one launch, ncu capture of this workload (profiles/rope_kernel_config2.md)
                     "traffic": ROPE_TRAFFIC, "traffic_unit": "bytes per launch",
                     "kernel": "rope_kernel (1 launch rotates Q and K)"},
    }

    # ---- sampling the next token from the decoding step's logits ----
    scfg = dict(b=DECODE["b"], v=151936)
    zl = (torch.randn((scfg["b"], scfg["v"]), generator=torch.Generator(device=dev).manual_seed(3000 + rank), device=dev) * 3).to(torch.bfloat16)
    sample_leg = {"workload": f"logits [{scfg['b']}, {scfg['v']}] bf16, N(0, 3): every token within reach of the draw (the worst case)"}
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
        s_bytes = zl.numel() * 2
        sample_leg[name] = {"ms_per_step": s_ms, "tokens_per_s": sum_over_ranks(scfg["b"]) / (s_ms * 1e-3),
                            "gpu_launches_per_step": (_lib.probe("kernel_launches") - sl0) / sreps,
                            # the logits are read from L2 after the first pass: the kernel is bound by the
                            # generator's and the logarithms' instructions, not by HBM; the fraction says so
                            "roofline": {"bound": "hbm", "achieved": s_bytes / (s_ms * 1e-3) / 1e9, "peak": pk["hbm"], "unit": "GB/s",
                                         "frac": s_bytes / (s_ms * 1e-3) / 1e9 / pk["hbm"],
                                         # dram read of one launch = the logits once (profiles/sample_kernel_batch64.md)
                                         "traffic": 19.53e6, "traffic_unit": "bytes per launch",
                                         "kernel": "sample_kernel (1 launch, a cluster of blocks per row)"}}
    del zl

    # ---- decoding leg ----
    decode = None
    if not args.skip_decode:
        dcfg = dict(DECODE, b=args.decode_batch)
        rng = np.random.default_rng(77 + rank)
        dl = rng.integers(dcfg["lo"], dcfg["hi"] + 1, size=dcfg["b"])
        lengths = torch.tensor(dl, dtype=torch.int32, device=dev)
        g2 = torch.Generator(device=dev).manual_seed(2000 + rank)
        shape = (dcfg["b"], dcfg["s"], dcfg["hkv"], dcfg["d"])
        kc = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        vc = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        for t in (kc, vc):  # filled in slices: no f32 temporary of the whole cache
            for b0 in range(0, dcfg["b"], 8):
                t[b0:b0 + 8] = torch.randn((min(8, dcfg["b"] - b0),) + shape[1:], generator=g2, device=dev, dtype=torch.float32).to(torch.bfloat16)
        qd_host = torch.randn((dcfg["b"], dcfg["hq"], dcfg["d"]), dtype=torch.float32).to(torch.bfloat16).pin_memory()
        qd = qd_host.to(dev)
        out_host = torch.empty_like(qd_host).pin_memory()
        dec_bytes = int(dl.sum()) * dcfg["hkv"] * dcfg["d"] * 2 * 2
        dec_options = AttentionOptions()
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
        total_dec_bytes = sum_over_ranks(dec_bytes)
        gbs = total_dec_bytes / (dec_ms * 1e-3) / 1e9
        decode = {
            "metric": "decode_cache_read", "value": gbs, "unit": "GB/s", "ms_per_step": dec_ms,
            "bytes_per_step": dec_bytes, "gpu_launches_per_step": dec_launches / reps,
            "e2e": {"value": total_dec_bytes / (dec_e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": qd_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 2},
            "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": pk["hbm"], "unit": "GB/s",
                         "frac": gbs / world / pk["hbm"], "frac_of_nominal_8TBs": gbs / world / 8000.0,
                         # ncu at batch 8 read 1.011 x the algorithmic bytes; traffic grows with the cache read
                         # (profiles/decode_split_mma_batch8.md)
                         "traffic": dec_bytes * 1.011, "traffic_unit": "bytes per pass (scaled from the batch-8 capture)",
                         "kernels": "decode_split_mma_kernel + decode_merge_kernel (pass-level)"},
        }
        del kc, vc

    if rank == 0:
        fwd_tf = fwd_flops / (fwd_ms * 1e-3) / 1e12
        bwd_tf = bwd_flops / (bwd_ms * 1e-3) / 1e12
        tensor_peak = pk["tensor_burst"]
        line = {
            "metric": "attention_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world),
            "fwd": {"ms": fwd_ms, "tflops": fwd_tf, "flops": fwd_flops},
            "bwd": {"ms": bwd_ms, "tflops": bwd_tf, "flops": bwd_flops},
            "e2e": {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": fwd_tf, "peak": tensor_peak, "unit": "TFLOP/s",
                         "frac": fwd_tf / tensor_peak, "frac_of_nominal_2250": fwd_tf / 2250.0,
                         "frac_of_sustained_peak": fwd_tf / pk["tensor_sustained"],
                         "peak_source": pk["source"] + " burst (kernel timed alone)",
                         # dram read + write of one launch, ncu capture of this workload (profiles/fwd2_sm100_config2.md)
                         "traffic": 307.8e6, "traffic_unit": "bytes per launch",
                         "kernel": "fwd2_sm100_kernel (1 launch per pass)"},
            "roofline_backward": {"bound": "tensor", "achieved": bwd_tf, "peak": tensor_peak, "unit": "TFLOP/s",
                                  "frac": bwd_tf / tensor_peak, "frac_of_nominal_2250": bwd_tf / 2250.0,
                                  "frac_of_sustained_peak": bwd_tf / pk["tensor_sustained"],
                                  # delta 0.27 GB + dq 0.45 GB + dkdv 0.99 GB (profiles/bwd_*_config2.md)
                                  "traffic": 1.71e9, "traffic_unit": "bytes per pass",
                                  "kernel": "backward pass: delta_rows + bwd_dq_sm100 + bwd_plan + bwd_dkdv_sm100"},
            "rope": rope_leg,
            "sample": sample_leg,
            "decode": decode,
            "cpu_baseline": None if args.skip_cpu else cpu_baseline(),
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
