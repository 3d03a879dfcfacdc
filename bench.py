#!/usr/bin/env python
"""Benchmark of the quantized projection hot path on B200.

Headline workload (all N): the FP8 LM head with fused greedy argmax of the third benchmark
configuration -- K = 5120, vocabulary 248320, M decode tokens (default 1), E4M3 weights
~N(0, 0.02) with one BF16 scale per row, BF16 hidden ~N(0, 1), fp32 logits + int32 argmax
out -- the largest single-GPU configuration of the path and the one that shards: the
vocabulary is split contiguously over the N ranks, every rank streams its shard once per
step and the per-shard (max, index) pairs are exchanged over NVLink and merged.

One step = quantise the hidden rows + stream the weight shard through the tcgen05
projection kernel, whose last CTA to finish unpacks the maxima (N = 1) or exchanges them with
the peers over NVLink and merges (N > 1): two kernel launches per step.

  value     whole-job algorithmic GB/s with the hidden rows resident in HBM, from EXACTLY
            `--steps` graph replays between two barriers (max over ranks)
  protocol  the same step timed the way the reference times its operators
            (qual/src/device_benchmark.rs:993-1101): 40 samples, median / p10 / p90
  e2e       the same through the public operator call with HOST buffers: pinned-host ->
            device copy of the hidden rows and device -> host read of the argmax pairs
            inside the timed region, one stream synchronisation per step (graph replay, and
            `e2e.eager` with every operator call made from the host)
  roofline  the projection kernel alone against the measured HBM copy bandwidth
  configs   (N = 1) every other benchmark configuration as its own measured row with its
            roofline and the CPU oracle beside it

`--impl reference` times the CPU restatement of the reference's qualification oracle for
the same workload on the host cores (the reference is Rust + cuda-oxide for sm_120 and can
neither be built nor run here).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN = 5120
VOCAB = 248320
SEED = 20260425
SAMPLES = 40  # qual/src/device_benchmark.rs: 40 samples per case
# DRAM bytes (read + write) that ncu counted for one LM-head projection launch at vocab 248320,
# M = 1, over that launch's algorithmic bytes (1 272 757 504 / 1 272 893 444): every weight byte
# crosses HBM once (ncu: dram__bytes_read.sum + dram__bytes_write.sum of one captured launch).
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1272757504 / 1272893444
FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0
NOMINAL_FP8_TFLOPS = 4500.0
NOMINAL_FP4_TFLOPS = 9000.0


def algorithmic_bytes(rows: int, out_rows: int, k: int, out_bytes: int) -> int:
    """weights + row scales + activation codes + activation scales + outputs."""
    return out_rows * k + 2 * out_rows + rows * k + 4 * rows + out_bytes * rows * out_rows


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_tensor_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 1590.0, 1400.0, "fallback"


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def workload_config(rows: int, vocab: int, world: int) -> dict:
    """The `config` object: the same keys and values in the GPU arm and the reference arm."""
    return {"workload": f"fp8_lm_head_argmax K={HIDDEN} vocab={vocab} M={rows}",
            "rows": rows, "vocab": vocab, "hidden": HIDDEN,
            "parallelism": f"vocab-shard x{world}",
            "l2": "weight shard (%.0f MB) larger than L2, streamed once per step"
                  % (vocab // world * HIDDEN / 1e6)}


class ClockSampler:
    """Polls nvidia-smi for SM clocks and throttle reasons from before the warm-up until the
    last timed region ends (the GPU is under load for the whole span)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def wait_for_first_sample(self, limit_s: float = 3.0):
        t0 = time.time()
        while self.proc is not None and not self.samples and time.time() - t0 < limit_s:
            time.sleep(0.01)

    def mark(self) -> int:
        return len(self.samples)

    def stop(self, first: int = 0):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        sm, mx, reasons = [], 0.0, set()
        for p in self.samples[first:]:
            try:
                sm.append(float(p[0]))
                mx = max(mx, float(p[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------- CPU arm

def cpu_threads_all() -> int:
    """Gives the oracle's OpenMP loops every online core, whatever OMP_NUM_THREADS a launcher
    exported to its ranks (torch.distributed.run sets it to 1)."""
    from oracle import tuisko_oracle as O

    O.lib()
    return O.set_num_threads(host_cores())


def cpu_lm_head(rows: int, steps: int, warmup: int, budget_s: float, sample_rows: int = 0):
    """Times the oracle's LM-head formula (quantise + f64 FP8 dot + greedy pick) on a
    bounded sample of vocabulary rows sized so that all steps take about `budget_s` seconds;
    returns (GB/s, seconds/step, threads, note, sampled rows)."""
    import numpy as np

    from oracle import tuisko_oracle as O
    from tuiskollm_b200 import synth

    threads = cpu_threads_all()
    x = synth.normal_bf16(SEED, 2, (rows, HIDDEN))

    def make_step(wc, ws):
        def step():
            codes, scales = O.quantize_e4m3(x)
            logits = O.fp8_projection(codes, scales, wc, ws)
            bits = O.f32_to_bf16(logits.astype(np.float32))
            return [O.greedy_index(bits[t]) for t in range(rows)]
        return step

    if sample_rows <= 0:
        probe_rows = 2048
        probe = make_step(*synth.fp8_weights(SEED, 1, probe_rows, HIDDEN))
        probe()
        t0 = time.perf_counter()
        probe()
        rate = probe_rows / max(time.perf_counter() - t0, 1e-6)  # vocabulary rows per second
        sample_rows = int(rate * budget_s / max(1, steps + warmup))
        sample_rows = max(1024, min(32768, sample_rows // 128 * 128))  # bounded host memory
    step = make_step(*synth.fp8_weights(SEED, 1, sample_rows, HIDDEN))
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    nbytes = algorithmic_bytes(rows, sample_rows, HIDDEN, 4)
    note = (f"{sample_rows} of {VOCAB} vocabulary rows x {HIDDEN}, M={rows}: per-token E4M3 "
            f"quantise, f64 dot of decoded codes, greedy pick; OpenMP over rows")
    return nbytes / dt / 1e9, dt, threads, note, sample_rows


def cpu_time(fn, budget_s: float = 1.0) -> float:
    """Seconds per call of fn: one warm-up call, then repeats for about `budget_s`."""
    fn()
    t0 = time.perf_counter()
    n = 0
    while True:
        fn()
        n += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s or n >= 50:
            return dt / n


_CPU_PLANES = {}


def cpu_fp8_plane(k: int):
    """One 8192-row E4M3 plane per reduction length, drawn once and sliced by the CPU rows."""
    import numpy as np
    import torch

    from tuiskollm_b200 import synth

    if k not in _CPU_PLANES:
        if torch.cuda.is_available():  # same recipe, drawn on the device and copied back: seconds faster
            c, sc = synth.torch_fp8_weights(SEED, 3, 8192, k, "cuda")
            _CPU_PLANES[k] = (c.cpu().numpy(), sc.view(torch.int16).cpu().numpy().view(np.uint16))
        else:
            _CPU_PLANES[k] = synth.fp8_weights(SEED, 3, 8192, k)
    return _CPU_PLANES[k]


def cpu_fp8_projection(rows: int, out_rows: int, k: int, gpu_us: float, out_bytes: int = 2):
    """Oracle port of one FP8 projection on a bounded sample of the weight rows (all tokens),
    extrapolated linearly in the row count."""
    from oracle import tuisko_oracle as O
    from tuiskollm_b200 import synth

    threads = cpu_threads_all()
    sample = min(out_rows, 8192, max(256, int(4.0e8 / (rows * k)) // 128 * 128))
    x = synth.normal_bf16(SEED, 2, (rows, k))
    wc, ws = cpu_fp8_plane(k)
    wc, ws = wc[:sample], ws[:sample]
    codes, scales = O.quantize_e4m3(x)
    dt = cpu_time(lambda: O.fp8_projection(codes, scales, wc, ws), 0.6) * out_rows / sample
    b = algorithmic_bytes(rows, out_rows, k, out_bytes)
    return {"value": b / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "us_full_shape": dt * 1e6, "gpu_speedup": dt * 1e6 / gpu_us,
            "sample": f"{sample} of {out_rows} weight rows x {k}, M={rows}, f64 dot of decoded "
                      f"codes" + ("" if sample == out_rows else "; extrapolated to the full plane")}


def cpu_norm_quant(rows: int, gpu_us: float):
    from oracle import tuisko_oracle as O
    from tuiskollm_b200 import synth

    threads = cpu_threads_all()
    sample = min(rows, 64)
    x = synth.normal_bf16(SEED, 90, (sample, HIDDEN))
    b = synth.normal_bf16(SEED, 190, (sample, HIDDEN))
    w = synth.normal_bf16(SEED, 5, (HIDDEN,), std=0.1)

    def fn():
        _res, nrm = O.residual_rms_norm(x, b, w, 1e-6)
        O.quantize_e4m3(nrm)

    dt = cpu_time(fn, 0.4) * rows / sample
    nbytes = 11 * rows * HIDDEN + 4 * rows
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "us_full_shape": dt * 1e6, "gpu_speedup": dt * 1e6 / gpu_us,
            "sample": f"{sample} of {rows} rows x {HIDDEN}: residual add, f64 RMSNorm, E4M3 quantise"
                      + ("" if sample == rows else "; extrapolated")}


def cpu_gdn(which: str, batch: int, gpu_us: float):
    """FP64 oracle (numpy, one thread) of one gated-delta-net decode step on the same shapes."""
    import numpy as np

    from oracle import gdn_oracle as G
    from tuiskollm_b200 import synth

    rows = np.arange(batch, dtype=np.uint32)
    proj = synth.normal_bf16(SEED, 404, (batch, G.INPUT_ROWS))
    if which == "prepare":
        x = synth.normal_bf16(SEED, 400, (batch, HIDDEN))
        cw = synth.normal_bf16(SEED, 401, (2 * G.CONTROL_ROWS, HIDDEN), std=0.02)
        a_log, dt_bias = synth.normal_bf16(SEED, 402, (G.CONTROL_ROWS,)), synth.normal_bf16(SEED, 403, (G.CONTROL_ROWS,))
        convw = synth.normal_bf16(SEED, 405, (G.QKV_ROWS, 4), std=0.5)
        hist = synth.normal_bf16(SEED, 406, (batch, G.QKV_ROWS, 3))

        def fn():
            G.gdn_controls(x, cw, a_log, dt_bias)
            G.gdn_convolution(proj, convw, rows, hist)
    else:
        qkv = synth.normal_bf16(SEED, 409, (batch, G.QKV_ROWS))
        norm = synth.normal_bf16(SEED, 408, (G.HEAD_DIM,))
        decay = -np.abs(np.random.default_rng(SEED).normal(0.5, 0.2, (batch, G.VALUE_HEADS))).astype(np.float32)
        beta = np.full((batch, G.VALUE_HEADS), 0.5, dtype=np.float32)
        state = np.zeros((batch, G.VALUE_HEADS, G.HEAD_DIM, G.HEAD_DIM), dtype=np.float32)

        def fn():
            G.gdn_recurrence(qkv, proj, decay, beta, norm, rows, state)

    dt = cpu_time(fn, 0.4)
    return {"value": dt * 1e6, "unit": "us per step", "cores": 1, "kind": "port",
            "us_full_shape": dt * 1e6, "gpu_speedup": dt * 1e6 / gpu_us,
            "sample": f"GDN {which}, batch {batch}: the FP64 formulas of the reference's qualification in numpy"}


def cpu_sampler(batch: int, vocab: int, gpu_us: float):
    """The C oracle of the host sampler (top-k 20, top-p 0.95) on `batch` full-vocabulary rows,
    one thread -- what the reference's engine does per token after copying the row to the host."""
    from oracle import tuisko_oracle as O
    from tuiskollm_b200 import synth

    rows = [synth.normal_bf16(SEED, 500 + i, (vocab,), std=3.0) for i in range(batch)]
    samplers = [O.Sampler(1.0, 0.95, 20, i, (1, 2)) for i in range(batch)]

    def fn():
        for sampler, row in zip(samplers, rows):
            sampler.sample(row)

    dt = cpu_time(fn, 0.4)
    return {"value": dt * 1e6, "unit": "us per batch", "cores": 1, "kind": "port",
            "us_full_shape": dt * 1e6, "gpu_speedup": dt * 1e6 / gpu_us,
            "sample": f"{batch} rows x {vocab} BF16 logits: top-k select, softmax weights, top-p, xorshift64 draw "
                      "(the host copy of the rows is not included)"}


def cpu_nvfp4(rows: int, out_rows: int, k: int, gate_up: bool, gpu_us: float):
    """Oracle port of one NVFP4 projection on a stratified sample (64 tokens x 512 weight rows),
    reported per output element and extrapolated to the full shape, labelled as such."""
    from oracle import tuisko_oracle as O
    from tuiskollm_b200 import synth

    threads = cpu_threads_all()
    st, sr = min(rows, 64), min(out_rows, 512)
    n_w = sr * (2 if gate_up else 1)
    x = synth.normal_bf16(SEED, 310, (st, k))
    if ("nvfp4", n_w, k) not in _CPU_PLANES:
        _CPU_PLANES[("nvfp4", n_w, k)] = synth.nvfp4_weights(SEED, 320, n_w, k)
    wc, ws, wd = _CPU_PLANES[("nvfp4", n_w, k)]
    a_div = 448.0
    oc, osc = O.nvfp4_quantize(x, a_div)

    def fn():
        d = O.nvfp4_w4a4_dot(oc, osc, a_div, wc, ws, float(wd))
        if gate_up:
            O.silu_mul(d[:, :sr], d[:, sr:])

    dt_sample = cpu_time(fn, 0.6)
    per_elem = dt_sample / (st * sr)
    dt = per_elem * rows * out_rows
    flops = 2.0 * rows * out_rows * k * (2 if gate_up else 1)
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "us_per_output_element": per_elem * 1e6, "us_full_shape": dt * 1e6,
            "gpu_speedup": dt * 1e6 / gpu_us,
            "sample": f"{st} tokens x {sr} outputs of {rows} x {out_rows}, K={k}: integer dot of "
                      f"E2M1 codes per 16-block, f64 scale product; extrapolated to the full shape"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    gbs, dt, threads, note, sample = cpu_lm_head(args.rows, max(1, args.steps), args.warmup,
                                                 budget_s=90.0, sample_rows=args.cpu_sample_rows)
    line = {
        "impl": "reference", "metric": "fp8_lm_head_gbs", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "e4m3",
        "data": "synthetic",
        "config": workload_config(args.rows, args.vocab, args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": note, "sampled_vocab_rows": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ----------------------------------------------------------------- GPU arm

def time_region(torch, fn, steps, sync_each=False):
    """CUDA-event time (ms) of `steps` calls of fn on the current stream."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        fn()
        if sync_each:
            torch.cuda.current_stream().synchronize()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop)


def capture(torch, fn, reps=1):
    """Records `reps` calls of fn into one CUDA graph (the reference times its operators as
    graph replays too: qual/src/device_benchmark.rs:1026-1054)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()  # tensor maps are encoded and cached here, outside the capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    return graph


def percentile(sorted_values, q):
    if not sorted_values:
        return None
    i = min(len(sorted_values) - 1, max(0, int(round(q * (len(sorted_values) - 1)))))
    return sorted_values[i]


class Protocol:
    """The reference's measurement loop (qual/src/device_benchmark.rs:993-1101, order
    :1228-1239): every case is a CUDA graph of `ops` operations; each of the 40 samples times
    every case once with CUDA events, visiting the cases in an order that reverses on odd samples
    and rotates by the sample number; a case reports median / p10 / p90 microseconds per
    operation.  Between the two events the graph is launched as often as it takes to reach
    OPS_PER_SAMPLE operations (the reference launches its graph 256 times per sample, :39,
    :1028-1031): the device idles for one host-side graph launch (a few microseconds) after the
    start event, and that idle time belongs to no operation."""

    OPS_PER_SAMPLE = 32

    def __init__(self, torch):
        self.torch = torch
        self.cases = []  # (name, replay, ops, replays per sample)

    def add(self, name, replay, ops, inner=None):
        if inner is None:
            inner = max(1, -(-self.OPS_PER_SAMPLE // ops))
        self.cases.append((name, replay, ops, inner))

    @staticmethod
    def order(sample, count):
        order = list(range(count))
        if sample % 2 == 1:
            order.reverse()
        r = sample % count
        return order[r:] + order[:r]

    def run(self, samples=SAMPLES, warmup=3):
        torch = self.torch
        times = {name: [] for name, *_ in self.cases}
        for _name, replay, _ops, inner in self.cases:
            for _ in range(warmup):
                replay()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for s in range(samples):
            for i in self.order(s, len(self.cases)):
                name, replay, ops, inner = self.cases[i]
                start.record()
                for _ in range(inner):
                    replay()
                stop.record()
                stop.synchronize()
                times[name].append(start.elapsed_time(stop) * 1e3 / (ops * inner))
        out = {}
        for name, v in times.items():
            v.sort()
            out[name] = {"median": statistics.median(v), "p10": percentile(v, 0.1),
                         "p90": percentile(v, 0.9), "samples": len(v)}
        for name, _replay, ops, inner in self.cases:
            out[name]["operations_per_sample"] = ops * inner
        return out


def hbm_roofline(kernel, nbytes, us, peak, peak_kind):
    gbs = nbytes / us / 1e3
    return {"bound": "hbm", "kernel": kernel, "algorithmic_bytes": int(nbytes), "us": us,
            "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
            "peak_kind": peak_kind, "frac_of_8TBs": gbs / NOMINAL_HBM_GBS}


def tensor_roofline(kernel, flops, nbytes, us, nominal_tflops, proxy_factor, hbm_peak):
    burst, sustained, kind = measured_tensor_peaks()
    tf = flops / us / 1e6
    proxy = proxy_factor * burst
    # near the ridge the bound is the slower of the byte stream and the flops
    bound_us = max(nbytes / hbm_peak / 1e3, flops / (proxy * 1e6))
    return {"bound": "tensor", "kernel": kernel, "algorithmic_flops": flops,
            "algorithmic_bytes": int(nbytes), "us": us, "achieved": tf, "peak": proxy,
            "unit": "TFLOP/s", "frac": tf / proxy,
            "peak_kind": f"{proxy_factor} x {kind} bf16 burst ({burst:.0f} TFLOP/s)",
            "frac_of_nominal": tf / nominal_tflops, "nominal_tflops": nominal_tflops,
            "frac_of_sustained_proxy": tf / (proxy_factor * sustained),
            "bound_us_max_of_bytes_and_flops": bound_us, "frac_of_bound": bound_us / us}


class MlpPlanes:
    """Synthetic NVFP4 MLP weights (shared between token counts) + activation planes."""

    def __init__(self, torch, ops, synth, m, weights, dev="cuda"):
        inter = synth.INTERMEDIATE
        self.m = m
        (self.gu_codes, self.gu_scales, self.gu_div), (self.dn_codes, self.dn_scales, self.dn_div) = weights
        self.a_codes = torch.empty((m, HIDDEN // 2), dtype=torch.uint8, device=dev)
        self.a_scales = torch.zeros((ops.nvfp4_scale_plane_bytes(m, HIDDEN),), dtype=torch.uint8,
                                    device=dev)
        self.mid = torch.empty((m, inter), dtype=torch.bfloat16, device=dev)
        self.m_codes = torch.empty((m, inter // 2), dtype=torch.uint8, device=dev)
        self.m_scales = torch.zeros((ops.nvfp4_scale_plane_bytes(m, inter),), dtype=torch.uint8,
                                    device=dev)
        self.out = torch.empty((m, HIDDEN), dtype=torch.bfloat16, device=dev)
        # activation divisors: a calibration constant for ~N(0,1) rows and for the SwiGLU
        # output of these weights (|silu(g) * u| stays below ~8)
        self.a_div = 448.0 * 6.0 / 6.0
        self.m_div = 448.0 * 6.0 / 8.0


def mlp_weights(synth):
    inter = synth.INTERMEDIATE
    return (synth.torch_nvfp4_weights(SEED, 300, 2 * inter, HIDDEN, "cuda"),
            synth.torch_nvfp4_weights(SEED, 301, HIDDEN, inter, "cuda"))


def w4a4_vs_a16(torch, pl, x):
    """How far the W4A4 result lies from the reference's A16 definition
    (tuisko-kernels-sm89/src/nvfp4/swiglu.rs:166-320: BF16 activations times decoded NVFP4
    weights) on the benchmark's own inputs: max and mean relative deviation of sampled tiles of
    the gate_up + SwiGLU output and of the down output (its input being the BF16 intermediate the
    device wrote).  A reported fact, not a gate."""
    import numpy as np

    from oracle import tuisko_oracle as O
    from tuiskollm_b200 import synth

    inter = synth.INTERMEDIATE
    host16 = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)
    tok = slice(0, 64)
    xs = host16(x[tok])
    out = {}
    g_w = HIDDEN // 16
    devs = []
    sc_all = pl.gu_scales.cpu().numpy()
    tile = lambda t: sc_all[t * 128 * g_w:(t + 1) * 128 * g_w]
    for wt in (0, 77):
        rows_g = slice(wt * 128, (wt + 1) * 128)
        rows_u = slice(inter + wt * 128, inter + (wt + 1) * 128)
        wc = np.concatenate([pl.gu_codes[rows_g].cpu().numpy(), pl.gu_codes[rows_u].cpu().numpy()])
        ws = np.concatenate([tile(wt), tile(inter // 128 + wt)])
        dots = O.nvfp4_a16_dot(xs, wc, ws, float(pl.gu_div))
        exp = O.silu_mul(dots[:, :128], dots[:, 128:])
        got = O.bf16_to_f32(host16(pl.mid[tok])[:, rows_g]).astype(np.float64)
        devs.append(np.abs(got - exp) / np.maximum(np.abs(exp), 4 * np.abs(exp).mean()))
    d = np.concatenate([v.reshape(-1) for v in devs])
    out["gate_up_swiglu"] = {"max_rel": float(d.max()), "mean_rel": float(d.mean()),
                             "sample": "64 tokens x 2 tiles of 128 outputs"}
    mids = host16(pl.mid[tok])
    g_d = inter // 16
    dsc = pl.dn_scales.cpu().numpy()
    devs = []
    for wt in (0, 31):
        rows_w = slice(wt * 128, (wt + 1) * 128)
        wc = pl.dn_codes[rows_w].cpu().numpy()
        ws = dsc[wt * 128 * g_d:(wt + 1) * 128 * g_d]
        exp = O.nvfp4_a16_dot(mids, wc, ws, float(pl.dn_div))
        got = O.bf16_to_f32(host16(pl.out[tok])[:, rows_w]).astype(np.float64)
        devs.append(np.abs(got - exp) / np.maximum(np.abs(exp), 4 * np.abs(exp).mean()))
    d = np.concatenate([v.reshape(-1) for v in devs])
    out["down"] = {"max_rel": float(d.max()), "mean_rel": float(d.mean()),
                   "sample": "64 tokens x 2 tiles of 128 outputs"}
    out["definition"] = ("|w4a4 - a16| / max(|a16|, 4 x mean|a16|); a16 = the reference's BF16-"
                         "activation product in f64 on the same inputs")
    return out


def config_rows(torch, tk, ctx, peak_gbs, peak_kind, lm, with_cpu=True):
    """Configurations 1, 2, 4 and 5 (and the other LM-head token counts of 3) on one GPU, each
    operator as a graph of several launches timed with the 40-sample protocol.  Decode planes
    rotate over enough weight copies (> 3 x L2) that every launch streams from HBM."""
    from tuiskollm_b200 import ops, synth

    dev = "cuda"
    proto = Protocol(torch)
    meta = {}   # case name -> dict(describing the row)
    keep = []   # tensors that must outlive the graphs
    inter = synth.INTERMEDIATE

    # ---- configurations 1 and 2: FP8 decode projections, weights rotated over > 3 x L2
    for name, n_rows, cfg in (("fp8_qkv", synth.QKV_ROWS, 1), ("fp8_gdn_input", synth.GDN_ROWS, 2),
                              ("fp8_qkv_refN", synth.QKV_ROWS_REF, 1),
                              ("fp8_gdn_input_refN", synth.GDN_ROWS_REF, 2)):
        copies = max(4, int(3 * 126e6 / (n_rows * HIDDEN)) + 1)
        planes = [synth.torch_fp8_weights(SEED, 50 + c, n_rows, HIDDEN, dev) for c in range(copies)]
        keep.append(planes)
        for m in (1, 8, 32):
            if name.endswith("refN") and m != 1:
                continue
            x = synth.torch_normal_bf16(SEED, 7, (m, HIDDEN), dev)
            codes = torch.empty((m, HIDDEN), dtype=torch.uint8, device=dev)
            scales = torch.empty((m,), dtype=torch.float32, device=dev)
            outp = torch.empty((m, n_rows), dtype=torch.bfloat16, device=dev)
            op = tk.GdnInputProjectionOp(ctx, n_rows)
            op.launch(None, m, x, codes, scales, planes[0][0], planes[0][1], outp)
            state = {"i": 0}

            def proj(op=op, m=m, codes=codes, scales=scales, outp=outp, planes=planes, state=state,
                     copies=copies):
                w, s = planes[state["i"] % copies]
                state["i"] += 1
                op.launch(None, m, None, codes, scales, w, s, outp)

            graph = capture(torch, proj, copies)  # one launch per weight copy, in rotation
            case = f"{name}:M{m}"
            proto.add(case, graph.replay, copies)
            meta[case] = {"config": cfg, "op": name, "M": m, "N": n_rows, "K": HIDDEN,
                          "kernel": ctx.last_kernel, "weight_copies": copies,
                          "bytes": algorithmic_bytes(m, n_rows, HIDDEN, 2), "kind": "hbm",
                          "cpu": ("fp8", m, n_rows, HIDDEN)}
            keep.append((graph, x, codes, scales, outp))

    # ---- FP8 prefill shapes (tensor-bound): one weight plane, graph of 8 launches
    for name, n_rows in (("fp8_qkv", synth.QKV_ROWS), ("fp8_gdn_input", synth.GDN_ROWS)):
        w, s = synth.torch_fp8_weights(SEED, 60, n_rows, HIDDEN, dev)
        for m in (256, 512, 2048):
            x = synth.torch_normal_bf16(SEED, 8, (m, HIDDEN), dev)
            codes = torch.empty((m, HIDDEN), dtype=torch.uint8, device=dev)
            scales = torch.empty((m,), dtype=torch.float32, device=dev)
            outp = torch.empty((m, n_rows), dtype=torch.bfloat16, device=dev)
            op = tk.GdnInputProjectionOp(ctx, n_rows)
            op.launch(None, m, x, codes, scales, w, s, outp)
            graph = capture(torch, lambda op=op, m=m, codes=codes, scales=scales, outp=outp, w=w, s=s:
                            op.launch(None, m, None, codes, scales, w, s, outp), 8)
            case = f"{name}:M{m}"
            proto.add(case, graph.replay, 8)
            meta[case] = {"config": 5 if m == 256 else "metric", "op": name, "M": m, "N": n_rows,
                          "K": HIDDEN, "kernel": ctx.last_kernel, "kind": "fp8_tensor",
                          "flops": 2.0 * m * n_rows * HIDDEN,
                          "bytes": algorithmic_bytes(m, n_rows, HIDDEN, 2),
                          "cpu": ("fp8", m, n_rows, HIDDEN)}
            keep.append((graph, x, codes, scales, outp, w, s))

    # ---- the next rows of the path: dense-FP8 MLP (gate/up + SwiGLU, down) and the GDN output projection
    gdn_value = 6144
    for m in (1, 32, 256):
        copies = 3 if m <= 32 else 1
        gu_planes = [synth.torch_fp8_weights(SEED, 70 + c, 2 * inter, HIDDEN, dev) for c in range(copies)]
        dn_planes = [synth.torch_fp8_weights(SEED, 75 + c, HIDDEN, inter, dev) for c in range(copies)]
        go_planes = [synth.torch_fp8_weights(SEED, 80 + c, HIDDEN, gdn_value, dev) for c in range(max(copies, 4 if m <= 32 else 1))]
        x = synth.torch_normal_bf16(SEED, 9, (m, HIDDEN), dev)
        xi = synth.torch_normal_bf16(SEED, 10, (m, inter), dev)
        xg = synth.torch_normal_bf16(SEED, 11, (m, gdn_value), dev)
        c1 = torch.empty((m, HIDDEN), dtype=torch.uint8, device=dev)
        c2 = torch.empty((m, inter), dtype=torch.uint8, device=dev)
        c3 = torch.empty((m, gdn_value), dtype=torch.uint8, device=dev)
        s1, s2, s3 = (torch.empty((m,), dtype=torch.float32, device=dev) for _ in range(3))
        mid = torch.empty((m, inter), dtype=torch.bfloat16, device=dev)
        out = torch.empty((m, HIDDEN), dtype=torch.bfloat16, device=dev)
        out_g = torch.empty((m, HIDDEN), dtype=torch.bfloat16, device=dev)
        sw_op, dn_op, go_op = tk.Fp8SwiGluOp(ctx), tk.Fp8DownOp(ctx), tk.GdnOutputProjectionOp(ctx, gdn_value)
        sw_op.launch(None, m, x, c1, s1, gu_planes[0][0], gu_planes[0][1], mid)
        dn_op.launch(None, m, xi, c2, s2, dn_planes[0][0], dn_planes[0][1], out)
        go_op.launch(None, m, xg, c3, s3, go_planes[0][0], go_planes[0][1], out_g)
        for nm, op_, planes_, args, by, fl in (
                ("fp8_swiglu", sw_op, gu_planes, (c1, s1, mid), 2 * inter * HIDDEN + 4 * inter + m * HIDDEN + 4 * m + 2 * m * inter,
                 2.0 * m * 2 * inter * HIDDEN),
                ("fp8_down", dn_op, dn_planes, (c2, s2, out), algorithmic_bytes(m, HIDDEN, inter, 2), 2.0 * m * HIDDEN * inter),
                ("fp8_gdn_output", go_op, go_planes, (c3, s3, out_g), algorithmic_bytes(m, HIDDEN, gdn_value, 2),
                 2.0 * m * HIDDEN * gdn_value)):
            state = {"i": 0}

            def run(op_=op_, planes_=planes_, args=args, state=state, m=m):
                w, sc = planes_[state["i"] % len(planes_)]
                state["i"] += 1
                op_.launch(None, m, None, args[0], args[1], w, sc, args[2])

            run()
            kernel = ctx.last_kernel
            graph = capture(torch, run, len(planes_))
            case = f"{nm}:M{m}"
            proto.add(case, graph.replay, len(planes_))
            meta[case] = {"config": "next", "op": nm, "M": m, "kernel": kernel,
                          "kind": "hbm" if m <= 32 else "fp8_tensor", "bytes": by, "flops": fl, "cpu": None}
            keep.append(graph)
        keep.append((gu_planes, dn_planes, go_planes, x, xi, xg, c1, c2, c3, s1, s2, s3, mid, out, out_g))

    # ---- the steps either side of the GDN projections: control mat-vecs + convolution, and the
    # FP32 state recurrence, at decode batches 1 and 8.  State slots rotate so that the 6.29 MB of
    # state per token come from HBM, not from L2.
    qkv_rows, in_rows, slots = 10240, 16384, 48
    prep_op, rec_op = tk.GdnPrepareOp(ctx), tk.GdnRecurrenceOp(ctx)
    g_x = synth.torch_normal_bf16(SEED, 400, (8, HIDDEN), dev)
    g_cw = synth.torch_normal_bf16(SEED, 401, (96, HIDDEN), dev, std=0.02)
    g_alog = synth.torch_normal_bf16(SEED, 402, (48,), dev)
    g_dt = synth.torch_normal_bf16(SEED, 403, (48,), dev)
    g_proj = synth.torch_normal_bf16(SEED, 404, (8, in_rows), dev)
    g_convw = synth.torch_normal_bf16(SEED, 405, (qkv_rows, 4), dev, std=0.5)
    g_hist = synth.torch_normal_bf16(SEED, 406, (slots, qkv_rows, 3), dev)
    g_state = torch.zeros((slots, 48, 128, 128), dtype=torch.float32, device=dev)
    g_state.normal_(0.0, 0.05, generator=torch.Generator(device=dev).manual_seed(SEED + 407))
    g_norm = synth.torch_normal_bf16(SEED, 408, (128,), dev)
    g_decay = torch.empty((8, 48), dtype=torch.float32, device=dev)
    g_beta = torch.empty((8, 48), dtype=torch.float32, device=dev)
    g_conv = torch.empty((8, qkv_rows), dtype=torch.bfloat16, device=dev)
    g_out = torch.empty((8, 6144), dtype=torch.bfloat16, device=dev)
    for b in (1, 8):
        groups = slots // b
        rows = [torch.arange(g * b, (g + 1) * b, dtype=torch.int32, device=dev) for g in range(groups)]
        keep.append(rows)  # the captured launches read their slot indices from these tensors
        st = {"p": 0, "r": 0}

        def prep(b=b, rows=rows, st=st, groups=groups):
            prep_op.launch(None, b, g_x, g_cw, g_alog, g_dt, g_proj, g_convw, rows[st["p"] % groups],
                           g_hist, g_decay, g_beta, g_conv)
            st["p"] += 1

        def rec(b=b, rows=rows, st=st, groups=groups):
            rec_op.launch(None, b, g_conv, g_proj, g_decay, g_beta, g_norm, rows[st["r"] % groups],
                          g_state, g_out)
            st["r"] += 1

        def step(b=b, rows=rows, st=st, groups=groups):
            # one decode step: prepare, then the recurrence on the same slots
            r = rows[st["s"] % groups]
            st["s"] += 1
            prep_op.launch(None, b, g_x, g_cw, g_alog, g_dt, g_proj, g_convw, r, g_hist, g_decay, g_beta, g_conv)
            rec_op.launch(None, b, g_conv, g_proj, g_decay, g_beta, g_norm, r, g_state, g_out)

        st["s"] = 0
        state_bytes = b * (2 * 48 * 128 * 128 * 4 + 2 * (qkv_rows + 2 * 6144) + 2 * 48 * 4)
        prep_bytes = 2 * 96 * HIDDEN + b * (2 * HIDDEN + qkv_rows * (2 + 6 + 6 + 2) + 2 * 48 * 4) + 8 * qkv_rows
        for nm in ("gdn_step",):
            step()
            graph = capture(torch, step, groups)
            case = f"{nm}:B{b}"
            proto.add(case, graph.replay, groups)
            meta[case] = {"config": "next", "op": nm, "M": b, "kernel": "gdn_prepare_kernel + gdn_recurrence_kernel",
                          "kind": "hbm", "bytes": state_bytes + prep_bytes, "cpu": None}
            keep.append(graph)

        prep()
        rec()
        for nm, fn, by in (
                ("gdn_prepare", prep, 2 * 96 * HIDDEN + b * (2 * HIDDEN + qkv_rows * (2 + 6 + 6 + 2) + 2 * 48 * 4)
                 + 8 * qkv_rows),
                ("gdn_recurrence", rec, b * (2 * 48 * 128 * 128 * 4 + 2 * (qkv_rows + 2 * 6144) + 2 * 48 * 4))):
            graph = capture(torch, fn, groups)
            case = f"{nm}:B{b}"
            proto.add(case, graph.replay, groups)
            meta[case] = {"config": "next", "op": nm, "M": b, "kernel": nm + "_kernel", "kind": "hbm",
                          "bytes": by, "cpu": ("gdn", nm.split("_")[1], b)}
            keep.append(graph)
    keep.append((g_x, g_cw, g_alog, g_dt, g_proj, g_convw, g_hist, g_state, g_norm, g_decay, g_beta,
                 g_conv, g_out))

    # ---- device sampler on BF16 logit rows of the full vocabulary (top-k 20, top-p 0.95), and the
    # load-time NVFP4 scale permutation of the gate/up planes
    vocab_s = lm["vocab"]
    for b in (1, 8):
        copies_s = max(2, int(3 * 126e6 / (b * vocab_s * 2)) + 1)
        rows_s = [synth.torch_normal_bf16(SEED, 500 + c, (b, vocab_s), dev, std=3.0) for c in range(copies_s)]
        samp = tk.Sampler(ctx, vocab_s, [tk.SamplingOptions(seed=i) for i in range(b)], [(1, 2)] * b)
        st_s = {"i": 0}

        def draw(samp=samp, rows_s=rows_s, st_s=st_s, copies_s=copies_s):
            samp.sample(None, rows_s[st_s["i"] % copies_s])
            st_s["i"] += 1

        draw()
        graph = capture(torch, draw, copies_s)
        case = f"device_sampler:B{b}"
        proto.add(case, graph.replay, copies_s)
        meta[case] = {"config": "next", "op": "device_sampler_top20_p95", "M": b, "kernel": "sampler_kernel",
                      "kind": "hbm", "bytes": b * vocab_s * 2 + b * 16, "cpu": ("sampler", b, vocab_s)}
        keep.append((graph, rows_s, samp))
    mat = tk.Materializer(ctx)
    sc_src = [torch.randint(0, 0x7F, (inter, HIDDEN // 16), dtype=torch.uint8, device=dev) for _ in range(2)]
    sc_out = torch.empty(2 * inter * (HIDDEN // 16), dtype=torch.uint8, device=dev)
    sc_ptrs = (ctypes.c_void_p * 2)(sc_src[0].data_ptr(), sc_src[1].data_ptr())

    def swizzle():
        ctx.check(ctx._lib.tk100_materialize_nvfp4_scales(ctx.handle, ops._stream(None), 2, sc_ptrs, inter,
                                                          HIDDEN // 16, sc_out.data_ptr()))

    swizzle()
    graph = capture(torch, swizzle, 4)
    proto.add("nvfp4_scale_layout", graph.replay, 4)
    meta["nvfp4_scale_layout"] = {"config": "next", "op": "materialize_nvfp4_scales_gate_up", "M": 0,
                                  "kernel": "swizzle_scales_kernel", "kind": "hbm",
                                  "bytes": 2 * 2 * inter * (HIDDEN // 16), "cpu": None}
    keep.append((graph, sc_src, sc_out, sc_ptrs, mat))

    # ---- fused residual + RMSNorm + quantise (configurations 1 and 5, and the metric's M = 512)
    normop = tk.ResidualNormOp(ctx)
    nw = synth.torch_normal_bf16(SEED, 5, (HIDDEN,), dev, std=0.1)
    for m in (1, 256, 512):
        copies = 1 if m == 1 else max(2, int(2 * 126e6 / (m * HIDDEN * 11)) + 1)
        xs = [synth.torch_normal_bf16(SEED, 90 + c, (m, HIDDEN), dev) for c in range(copies)]
        bs = [synth.torch_normal_bf16(SEED, 190 + c, (m, HIDDEN), dev) for c in range(copies)]
        res = [torch.empty_like(xs[0]) for _ in range(copies)]
        nrm = [torch.empty_like(xs[0]) for _ in range(copies)]
        codes = [torch.empty((m, HIDDEN), dtype=torch.uint8, device=dev) for _ in range(copies)]
        scales = torch.empty((m,), dtype=torch.float32, device=dev)
        state = {"i": 0}

        def norm(m=m, xs=xs, bs=bs, res=res, nrm=nrm, codes=codes, scales=scales, state=state,
                 copies=copies):
            i = state["i"] % copies
            state["i"] += 1
            normop.launch_quantize(None, m, xs[i], bs[i], nw, res[i], nrm[i], codes[i], scales)

        graph = capture(torch, norm, copies * 4)
        case = f"residual_rmsnorm_quant_e4m3:M{m}"
        proto.add(case, graph.replay, copies * 4)
        meta[case] = {"config": 1 if m == 1 else 5 if m == 256 else "metric",
                      "op": "residual_rmsnorm_quant_e4m3", "M": m, "kind": "hbm",
                      "kernel": "resnorm_quant_kernel<1,1,1,1>",
                      "bytes": 11 * m * HIDDEN + 4 * m, "cpu": ("norm", m)}
        keep.append((graph, xs, bs, res, nrm, codes, scales))

    # ---- configuration 3 at the other token counts (the headline run has M = lm['m'])
    for m in (1, 4, 32):
        if m == lm["m"]:
            continue
        x = synth.torch_normal_bf16(SEED, 2, (m, HIDDEN), dev)
        codes = torch.empty((m, HIDDEN), dtype=torch.uint8, device=dev)
        scales = torch.empty((m,), dtype=torch.float32, device=dev)
        logits = torch.empty((m, lm["vocab"]), dtype=torch.float32, device=dev)
        scratch = torch.zeros((m,), dtype=torch.int64, device=dev)
        pairs = torch.zeros((m, 2), dtype=torch.int32, device=dev)
        op = tk.LmHeadOp(ctx, lm["vocab"], 0)
        op.launch(None, m, x, codes, scales, lm["wc"], lm["ws"], None, logits, scratch, pairs)
        graph = capture(torch, lambda op=op, m=m, codes=codes, scales=scales, logits=logits,
                        scratch=scratch, pairs=pairs:
                        op.launch(None, m, None, codes, scales, lm["wc"], lm["ws"], None, logits,
                                  scratch, pairs), 1)
        case = f"fp8_lm_head_argmax:M{m}"
        proto.add(case, graph.replay, 1)
        meta[case] = {"config": 3, "op": "fp8_lm_head_argmax", "M": m, "N": lm["vocab"], "K": HIDDEN,
                      "kernel": ctx.last_kernel + " (finalize in its last CTA)", "kind": "hbm",
                      "bytes": algorithmic_bytes(m, lm["vocab"], HIDDEN, 4),
                      "cpu": ("fp8", m, lm["vocab"], HIDDEN, 4)}
        keep.append((graph, x, codes, scales, logits, scratch, pairs))

    # ---- configuration 4 (M = 2048) and the decode / batched-decode shapes of the NVFP4 MLP
    weights = mlp_weights(synth)
    gu, dn = tk.Nvfp4SwiGluOp(ctx), tk.Nvfp4DownOp(ctx)
    mlp_planes = {}
    for m in (2048, 256, 32, 8, 1):
        pl = MlpPlanes(torch, ops, synth, m, weights)
        mlp_planes[m] = pl
        x = synth.torch_normal_bf16(SEED, 310, (m, HIDDEN), dev)
        pl.x = x

        def quant_in(pl=pl, m=m, x=x):
            gu.quantize(None, m, HIDDEN, x, pl.a_div, pl.a_codes, pl.a_scales)

        def gate_up(pl=pl, m=m):
            gu.launch(None, m, None, pl.gu_codes, pl.gu_scales, pl.gu_div, pl.mid,
                      activation_codes=pl.a_codes, activation_scales=pl.a_scales,
                      input_global_divisor=pl.a_div)

        def quant_mid(pl=pl, m=m):
            dn.quantize(None, m, inter, pl.mid, pl.m_div, pl.m_codes, pl.m_scales)

        def down(pl=pl, m=m):
            dn.launch(None, m, None, pl.dn_codes, pl.dn_scales, pl.dn_div, pl.out,
                      activation_codes=pl.m_codes, activation_scales=pl.m_scales,
                      input_global_divisor=pl.m_div)

        def gate_up_q(pl=pl, m=m):  # the same projection also leaving the NVFP4 form of its output
            gu.launch_quantize(None, m, None, pl.gu_codes, pl.gu_scales, pl.gu_div, pl.mid,
                               activation_codes=pl.a_codes, activation_scales=pl.a_scales,
                               input_global_divisor=pl.a_div, output_global_divisor=pl.m_div,
                               output_codes=pl.m_codes, output_scales=pl.m_scales)

        def mlp(quant_in=quant_in, gate_up_q=gate_up_q, down=down):
            quant_in(); gate_up_q(); down()

        for fn in (quant_in, gate_up, quant_mid, down):
            fn()
        torch.cuda.synchronize()
        f_gu = 2.0 * m * 2 * inter * HIDDEN
        f_dn = 2.0 * m * HIDDEN * inter
        b_gu = 2 * inter * HIDDEN // 2 + 2 * inter * HIDDEN // 16 + m * HIDDEN // 2 + m * HIDDEN // 16 + 2 * m * inter
        b_dn = HIDDEN * inter // 2 + HIDDEN * inter // 16 + m * inter // 2 + m * inter // 16 + 2 * m * HIDDEN
        for nm, fn, fl, by, cpu in (("quant_in", quant_in, 0.0, m * HIDDEN * (2 + 9 / 16), None),
                                    ("gate_up_swiglu", gate_up, f_gu, b_gu, ("nvfp4", m, inter, HIDDEN, True)),
                                    ("quant_mid", quant_mid, 0.0, m * inter * (2 + 9 / 16), None),
                                    ("gate_up_swiglu_quantize", gate_up_q, f_gu, b_gu + m * inter * 9 // 16, None),
                                    ("down", down, f_dn, b_dn, ("nvfp4", m, HIDDEN, inter, False)),
                                    ("mlp_total", mlp, f_gu + f_dn, b_gu + b_dn, None)):
            fn()
            kernel = ctx.last_kernel if nm in ("gate_up_swiglu", "down") else nm
            graph = capture(torch, fn, 4)
            case = f"nvfp4_{nm}:M{m}"
            proto.add(case, graph.replay, 4)
            meta[case] = {"config": 4 if m == 2048 else 5 if m == 256 else "decode",
                          "op": f"nvfp4_{nm}", "M": m, "kernel": kernel,
                          "kind": "fp4_tensor" if (m >= 256 and fl > 0) else "hbm",
                          "flops": fl, "bytes": by, "cpu": cpu}
            keep.append(graph)

    # ---- configuration 5: the layer slice on one GPU (M = 1 decode slice of configuration 1 too)
    qkv_w = synth.torch_fp8_weights(SEED, 400, synth.QKV_ROWS, HIDDEN, dev)
    gdn_w = synth.torch_fp8_weights(SEED, 401, synth.GDN_ROWS, HIDDEN, dev)
    weight_bytes = (synth.QKV_ROWS + synth.GDN_ROWS) * HIDDEN + 3 * inter * HIDDEN * 9 // 16
    slice_e2e = {}
    for m in (1, 256, 512):
        pl = MlpPlanes(torch, ops, synth, m, weights)
        x = synth.torch_normal_bf16(SEED, 410, (m, HIDDEN), dev)
        br = synth.torch_normal_bf16(SEED, 411, (m, HIDDEN), dev)
        x_host, br_host = x.cpu().pin_memory(), br.cpu().pin_memory()
        out_host = torch.empty((m, HIDDEN), dtype=torch.bfloat16).pin_memory()
        res = torch.empty_like(x)
        nrm = torch.empty_like(x)
        codes = torch.empty((m, HIDDEN), dtype=torch.uint8, device=dev)
        scales = torch.empty((m,), dtype=torch.float32, device=dev)
        qkv = torch.empty((m, synth.QKV_ROWS), dtype=torch.bfloat16, device=dev)
        gdn = torch.empty((m, synth.GDN_ROWS), dtype=torch.bfloat16, device=dev)
        qkv_op = tk.FullAttentionQkvOp(ctx, synth.QKV_ROWS)
        gdn_op = tk.GdnInputProjectionOp(ctx, synth.GDN_ROWS)

        def slice_(m=m, pl=pl, x=x, br=br, res=res, nrm=nrm, codes=codes, scales=scales, qkv=qkv,
                   gdn=gdn, qkv_op=qkv_op, gdn_op=gdn_op):
            normop.launch_quantize_nvfp4(None, m, x, br, nw, res, nrm, codes, scales, pl.a_div,
                                         pl.a_codes, pl.a_scales)
            qkv_op.launch(None, m, None, codes, scales, qkv_w[0], qkv_w[1], qkv)
            gdn_op.launch(None, m, None, codes, scales, gdn_w[0], gdn_w[1], gdn)
            gu.launch_quantize(None, m, None, pl.gu_codes, pl.gu_scales, pl.gu_div, pl.mid,
                               activation_codes=pl.a_codes, activation_scales=pl.a_scales,
                               input_global_divisor=pl.a_div, output_global_divisor=pl.m_div,
                               output_codes=pl.m_codes, output_scales=pl.m_scales)
            dn.launch(None, m, None, pl.dn_codes, pl.dn_scales, pl.dn_div, pl.out,
                      activation_codes=pl.m_codes, activation_scales=pl.m_scales,
                      input_global_divisor=pl.m_div)

        def slice_e2e_(slice_=slice_, x=x, br=br, x_host=x_host, br_host=br_host, pl=pl,
                       out_host=out_host):
            x.copy_(x_host, non_blocking=True)
            br.copy_(br_host, non_blocking=True)
            slice_()
            out_host.copy_(pl.out, non_blocking=True)

        slice_()
        torch.cuda.synchronize()
        graph = capture(torch, slice_, 1)
        case = f"layer_slice:M{m}"
        proto.add(case, graph.replay, 1)
        flops = 2.0 * m * HIDDEN * (synth.QKV_ROWS + synth.GDN_ROWS + 3 * inter)
        meta[case] = {"config": 1 if m == 1 else 5 if m == 256 else "metric", "op": "layer_slice",
                      "M": m, "kernel": "5 kernels" if m <= 32 else "6 kernels",
                      "kind": "slice", "flops": flops, "bytes": weight_bytes, "cpu": ("slice", m)}
        graph_e2e = capture(torch, slice_e2e_, 1)
        for _ in range(3):
            graph_e2e.replay()
        reps = 40
        ms = time_region(torch, graph_e2e.replay, reps, sync_each=True) / reps
        slice_e2e[case] = {"us": ms * 1e3, "h2d_bytes_per_step": 2 * m * HIDDEN * 2,
                           "d2h_bytes_per_step": m * HIDDEN * 2, "launch": "graph",
                           "note": "host x and branch in, BF16 down output out, one sync per step"}
        keep.append((graph, graph_e2e, pl, x, br, res, nrm, codes, scales, qkv, gdn))

    results = proto.run()

    rows = []
    for case, r in results.items():
        md = meta[case]
        us = r["median"]
        row = {"config": md["config"], "op": md["op"], "M": md["M"],
               "us": {"median": us, "p10": r["p10"], "p90": r["p90"], "samples": r["samples"],
                      "operations_per_sample": r["operations_per_sample"]}}
        for key in ("N", "K", "weight_copies"):
            if key in md:
                row[key] = md[key]
        if md["kind"] == "hbm":
            row["roofline"] = hbm_roofline(md["kernel"], md["bytes"], us, peak_gbs, peak_kind)
        elif md["kind"] == "fp8_tensor":
            row["roofline"] = tensor_roofline(md["kernel"], md["flops"], md["bytes"], us,
                                              NOMINAL_FP8_TFLOPS, 2, peak_gbs)
        elif md["kind"] == "fp4_tensor":
            row["roofline"] = tensor_roofline(md["kernel"], md["flops"], md["bytes"], us,
                                              NOMINAL_FP4_TFLOPS, 4, peak_gbs)
        else:  # the slice: bounded by its weight stream at decode, by its flops at 256 and more
            floor_us = md["bytes"] / peak_gbs / 1e3
            row["roofline"] = {"bound": "hbm" if md["M"] <= 32 else "tensor",
                               "kernel": md["kernel"], "weight_bytes": md["bytes"],
                               "algorithmic_flops": md["flops"], "us": us,
                               "weight_stream_GBs": md["bytes"] / us / 1e3,
                               "TFLOPs": md["flops"] / us / 1e6,
                               "floor_us_at_measured_hbm": floor_us, "frac": floor_us / us,
                               "peak_kind": peak_kind}
            row["e2e"] = slice_e2e[case]
        if with_cpu and md.get("cpu"):
            c = md["cpu"]
            try:
                if c[0] == "fp8":
                    row["cpu_baseline"] = cpu_fp8_projection(c[1], c[2], c[3], us, *(c[4:5] or (2,)))
                elif c[0] == "norm":
                    row["cpu_baseline"] = cpu_norm_quant(c[1], us)
                elif c[0] == "nvfp4":
                    row["cpu_baseline"] = cpu_nvfp4(c[1], c[2], c[3], c[4], us)
                elif c[0] == "gdn":
                    row["cpu_baseline"] = cpu_gdn(c[1], c[2], us)
                elif c[0] == "sampler":
                    row["cpu_baseline"] = cpu_sampler(c[1], c[2], us)
                elif c[0] == "slice":
                    row["cpu_baseline"] = None  # filled below from the operators' own rows
            except Exception as exc:  # the row stays, the baseline says why it is absent
                row["cpu_baseline"] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
        rows.append(row)
    # the slice's CPU figure = the sum of its operators' extrapolated CPU times
    by_key = {(r["op"], r["M"]): r for r in rows}
    for r in rows:
        if r["op"] != "layer_slice" or not with_cpu:
            continue
        m = r["M"]
        parts = [by_key.get(("residual_rmsnorm_quant_e4m3", m)), by_key.get(("fp8_qkv", m)),
                 by_key.get(("fp8_gdn_input", m)), by_key.get(("nvfp4_gate_up_swiglu", m)),
                 by_key.get(("nvfp4_down", m))]
        if all(p and isinstance(p.get("cpu_baseline"), dict) and "us_full_shape" in p["cpu_baseline"]
               for p in parts):
            total = sum(p["cpu_baseline"]["us_full_shape"] for p in parts)
            r["cpu_baseline"] = {"value": total, "unit": "us per slice", "kind": "port",
                                 "cores": parts[0]["cpu_baseline"]["cores"],
                                 "gpu_speedup": total / r["us"]["median"],
                                 "sample": "sum of the five operators' CPU rows (extrapolated)"}
        else:
            r.pop("cpu_baseline", None)
    deviation = None
    if with_cpu:
        try:
            pl = mlp_planes[2048]
            gu.quantize(None, 2048, HIDDEN, pl.x, pl.a_div, pl.a_codes, pl.a_scales)
            gu.launch_quantize(None, 2048, None, pl.gu_codes, pl.gu_scales, pl.gu_div, pl.mid,
                               activation_codes=pl.a_codes, activation_scales=pl.a_scales,
                               input_global_divisor=pl.a_div, output_global_divisor=pl.m_div,
                               output_codes=pl.m_codes, output_scales=pl.m_scales)
            dn.launch(None, 2048, None, pl.dn_codes, pl.dn_scales, pl.dn_div, pl.out,
                      activation_codes=pl.m_codes, activation_scales=pl.m_scales,
                      input_global_divisor=pl.m_div)
            torch.cuda.synchronize()
            deviation = w4a4_vs_a16(torch, pl, pl.x)
        except Exception as exc:
            deviation = {"error": f"{type(exc).__name__}: {exc}"[:200]}
    del keep
    return rows, deviation


def tp_layer_slice(torch, tk, dist, rank, world, m, local, nccl_reduce=False):
    """Configuration 5 on `world` GPUs: norm + quantise replicated; QKV / GDN-input / gate-up
    column-parallel; down row-parallel with fp32 partial sums, which the library's peer-memory
    kernel adds over NVLink and rounds to BF16 once (`nccl_reduce`: an NCCL all-reduce of
    [m, hidden] fp32 and a rounding kernel instead).  Before timing, the two routes are compared.
    Returns (device time per replay in ms, launch mode, reduce route)."""
    from tuiskollm_b200 import dist as tkd, ops, synth

    dev = "cuda"
    inter = synth.INTERMEDIATE
    qkv_rows = tkd.column_shard(synth.QKV_ROWS, world, rank).rows
    gdn_rows = tkd.column_shard(synth.GDN_ROWS, world, rank).rows
    i_shard = tkd.column_shard(inter, world, rank).rows
    ctx = tk.Context(device=local, hidden=HIDDEN, intermediate=i_shard, max_rows=max(2048, m))
    qkv_w = synth.torch_fp8_weights(SEED, 500 + rank, qkv_rows, HIDDEN, dev)
    gdn_w = synth.torch_fp8_weights(SEED, 520 + rank, gdn_rows, HIDDEN, dev)
    gu_codes, gu_scales, gu_div = synth.torch_nvfp4_weights(SEED, 540 + rank, 2 * i_shard, HIDDEN, dev)
    dn_codes, dn_scales, dn_div = synth.torch_nvfp4_weights(SEED, 560 + rank, HIDDEN, i_shard, dev)
    nw = synth.torch_normal_bf16(SEED, 5, (HIDDEN,), dev, std=0.1)
    x = synth.torch_normal_bf16(SEED, 410, (m, HIDDEN), dev)
    br = synth.torch_normal_bf16(SEED, 411, (m, HIDDEN), dev)
    res, nrm = torch.empty_like(x), torch.empty_like(x)
    codes = torch.empty((m, HIDDEN), dtype=torch.uint8, device=dev)
    scales = torch.empty((m,), dtype=torch.float32, device=dev)
    qkv = torch.empty((m, qkv_rows), dtype=torch.bfloat16, device=dev)
    gdn = torch.empty((m, gdn_rows), dtype=torch.bfloat16, device=dev)
    a_codes = torch.empty((m, HIDDEN // 2), dtype=torch.uint8, device=dev)
    a_scales = torch.zeros((ops.nvfp4_scale_plane_bytes(m, HIDDEN),), dtype=torch.uint8, device=dev)
    mid = torch.empty((m, i_shard), dtype=torch.bfloat16, device=dev)
    m_codes = torch.empty((m, i_shard // 2), dtype=torch.uint8, device=dev)
    m_scales = torch.zeros((ops.nvfp4_scale_plane_bytes(m, i_shard),), dtype=torch.uint8, device=dev)
    partial = torch.empty((m, HIDDEN), dtype=torch.float32, device=dev)
    out = torch.empty((m, HIDDEN), dtype=torch.bfloat16, device=dev)
    norm = tk.ResidualNormOp(ctx)
    qkv_op = tk.FullAttentionQkvOp(ctx, qkv_rows)
    gdn_op = tk.GdnInputProjectionOp(ctx, gdn_rows)
    gu, dn = tk.Nvfp4SwiGluOp(ctx), tk.Nvfp4DownOp(ctx)
    a_div, m_div = 448.0 * 6.0 / 6.0, 448.0 * 6.0 / 8.0
    route = "nccl all_reduce + rounding kernel"
    peer_addrs = None
    if world > 1 and not nccl_reduce:
        try:
            _rbuf, _rhdl, peer_addrs = tkd.alloc_peer_sum(m * HIDDEN, world, torch.device("cuda", local))
            route = "peer-memory sum kernel over NVLink (one launch)"
        except Exception as exc:  # symmetric memory unavailable: keep the NCCL route
            route += f" (peer sum unavailable: {type(exc).__name__}: {exc})"[:200]
        flag = torch.tensor([1 if peer_addrs is not None else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)  # all ranks must agree on the route
        if int(flag.item()) == 0:
            peer_addrs = None

    def reduce_():
        if peer_addrs is not None:
            ops.peer_sum_bf16(ctx, None, m * HIDDEN, m * HIDDEN, world, rank, partial, peer_addrs, out)
            return
        if world > 1:
            dist.all_reduce(partial)
        ops.f32_to_bf16(ctx, None, m * HIDDEN, partial, out)

    def slice_():
        norm.launch_quantize_nvfp4(None, m, x, br, nw, res, nrm, codes, scales, a_div, a_codes,
                                   a_scales)
        qkv_op.launch(None, m, None, codes, scales, qkv_w[0], qkv_w[1], qkv)
        gdn_op.launch(None, m, None, codes, scales, gdn_w[0], gdn_w[1], gdn)
        gu.launch_quantize(None, m, None, gu_codes, gu_scales, gu_div, mid,
                           activation_codes=a_codes, activation_scales=a_scales,
                           input_global_divisor=a_div, output_global_divisor=m_div,
                           output_codes=m_codes, output_scales=m_scales)
        dn.launch_partial(None, m, None, dn_codes, dn_scales, dn_div, partial,
                          activation_codes=m_codes, activation_scales=m_scales,
                          input_global_divisor=m_div)
        reduce_()

    slice_()
    torch.cuda.synchronize()
    if peer_addrs is not None:
        # the peer sum against NCCL on the same partials: same values up to the order of the
        # fp32 additions, i.e. at most one BF16 step apart, and identical on every rank
        mine = out.clone()
        check = partial.clone()
        dist.all_reduce(check)
        want = check.to(torch.bfloat16).float()
        got = mine.float()
        tol = want.abs() * 2.0 ** -7 + 1e-6
        bad = int(((got - want).abs() > tol).sum())
        assert bad == 0, f"peer sum differs from the NCCL all-reduce in {bad} values"
        ref = mine.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(ref.view(torch.int16), mine.view(torch.int16)), "ranks hold different sums"
    mode = "graph"
    try:
        graph = capture(torch, slice_, 1)
        run = graph.replay
    except Exception as exc:
        mode = f"eager ({type(exc).__name__})"
        run = slice_
        torch.cuda.synchronize()
    for _ in range(5):
        run()
    if world > 1:
        dist.barrier()
    reps = 50
    ms = time_region(torch, run, reps) / reps
    assert ctx.device_status() == 0
    return ms, mode, route


def run_case(args):
    """One small side case on one GPU (for profiling): `nvfp4:M`, `fp8:N:M`, `norm:M`,
    `fp8mlp:M`, `gdn:B`, `sampler:B`, `exchange`, `stamps:N:M` (per-CTA time stamps, experiment build) or
    `issue` (the tcgen05 issue-rate micro-benchmark beside this file)."""
    if args.case == "issue":
        src = os.path.join(ROOT, "bench_tcgen05_issue.cu")
        exe = os.path.join(ROOT, "bench_tcgen05_issue")
        if not os.path.exists(exe) or os.path.getmtime(exe) < os.path.getmtime(src):
            cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17",
                   "-I", ROOT, "-o", exe, src]
            if os.path.exists("/usr/bin/g++"):
                cmd[1:1] = ["-ccbin", "/usr/bin/g++"]
            subprocess.run(cmd, check=True)
        return subprocess.run([exe]).returncode

    import torch

    parts = args.case.split(":")
    stamps = None
    if parts[0] == "stamps":
        # the plane's address has to be in the environment before the library reads its switches
        torch.cuda.set_device(0)
        stamps = torch.zeros(8192 * 8, dtype=torch.int64, device="cuda")
        os.environ["TK100_STAMPS_PTR"] = hex(stamps.data_ptr())

    import tuiskollm_b200 as tk
    from tuiskollm_b200 import ops, synth

    torch.cuda.set_device(0)
    ctx = tk.Context(device=0)
    reps = args.case_reps
    if parts[0] == "stamps":
        # Where a decode CTA's time goes: %globaltimer stamps of every CTA of the FP8 projection
        # kernel (entry, set-up done, predecessor complete, first stage full, last MMA issued,
        # accumulator complete, epilogue done, exit), taken from the last launch of a back-to-back
        # sequence over rotating weight copies.  Needs a library built with TK100_EXPERIMENT=1.
        import numpy as np
        n_rows, m = int(parts[1]), int(parts[2])
        copies = max(4, int(3 * 126e6 / (n_rows * HIDDEN)) + 1)
        planes = [synth.torch_fp8_weights(SEED, 50 + c, n_rows, HIDDEN, "cuda") for c in range(copies)]
        x = synth.torch_normal_bf16(SEED, 7, (m, HIDDEN), "cuda")
        codes = torch.empty((m, HIDDEN), dtype=torch.uint8, device="cuda")
        scales = torch.empty((m,), dtype=torch.float32, device="cuda")
        out = torch.empty((m, n_rows), dtype=torch.bfloat16, device="cuda")
        op = tk.GdnInputProjectionOp(ctx, n_rows)
        op.launch(None, m, x, codes, scales, planes[0][0], planes[0][1], out)
        for _ in range(3):
            for c in range(copies):
                op.launch(None, m, None, codes, scales, planes[c][0], planes[c][1], out)
        torch.cuda.synchronize()
        stamps.zero_()
        for c in range(copies):
            op.launch(None, m, None, codes, scales, planes[c][0], planes[c][1], out)
        torch.cuda.synchronize()
        kernel = ctx.last_kernel
        splits = int(kernel.split("splits=")[1].split()[0])
        ctas = ((n_rows + 127) // 128) * splits * ((m + 127) // 128)
        st = stamps[: ctas * 8].cpu().numpy().reshape(ctas, 8).astype(np.float64)
        if not st.any():
            print(json.dumps({"case": args.case, "error": "no stamps: build the library with "
                              "TK100_EXPERIMENT=1 python -m tuiskollm_b200.build"}), flush=True)
            return 1
        d = (st - st[:, 0].min()) / 1e3
        med = lambda v: round(float(np.median(v)), 2)
        rows = [{"kernel": kernel, "ctas": ctas,
                 "us_median_per_cta": {"entry_to_setup_done": med(d[:, 1] - d[:, 0]),
                                       "entry_to_first_stage_full": med(d[:, 3] - d[:, 0]),
                                       "first_full_to_last_mma": med(d[:, 4] - d[:, 3]),
                                       "accumulator_complete_to_epilogue_done": med(d[:, 6] - d[:, 5]),
                                       "epilogue_done_to_exit": med(d[:, 7] - d[:, 6])},
                 "us_spread_of_cta_entries": round(float(d[:, 0].max()), 2),
                 "us_first_entry_to_last_exit": round(float(d[:, 7].max()), 2)}]
    elif parts[0] == "nvfp4":
        m = int(parts[1])
        which = parts[2] if len(parts) > 2 else "all"
        pl = MlpPlanes(torch, ops, synth, m, mlp_weights(synth))
        x = synth.torch_normal_bf16(SEED, 310, (m, HIDDEN), "cuda")
        gu, dn = tk.Nvfp4SwiGluOp(ctx), tk.Nvfp4DownOp(ctx)
        gu.quantize(None, m, HIDDEN, x, pl.a_div, pl.a_codes, pl.a_scales)
        rows = []

        def gate_up():
            gu.launch(None, m, None, pl.gu_codes, pl.gu_scales, pl.gu_div, pl.mid,
                      activation_codes=pl.a_codes, activation_scales=pl.a_scales,
                      input_global_divisor=pl.a_div)

        def quant_mid():
            dn.quantize(None, m, synth.INTERMEDIATE, pl.mid, pl.m_div, pl.m_codes, pl.m_scales)

        def down():
            dn.launch(None, m, None, pl.dn_codes, pl.dn_scales, pl.dn_div, pl.out,
                      activation_codes=pl.m_codes, activation_scales=pl.m_scales,
                      input_global_divisor=pl.m_div)

        gate_up(); quant_mid(); down()
        torch.cuda.synchronize()
        for nm, fn in (("gate_up", gate_up), ("down", down)):
            if which not in ("all", nm):
                continue
            for _ in range(2):
                fn()
            ms = time_region(torch, fn, reps) / reps
            rows.append({"op": nm, "M": m, "us": ms * 1e3, "kernel": ctx.last_kernel})
    elif parts[0] == "fp8":
        n_rows, m = int(parts[1]), int(parts[2])
        copies = max(4, int(3 * 126e6 / (n_rows * HIDDEN)) + 1)  # as in config_rows: 3 x L2
        planes = [synth.torch_fp8_weights(SEED, 50 + c, n_rows, HIDDEN, "cuda")
                  for c in range(copies)]
        x = synth.torch_normal_bf16(SEED, 7, (m, HIDDEN), "cuda")
        codes = torch.empty((m, HIDDEN), dtype=torch.uint8, device="cuda")
        scales = torch.empty((m,), dtype=torch.float32, device="cuda")
        outp = torch.empty((m, n_rows), dtype=torch.bfloat16, device="cuda")
        op = tk.GdnInputProjectionOp(ctx, n_rows)
        op.launch(None, m, x, codes, scales, planes[0][0], planes[0][1], outp)
        state = {"i": 0}

        def proj():
            w, sc = planes[state["i"] % copies]
            state["i"] += 1
            op.launch(None, m, None, codes, scales, w, sc, outp)

        graph = capture(torch, proj, copies)
        for _ in range(3):
            graph.replay()
        ms = time_region(torch, graph.replay, reps) / (reps * copies)
        rows = [{"op": "fp8", "N": n_rows, "M": m, "us": ms * 1e3, "kernel": ctx.last_kernel,
                 "GB/s": algorithmic_bytes(m, n_rows, HIDDEN, 2) / ms / 1e6}]
    elif parts[0] == "norm":
        m = int(parts[1])
        copies = max(2, int(2 * 126e6 / (m * HIDDEN * 11)) + 1)
        xs = [synth.torch_normal_bf16(SEED, 90 + c, (m, HIDDEN), "cuda") for c in range(copies)]
        bs = [synth.torch_normal_bf16(SEED, 190 + c, (m, HIDDEN), "cuda") for c in range(copies)]
        nw = synth.torch_normal_bf16(SEED, 5, (HIDDEN,), "cuda", std=0.1)
        res, nrm = torch.empty_like(xs[0]), torch.empty_like(xs[0])
        codes = torch.empty((m, HIDDEN), dtype=torch.uint8, device="cuda")
        scales = torch.empty((m,), dtype=torch.float32, device="cuda")
        normop = tk.ResidualNormOp(ctx)
        state = {"i": 0}

        def norm():
            i = state["i"] % copies
            state["i"] += 1
            normop.launch_quantize(None, m, xs[i], bs[i], nw, res, nrm, codes, scales)

        for _ in range(3):
            norm()
        ms = time_region(torch, norm, reps) / reps
        rows = [{"op": "norm", "M": m, "us": ms * 1e3, "GB/s": (11 * m * HIDDEN + 4 * m) / ms / 1e6}]
    elif parts[0] == "fp8mlp":
        # dense-FP8 gate/up + SwiGLU and down at M tokens, weight planes rotating through > L2
        m = int(parts[1])
        inter = synth.INTERMEDIATE
        copies = 3 if m <= 32 else 1
        gu_planes = [synth.torch_fp8_weights(SEED, 70 + c, 2 * inter, HIDDEN, "cuda") for c in range(copies)]
        dn_planes = [synth.torch_fp8_weights(SEED, 75 + c, HIDDEN, inter, "cuda") for c in range(copies)]
        x = synth.torch_normal_bf16(SEED, 9, (m, HIDDEN), "cuda")
        xi = synth.torch_normal_bf16(SEED, 10, (m, inter), "cuda")
        c1 = torch.empty((m, HIDDEN), dtype=torch.uint8, device="cuda")
        c2 = torch.empty((m, inter), dtype=torch.uint8, device="cuda")
        s1, s2 = (torch.empty((m,), dtype=torch.float32, device="cuda") for _ in range(2))
        mid = torch.empty((m, inter), dtype=torch.bfloat16, device="cuda")
        out = torch.empty((m, HIDDEN), dtype=torch.bfloat16, device="cuda")
        go_planes = [synth.torch_fp8_weights(SEED, 80 + c, HIDDEN, 6144, "cuda") for c in range(4 if m <= 32 else 1)]
        xg = synth.torch_normal_bf16(SEED, 11, (m, 6144), "cuda")
        c3 = torch.empty((m, 6144), dtype=torch.uint8, device="cuda")
        s3 = torch.empty((m,), dtype=torch.float32, device="cuda")
        out_g = torch.empty((m, HIDDEN), dtype=torch.bfloat16, device="cuda")
        sw_op, dn_op, go_op = tk.Fp8SwiGluOp(ctx), tk.Fp8DownOp(ctx), tk.GdnOutputProjectionOp(ctx, 6144)
        sw_op.launch(None, m, x, c1, s1, gu_planes[0][0], gu_planes[0][1], mid)
        dn_op.launch(None, m, xi, c2, s2, dn_planes[0][0], dn_planes[0][1], out)
        go_op.launch(None, m, xg, c3, s3, go_planes[0][0], go_planes[0][1], out_g)
        rows = []
        for nm, op_, planes_, args_ in (("fp8_swiglu", sw_op, gu_planes, (c1, s1, mid)),
                                        ("fp8_down", dn_op, dn_planes, (c2, s2, out)),
                                        ("fp8_gdn_output", go_op, go_planes, (c3, s3, out_g))):
            state = {"i": 0}

            def run(op_=op_, planes_=planes_, args_=args_, state=state):
                w, sc = planes_[state["i"] % len(planes_)]
                state["i"] += 1
                op_.launch(None, m, None, args_[0], args_[1], w, sc, args_[2])

            for _ in range(3):
                run()
            kernel = ctx.last_kernel
            ms = time_region(torch, run, reps) / reps
            rows.append({"op": nm, "M": m, "us": ms * 1e3, "kernel": kernel})
    elif parts[0] == "gdn":
        # one GDN decode step (prepare, recurrence) per call, state slots rotating through > L2
        b = int(parts[1])
        slots = 48
        g_x = synth.torch_normal_bf16(SEED, 400, (8, HIDDEN), "cuda")
        g_cw = synth.torch_normal_bf16(SEED, 401, (96, HIDDEN), "cuda", std=0.02)
        g_alog = synth.torch_normal_bf16(SEED, 402, (48,), "cuda")
        g_dt = synth.torch_normal_bf16(SEED, 403, (48,), "cuda")
        g_proj = synth.torch_normal_bf16(SEED, 404, (8, 16384), "cuda")
        g_convw = synth.torch_normal_bf16(SEED, 405, (10240, 4), "cuda", std=0.5)
        g_hist = synth.torch_normal_bf16(SEED, 406, (slots, 10240, 3), "cuda")
        g_state = torch.zeros((slots, 48, 128, 128), dtype=torch.float32, device="cuda")
        g_state.normal_(0.0, 0.05, generator=torch.Generator(device="cuda").manual_seed(SEED + 407))
        g_norm = synth.torch_normal_bf16(SEED, 408, (128,), "cuda")
        g_decay = torch.empty((8, 48), dtype=torch.float32, device="cuda")
        g_beta = torch.empty((8, 48), dtype=torch.float32, device="cuda")
        g_conv = torch.empty((8, 10240), dtype=torch.bfloat16, device="cuda")
        g_out = torch.empty((8, 6144), dtype=torch.bfloat16, device="cuda")
        groups = slots // b
        slot_rows = [torch.arange(g * b, (g + 1) * b, dtype=torch.int32, device="cuda") for g in range(groups)]
        prep_op, rec_op = tk.GdnPrepareOp(ctx), tk.GdnRecurrenceOp(ctx)
        state = {"i": 0}

        def gdn_step():
            r = slot_rows[state["i"] % groups]
            state["i"] += 1
            prep_op.launch(None, b, g_x, g_cw, g_alog, g_dt, g_proj, g_convw, r, g_hist, g_decay, g_beta, g_conv)
            rec_op.launch(None, b, g_conv, g_proj, g_decay, g_beta, g_norm, r, g_state, g_out)

        for _ in range(3):
            gdn_step()
        ms = time_region(torch, gdn_step, reps) / reps
        rows = [{"op": "gdn_step (eager launches)", "B": b, "us": ms * 1e3}]
    elif parts[0] == "sampler":
        b = int(parts[1])
        vocab = 248320
        copies = 8
        logit_rows = [synth.torch_normal_bf16(SEED, 500 + c, (b, vocab), "cuda", std=3.0) for c in range(copies)]
        samp = tk.Sampler(ctx, vocab, [tk.SamplingOptions(seed=i) for i in range(b)], [(1, 2)] * b)
        state = {"i": 0}

        def draw():
            samp.sample(None, logit_rows[state["i"] % copies])
            state["i"] += 1

        for _ in range(3):
            draw()
        ms = time_region(torch, draw, reps) / reps
        rows = [{"op": "device sampler (eager launches)", "B": b, "us": ms * 1e3}]
    elif parts[0] == "exchange":
        # the fused exchange kernel with world = 1: its fixed cost without NVLink or rank skew
        m = 1
        buf = torch.zeros((ops.exchange_bytes(m, 1) + 7) // 8, dtype=torch.int64, device="cuda")
        scratch = torch.zeros((m,), dtype=torch.int64, device="cuda")
        merged = torch.zeros((m, 2), dtype=torch.int32, device="cuda")
        op = tk.LmHeadOp(ctx, 4096, 0)
        fn = lambda: op.exchange(None, m, 1, 0, scratch, [buf.data_ptr()], merged)
        for _ in range(3):
            fn()
        ms = time_region(torch, fn, reps) / reps
        rows = [{"op": "argmax_exchange world=1", "us": ms * 1e3}]
    else:
        raise SystemExit(f"unknown case {args.case}")
    status = ctx.device_status()
    print(json.dumps({"status": status, "case": args.case, "rows": rows}), flush=True)
    return 0


def first_maximum_merge(gathered):
    """Host restatement of the merge rule (tuisko-engine/src/sampling.rs:162-173 over shards):
    `gathered` [world, rows, 2] int32 (value bits, global index, -1 = none) -> [rows, 2]; the
    greater value in IEEE total order wins, equal values go to the lowest global index."""
    import numpy as np

    world, rows, _ = gathered.shape
    out = np.zeros((rows, 2), np.int32)
    for t in range(rows):
        best = None
        for r in range(world):
            bits, idx = int(gathered[r, t, 0]) & 0xFFFFFFFF, int(gathered[r, t, 1])
            if idx < 0:
                continue
            key = bits ^ (0xFFFFFFFF if bits & 0x80000000 else 0x80000000)
            if best is None or (key, -idx) > (best[0], -best[1]):
                best = (key, idx, int(gathered[r, t, 0]))
        out[t] = (best[2], best[1]) if best else (0, -1)
    return out


def run_native(args):
    import numpy as np
    import torch

    import tuiskollm_b200 as tk
    from tuiskollm_b200 import synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    m = args.rows
    vocab = args.vocab
    assert vocab % (world * 16) == 0, "vocabulary must split into shards of a multiple of 16 rows"
    shard = vocab // world
    offset = rank * shard
    ctx = tk.Context(device=local, max_rows=max(2048, m))
    dev = "cuda"
    # every rank draws the same hidden rows; weights are drawn per shard (stream = rank)
    wc, ws = synth.torch_fp8_weights(SEED, 1000 + rank, shard, HIDDEN, dev)
    x_host = torch.from_numpy(synth.normal_bf16(SEED, 2, (m, HIDDEN)).view(np.int16)).pin_memory()
    x = x_host.to(dev)
    codes = torch.empty((m, HIDDEN), dtype=torch.uint8, device=dev)
    scales = torch.empty((m,), dtype=torch.float32, device=dev)
    logits = torch.empty((m, shard), dtype=torch.float32, device=dev)
    scratch = torch.zeros((m,), dtype=torch.int64, device=dev)
    pairs = torch.zeros((m, 2), dtype=torch.int32, device=dev)
    gathered = torch.zeros((world, m, 2), dtype=torch.int32, device=dev)
    merged = torch.zeros((m, 2), dtype=torch.int32, device=dev)
    merged_host = torch.zeros((m, 2), dtype=torch.int32).pin_memory()
    op = tk.LmHeadOp(ctx, shard, offset)
    exchange = "none"
    peer_addresses = None
    if world > 1:
        exchange = "nccl all_gather + merge kernel"
        if not args.nccl_gather:
            try:
                from tuiskollm_b200 import dist as tkd
                _xbuf, _xhdl, peer_addresses = tkd.alloc_exchange(m, world, torch.device("cuda", local))
                exchange = ("peer stores over NVLink fused with the merge (one kernel behind the projection)"
                            if args.split_exchange else
                            "peer stores over NVLink and merge by the projection kernel's last CTA")
            except Exception as exc:  # symmetric memory unavailable: keep the NCCL route
                exchange += f" (peer exchange unavailable: {type(exc).__name__}: {exc})"[:300]
    # all ranks must agree on the route
    if world > 1:
        flag = torch.tensor([1 if peer_addresses is not None else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            peer_addresses = None

    def step():
        if peer_addresses is not None:
            if args.split_exchange:  # projection, then the exchange + merge as its own launch
                op.launch(None, m, x, codes, scales, wc, ws, None, logits, scratch, None)
                op.exchange(None, m, world, rank, scratch, peer_addresses, merged)
            else:  # quantiser, then ONE launch: projection + argmax + peer exchange + merge
                op.launch_sharded(None, m, x, codes, scales, wc, ws, None, logits, scratch, world,
                                  rank, peer_addresses, merged)
            return
        op.launch(None, m, x, codes, scales, wc, ws, None, logits, scratch, pairs)
        if world > 1:
            dist.all_gather_into_tensor(gathered.view(-1), pairs.view(-1))
            op.merge(None, m, world, gathered, merged)

    def step_e2e():
        x.copy_(x_host, non_blocking=True)
        step()
        merged_host.copy_(merged if world > 1 else pairs, non_blocking=True)

    def projection_only():
        op.launch(None, m, None, codes, scales, wc, ws, None, logits, scratch, pairs)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def meet():
        """barrier + synchronize, after which all ranks leave at the same instant of the host's
        monotonic clock (one box, one clock): rank 0 names an instant 2 ms ahead before the
        barrier and everybody spins up to it.  Without this the ranks leave the barrier tens of
        microseconds apart and a short timed region measures that scatter in its first exchange."""
        if world == 1:
            torch.cuda.synchronize()
            return
        when = torch.zeros(1, dtype=torch.int64, device=dev)
        if rank == 0:
            when[0] = time.monotonic_ns() + 2_000_000
        dist.broadcast(when, 0)
        dist.barrier()
        torch.cuda.synchronize()
        target = int(when.item())
        while time.monotonic_ns() < target:
            pass

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(3):
        step()
    kernel_name = ctx.last_kernel
    barrier()
    # One step as a CUDA graph (kernels + the NCCL gather), replayed: the way the reference's
    # engine runs this path (tuisko-engine/src/program.rs:149-154, 303-319).
    mode = "graph"
    launches0 = ctx.launch_count
    try:
        if args.eager:
            raise RuntimeError("eager requested")
        graph = capture(torch, step, 1)
        run_step = graph.replay
    except Exception as exc:  # capture of the collective can be refused by the backend
        mode = f"eager ({type(exc).__name__})"
        run_step = step
        torch.cuda.synchronize()
    launches_per_step = (ctx.launch_count - launches0) // 2 if mode == "graph" else None
    if rank == 0:
        sampler.wait_for_first_sample()
    for _ in range(max(3, args.warmup)):
        run_step()
    # rank 0 alone spent host time on the sampler; the exchange kernels of the other ranks give a
    # late peer 2 s, so the ranks meet again before the timed region
    barrier()
    first_clock_sample = sampler.mark()
    launches0 = ctx.launch_count
    meet()
    ms = time_region(torch, run_step, args.steps)
    launches = (launches_per_step * args.steps if launches_per_step is not None
                else ctx.launch_count - launches0)
    barrier()
    # The reference's protocol on the same step: 40 samples of `inner` replays each (at least
    # half a second of load in total, which also gives the clock sampler something to see).
    # (every rank must replay the same number of steps: the count comes from the slowest rank's time)
    ms_all = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms_all, op=dist.ReduceOp.MAX)
    inner = max(1, min(256, int(0.5e3 / SAMPLES / max(float(ms_all.item()) / args.steps, 1e-3)) + 1))
    sample_us = []
    for _ in range(SAMPLES):
        meet()
        sample_us.append(time_region(torch, run_step, inner) * 1e3 / inner)
    st = torch.tensor(sample_us, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
    sample_us = sorted(float(v) for v in st.tolist())
    barrier()
    # End to end: the same step with the pinned-host -> device copy of the hidden rows in front
    # and the device -> pinned-host copy of the selected (value, index) pairs behind, recorded
    # into one graph like the step itself; the host waits for every step's result.
    run_e2e, e2e_mode = step_e2e, "eager"
    if mode == "graph":
        try:
            graph_e2e = capture(torch, step_e2e, 1)
            run_e2e, e2e_mode = graph_e2e.replay, "graph"
        except Exception:  # keep the eager calls
            torch.cuda.synchronize()
    for _ in range(3):
        run_e2e()
    meet()
    ms_e2e = time_region(torch, run_e2e, args.steps, sync_each=True)
    barrier()
    # ... and without a graph: every operator call made from the host, per step (C-ABI cost)
    for _ in range(3):
        step_e2e()
        torch.cuda.synchronize()
    meet()
    ms_e2e_eager = time_region(torch, step_e2e, args.steps, sync_each=True)
    barrier()
    for _ in range(3):
        projection_only()
    ms_proj = time_region(torch, projection_only, max(args.steps, 20))
    ms_proj = ms_proj / max(args.steps, 20) * args.steps
    clocks = sampler.stop(first_clock_sample) if rank == 0 else None

    tp = []
    if world > 1 and not args.no_extra:
        for m_tp in (256, 1):
            t_ms, t_mode, t_route = tp_layer_slice(torch, tk, dist, rank, world, m_tp, local,
                                                   nccl_reduce=args.nccl_reduce)
            tp.append([m_tp, t_ms, t_mode, t_route])
    times = torch.tensor([ms, ms_e2e, ms_proj, ms_e2e_eager] + [t[1] for t in tp],
                         dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    vals = [float(v) for v in times.tolist()]
    ms, ms_e2e, ms_proj, ms_e2e_eager = vals[:4]
    for t, v in zip(tp, vals[4:]):
        t[1] = v

    # ---- correctness of what was timed
    def local_pairs():
        """This rank's own (max, index) pairs for the current inputs (finalize route)."""
        op.launch(None, m, x, codes, scales, wc, ws, None, logits, scratch, pairs)
        torch.cuda.synchronize()
        return pairs.cpu().numpy().copy()

    def check_step(tag):
        """One step; the device argmax must equal the first maximum of the logits this rank
        wrote, and at N > 1 the merged pair must equal, bit for bit and on every rank, the host
        merge of all ranks' local pairs (gathered with NCCL)."""
        run_step()
        torch.cuda.synchronize()
        final = (merged if world > 1 else pairs).cpu().numpy().copy()
        mine = local_pairs()
        rounded = logits.to(torch.bfloat16).float()
        for t in range(m):
            first = int(torch.nonzero(rounded[t] == rounded[t].max())[0, 0]) + offset
            assert int(mine[t, 1]) == first, f"{tag}: device argmax disagrees with its own logits"
        if world == 1:
            return {"scenario": tag, "token0_index": int(final[0, 1])}
        all_local = torch.zeros((world, m, 2), dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(all_local.view(-1), torch.from_numpy(mine).to(dev).view(-1))
        expect = first_maximum_merge(all_local.cpu().numpy())
        assert np.array_equal(final, expect), (
            f"{tag}: rank {rank} merged pair {final.tolist()} != host merge {expect.tolist()}")
        all_final = torch.zeros((world, m, 2), dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(all_final.view(-1), torch.from_numpy(final).to(dev).view(-1))
        af = all_final.cpu().numpy()
        assert all(np.array_equal(af[r], af[0]) for r in range(world)), f"{tag}: ranks disagree"
        return {"scenario": tag, "token0_index": int(final[0, 1]),
                "winner_rank": int(final[0, 1]) // shard,
                "local_indices_token0": [int(v) for v in all_local[:, 0, 1].tolist()]}

    checks = [check_step("random weights")]
    if world > 1:
        # Plant a row that wins by a wide margin -- its codes are the token's own activation
        # codes, so its logit is the sum of their squares -- in the LAST rank's shard, then the
        # same row in a second shard so that the maximum is an exact cross-shard tie.
        planted_row = 5
        def plant(in_rank, local_row):
            if rank == in_rank:
                wc[local_row].copy_(codes[0])
                ws.view(torch.int16)[local_row] = 0x3F80  # BF16 1.0
            torch.cuda.synchronize()
            dist.barrier()
        plant(world - 1, planted_row)
        c = check_step("winner planted in the last rank's shard")
        assert c["token0_index"] == (world - 1) * shard + planted_row, c
        checks.append(c)
        tie_rank = 1 if world > 2 else 0
        plant(tie_rank, planted_row + 4)
        c = check_step("exact tie between two shards")
        assert c["token0_index"] == tie_rank * shard + planted_row + 4, c
        checks.append(c)
    status = ctx.device_status()
    assert status == 0, f"device status word {status:#x}"

    if rank == 0:
        peak, peak_kind = measured_peak()
        total_bytes = algorithmic_bytes(m, vocab, HIDDEN, 4) + (world - 1) * (m * HIDDEN + 4 * m)
        per_step = ms / args.steps
        value = total_bytes / per_step / 1e6
        e2e_value = total_bytes / (ms_e2e / args.steps) / 1e6
        shard_bytes = algorithmic_bytes(m, shard, HIDDEN, 4)
        proj_ms = ms_proj / args.steps
        achieved = shard_bytes / proj_ms / 1e6
        cfg = workload_config(m, vocab, world)
        line = {
            "metric": "fp8_lm_head_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "e4m3",
            "data": "synthetic", "config": cfg,
            "run": {"vocab_shard_rows": shard, "launch": mode, "exchange": exchange,
                    "tokens_per_s": m / (per_step * 1e-3), "us_per_step": per_step * 1e3},
            "protocol": {"samples": SAMPLES, "replays_per_sample": inner,
                         "us_per_step": {"median": statistics.median(sample_us),
                                         "p10": percentile(sample_us, 0.1),
                                         "p90": percentile(sample_us, 0.9)},
                         "source": "qual/src/device_benchmark.rs:993-1101 (40 samples, median/p10/p90)"},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": m * HIDDEN * 2,
                    "d2h_bytes_per_step": m * 8, "us_per_step": ms_e2e / args.steps * 1e3,
                    "launch": e2e_mode,
                    "eager": {"value": total_bytes / (ms_e2e_eager / args.steps) / 1e6,
                              "us_per_step": ms_e2e_eager / args.steps * 1e3,
                              "note": "every operator call made from the host each step, no graph"}},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "traffic": int(round(shard_bytes * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE)),
                         "traffic_source": "ncu dram read+write bytes of this kernel at vocab "
                                           "248320, M=1 (1 272 757 504 B), scaled by algorithmic bytes",
                         "peak_kind": peak_kind,
                         "kernel": kernel_name + " (finalize / peer exchange in its last CTA)",
                         "algorithmic_bytes": shard_bytes,
                         "us_per_launch": proj_ms * 1e3, "frac_of_8TBs": achieved / NOMINAL_HBM_GBS},
            "clocks": clocks,
            "checks": checks,
            "selected_tokens": [c["token0_index"] for c in checks],
        }
        if tp:
            # per rank: its share of the slice's weight bytes (FP8 QKV + GDN-in planes, NVFP4 codes and
            # scales of gate_up and down) against the measured copy rate, and the fp32 partial sums
            # that cross NVLink (each rank sends and receives (world - 1) / world of them, two-shot)
            from tuiskollm_b200 import synth as _synth
            slice_weight_bytes = ((_synth.QKV_ROWS + _synth.GDN_ROWS) * HIDDEN
                                  + 3 * _synth.INTERMEDIATE * HIDDEN * 9 // 16)
            line["tp_layer_slice"] = [
                {"M": t[0], "us": t[1] * 1e3, "launch": t[2], "partial_bytes": t[0] * HIDDEN * 4,
                 "reduce": t[3],
                 "parallelism": f"column(QKV,GDN-in,gate_up) + row(down) x{world}, fp32 partial sums",
                 "roofline": {"bound": "hbm" if t[0] <= 32 else "tensor",
                              "weight_bytes_per_rank": slice_weight_bytes // world,
                              "floor_us_at_measured_hbm": slice_weight_bytes / world / peak / 1e3,
                              "frac": slice_weight_bytes / world / peak / 1e3 / (t[1] * 1e3),
                              "nvlink_bytes_per_rank": t[0] * HIDDEN * 4 * (world - 1) // world,
                              "nvlink_floor_us_at_770GBs": t[0] * HIDDEN * 4 * (world - 1) / world / 770e3,
                              "peak_kind": peak_kind}}
                for t in tp]
        if world == 1 and not args.no_cpu:
            gbs, dt, threads, note, srows = cpu_lm_head(m, 3, 1, budget_s=15.0,
                                                        sample_rows=args.cpu_sample_rows)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                    "sample": note, "seconds_per_sample": dt,
                                    "sampled_vocab_rows": srows}
        if world == 1 and not args.no_extra:
            # clocks while the configuration rows run (their cases are visited in rotating order,
            # so one median covers them all); each row also carries time x that median, which
            # compares runs taken at different sustained clocks
            row_sampler = ClockSampler(local)
            row_sampler.start()
            rows, deviation = config_rows(torch, tk, ctx, peak, peak_kind,
                                          {"m": m, "vocab": vocab, "wc": wc, "ws": ws},
                                          with_cpu=not args.no_cpu)
            row_clocks = row_sampler.stop()
            line["clocks_configs"] = row_clocks
            if row_clocks.get("sm_mhz"):
                for r in rows:
                    r["kilocycles_at_median_sm_clock"] = r["us"]["median"] * row_clocks["sm_mhz"] / 1e3
            line["configs"] = rows
            if deviation is not None:
                line["w4a4_vs_a16"] = deviation
        print(json.dumps(line), flush=True)
    if world > 1:
        # Graphs that hold NCCL kernels are still alive here and tearing the process group
        # down under them can block; everything is flushed and synchronised, so leave directly.
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--rows", type=int, default=1, help="decode tokens M (1, 4 or 32 in the config)")
    ap.add_argument("--cpu-sample-rows", type=int, default=0,
                    help="vocabulary rows per CPU step (0 = sized from a probe)")
    ap.add_argument("--vocab", type=int, default=VOCAB,
                    help="vocabulary rows (a smaller plane makes a small profiling case)")
    ap.add_argument("--eager", action="store_true", help="launch every step from the host")
    ap.add_argument("--nccl-reduce", action="store_true",
                    help="tensor-parallel slice: NCCL all-reduce + rounding kernel instead of the peer sum")
    ap.add_argument("--nccl-gather", action="store_true",
                    help="N > 1: gather the pairs with NCCL instead of the fused peer exchange")
    ap.add_argument("--split-exchange", action="store_true",
                    help="N > 1: the peer exchange as a launch of its own behind the projection")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--case", default="",
                    help="run one side case only: nvfp4:M[:gate_up|down], fp8:N:M, norm:M, exchange, issue")
    ap.add_argument("--case-reps", type=int, default=20, help="timed launches of a --case run")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.case:
        return run_case(args)
    return run_native(args)


if __name__ == "__main__":
    sys.exit(main())
