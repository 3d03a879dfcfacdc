#!/usr/bin/env python
"""Benchmark of the quantized projection hot path on B200.

Workload (all N): the FP8 LM head with fused greedy argmax of the third benchmark
configuration -- K = 5120, vocabulary 248320, M decode tokens (default 1), E4M3 weights
~N(0, 0.02) with one BF16 scale per row, BF16 hidden ~N(0, 1), fp32 logits + int32 argmax
out -- the largest single-GPU configuration of the path and the one that shards: the
vocabulary is split contiguously over the N ranks, every rank streams its shard once per
step and the per-shard (max, index) pairs are gathered with NCCL and merged.

One step = quantise the hidden rows + stream the weight shard through the tcgen05
projection kernel + argmax finalize (+ all-gather + merge when N > 1).

  value   whole-job algorithmic GB/s with the hidden rows resident in HBM
  e2e     the same through the public operator call with HOST buffers: pinned-host ->
          device copy of the hidden rows and device -> host read of the argmax pairs
          inside the timed region, one stream synchronisation per step
  roofline  the projection kernel alone against the measured HBM copy bandwidth

`--impl reference` times the CPU restatement of the reference's qualification oracle for
the same workload on the host cores (the reference is Rust + cuda-oxide for sm_120 and can
neither be built nor run here).
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

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN = 5120
VOCAB = 248320
SEED = 20260425
# DRAM bytes (read + write) that ncu counted for one LM-head projection launch at vocab 248320,
# M = 1, over that launch's algorithmic bytes (1 272 757 504 / 1 272 893 444): every weight byte
# crosses HBM once (ncu: dram__bytes_read.sum + dram__bytes_write.sum of one captured launch).
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1272757504 / 1272893444
FALLBACK_HBM_GBS = 6650.0


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


class ClockSampler:
    """Polls nvidia-smi for SM clocks and throttle reasons while the timed region runs."""

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

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        sm, mx, reasons = [], 0.0, set()
        for p in self.samples:
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

def cpu_lm_head(rows: int, steps: int, warmup: int, budget_s: float, sample_rows: int = 0):
    """Times the oracle's LM-head formula (quantise + f64 FP8 dot + greedy pick) on a
    bounded sample of vocabulary rows sized so that all steps take about `budget_s` seconds;
    returns (GB/s, seconds/step, threads, note)."""
    import numpy as np

    from oracle import tuisko_oracle as O
    from tuiskollm_b200 import synth

    O.lib()
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
    return nbytes / dt / 1e9, dt, O.num_threads(), note, sample_rows


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
        "config": {"workload": f"fp8_lm_head_argmax K={HIDDEN} vocab={VOCAB} M={args.rows}",
                   "rows": args.rows, "sampled_vocab_rows": sample},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": note},
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


def extra_rows(torch, tk, ctx, peak_gbs):
    """Other configurations of the path on one GPU: decode projections with the weight plane
    rotated over several copies so that every launch streams from HBM, not from L2."""
    import numpy as np

    from tuiskollm_b200 import synth

    out = []
    dev = "cuda"
    for name, n_rows in (("fp8_qkv", synth.QKV_ROWS), ("fp8_gdn_input", synth.GDN_ROWS),
                         ("fp8_qkv_refN", synth.QKV_ROWS_REF),
                         ("fp8_gdn_input_refN", synth.GDN_ROWS_REF)):
        copies = max(4, int(3 * 126e6 / (n_rows * HIDDEN)) + 1)
        planes = [synth.torch_fp8_weights(SEED, 50 + c, n_rows, HIDDEN, dev) for c in range(copies)]
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

            def proj():
                w, s = planes[state["i"] % copies]
                state["i"] += 1
                op.launch(None, m, None, codes, scales, w, s, outp)

            state["i"] = 0
            graph = capture(torch, proj, copies)  # one launch per weight copy, in rotation
            for _ in range(3):
                graph.replay()
            reps = 20
            ms = time_region(torch, graph.replay, reps) / (reps * copies)
            b = algorithmic_bytes(m, n_rows, HIDDEN, 2)
            out.append({"op": name, "M": m, "N": n_rows, "us": ms * 1e3, "GB/s": b / ms / 1e6,
                        "frac_of_measured_hbm": b / ms / 1e6 / peak_gbs,
                        "frac_of_8TBs": b / ms / 1e6 / 8000.0, "weight_copies": copies})
        del planes
    # prefill-shaped FP8 projections (tensor-bound): one weight plane, graph of 8 launches
    burst, _sustained, tkind = measured_tensor_peaks()
    for name, n_rows in (("fp8_qkv", synth.QKV_ROWS), ("fp8_gdn_input", synth.GDN_ROWS)):
        w, s = synth.torch_fp8_weights(SEED, 60, n_rows, HIDDEN, dev)
        for m in (256, 512, 2048):
            x = synth.torch_normal_bf16(SEED, 8, (m, HIDDEN), dev)
            codes = torch.empty((m, HIDDEN), dtype=torch.uint8, device=dev)
            scales = torch.empty((m,), dtype=torch.float32, device=dev)
            outp = torch.empty((m, n_rows), dtype=torch.bfloat16, device=dev)
            op = tk.GdnInputProjectionOp(ctx, n_rows)
            op.launch(None, m, x, codes, scales, w, s, outp)
            graph = capture(torch, lambda: op.launch(None, m, None, codes, scales, w, s, outp), 8)
            for _ in range(3):
                graph.replay()
            ms = time_region(torch, graph.replay, 10) / 80
            tf = 2.0 * m * n_rows * HIDDEN / ms / 1e9
            out.append({"op": name, "M": m, "N": n_rows, "us": ms * 1e3, "TFLOPs": tf,
                        "frac_of_4.5PF": tf / 4500.0, "frac_of_2x_measured_bf16": tf / (2 * burst),
                        "tensor_peak_kind": tkind})
        del w, s
    # fused residual + RMSNorm + quantise
    normop = tk.ResidualNormOp(ctx)
    for m in (1, 256, 512):
        copies = 1 if m == 1 else max(2, int(2 * 126e6 / (m * HIDDEN * 11)) + 1)
        xs = [synth.torch_normal_bf16(SEED, 90 + c, (m, HIDDEN), dev) for c in range(copies)]
        bs = [synth.torch_normal_bf16(SEED, 190 + c, (m, HIDDEN), dev) for c in range(copies)]
        w = synth.torch_normal_bf16(SEED, 5, (HIDDEN,), dev, std=0.1)
        res = [torch.empty_like(xs[0]) for _ in range(copies)]
        nrm = [torch.empty_like(xs[0]) for _ in range(copies)]
        codes = [torch.empty((m, HIDDEN), dtype=torch.uint8, device=dev) for _ in range(copies)]
        scales = torch.empty((m,), dtype=torch.float32, device=dev)
        state = {"i": 0}

        def norm():
            i = state["i"] % copies
            state["i"] += 1
            normop.launch_quantize(None, m, xs[i], bs[i], w, res[i], nrm[i], codes[i], scales)

        state["i"] = 0
        graph = capture(torch, norm, copies * 4)
        for _ in range(3):
            graph.replay()
        reps = 20
        ms = time_region(torch, graph.replay, reps) / (reps * copies * 4)
        b = 10 * m * HIDDEN + m * HIDDEN + 4 * m
        out.append({"op": "residual_rmsnorm_quant_e4m3", "M": m, "us": ms * 1e3,
                    "GB/s": b / ms / 1e6, "frac_of_measured_hbm": b / ms / 1e6 / peak_gbs})
    out.extend(nvfp4_rows(torch, tk, ctx))
    out.extend(layer_slice_rows(torch, tk, ctx))
    return out


def measured_tensor_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 1590.0, 1400.0, "fallback"


class MlpPlanes:
    """Synthetic NVFP4 MLP weights + activation planes for `m` tokens."""

    def __init__(self, torch, ops, synth, m, dev="cuda"):
        inter = synth.INTERMEDIATE
        self.m = m
        self.gu_codes, self.gu_scales, self.gu_div = synth.torch_nvfp4_weights(
            SEED, 300, 2 * inter, HIDDEN, dev)
        self.dn_codes, self.dn_scales, self.dn_div = synth.torch_nvfp4_weights(
            SEED, 301, HIDDEN, inter, dev)
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


def nvfp4_rows(torch, tk, ctx, row_counts=(2048, 256, 32, 8, 1)):
    """NVFP4 MLP (configuration 4 at M = 2048, and decode shapes): each kernel as graph
    replays; prefill in TFLOP/s against the block-scaled FP4 peak, decode in GB/s."""
    from tuiskollm_b200 import ops, synth

    inter = synth.INTERMEDIATE
    burst, sustained, kind = measured_tensor_peaks()
    hbm, _ = measured_peak()
    out = []
    for m in row_counts:
        pl = MlpPlanes(torch, ops, synth, m)
        x = synth.torch_normal_bf16(SEED, 310, (m, HIDDEN), "cuda")
        gu, dn = tk.Nvfp4SwiGluOp(ctx), tk.Nvfp4DownOp(ctx)

        def quant_in():
            gu.quantize(None, m, HIDDEN, x, pl.a_div, pl.a_codes, pl.a_scales)

        def gate_up():
            gu.launch(None, m, None, pl.gu_codes, pl.gu_scales, pl.gu_div, pl.mid,
                      activation_codes=pl.a_codes, activation_scales=pl.a_scales,
                      input_global_divisor=pl.a_div)

        def quant_mid():
            dn.quantize(None, m, inter, pl.mid, pl.m_div, pl.m_codes, pl.m_scales)

        def down():
            dn.launch(None, m, None, pl.dn_codes, pl.dn_scales, pl.dn_div, pl.out,
                      activation_codes=pl.m_codes, activation_scales=pl.m_scales,
                      input_global_divisor=pl.m_div)

        def gate_up_q():  # the same projection also leaving the NVFP4 form of its output
            gu.launch_quantize(None, m, None, pl.gu_codes, pl.gu_scales, pl.gu_div, pl.mid,
                               activation_codes=pl.a_codes, activation_scales=pl.a_scales,
                               input_global_divisor=pl.a_div, output_global_divisor=pl.m_div,
                               output_codes=pl.m_codes, output_scales=pl.m_scales)

        def mlp():
            quant_in(); gate_up_q(); down()

        for fn in (quant_in, gate_up, quant_mid, down):
            fn()
        torch.cuda.synchronize()
        times = {}
        for name, fn in (("quant_in", quant_in), ("gate_up_swiglu", gate_up),
                         ("quant_mid", quant_mid), ("gate_up_swiglu_quantize", gate_up_q),
                         ("down", down), ("mlp_total", mlp)):
            graph = capture(torch, fn, 4)
            for _ in range(3):
                graph.replay()
            reps = 10
            times[name] = time_region(torch, graph.replay, reps) / (reps * 4)
        f_gu = 2.0 * m * 2 * inter * HIDDEN
        f_dn = 2.0 * m * HIDDEN * inter
        b_gu = 2 * inter * HIDDEN // 2 + 2 * inter * HIDDEN // 16 + m * HIDDEN // 2 + m * HIDDEN // 16 + 2 * m * inter
        b_dn = HIDDEN * inter // 2 + HIDDEN * inter // 16 + m * inter // 2 + m * inter // 16 + 2 * m * HIDDEN
        row = {"op": "nvfp4_mlp", "M": m, "us": {k: v * 1e3 for k, v in times.items()},
               "gate_up_TFLOPs": f_gu / times["gate_up_swiglu"] / 1e9,
               "down_TFLOPs": f_dn / times["down"] / 1e9,
               "mlp_TFLOPs": (f_gu + f_dn) / times["mlp_total"] / 1e9,
               "gate_up_GBs": b_gu / times["gate_up_swiglu"] / 1e6,
               "down_GBs": b_dn / times["down"] / 1e6}
        if m >= 256:
            row["gemm_frac_of_9PF"] = (f_gu + f_dn) / (times["gate_up_swiglu"] + times["down"]) / 1e9 / 9000.0
            row["gemm_frac_of_4x_measured_bf16"] = ((f_gu + f_dn) / (times["gate_up_swiglu"] + times["down"])
                                                    / 1e9 / (4 * burst))
            row["tensor_peak_kind"] = kind
        else:
            row["gate_up_frac_of_measured_hbm"] = row["gate_up_GBs"] / hbm
            row["down_frac_of_measured_hbm"] = row["down_GBs"] / hbm
        out.append(row)
        del pl
    return out


def layer_slice_rows(torch, tk, ctx):
    """Configuration 5, one GPU: residual add + RMSNorm + E4M3 and NVFP4 quantise (one kernel)
    -> FP8 QKV (N = 8192) -> FP8 GDN-input (N = 12288) -> NVFP4 gate_up + SwiGLU (its epilogue
    leaves the NVFP4 form of the intermediate at decode sizes, a quantiser launch otherwise) ->
    NVFP4 down, as one CUDA graph of five or six kernels."""
    from tuiskollm_b200 import ops, synth

    out = []
    dev = "cuda"
    qkv_w = synth.torch_fp8_weights(SEED, 400, synth.QKV_ROWS, HIDDEN, dev)
    gdn_w = synth.torch_fp8_weights(SEED, 401, synth.GDN_ROWS, HIDDEN, dev)
    nw = synth.torch_normal_bf16(SEED, 5, (HIDDEN,), dev, std=0.1)
    weight_bytes = (synth.QKV_ROWS + synth.GDN_ROWS) * HIDDEN + 3 * synth.INTERMEDIATE * HIDDEN * 9 // 16
    for m in (1, 256, 512):
        pl = MlpPlanes(torch, ops, synth, m)
        x = synth.torch_normal_bf16(SEED, 410, (m, HIDDEN), dev)
        br = synth.torch_normal_bf16(SEED, 411, (m, HIDDEN), dev)
        res = torch.empty_like(x)
        nrm = torch.empty_like(x)
        codes = torch.empty((m, HIDDEN), dtype=torch.uint8, device=dev)
        scales = torch.empty((m,), dtype=torch.float32, device=dev)
        qkv = torch.empty((m, synth.QKV_ROWS), dtype=torch.bfloat16, device=dev)
        gdn = torch.empty((m, synth.GDN_ROWS), dtype=torch.bfloat16, device=dev)
        norm = tk.ResidualNormOp(ctx)
        qkv_op = tk.FullAttentionQkvOp(ctx, synth.QKV_ROWS)
        gdn_op = tk.GdnInputProjectionOp(ctx, synth.GDN_ROWS)
        gu, dn = tk.Nvfp4SwiGluOp(ctx), tk.Nvfp4DownOp(ctx)

        def slice_():
            norm.launch_quantize_nvfp4(None, m, x, br, nw, res, nrm, codes, scales, pl.a_div,
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

        slice_()
        torch.cuda.synchronize()
        graph = capture(torch, slice_, 1)
        for _ in range(5):
            graph.replay()
        reps = 50
        ms = time_region(torch, graph.replay, reps) / reps
        flops = 2.0 * m * HIDDEN * (synth.QKV_ROWS + synth.GDN_ROWS + 3 * synth.INTERMEDIATE)
        out.append({"op": "layer_slice", "M": m, "us": ms * 1e3, "kernels": 5 if m <= 32 else 6,
                    "weight_stream_GBs": weight_bytes / ms / 1e6, "TFLOPs": flops / ms / 1e9,
                    "floor_us_at_measured_hbm": weight_bytes / measured_peak()[0] / 1e3})
        del pl
    return out


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
    """One small side case on one GPU (for profiling): `nvfp4:M` or `fp8:N:M`."""
    import torch

    import tuiskollm_b200 as tk
    from tuiskollm_b200 import synth

    torch.cuda.set_device(0)
    ctx = tk.Context(device=0)
    parts = args.case.split(":")
    if parts[0] == "nvfp4":
        rows = nvfp4_rows(torch, tk, ctx, (int(parts[1]),))
    elif parts[0] == "fp8":
        n_rows, m = int(parts[1]), int(parts[2])
        copies = max(4, int(3 * 126e6 / (n_rows * HIDDEN)) + 1)  # as in extra_rows: 3 x L2
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
        ms = time_region(torch, graph.replay, 20) / (20 * copies)
        rows = [{"op": "fp8", "N": n_rows, "M": m, "us": ms * 1e3,
                 "GB/s": algorithmic_bytes(m, n_rows, HIDDEN, 2) / ms / 1e6}]
    else:
        raise SystemExit(f"unknown case {args.case}")
    status = ctx.device_status()
    print(json.dumps({"debug": os.environ.get("TK100_DEBUG", "0"), "status": status, "case": args.case, "rows": rows}), flush=True)
    return 0


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
                exchange = "peer stores over NVLink fused with the merge (one kernel)"
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
            op.launch(None, m, x, codes, scales, wc, ws, None, logits, scratch, None)
            op.exchange(None, m, world, rank, scratch, peer_addresses, merged)
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

    def local_pairs():
        """This rank's own (max, index) pairs of the last step, for the sanity check."""
        if peer_addresses is None:
            return pairs.cpu().numpy()
        op.launch(None, m, x, codes, scales, wc, ws, None, logits, scratch, pairs)
        torch.cuda.synchronize()
        return pairs.cpu().numpy()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(3):
        step()
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
    for _ in range(max(3, args.warmup)):
        run_step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # rank 0 alone just spent host time starting the sampler; the exchange kernels of the other
    # ranks give a late peer 2 s, so the ranks meet again before the timed region
    barrier()
    launches0 = ctx.launch_count
    ms = time_region(torch, run_step, args.steps)
    launches = (launches_per_step * args.steps if launches_per_step is not None
                else ctx.launch_count - launches0)
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
    barrier()
    ms_e2e = time_region(torch, run_e2e, args.steps, sync_each=True)
    barrier()
    for _ in range(3):
        projection_only()
    ms_proj = time_region(torch, projection_only, args.steps)
    clocks = sampler.stop() if rank == 0 else None

    tp = []
    if world > 1 and not args.no_extra:
        for m_tp in (256, 1):
            t_ms, t_mode, t_route = tp_layer_slice(torch, tk, dist, rank, world, m_tp, local,
                                                   nccl_reduce=args.nccl_reduce)
            tp.append([m_tp, t_ms, t_mode, t_route])
    times = torch.tensor([ms, ms_e2e, ms_proj] + [t[1] for t in tp], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    vals = [float(v) for v in times.tolist()]
    ms, ms_e2e, ms_proj = vals[:3]
    for t, v in zip(tp, vals[3:]):
        t[1] = v

    # sanity: the selected token is the arg-max of the logits this step wrote
    run_step()
    torch.cuda.synchronize()
    final = (merged if world > 1 else pairs).cpu().numpy()
    mine = local_pairs()
    rounded = logits.to(torch.bfloat16).float()
    for t in range(m):
        first = int(torch.nonzero(rounded[t] == rounded[t].max())[0, 0]) + offset
        assert int(mine[t, 1]) == first, "device argmax disagrees with its own logits"
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
        line = {
            "metric": "fp8_lm_head_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "e4m3",
            "data": "synthetic",
            "config": {"workload": f"fp8_lm_head_argmax K={HIDDEN} vocab={vocab} M={m}",
                       "rows": m, "vocab_shard_rows": shard, "parallelism": f"vocab-shard x{world}",
                       "launch": mode, "exchange": exchange,
                       "l2": "weight shard (%.0f MB) larger than L2, streamed once per step"
                             % (shard * HIDDEN / 1e6),
                       "tokens_per_s": m / (per_step * 1e-3), "us_per_step": per_step * 1e3},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": m * HIDDEN * 2,
                    "d2h_bytes_per_step": m * 8, "us_per_step": ms_e2e / args.steps * 1e3,
                    "launch": e2e_mode},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "traffic": int(round(shard_bytes * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE)),
                         "traffic_source": "ncu dram read+write bytes of this kernel at vocab "
                                           "248320, M=1 (1 272 757 504 B), scaled by algorithmic bytes",
                         "peak_kind": peak_kind,
                         "kernel": "fp8_projection_kernel<16> (+ argmax finalize, < 2 us)",
                         "us_per_launch": proj_ms * 1e3, "frac_of_8TBs": achieved / 8000.0},
            "clocks": clocks,
            "selected_tokens": final[:, 1].tolist()[:8],
        }
        if tp:
            line["tp_layer_slice"] = [
                {"M": t[0], "us": t[1] * 1e3, "launch": t[2], "partial_bytes": t[0] * HIDDEN * 4,
                 "reduce": t[3],
                 "parallelism": f"column(QKV,GDN-in,gate_up) + row(down) x{world}, fp32 partial sums"}
                for t in tp]
        if world == 1 and not args.no_cpu:
            gbs, dt, threads, note, _ = cpu_lm_head(m, 3, 1, budget_s=15.0,
                                                    sample_rows=args.cpu_sample_rows)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                    "sample": note, "seconds_per_sample": dt}
        if world == 1 and not args.no_extra:
            line["extra"] = extra_rows(torch, tk, ctx, peak)
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
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--case", default="", help="run one side case only: nvfp4:M or fp8:N:M")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.case:
        return run_case(args)
    return run_native(args)


if __name__ == "__main__":
    sys.exit(main())
