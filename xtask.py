#!/usr/bin/env python
"""Qualification and performance commands for the sm100 target, after the reference's
`cargo run -p xtask -- <command>` (xtask/src/main.rs:160-195):

  python xtask.py qualify-<suite> [--target sm100]   parity suite against the CPU oracle (needs a B200)
  python xtask.py qualify-all                        every suite
  python xtask.py gate-resources [--bless]           registers / spills / shared bytes per kernel against
                                                     qual/baselines/resources-sm100.txt (no GPU needed)
  python xtask.py perf smoke|gate|bless              bench.py on one GPU; `gate` compares every row's median
                                                     with qual/baselines/perf-sm100.json, `bless` rewrites it

The suites are the reference's (`qualify-residual-norm`, `qualify-fp8-qkv`, `qualify-fp8-gdn-input`,
`qualify-fp8-lm-head`, `qualify-nvfp4-swiglu`, `qualify-nvfp4-down`, ...); each maps to the pytest
file that restates that suite's checks through the C ABI.  The resource gate follows
xtask/src/main.rs:1328-1425 (launch bounds kept, no spills, pinned register counts), reading the
numbers from `nvcc -Xptxas -v` instead of a dump of the binary.  The timing gate follows
xtask/src/performance.rs:9-17,187-283: a row fails when its median exceeds the blessed median by
more than max(5 %, 0.05 us).
"""
from __future__ import annotations

import argparse
import concurrent.futures
import json
import os
import re
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
BASELINES = os.path.join(ROOT, "qual", "baselines")
RESOURCE_BASELINE = os.path.join(BASELINES, "resources-sm100.txt")
PERF_BASELINE = os.path.join(BASELINES, "perf-sm100.json")
DEVICE_RELATIVE_TOLERANCE_PERCENT = 5.0        # xtask/src/performance.rs:13
DEVICE_ABSOLUTE_TOLERANCE_MICROSECONDS = 0.05  # xtask/src/performance.rs:14

SUITES = {
    "residual-norm": ["tests/test_gpu_norm_quant.py"],
    "fp8-qkv": ["tests/test_gpu_fp8_projection.py"],
    "fp8-gdn-input": ["tests/test_gpu_fp8_projection.py"],
    "fp8-lm-head": ["tests/test_gpu_lm_head.py"],
    "fp8-swiglu": ["tests/test_gpu_fp8_mlp.py"],
    "fp8-down": ["tests/test_gpu_fp8_mlp.py"],
    "gdn-output": ["tests/test_gpu_fp8_mlp.py"],
    "gdn-prepare": ["tests/test_gpu_gdn.py"],
    "gdn-recurrence": ["tests/test_gpu_gdn.py"],
    "nvfp4-swiglu": ["tests/test_gpu_nvfp4.py"],
    "nvfp4-down": ["tests/test_gpu_nvfp4.py"],
    "peer-exchange": ["tests/test_gpu_peer_sum.py", "tests/test_gpu_multi.py"],
    "static-entry": ["tests/test_zz_no_alloc.py"],
    "host-codecs": ["tests/test_oracle_kat.py", "tests/test_oracle_gdn.py"],
}


def qualify(suite: str) -> int:
    files = sorted({f for s in (SUITES if suite == "all" else [suite]) for f in SUITES[s]})
    files = [f for f in files if os.path.exists(os.path.join(ROOT, f))]
    cmd = [sys.executable, "-m", "pytest", "-q", "-x"] + files
    if suite != "host-codecs":
        cmd += ["-m", "gpu"]
    print("+", " ".join(cmd), flush=True)
    return subprocess.call(cmd, cwd=ROOT)


# ------------------------------------------------------------------ resource gate

def demangle(names):
    tool = shutil.which("cu++filt") or "/usr/local/cuda/bin/cu++filt"
    if not os.path.exists(tool):
        tool = shutil.which("c++filt")
    if not tool:
        return {n: n for n in names}
    out = subprocess.run([tool], input="\n".join(names), capture_output=True, text=True).stdout.splitlines()
    return dict(zip(names, out)) if len(out) == len(names) else {n: n for n in names}


def short_name(demangled: str) -> str:
    """`void tk100::(anonymous namespace)::kernel<16, 0>(args)` -> `kernel<16, 0>`."""
    s = re.sub(r"^void\s+", "", demangled)
    depth, cut = 0, len(s)
    for i, ch in enumerate(s):  # strip the argument list (the first '(' outside template brackets)
        if ch == "<":
            depth += 1
        elif ch == ">":
            depth -= 1
        elif ch == "(" and depth == 0 and not s.startswith("(anonymous namespace)", i):
            cut = i
            break
    s = s[:cut]
    return s.replace("tk100::", "").replace("(anonymous namespace)::", "").replace(", ", ",")


def kernel_resources():
    """{kernel: (registers, spill bytes, static shared bytes)} from `nvcc -Xptxas -v` of every source."""
    from tuiskollm_b200 import build as cuda_build

    nvcc = cuda_build.nvcc_path()
    csrc = cuda_build.CSRC

    def one(source):
        cmd = [nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xptxas", "-v", "-c", "-o", os.devnull, os.path.join(csrc, source)]
        if os.path.exists("/usr/bin/g++"):
            cmd[1:1] = ["-ccbin", "/usr/bin/g++"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {source}:\n{res.stderr}")
        return res.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=4) as pool:
        logs = list(pool.map(one, cuda_build.SOURCES))
    found = {}
    for log in logs:
        entry = None
        spill = 0
        for line in log.splitlines():
            m = re.search(r"Compiling entry function '([^']+)'", line)
            if m:
                entry, spill = m.group(1), 0
                continue
            m = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", line)
            if m and entry:
                spill = int(m.group(2)) + int(m.group(3))
                continue
            m = re.search(r"Used (\d+) registers", line)
            if m and entry:
                smem = re.search(r"(\d+) bytes smem", line)
                found[entry] = (int(m.group(1)), spill, int(smem.group(1)) if smem else 0)
                entry = None
    names = demangle(sorted(found))
    return {short_name(names[k]): v for k, v in found.items()}


def read_resource_baseline():
    out = {}
    with open(RESOURCE_BASELINE) as f:
        for line in f:
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            name, rest = line.split(" = ")
            regs, spill, smem = (int(v.split(":")[1]) for v in rest.split())
            out[name] = (regs, spill, smem)
    return out


def gate_resources(bless: bool) -> int:
    now = kernel_resources()
    if bless:
        os.makedirs(BASELINES, exist_ok=True)
        with open(RESOURCE_BASELINE, "w") as f:
            f.write("# nvcc -Xptxas -v, arch sm_100a: registers per thread, spill bytes (stores + loads), static\n"
                    "# shared bytes, per kernel entry.  Rewritten by `python xtask.py gate-resources --bless`.\n")
            for name in sorted(now):
                r, s, m = now[name]
                f.write(f"{name} = REG:{r} SPILL:{s} SHARED:{m}\n")
        print(f"blessed {len(now)} kernel entries -> {os.path.relpath(RESOURCE_BASELINE, ROOT)}")
        return 0
    want = read_resource_baseline()
    failures = 0
    for name in sorted(set(now) | set(want)):
        if name not in now or name not in want:
            print(f"FAIL  {name}: {'missing from the build' if name not in now else 'not in the baseline'}")
            failures += 1
            continue
        (r, s, m), (wr, ws, wm) = now[name], want[name]
        ok = s == 0 and r == wr and m == wm
        print(f"{'PASS' if ok else 'FAIL'}  {name}: REG {r} (baseline {wr}) SPILL {s} SHARED {m} (baseline {wm})")
        failures += 0 if ok else 1
    if failures:
        print(f"{failures} kernel entries differ from the resource baseline (spills are never admitted)")
        return 1
    print(f"sm100 resource gate passed: {len(now)} kernel entries, STACK SPILL 0")
    return 0


# -------------------------------------------------------------------- timing gate

def perf_rows(line: dict):
    rows = {("fp8_lm_head_argmax step", line["config"]["rows"], line["config"]["vocab"]):
            line["protocol"]["us_per_step"]["median"]}
    for r in line.get("configs", []):
        rows[(r["op"], r["M"], r.get("N", 0))] = r["us"]["median"]
    return rows


def perf(mode: str, extra) -> int:
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "1"] + list(extra)
    if mode == "smoke":
        cmd += ["--no-extra", "--no-cpu", "--steps", "20", "--warmup", "5"]
    else:
        cmd += ["--no-cpu"]
    print("+", " ".join(cmd), flush=True)
    res = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True)
    sys.stderr.write(res.stderr)
    if res.returncode != 0:
        print(res.stdout)
        return res.returncode
    line = json.loads(res.stdout.strip().splitlines()[-1])
    rows = perf_rows(line)
    if mode == "smoke":
        for k, v in rows.items():
            print(f"{k[0]:<36} M={k[1]:<5} N={k[2]:<7} {v:10.3f} us")
        return 0
    if mode == "bless":
        os.makedirs(BASELINES, exist_ok=True)
        doc = {"schema_version": 1, "target": "sm100", "device": "NVIDIA B200",
               "clocks": line.get("clocks"), "samples": line["protocol"]["samples"],
               "metrics": [{"op": k[0], "M": k[1], "N": k[2], "median_microseconds": v}
                           for k, v in sorted(rows.items(), key=lambda kv: str(kv[0]))]}
        with open(PERF_BASELINE, "w") as f:
            json.dump(doc, f, indent=1)
            f.write("\n")
        print(f"blessed {len(rows)} timing rows -> {os.path.relpath(PERF_BASELINE, ROOT)}")
        return 0
    with open(PERF_BASELINE) as f:
        base = {(m["op"], m["M"], m["N"]): m["median_microseconds"] for m in json.load(f)["metrics"]}
    if set(base) != set(rows):
        print("performance report and baseline metric inventories differ:",
              sorted(map(str, set(base) ^ set(rows))))
        return 1
    failures = 0
    print("status op                                   M     N        reference  candidate    delta")
    for k in sorted(rows, key=str):
        ref, cand = base[k], rows[k]
        limit = max(ref * (1 + DEVICE_RELATIVE_TOLERANCE_PERCENT / 100),
                    ref + DEVICE_ABSOLUTE_TOLERANCE_MICROSECONDS)
        ok = cand <= limit
        failures += 0 if ok else 1
        print(f"{'PASS' if ok else 'FAIL':<6} {k[0]:<36} {k[1]:<5} {k[2]:<7} {ref:9.3f} us {cand:9.3f} us "
              f"{(cand / ref - 1) * 100:+7.2f}%")
    if failures:
        print(f"{failures} timing rows regressed")
        return 1
    print(f"performance gate passed: {len(rows)} timing rows")
    return 0


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("command")
    ap.add_argument("mode", nargs="?")
    ap.add_argument("--target", default="sm100", choices=["sm100"])
    ap.add_argument("--bless", action="store_true")
    args, extra = ap.parse_known_args()
    if args.command.startswith("qualify-"):
        suite = args.command[len("qualify-"):]
        if suite != "all" and suite not in SUITES:
            print(f"unknown suite {suite}; known: {', '.join(sorted(SUITES))}")
            return 2
        return qualify(suite)
    if args.command == "gate-resources":
        return gate_resources(args.bless)
    if args.command == "perf":
        if args.mode not in ("smoke", "gate", "bless"):
            print("perf needs a mode: smoke, gate or bless")
            return 2
        return perf(args.mode, extra)
    print(__doc__)
    return 2


if __name__ == "__main__":
    sys.exit(main())
