"""The resource gate of `xtask.py gate-resources` as a CPU test (the reference's static gate,
xtask/src/main.rs:1328-1425: pinned register counts, no spills): every kernel entry compiled for
sm_100a must match qual/baselines/resources-sm100.txt."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_kernel_resources_match_the_blessed_baseline(capsys):
    import xtask

    rc = xtask.gate_resources(bless=False)
    out = capsys.readouterr().out
    assert rc == 0, out[-3000:]


def test_timing_gate_arithmetic():
    import xtask

    line = {"config": {"rows": 1, "vocab": 248320}, "protocol": {"us_per_step": {"median": 186.0}},
            "configs": [{"op": "fp8_qkv", "M": 1, "N": 8192, "us": {"median": 9.5}}]}
    rows = xtask.perf_rows(line)
    assert rows[("fp8_qkv", 1, 8192)] == 9.5 and len(rows) == 2
    assert set(xtask.SUITES) >= {"residual-norm", "fp8-qkv", "fp8-gdn-input", "fp8-lm-head",
                                 "nvfp4-swiglu", "nvfp4-down"}
