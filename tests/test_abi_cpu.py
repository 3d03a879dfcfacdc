"""CPU-side checks of the boundary: the shared library builds, loads and exports every
symbol the public header declares; host-side builders agree with the oracle."""
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "tuisko_sm100.h")).read()
    return sorted(set(re.findall(r"TK100_API[^;(]*?\b(tk100_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from tuiskollm_b200 import _lib

    names = header_symbols()
    assert len(names) >= 14
    lib = _lib.load()
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signature table and header disagree"


def test_config_struct_matches_header_layout():
    from tuiskollm_b200 import _lib
    import ctypes as C

    assert C.sizeof(_lib.Config) == 32 and _lib.Config.workspace_bytes.offset == 24
    assert C.sizeof(_lib.ArgmaxPair) == 8


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device failure path")
def test_create_fails_loudly_without_a_device():
    import tuiskollm_b200 as tk

    with pytest.raises(tk.GpuError) as info:
        tk.Context()
    assert info.value.code in ("gpu.driver", "gpu.module")


def test_host_planes_are_rejected_before_any_launch():
    from tuiskollm_b200 import ops

    with pytest.raises(ops.GpuError) as info:
        ops._ptr(torch.zeros(4))
    assert info.value.code == "gpu.context"


def test_synth_codecs_agree_with_oracle(oracle):
    from tuiskollm_b200 import synth

    rng = np.random.default_rng(11)
    v = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 100,
                        rng.standard_normal(20000).astype(np.float32) * 0.01,
                        np.array([0.0, -0.0, 448.0, -448.0, 1e6, -1e6, 2.0 ** -10, -(2.0 ** -10), 2.0 ** -9 * 7.5], np.float32)])
    got = synth.e4m3_encode(v)
    exp = np.array([oracle.e4m3_encode(float(x)) for x in v], np.uint8)
    assert np.array_equal(got, exp)
    tab = synth.e4m3_table()
    ref = oracle.e4m3_decode_table()
    assert np.array_equal(tab[~np.isnan(ref)], ref[~np.isnan(ref)]) and np.isnan(tab[0x7F])
    q = rng.standard_normal(5000).astype(np.float32) * 3
    q = np.concatenate([q, np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -5.0, 7.0, -0.0], np.float32)])
    assert np.array_equal(synth.e2m1_encode(q), np.array([oracle.e2m1_encode(float(x)) for x in q], np.uint8))
    assert np.array_equal(synth.nvfp4_scale_offsets(256, 320), oracle.nvfp4_scale_offsets(256, 320))
    bits = synth.f32_to_bf16_bits(v)
    assert np.array_equal(bits, oracle.f32_to_bf16(v))


def test_synth_fp8_weights_follow_the_stated_recipe(oracle):
    from tuiskollm_b200 import synth

    codes, scale_bits = synth.fp8_weights(1234, 3, 64, 1024)
    assert codes.shape == (64, 1024) and scale_bits.shape == (64,)
    assert not np.isin(codes, [0x7F, 0xFF]).any()
    # every row uses the top of the E4M3 range: |code| reaches 448 or the value next to it
    tab = oracle.e4m3_decode_table()
    assert (np.abs(tab[codes]).max(axis=1) >= 416).all()
    again, _ = synth.fp8_weights(1234, 3, 64, 1024)
    assert np.array_equal(codes, again)


def test_synth_nvfp4_weights_match_oracle_definition(oracle):
    from tuiskollm_b200 import synth

    rng = np.random.default_rng(5)
    w = (rng.standard_normal((128, 256)) * 0.02).astype(np.float32)
    # bf16-representable weights so that the oracle (BF16 in) sees the same numbers
    w = oracle.bf16_to_f32(oracle.f32_to_bf16(w))
    codes, scales, div = synth.nvfp4_quantize_weights(w)
    ocodes, oscales = oracle.nvfp4_quantize(oracle.f32_to_bf16(w), float(div))
    assert np.array_equal(codes, ocodes) and np.array_equal(scales, oscales)
    assert scales.max() <= 0x7E and div == np.float32(448.0 * 6.0) / np.abs(w).max()


def test_rust_ffi_declares_exactly_the_header_symbols():
    """The Rust side of the boundary (crates/tuisko-gpu/src/ffi_sm100.rs, not compiled in this
    image) must declare every exported function, no more and no fewer, and the crate's build
    script must compile the same sources as the Python build."""
    from tuiskollm_b200 import build as cuda_build

    ffi = open(os.path.join(ROOT, "crates", "tuisko-gpu", "src", "ffi_sm100.rs")).read()
    declared = sorted(set(re.findall(r"pub fn (tk100_[a-z0-9_]+)\s*\(", ffi)))
    assert declared == header_symbols()
    build_rs = open(os.path.join(ROOT, "crates", "tuisko-kernels-sm100", "build.rs")).read()
    listed = re.findall(r'"([a-z0-9_]+\.cu)"', build_rs.split("const SOURCES", 1)[1].split("];", 1)[0])
    assert listed == cuda_build.SOURCES
    lib_rs = open(os.path.join(ROOT, "crates", "tuisko-kernels-sm100", "src", "lib.rs")).read()
    used = set(re.findall(r"ffi::(tk100_[a-z0-9_]+)", lib_rs))
    assert used <= set(declared), used - set(declared)


def test_no_launch_function_reads_the_environment():
    """Route selectors are read once (Tuning::from_environment at tk100_create,
    read_process_switches); nothing else in the library calls getenv."""
    csrc = os.path.join(ROOT, "tuiskollm_b200", "csrc")
    hits = []
    for name in sorted(os.listdir(csrc)):
        text = open(os.path.join(csrc, name)).read()
        for m in re.finditer(r"getenv", text):
            line = text[:m.start()].count("\n") + 1
            hits.append((name, line))
    allowed = {"ops.cu", "norm_quant.cu"}
    assert {n for n, _ in hits} <= allowed, hits
    ops = open(os.path.join(csrc, "ops.cu")).read()
    assert ops.count("getenv") == 1  # inside env_int(), which only Tuning::from_environment calls
    body = ops.split("Tuning Tuning::from_environment()", 1)[1].split("\n}\n", 1)[0]
    assert ops.count("env_int(") == body.count("env_int(") + 1  # + its definition
