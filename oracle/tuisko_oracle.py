"""ctypes/numpy front end of the CPU oracle (``tuisko_oracle.c``).

Test infrastructure only: imported by ``tests/``, by the smoke check and by the
benchmark's CPU-baseline leg.  The shipped package never imports it.

All arrays are numpy, C-contiguous: BF16 planes travel as ``uint16`` bit
patterns, E4M3/E2M1 codes as ``uint8``, scales as ``float32``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtuisko_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file; returns the .so path."""
    src = os.path.join(_HERE, "tuisko_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libtuisko_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        u8p, u16p, f32p, f64p = (C.POINTER(C.c_uint8), C.POINTER(C.c_uint16),
                                 C.POINTER(C.c_float), C.POINTER(C.c_double))
        sz = C.c_size_t
        L.tko_init.restype = None
        L.tko_bf16_to_f32.restype = C.c_float
        L.tko_bf16_to_f32.argtypes = [C.c_uint16]
        L.tko_f32_to_bf16.restype = C.c_uint16
        L.tko_f32_to_bf16.argtypes = [C.c_float]
        L.tko_e4m3_decode.restype = C.c_int
        L.tko_e4m3_decode.argtypes = [C.c_uint8, f32p]
        L.tko_e4m3_encode_search.restype = C.c_int
        L.tko_e4m3_encode_search.argtypes = [C.c_float]
        L.tko_e4m3_encode.restype = C.c_int
        L.tko_e4m3_encode.argtypes = [C.c_float]
        L.tko_e4m3_encoder_disagreements.restype = C.c_long
        L.tko_e4m3_encoder_disagreements.argtypes = [C.c_float, C.POINTER(C.c_uint32)]
        L.tko_e2m1_decode.restype = C.c_float
        L.tko_e2m1_decode.argtypes = [C.c_uint8]
        L.tko_e2m1_encode.restype = C.c_int
        L.tko_e2m1_encode.argtypes = [C.c_float]
        L.tko_nvfp4_scale_offset.restype = sz
        L.tko_nvfp4_scale_offset.argtypes = [sz, sz, sz]
        L.tko_residual_rms_norm_rows.restype = None
        L.tko_residual_rms_norm_rows.argtypes = [u16p, u16p, u16p, sz, sz, C.c_float, u16p, u16p]
        L.tko_quantize_e4m3.restype = C.c_int
        L.tko_quantize_e4m3.argtypes = [u16p, sz, C.c_int, u8p, f32p, f64p]
        L.tko_quantize_e4m3_rows.restype = C.c_int
        L.tko_quantize_e4m3_rows.argtypes = [u16p, sz, sz, C.c_int, u8p, f32p]
        L.tko_fp8_projection.restype = C.c_int
        L.tko_fp8_projection.argtypes = [u8p, f32p, u8p, u16p, sz, sz, sz, f64p]
        L.tko_greedy_index.restype = C.c_long
        L.tko_greedy_index.argtypes = [u16p, sz]
        L.tko_nvfp4_a16_dot.restype = C.c_int
        L.tko_nvfp4_a16_dot.argtypes = [u16p, sz, sz, u8p, u8p, C.c_float, sz, f64p]
        L.tko_silu_mul.restype = C.c_double
        L.tko_silu_mul.argtypes = [C.c_double, C.c_double]
        L.tko_nvfp4_quantize_rows.restype = None
        L.tko_nvfp4_quantize_rows.argtypes = [u16p, sz, sz, C.c_float, u8p, u8p]
        L.tko_nvfp4_w4a4_dot.restype = C.c_int
        L.tko_nvfp4_w4a4_dot.argtypes = [u8p, u8p, C.c_float, sz, sz, u8p, u8p, C.c_float, sz, f64p]
        L.tko_top_k_select.restype = C.c_long
        L.tko_top_k_select.argtypes = [u16p, sz, sz, C.POINTER(C.c_uint32), f32p]
        L.tko_xorshift_new.restype = C.c_uint64
        L.tko_xorshift_new.argtypes = [C.c_uint64]
        L.tko_xorshift_unit.restype = C.c_double
        L.tko_xorshift_unit.argtypes = [C.POINTER(C.c_uint64)]
        L.tko_sample.restype = C.c_long
        L.tko_sample.argtypes = [u16p, sz, C.c_float, C.c_float, sz, C.POINTER(C.c_uint64)]
        L.tko_num_threads.restype = C.c_int
        L.tko_set_num_threads.restype = None
        L.tko_set_num_threads.argtypes = [C.c_int]
        L.tko_init()
        _lib = L
    return _lib


def _p(a: np.ndarray, ctype):
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(C.POINTER(ctype))


def _u16(a):
    return np.ascontiguousarray(a, dtype=np.uint16)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


# ------------------------------------------------------------------ codecs

def bf16_to_f32(bits) -> np.ndarray:
    """BF16 bit patterns -> float32 (qual/src/fp8_projection_oracle.rs:106-108)."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(values) -> np.ndarray:
    """float32 -> BF16 bits, nearest-even (qual/src/fp8_projection_oracle.rs:99-104)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFFFFFF
    return (rounded >> 16).astype(np.uint16)


def e4m3_decode_table() -> np.ndarray:
    """float32[256]; NaN at the two NaN codes (qual/src/fp8_projection_oracle.rs:81-97)."""
    out = np.empty(256, dtype=np.float32)
    v = C.c_float()
    for code in range(256):
        out[code] = v.value if lib().tko_e4m3_decode(code, C.byref(v)) == 0 else np.nan
    return out


def e4m3_encode(value: float, search: bool = False) -> int:
    f = lib().tko_e4m3_encode_search if search else lib().tko_e4m3_encode
    return int(f(C.c_float(value)))


def e2m1_decode(code: int) -> float:
    return float(lib().tko_e2m1_decode(code & 0xFF))


def e2m1_encode(value: float) -> int:
    return int(lib().tko_e2m1_encode(C.c_float(value)))


def nvfp4_scale_offset(row: int, group: int, groups_per_row: int) -> int:
    return int(lib().tko_nvfp4_scale_offset(row, group, groups_per_row))


def nvfp4_scale_offsets(rows: int, groups: int) -> np.ndarray:
    """int64[rows, groups] table of swizzled byte offsets (materialize.rs:410-422)."""
    r = np.arange(rows, dtype=np.int64)[:, None]
    g = np.arange(groups, dtype=np.int64)[None, :]
    return ((r // 128) * (groups // 4) + g // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4


# ------------------------------------------------------------ norm / quant

def residual_rms_norm(x, branch, weight, eps=1e-6):
    """Returns (residual_bits or None, normalized_bits); rows x hidden BF16 planes."""
    x = _u16(x)
    rows, hidden = x.shape
    weight = _u16(weight)
    normalized = np.empty_like(x)
    if branch is None:
        lib().tko_residual_rms_norm_rows(_p(x, C.c_uint16), None, _p(weight, C.c_uint16), rows,
                                         hidden, C.c_float(eps), None, _p(normalized, C.c_uint16))
        return None, normalized
    branch = _u16(branch)
    residual = np.empty_like(x)
    lib().tko_residual_rms_norm_rows(_p(x, C.c_uint16), _p(branch, C.c_uint16),
                                     _p(weight, C.c_uint16), rows, hidden, C.c_float(eps),
                                     _p(residual, C.c_uint16), _p(normalized, C.c_uint16))
    return residual, normalized


def quantize_e4m3(x, search: bool = False):
    """Per-token E4M3 quantisation; returns (codes u8 [rows,h], scales f32 [rows])."""
    x = _u16(x)
    rows, hidden = x.shape
    codes = np.empty((rows, hidden), dtype=np.uint8)
    scales = np.empty(rows, dtype=np.float32)
    rc = lib().tko_quantize_e4m3_rows(_p(x, C.c_uint16), rows, hidden, int(search),
                                      _p(codes, C.c_uint8), _p(scales, C.c_float))
    if rc != 0:
        raise ValueError("oracle E4M3 input is not finite")
    return codes, scales


def quantize_e4m3_token(x, search: bool = True):
    """One token, also returning the f64 sum of represented codes (TokenOracle)."""
    x = _u16(x).reshape(-1)
    codes = np.empty(x.size, dtype=np.uint8)
    scale = C.c_float()
    rsum = C.c_double()
    rc = lib().tko_quantize_e4m3(_p(x, C.c_uint16), x.size, int(search), _p(codes, C.c_uint8),
                                 C.byref(scale), C.byref(rsum))
    if rc != 0:
        raise ValueError("oracle E4M3 input is not finite")
    return codes, np.float32(scale.value), float(rsum.value)


def fp8_projection(act_codes, act_scales, w_codes, w_scales_bf16) -> np.ndarray:
    """f64 [rows, out_rows] FP8 projection oracle."""
    a = _u8(act_codes)
    w = _u8(w_codes)
    rows, k = a.shape
    out_rows = w.shape[0]
    assert w.shape[1] == k
    s = np.ascontiguousarray(act_scales, dtype=np.float32)
    ws = _u16(w_scales_bf16)
    out = np.empty((rows, out_rows), dtype=np.float64)
    rc = lib().tko_fp8_projection(_p(a, C.c_uint8), _p(s, C.c_float), _p(w, C.c_uint8),
                                  _p(ws, C.c_uint16), rows, out_rows, k, _p(out, C.c_double))
    if rc != 0:
        raise ValueError("oracle encountered an E4M3FN NaN code")
    return out


def greedy_index(logits_bf16) -> int:
    """First maximum in total order; raises on a non-finite logit (sampling.rs:162-173)."""
    l = _u16(logits_bf16).reshape(-1)
    r = int(lib().tko_greedy_index(_p(l, C.c_uint16), l.size))
    if r < 0:
        raise ValueError(f"sampling received a non-finite logit at token {-1 - r}")
    return r


# ------------------------------------------------------------------ NVFP4

def top_k_select(logits_bf16, k: int):
    """tuisko-engine/src/sampling.rs:212-231: (indices uint32, values float32) of the k best, or
    raises on a non-finite logit."""
    logits = _u16(logits_bf16)
    index = np.zeros(k, dtype=np.uint32)
    value = np.zeros(k, dtype=np.float32)
    kept = lib().tko_top_k_select(_p(logits, C.c_uint16), logits.size, k,
                                  _p(index, C.c_uint32), _p(value, C.c_float))
    if kept < 0:
        raise ValueError(f"sampling received a non-finite logit at token {-1 - kept}")
    return index[:kept], value[:kept]


class Sampler:
    """tuisko-engine/src/sampling.rs:56-101: one request's sampler with its xorshift64 state."""

    def __init__(self, temperature=1.0, top_p=0.95, top_k=20, seed=0, stop_ids=(0, 1)):
        self.temperature, self.top_p, self.top_k = temperature, top_p, top_k
        self.stop_ids = tuple(stop_ids)
        self.state = C.c_uint64(lib().tko_xorshift_new(seed))

    def sample(self, logits_bf16):
        logits = _u16(logits_bf16)
        token = lib().tko_sample(_p(logits, C.c_uint16), logits.size, self.temperature, self.top_p,
                                 self.top_k, C.byref(self.state))
        if token < 0:
            raise ValueError(f"sampling failed ({token})")
        return int(token), int(token) in self.stop_ids


def nvfp4_a16_dot(x_bf16, w_codes, w_scales_swz, weight_scale_divisor: float) -> np.ndarray:
    x = _u16(x_bf16)
    tokens, k = x.shape
    w = _u8(w_codes)
    rows_w = w.shape[0]
    assert w.shape[1] == k // 2
    s = _u8(w_scales_swz).reshape(-1)
    out = np.empty((tokens, rows_w), dtype=np.float64)
    rc = lib().tko_nvfp4_a16_dot(_p(x, C.c_uint16), tokens, k, _p(w, C.c_uint8), _p(s, C.c_uint8),
                                 C.c_float(weight_scale_divisor), rows_w, _p(out, C.c_double))
    if rc != 0:
        raise ValueError("oracle encountered an E4M3FN NaN")
    return out


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """qual/src/nvfp4_swiglu.rs:306-315 in f64."""
    gate = np.asarray(gate, dtype=np.float64)
    return gate / (1.0 + np.exp(-gate)) * np.asarray(up, dtype=np.float64)


def nvfp4_scale_plane_bytes(rows: int, k: int) -> int:
    return ((rows + 127) // 128) * 128 * (k // 16)


def nvfp4_quantize(x_bf16, divisor: float):
    """PARITY UNPINNED (own definition). Returns (codes u8 [rows,k/2], swizzled scales u8)."""
    x = _u16(x_bf16)
    rows, k = x.shape
    codes = np.empty((rows, k // 2), dtype=np.uint8)
    scales = np.zeros(nvfp4_scale_plane_bytes(rows, k), dtype=np.uint8)
    lib().tko_nvfp4_quantize_rows(_p(x, C.c_uint16), rows, k, C.c_float(divisor),
                                  _p(codes, C.c_uint8), _p(scales, C.c_uint8))
    return codes, scales


def nvfp4_w4a4_dot(a_codes, a_scales, a_divisor, w_codes, w_scales, w_divisor) -> np.ndarray:
    a = _u8(a_codes)
    w = _u8(w_codes)
    tokens, kh = a.shape
    rows_w = w.shape[0]
    assert w.shape[1] == kh
    out = np.empty((tokens, rows_w), dtype=np.float64)
    sa = _u8(a_scales).reshape(-1)
    sw = _u8(w_scales).reshape(-1)
    rc = lib().tko_nvfp4_w4a4_dot(_p(a, C.c_uint8), _p(sa, C.c_uint8), C.c_float(a_divisor), tokens,
                                  kh * 2, _p(w, C.c_uint8), _p(sw, C.c_uint8), C.c_float(w_divisor),
                                  rows_w, _p(out, C.c_double))
    if rc != 0:
        raise ValueError("oracle encountered an E4M3FN NaN")
    return out


def num_threads() -> int:
    return int(lib().tko_num_threads())


def set_num_threads(n: int) -> int:
    """OpenMP team size of the oracle's loops; returns the size now in force."""
    lib().tko_set_num_threads(int(n))
    return num_threads()
