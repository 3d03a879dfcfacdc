"""ctypes binding of ``libtuisko_sm100.so`` (the C ABI in ``include/tuisko_sm100.h``).

There is no fallback: if the shared library is missing it is built with nvcc, and if
that is impossible the import fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

ABI_VERSION = 1

STATUS_NAMES = {0: "ok", 1: "gpu.driver", 2: "gpu.arena", 3: "gpu.graph", 4: "gpu.context",
                5: "gpu.launch", 6: "gpu.module"}

DEVICE_WAIT_TIMEOUT = 1
DEVICE_NONFINITE_LOGIT = 2
DEVICE_NONFINITE_INPUT = 4
DEVICE_BAD_ARGUMENT = 8


class Config(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("device", C.c_int32), ("hidden", C.c_uint32),
                ("intermediate", C.c_uint32), ("rms_norm_epsilon", C.c_float),
                ("max_rows", C.c_uint32), ("workspace_bytes", C.c_uint64)]


class ArgmaxPair(C.Structure):
    _fields_ = [("value", C.c_float), ("index", C.c_int32)]


class SamplingOptions(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_uint32),
                ("stop_ids", C.c_uint32 * 2)]


_vp = C.c_void_p
_i = C.c_int

# name -> (restype, argtypes); every symbol include/tuisko_sm100.h declares
SIGNATURES = {
    "tk100_create": (_i, [C.POINTER(Config), C.POINTER(_vp)]),
    "tk100_destroy": (None, [_vp]),
    "tk100_last_error": (C.c_char_p, [_vp]),
    "tk100_device_status": (_i, [_vp, _vp, C.POINTER(C.c_uint32)]),
    "tk100_launch_count": (C.c_uint64, [_vp]),
    "tk100_last_kernel": (C.c_char_p, [_vp]),
    "tk100_rms_norm": (_i, [_vp, _vp, _i, _vp, _vp, _vp]),
    "tk100_residual_rms_norm": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp]),
    "tk100_residual_rms_norm_quantize": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tk100_residual_rms_norm_quantize_nvfp4": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                                    C.c_float, _vp, _vp]),
    "tk100_quantize_activation_e4m3": (_i, [_vp, _vp, _i, _i, _vp, _vp, _vp]),
    "tk100_fp8_qkv": (_i, [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tk100_fp8_gdn_input": (_i, [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tk100_fp8_projection": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tk100_fp8_swiglu": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tk100_fp8_down": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tk100_fp8_gdn_output": (_i, [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tk100_register_plane": (_i, [_vp, _vp, C.c_uint64, C.c_uint64]),
    "tk100_tensor_map_counts": (None, [_vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "tk100_materialize_gather": (_i, [_vp, _vp, _i, C.POINTER(_vp), C.POINTER(C.c_uint64), _vp]),
    "tk100_materialize_nvfp4_scales": (_i, [_vp, _vp, _i, C.POINTER(_vp), C.c_uint64, C.c_uint64, _vp]),
    "tk100_sample": (_i, [_vp, _vp, _i, _i, _vp, C.POINTER(SamplingOptions), _vp, _vp, _vp, _vp]),
    "tk100_sampler_initial_state": (C.c_uint64, [C.c_uint64]),
    "tk100_sampler_scratch_bytes": (C.c_size_t, [_i, _i]),
    "tk100_gdn_prepare": (_i, [_vp, _vp, _i] + [_vp] * 11),
    "tk100_gdn_recurrence": (_i, [_vp, _vp, _i] + [_vp] * 8),
    "tk100_fp8_lm_head": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tk100_fp8_lm_head_sharded": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                       _i, _i, C.POINTER(C.c_uint64), _vp]),
    "tk100_argmax_merge": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "tk100_argmax_exchange": (_i, [_vp, _vp, _i, _i, _i, _vp, C.POINTER(C.c_uint64), _vp]),
    "tk100_nvfp4_quantize_activation": (_i, [_vp, _vp, _i, _i, _vp, C.c_float, _vp, _vp]),
    "tk100_nvfp4_gate_up_swiglu": (_i, [_vp, _vp, _i, _vp, _vp, _vp, C.c_float, _vp, _vp, C.c_float,
                                        _vp]),
    "tk100_nvfp4_gate_up_swiglu_quantize": (_i, [_vp, _vp, _i, _vp, _vp, _vp, C.c_float, _vp, _vp,
                                                 C.c_float, _vp, C.c_float, _vp, _vp]),
    "tk100_nvfp4_down": (_i, [_vp, _vp, _i, _vp, _vp, _vp, C.c_float, _vp, _vp, C.c_float, _vp]),
    "tk100_nvfp4_down_partial": (_i, [_vp, _vp, _i, _vp, _vp, _vp, C.c_float, _vp, _vp, C.c_float,
                                      _vp]),
    "tk100_f32_to_bf16": (_i, [_vp, _vp, C.c_size_t, _vp, _vp]),
    "tk100_peer_sum_bytes": (C.c_size_t, [C.c_size_t, _i]),
    "tk100_peer_sum_bf16": (_i, [_vp, _vp, C.c_size_t, C.c_size_t, _i, _i, _vp,
                                 C.POINTER(C.c_uint64), _vp]),
    "tk100_fp8_projection_static": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, C.c_char_p,
                                         C.c_size_t]),
    "tk100_fp8_projection_static_status": (_i, [_vp, C.POINTER(C.c_uint32)]),
}

_lib = None


def library_path() -> str:
    return _build.LIB


def load() -> C.CDLL:
    """Loads (building first when stale or absent) the shared library."""
    global _lib
    if _lib is None:
        path = _build.build()
        if not os.path.exists(path):
            raise ImportError(f"{path} is missing and could not be built")
        lib = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here = a declared symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
