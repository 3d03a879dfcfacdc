"""Helpers shared by the GPU parity tests: device planes with 0xA5 sentinels (the
reference's inactive-row check, qual/src/fp8_qkv.rs:197-205,355-387), uploads and
tolerance checks."""
import numpy as np
import torch

SENTINEL = 0xA5


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t: torch.Tensor) -> np.ndarray:
    return t.cpu().numpy()


def sentinel_plane(shape, dtype) -> torch.Tensor:
    """Plane filled with 0xA5 bytes."""
    t = torch.empty(shape, dtype=dtype, device="cuda")
    t.view(torch.uint8).fill_(SENTINEL)
    return t


def assert_inactive_untouched(plane: torch.Tensor, active_rows: int):
    tail = plane[active_rows:].contiguous().view(torch.uint8)
    assert bool((tail == SENTINEL).all()), "rows beyond the active count were written"


def bf16_bits_to_f64(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def check_close(actual_bits, expected_f64, abs_tol, rel_tol, what=""):
    """Reference tolerance form max(abs_tol, rel_tol * |oracle|) (qual/src/fp8_qkv.rs:289)."""
    actual = bf16_bits_to_f64(np.asarray(actual_bits))
    expected = np.asarray(expected_f64, dtype=np.float64)
    err = np.abs(actual - expected)
    tol = np.maximum(abs_tol, rel_tol * np.abs(expected))
    bad = err > tol
    if bad.any():
        i = np.unravel_index(np.argmax(err - tol), err.shape)
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.size} values out of tolerance; worst at {i}: "
                             f"device={actual[i]}, oracle={expected[i]}, tol={tol[i]}")
    return float(err.max())


def max_relative_error(actual_bits, expected_f64, floor):
    """Max |a - e| / max(|e|, floor): the 1e-2 bound of the benchmark contract, with a floor
    so that outputs near zero are judged on an absolute scale."""
    actual = bf16_bits_to_f64(np.asarray(actual_bits))
    expected = np.asarray(expected_f64, dtype=np.float64)
    return float((np.abs(actual - expected) / np.maximum(np.abs(expected), floor)).max())


def graph_replay(fn, stream=None):
    """Captures fn() into a CUDA graph and returns a callable that replays it."""
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()  # warm-up on the side stream (tensor maps get encoded here, outside capture)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    with torch.cuda.graph(g):
        fn()
    return g
