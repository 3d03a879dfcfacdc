"""GPU parity: fused residual-add + RMSNorm + per-token E4M3 quantisation against the CPU
oracle, following qual/src/residual_norm.rs (exact batches, sentinels, graph replay)."""
import numpy as np
import pytest
import torch

import fixtures_ref as F
from gpu_util import (assert_inactive_untouched, check_close, dev, graph_replay, host,
                      sentinel_plane)

pytestmark = pytest.mark.gpu

MAX_ROWS = 8


@pytest.fixture(scope="module")
def tk():
    import tuiskollm_b200 as tk
    return tk


@pytest.fixture(scope="module")
def ctx(tk):
    return tk.Context(device=0)


def _u16(t):
    return host(t.view(torch.int16)).view(np.uint16)


def run_all(tk, ctx, x, b, w, rows, max_rows, hidden):
    op = tk.ResidualNormOp(ctx)
    plain = sentinel_plane((max_rows, hidden), torch.int16)
    res = sentinel_plane((max_rows, hidden), torch.int16)
    norm = sentinel_plane((max_rows, hidden), torch.int16)
    fres = sentinel_plane((max_rows, hidden), torch.int16)
    fnorm = sentinel_plane((max_rows, hidden), torch.int16)
    codes = sentinel_plane((max_rows, hidden), torch.uint8)
    scales = sentinel_plane((max_rows,), torch.float32)
    pcodes = sentinel_plane((max_rows, hidden), torch.uint8)
    pscales = sentinel_plane((max_rows,), torch.float32)
    pnorm = sentinel_plane((max_rows, hidden), torch.int16)

    def launch():
        op.launch_plain(None, rows, x, w, plain)
        op.launch_residual(None, rows, x, b, w, res, norm)
        op.launch_quantize(None, rows, x, b, w, fres, fnorm, codes, scales)
        op.launch_quantize(None, rows, x, None, w, None, pnorm, pcodes, pscales)

    planes = dict(plain=plain, res=res, norm=norm, fres=fres, fnorm=fnorm, codes=codes,
                  scales=scales, pcodes=pcodes, pscales=pscales, pnorm=pnorm)
    return launch, planes


def verify(oracle, planes, xb, bb, wb, rows, eps):
    res_o, norm_o = oracle.residual_rms_norm(xb[:rows], bb[:rows], wb, eps)
    _, plain_o = oracle.residual_rms_norm(xb[:rows], None, wb, eps)
    plain = _u16(planes["plain"])
    res, norm = _u16(planes["res"]), _u16(planes["norm"])
    fres, fnorm, pnorm = _u16(planes["fres"]), _u16(planes["fnorm"]), _u16(planes["pnorm"])
    # residual publication is bit exact (qual/src/residual_norm.rs:236-243)
    assert np.array_equal(res[:rows], res_o)
    assert np.array_equal(fres[:rows], res_o)
    # norm within max(1/64, 0.5 %) of the f64 oracle (qual/src/residual_norm.rs:364)
    f64 = lambda bits: oracle.bf16_to_f32(bits).astype(np.float64)
    worst = max(check_close(plain[:rows], f64(plain_o), 1 / 64, 0.005, "plain RMSNorm"),
                check_close(norm[:rows], f64(norm_o), 1 / 64, 0.005, "residual RMSNorm"))
    # the fused producer writes the same normalised words as the unfused launches
    assert np.array_equal(fnorm[:rows], norm[:rows]) and np.array_equal(pnorm[:rows], plain[:rows])
    # codes and scales are bit exact against the oracle applied to the row the device wrote
    for cplane, splane, nplane in (("codes", "scales", fnorm), ("pcodes", "pscales", pnorm)):
        oc, os_ = oracle.quantize_e4m3(nplane[:rows])
        assert np.array_equal(host(planes[cplane])[:rows], oc), cplane
        assert np.array_equal(host(planes[splane])[:rows].view(np.uint32), os_.view(np.uint32)), splane
    for name, p in planes.items():
        assert_inactive_untouched(p, rows)
    differing = int((norm[:rows] != norm_o).sum())
    return worst, differing


@pytest.mark.parametrize("rows", list(range(1, MAX_ROWS + 1)))
def test_reference_fixture_exact_batches(tk, ctx, oracle, rows):
    hidden = 5120
    xb, bb, wb = F.norm_fixture(MAX_ROWS, hidden)
    x, b, w = dev(xb.view(np.int16)), dev(bb.view(np.int16)), dev(wb.view(np.int16))
    launch, planes = run_all(tk, ctx, x, b, w, rows, MAX_ROWS, hidden)
    launch()
    torch.cuda.synchronize()
    worst, differing = verify(oracle, planes, xb, bb, wb, rows, 1e-6)
    assert worst <= 1 / 64
    eager = {k: host(v.view(torch.uint8)).copy() for k, v in planes.items()}
    # eager == two graph replays, bit for bit (qual/src/residual_norm.rs:116-123)
    for p in planes.values():
        p.view(torch.uint8).fill_(0xA5)
    g = graph_replay(launch)
    for p in planes.values():
        p.view(torch.uint8).fill_(0xA5)
    g.replay()
    g.replay()
    torch.cuda.synchronize()
    for k, v in planes.items():
        assert np.array_equal(host(v.view(torch.uint8)), eager[k]), k
    assert ctx.device_status() == 0


@pytest.mark.parametrize("rows", [1, 5, 32, 256, 512])
def test_random_rows_match_oracle(tk, oracle, rows):
    from tuiskollm_b200 import synth

    hidden = 5120
    ctx = tk.Context(device=0, max_rows=512)
    xb = synth.normal_bf16(2024, 1, (rows, hidden))
    bb = synth.normal_bf16(2024, 2, (rows, hidden))
    wb = synth.normal_bf16(2024, 3, (hidden,), std=0.1)
    x, b, w = dev(xb.view(np.int16)), dev(bb.view(np.int16)), dev(wb.view(np.int16))
    launch, planes = run_all(tk, ctx, x, b, w, rows, rows + 3, hidden)
    launch()
    torch.cuda.synchronize()
    worst, differing = verify(oracle, planes, xb, bb, wb, rows, 1e-6)
    # the device row differs from the f64 oracle's BF16 rounding in a handful of words at most
    assert differing <= max(4, rows * hidden // 2000), differing
    assert ctx.device_status() == 0


def test_small_geometry_and_edge_rows(tk, oracle):
    """The reference's test geometry (hidden 1024, eps 1e-5: tuisko-kernels-sm120/src/lib.rs:24-52)
    plus all-zero and signed-zero rows."""
    from tuiskollm_b200 import synth

    hidden, rows = 1024, 6
    ctx = tk.Context(device=0, hidden=hidden, rms_norm_epsilon=1e-5, max_rows=8)
    xb = synth.normal_bf16(7, 1, (rows, hidden))
    bb = synth.normal_bf16(7, 2, (rows, hidden))
    xb[2] = 0
    bb[2] = 0
    bb[2, 7] = 0x8000  # 0 + (-0) = +0 in round-to-nearest
    xb[3] = bb[3] ^ 0x8000  # x + branch cancels exactly
    wb = synth.normal_bf16(7, 3, (hidden,), std=0.1)
    x, b, w = dev(xb.view(np.int16)), dev(bb.view(np.int16)), dev(wb.view(np.int16))
    launch, planes = run_all(tk, ctx, x, b, w, rows, 8, hidden)
    launch()
    torch.cuda.synchronize()
    verify(oracle, planes, xb, bb, wb, rows, 1e-5)
    scales = host(planes["scales"])
    assert scales[2] == 1.0 and scales[3] == 1.0
    assert not host(planes["codes"])[2].any()


def test_in_place_residual_and_aliasing(tk, ctx, oracle):
    """x and branch may alias (tuisko-kernels-sm120/src/residual_norm.rs:463-465); the residual
    stream may be updated in place."""
    from tuiskollm_b200 import synth

    hidden, rows = 5120, 4
    xb = synth.normal_bf16(99, 1, (rows, hidden))
    wb = synth.normal_bf16(99, 3, (hidden,), std=0.1)
    x, w = dev(xb.view(np.int16)), dev(wb.view(np.int16))
    norm = sentinel_plane((rows, hidden), torch.int16)
    tk.ResidualNormOp(ctx).launch_residual(None, rows, x, x, w, x, norm)
    torch.cuda.synchronize()
    res_o, norm_o = oracle.residual_rms_norm(xb, xb, wb, 1e-6)
    assert np.array_equal(_u16(x), res_o)
    check_close(_u16(norm), oracle.bf16_to_f32(norm_o).astype(np.float64), 1 / 64, 0.005)


def test_standalone_quantiser_wide_rows(tk, ctx, oracle):
    """quantize_activation_e4m3 on 17408-wide rows (the dense-FP8 down input width,
    tuisko-kernels-sm120/src/fp8/down.rs:35-60) and on the reference fixture tokens."""
    from tuiskollm_b200 import synth

    for cols, xb in ((17408, synth.normal_bf16(5, 1, (3, 17408))), (5120, F.fp8_input(16, 5120))):
        rows = xb.shape[0]
        codes = sentinel_plane((rows + 1, cols), torch.uint8)
        scales = sentinel_plane((rows + 1,), torch.float32)
        tk.Fp8ProjectionOp(ctx).quantize(None, rows, cols, dev(xb.view(np.int16)), codes, scales)
        torch.cuda.synchronize()
        oc, os_ = oracle.quantize_e4m3(xb, search=(cols == 5120))
        assert np.array_equal(host(codes)[:rows], oc)
        assert np.array_equal(host(scales)[:rows].view(np.uint32), os_.view(np.uint32))
        assert_inactive_untouched(codes, rows)
        assert_inactive_untouched(scales, rows)


def test_rejected_launches_report_gpu_launch(tk, ctx):
    hidden = 5120
    x = torch.zeros((8, hidden), dtype=torch.int16, device="cuda")
    w = torch.zeros((hidden,), dtype=torch.int16, device="cuda")
    op = tk.ResidualNormOp(ctx)
    for rows in (0, -1, 100000):
        with pytest.raises(tk.GpuError) as info:
            op.launch_plain(None, rows, x, w, x)
        assert info.value.code == "gpu.launch" and "admitted" in str(info.value)
    with pytest.raises(tk.GpuError) as info:
        op.launch_plain(None, 1, x.data_ptr() + 2, w, x)
    assert info.value.code == "gpu.launch" and "aligned" in str(info.value)
    with pytest.raises(tk.GpuError) as info:
        op.launch_residual(None, 1, x, None, w, x, x)
    assert info.value.code == "gpu.launch" and "null" in str(info.value)
    with pytest.raises(tk.GpuError):
        tk.Context(device=0, hidden=1000)
    with pytest.raises(tk.GpuError) as info:
        tk.Context(device=99)
    assert info.value.code == "gpu.context"
