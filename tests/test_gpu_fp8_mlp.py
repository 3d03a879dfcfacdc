"""GPU parity of the dense-FP8 MLP operators and the GDN output projection through the C ABI,
on the reference's own structured fixtures (qual/src/fp8_swiglu.rs, qual/src/fp8_down.rs,
qual/src/gdn_output.rs: bit-exact activation codes and scales, outputs within the reference's
tolerances, 0xA5 sentinels beyond the active rows, eager == graph replay) and on seeded random
planes against the CPU oracle."""
import numpy as np
import pytest
import torch

import fixtures_ref as F
from gpu_util import (assert_inactive_untouched, check_close, dev, graph_replay, host,
                      max_relative_error, sentinel_plane)

pytestmark = pytest.mark.gpu

HIDDEN, INTER, GDN_VALUE = 5120, 17408, 6144


@pytest.fixture(scope="module")
def tk():
    import tuiskollm_b200 as tk
    return tk


@pytest.fixture(scope="module")
def ctx(tk):
    return tk.Context(device=0)


def _u16(t):
    return host(t.view(torch.int16)).view(np.uint16)


class Planes:
    def __init__(self, max_rows, k, out_cols):
        self.codes = sentinel_plane((max_rows, k), torch.uint8)
        self.scales = sentinel_plane((max_rows,), torch.float32)
        self.out = sentinel_plane((max_rows, out_cols), torch.int16)

    def all(self):
        return (self.codes, self.scales, self.out)

    def reset(self):
        for p in self.all():
            p.view(torch.uint8).fill_(0xA5)

    def check_inactive(self, rows):
        for p in self.all():
            assert_inactive_untouched(p, rows)


def check_quantiser(oracle, xb, planes, rows):
    reps = []
    for t in range(rows):
        c, sc, rsum = oracle.quantize_e4m3_token(xb[t], search=True)
        assert np.array_equal(host(planes.codes)[t], c), f"activation codes of token {t}"
        assert host(planes.scales)[t] == sc, f"activation scale of token {t}"
        reps.append((rsum, sc))
    return reps


def replay_is_identical(launch, planes):
    eager = [host(p.view(torch.uint8)).copy() for p in planes.all()]
    g = graph_replay(launch)
    planes.reset()
    g.replay()
    g.replay()
    torch.cuda.synchronize()
    for e, p in zip(eager, planes.all()):
        assert np.array_equal(host(p.view(torch.uint8)), e)


@pytest.fixture(scope="module")
def swiglu_weights():
    return F.fp8_swiglu_weights(INTER, HIDDEN, "cuda")


@pytest.mark.parametrize("rows", F.FP8_SWIGLU_ROUTES)
def test_reference_fixture_fp8_swiglu(tk, ctx, oracle, swiglu_weights, rows):
    """qual/src/fp8_swiglu.rs: every exact route 1..8, 32, 64, 128 at full size; closed-form
    expectation silu(gate) * up within max(1/8, 1.5 %) (:282)."""
    max_rows = 128
    xb = F.mlp_input(max_rows, HIDDEN)
    w, s = swiglu_weights
    planes = Planes(max_rows, HIDDEN, INTER)
    x = dev(xb.view(np.int16))
    op = tk.Fp8SwiGluOp(ctx)
    launch = lambda: op.launch(None, rows, x, planes.codes, planes.scales, w, s, planes.out)
    launch()
    torch.cuda.synchronize()
    assert ctx.last_kernel.startswith("fp8_swiglu_kernel")
    reps = check_quantiser(oracle, xb, planes, rows)
    got = _u16(planes.out)
    for t, (rsum, sc) in enumerate(reps):
        check_close(got[t], F.fp8_swiglu_expected(rsum, sc, INTER), 0.125, 0.015, f"token {t}")
    planes.check_inactive(rows)
    replay_is_identical(launch, planes)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("rows", [1, 2, 3, 4, 5, 6, 7, 8])
def test_reference_fixture_fp8_down(tk, ctx, oracle, rows):
    """qual/src/fp8_down.rs: routes 1..8 at full size (K = 17408: the activation quantiser runs
    over the whole intermediate row), weights varying along the row; tolerance max(1/8, 1.5 %)."""
    max_rows = 8
    xb = F.mlp_input(max_rows, INTER)
    w, s = F.fp8_down_weights(HIDDEN, INTER, "cuda")
    planes = Planes(max_rows, INTER, HIDDEN)
    x = dev(xb.view(np.int16))
    op = tk.Fp8DownOp(ctx)
    launch = lambda: op.launch(None, rows, x, planes.codes, planes.scales, w, s, planes.out)
    launch()
    torch.cuda.synchronize()
    check_quantiser(oracle, xb, planes, rows)
    oc, os_ = oracle.quantize_e4m3(xb[:rows])
    exp = oracle.fp8_projection(oc, os_, host(w), _u16(s))  # = the reference's weight_correlations form
    check_close(_u16(planes.out)[:rows], exp, 0.125, 0.015, "down projection")
    planes.check_inactive(rows)
    replay_is_identical(launch, planes)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("rows", [1, 2, 3, 4, 5, 6, 7, 8])
def test_reference_fixture_gdn_output(tk, ctx, oracle, rows):
    """qual/src/gdn_output.rs: K = 6144, N = 5120, routes 1..8; tolerance max(1/16, 1 %) (:250)."""
    max_rows = 8
    xb = F.mlp_input(max_rows, GDN_VALUE, F.GDN_OUT_INPUT_PATTERN)
    w, s = F.gdn_output_weights(HIDDEN, GDN_VALUE, "cuda")
    planes = Planes(max_rows, GDN_VALUE, HIDDEN)
    x = dev(xb.view(np.int16))
    op = tk.GdnOutputProjectionOp(ctx, GDN_VALUE)
    launch = lambda: op.launch(None, rows, x, planes.codes, planes.scales, w, s, planes.out)
    launch()
    torch.cuda.synchronize()
    reps = check_quantiser(oracle, xb, planes, rows)
    got = _u16(planes.out)
    for t, (rsum, sc) in enumerate(reps):
        check_close(got[t], F.fp8_expected(rsum, sc, HIDDEN), 0.0625, 0.01, f"token {t}")
    planes.check_inactive(rows)
    replay_is_identical(launch, planes)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("rows", [1, 20, 33, 200, 300])
def test_fp8_mlp_random_planes_match_oracle(tk, oracle, rows):
    """Seeded ~N(0,1) activations and ~N(0,0.02) weights on a small geometry, ragged token counts
    (both token tiles, zero-filled tile tails): SwiGLU -> down through the two operators, each
    stage against the f64 oracle of the codes it consumed, within 1e-2."""
    from tuiskollm_b200 import synth

    hidden, inter = 1024, 1536
    c = tk.Context(device=0, hidden=hidden, intermediate=inter, max_rows=512)
    xb = synth.normal_bf16(51, rows, (rows, hidden))
    gu_c, gu_s = synth.fp8_weights(51, 1, 2 * inter, hidden)
    dn_c, dn_s = synth.fp8_weights(51, 2, hidden, inter)
    p1 = Planes(rows + 1, hidden, inter)
    p2 = Planes(rows + 1, inter, hidden)
    tk.Fp8SwiGluOp(c).launch(None, rows, dev(xb.view(np.int16)), p1.codes, p1.scales, dev(gu_c),
                             dev(gu_s.view(np.int16)), p1.out)
    tk.Fp8DownOp(c).launch(None, rows, p1.out, p2.codes, p2.scales, dev(dn_c), dev(dn_s.view(np.int16)),
                           p2.out)
    torch.cuda.synchronize()
    oc, os_ = oracle.quantize_e4m3(xb)
    assert np.array_equal(host(p1.codes)[:rows], oc)
    assert np.array_equal(host(p1.scales)[:rows].view(np.uint32), os_.view(np.uint32))
    proj = oracle.fp8_projection(oc, os_, gu_c, gu_s)
    exp_mid = oracle.silu_mul(proj[:, :inter], proj[:, inter:])
    mid = _u16(p1.out)[:rows]
    assert max_relative_error(mid, exp_mid, 4 * float(np.abs(exp_mid).mean())) <= 1e-2
    mc, ms = oracle.quantize_e4m3(mid)
    assert np.array_equal(host(p2.codes)[:rows], mc)
    assert np.array_equal(host(p2.scales)[:rows].view(np.uint32), ms.view(np.uint32))
    exp_out = oracle.fp8_projection(mc, ms, dn_c, dn_s)
    assert max_relative_error(_u16(p2.out)[:rows], exp_out, 4 * float(np.abs(exp_out).mean())) <= 1e-2
    p1.check_inactive(rows)
    p2.check_inactive(rows)
    assert c.device_status() == 0


def test_fp8_swiglu_rejected_launches(tk, ctx):
    x = torch.zeros((4, HIDDEN), dtype=torch.int16, device="cuda")
    codes = torch.zeros((4, HIDDEN), dtype=torch.uint8, device="cuda")
    scales = torch.zeros((4,), dtype=torch.float32, device="cuda")
    w = torch.zeros((256, HIDDEN), dtype=torch.uint8, device="cuda")
    ws = torch.zeros((256,), dtype=torch.int16, device="cuda")
    out = torch.zeros((4, INTER), dtype=torch.int16, device="cuda")
    op = tk.Fp8SwiGluOp(ctx)
    for rows in (0, 2049):
        with pytest.raises(tk.GpuError) as info:
            op.launch(None, rows, x, codes, scales, w, ws, out)
        assert info.value.code == "gpu.launch" and "FP8 SwiGLU row count" in str(info.value)
    with pytest.raises(tk.GpuError) as info:
        op.launch(None, 1, x, codes, scales, w.data_ptr() + 16, ws, out)
    assert "128-byte aligned" in str(info.value)
    torch.cuda.synchronize()


@pytest.mark.parametrize("rows", [256, 512])
def test_benchmarked_fp8_down_and_gdn_output_sampled_rows(tk, ctx, oracle, rows):
    """The benchmarked batched shapes of the dense-FP8 down projection (K = 17408: at 256 tokens
    the one-CTA kernel with K split over clusters, at 512 the CTA pairs) and of the GDN output
    projection at full size: quantiser bit-exact, sampled output rows (first, middle and last
    128-row tile) of every token against the f64 oracle within 1e-2."""
    from tuiskollm_b200 import synth

    for columns, stream in ((INTER, 91), (GDN_VALUE, 92)):
        w, s = synth.torch_fp8_weights(7, stream, HIDDEN, columns, "cuda")
        xb = synth.normal_bf16(7, stream + 10, (rows, columns))
        planes = Planes(rows + 1, columns, HIDDEN)
        if columns == INTER:
            tk.Fp8DownOp(ctx).launch(None, rows, dev(xb.view(np.int16)), planes.codes, planes.scales, w, s,
                                     planes.out)
        else:
            tk.GdnOutputProjectionOp(ctx, columns).launch(None, rows, dev(xb.view(np.int16)), planes.codes,
                                                          planes.scales, w, s, planes.out)
        route = ctx.last_kernel
        torch.cuda.synchronize()
        oc, os_ = oracle.quantize_e4m3(xb)
        assert np.array_equal(host(planes.codes)[:rows], oc), route
        assert np.array_equal(host(planes.scales)[:rows].view(np.uint32), os_.view(np.uint32)), route
        sample = np.concatenate([np.arange(0, 16), np.arange(2560, 2576), np.arange(HIDDEN - 16, HIDDEN)])
        wc = host(w)[sample]
        ws = host(s.view(torch.int16)).view(np.uint16)[sample]
        exp = oracle.fp8_projection(oc, os_, wc, ws)
        got = _u16(planes.out)[:rows][:, sample]
        assert max_relative_error(got, exp, 4 * float(np.abs(exp).mean())) <= 1e-2, route
        planes.check_inactive(rows)
    assert ctx.device_status() == 0
