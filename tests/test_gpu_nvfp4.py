"""GPU parity for the NVFP4 MLP projections (W4A4 on block-scaled tcgen05).

Weight side: pinned by the reference's fixtures (qual/src/nvfp4_swiglu.rs:196-234,
qual/src/nvfp4_down.rs:196-230) -- their inputs are exactly representable in NVFP4 with a
power-of-two divisor, so the reference's A16 closed form applies unchanged.
Activation quantiser: PARITY UNPINNED (no reference counterpart); the GPU must match this
build's own oracle definition bit for bit."""
import numpy as np
import pytest
import torch

import fixtures_ref as F
from gpu_util import (assert_inactive_untouched, check_close, dev, graph_replay, host,
                      max_relative_error, sentinel_plane)

pytestmark = pytest.mark.gpu

HIDDEN, INTER = 5120, 17408


@pytest.fixture(scope="module")
def tk():
    import tuiskollm_b200 as tk
    return tk


@pytest.fixture(scope="module")
def ctx(tk):
    return tk.Context(device=0)


def _u16(t):
    return host(t.view(torch.int16)).view(np.uint16)


def act_planes(tk, max_rows, k):
    from tuiskollm_b200 import ops
    codes = sentinel_plane((max_rows, k // 2), torch.uint8)
    scales = sentinel_plane((ops.nvfp4_scale_plane_bytes(max_rows, k),), torch.uint8)
    return codes, scales


def check_quantiser(oracle, xb, divisor, codes, scales, rows):
    k = xb.shape[1]
    oc, osc = oracle.nvfp4_quantize(xb[:rows], divisor)
    assert np.array_equal(host(codes)[:rows], oc), "NVFP4 activation codes"
    offs = oracle.nvfp4_scale_offsets(rows, k // 16)
    got = host(scales)
    assert np.array_equal(got[offs], osc[offs]), "NVFP4 activation scales"
    # every other byte of the plane (rows >= `rows` of the padded tiles) is untouched
    mask = np.ones(got.size, bool)
    mask[offs.reshape(-1)] = False
    assert (got[mask] == 0xA5).all(), "scale entries of inactive rows were written"
    assert_inactive_untouched(codes, rows)
    return oc, osc


@pytest.mark.parametrize("rows,k", [(1, 5120), (5, 5120), (130, 5120), (3, 17408), (33, 256)])
def test_activation_quantiser_is_bit_exact(tk, ctx, oracle, rows, k):
    from tuiskollm_b200 import synth

    xb = synth.normal_bf16(21, rows + k, (rows, k))
    xb[0, :16] = 0          # an all-zero block (scale 0, signed-zero codes)
    xb[0, 3] = 0x8000
    xb[rows - 1, 16:32] = synth.f32_to_bf16_bits(np.full(16, 1e-30, np.float32))  # underflowing scale
    divisor = float(np.float32(448.0 * 6.0 / 4.5))
    codes, scales = act_planes(tk, rows + 2, k)
    tk.Nvfp4SwiGluOp(ctx).quantize(None, rows, k, dev(xb.view(np.int16)), divisor, codes, scales)
    torch.cuda.synchronize()
    check_quantiser(oracle, xb, divisor, codes, scales, rows)


@pytest.mark.parametrize("rows", [1, 7, 130])
def test_fused_producer_emits_nvfp4_and_e4m3(tk, ctx, oracle, rows):
    """Residual add + RMSNorm + E4M3 quantise + NVFP4 quantise in ONE kernel: every output is
    the oracle's function of the normalised row the kernel itself wrote, bit for bit, and the
    NVFP4 planes feed the gate_up projection directly (input == NULL)."""
    from tuiskollm_b200 import synth

    xb = synth.normal_bf16(33, rows, (rows, HIDDEN))
    bb = synth.normal_bf16(33, rows + 1, (rows, HIDDEN))
    nb = synth.normal_bf16(33, 3, (HIDDEN,), std=0.1)
    divisor = float(np.float32(448.0 * 6.0 / 6.0))
    res = sentinel_plane((rows + 1, HIDDEN), torch.int16)
    norm = sentinel_plane((rows + 1, HIDDEN), torch.int16)
    e_codes = sentinel_plane((rows + 1, HIDDEN), torch.uint8)
    e_scales = sentinel_plane((rows + 1,), torch.float32)
    codes, scales = act_planes(tk, rows + 1, HIDDEN)
    tk.ResidualNormOp(ctx).launch_quantize_nvfp4(None, rows, dev(xb.view(np.int16)), dev(bb.view(np.int16)),
                                                 dev(nb.view(np.int16)), res, norm, e_codes, e_scales,
                                                 divisor, codes, scales)
    torch.cuda.synchronize()
    res_o, _ = oracle.residual_rms_norm(xb, bb, nb, 1e-6)
    assert np.array_equal(_u16(res)[:rows], res_o)
    nd = _u16(norm)[:rows]
    oc, os_ = oracle.quantize_e4m3(nd)
    assert np.array_equal(host(e_codes)[:rows], oc)
    assert np.array_equal(host(e_scales)[:rows].view(np.uint32), os_.view(np.uint32))
    check_quantiser(oracle, nd, divisor, codes, scales, rows)
    for pl in (res, norm, e_codes, e_scales):
        assert_inactive_untouched(pl, rows)
    # E4M3 side optional
    codes2, scales2 = act_planes(tk, rows + 1, HIDDEN)
    tk.ResidualNormOp(ctx).launch_quantize_nvfp4(None, rows, dev(xb.view(np.int16)), None,
                                                 dev(nb.view(np.int16)), None, norm, None, None,
                                                 divisor, codes2, scales2)
    torch.cuda.synchronize()
    check_quantiser(oracle, _u16(norm)[:rows], divisor, codes2, scales2, rows)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("batch", [1, 2, 3, 4, 5, 6, 7, 8])
def test_reference_fixture_gate_up_swiglu(tk, ctx, oracle, batch):
    """qual/src/nvfp4_swiglu.rs: structured fixture at full size, exact batches 1..8; tolerance
    max(1/4, 2.5 %) of the f64 represented-value oracle (:248), sentinels, graph replay."""
    x = F.nvfp4_input(8, HIDDEN)
    wc, wsc = cached_fixture("gate_up")
    # amax of every 16-block is 0.5 * token factor, so divisor 12 makes every block scale a
    # power of two and every activation an exact E2M1 value: W4A4 == A16 on this fixture
    divisor = 12.0
    codes, scales = act_planes(tk, 8, HIDDEN)
    out = sentinel_plane((8, INTER), torch.int16)
    w, s, xd = dev(wc), dev(wsc), dev(x.view(np.int16))
    op = tk.Nvfp4SwiGluOp(ctx)
    launch = lambda: op.launch(None, batch, xd, w, s, F.NVFP4_WEIGHT_SCALE_DIVISOR, out,
                               activation_codes=codes, activation_scales=scales,
                               input_global_divisor=divisor)
    launch()
    torch.cuda.synchronize()
    oc, osc = check_quantiser(oracle, x, divisor, codes, scales, batch)
    dots = oracle.nvfp4_a16_dot(x[:batch], wc, wsc, F.NVFP4_WEIGHT_SCALE_DIVISOR)
    w4a4 = oracle.nvfp4_w4a4_dot(oc, osc, divisor, wc, wsc, F.NVFP4_WEIGHT_SCALE_DIVISOR)
    np.testing.assert_allclose(w4a4, dots, rtol=1e-12, atol=1e-12)  # lossless activations
    exp = oracle.silu_mul(dots[:, :INTER], dots[:, INTER:])
    for token in (0, batch - 1):
        for row in (0, 1, 127, 128, INTER - 1):
            g = F.nvfp4_closed_form_dot(x, token, row, wc, wsc, HIDDEN)
            u = F.nvfp4_closed_form_dot(x, token, row + INTER, wc, wsc, HIDDEN)
            assert exp[token, row] == pytest.approx(g / (1 + np.exp(-g)) * u, rel=1e-12, abs=1e-12)
    got = _u16(out)
    check_close(got[:batch], exp, 0.25, 0.025, "NVFP4 SwiGLU")
    assert_inactive_untouched(out, batch)
    eager = host(out.view(torch.uint8)).copy()
    g = graph_replay(launch)
    out.view(torch.uint8).fill_(0xA5)
    g.replay()
    g.replay()
    torch.cuda.synchronize()
    assert np.array_equal(host(out.view(torch.uint8)), eager)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("batch", [1, 4, 8])
def test_reference_fixture_down(tk, ctx, oracle, batch):
    """qual/src/nvfp4_down.rs: structured fixture at full size (K = 17408, split-K route)."""
    x = F.nvfp4_input(8, INTER)
    wc, wsc = cached_fixture("down")
    divisor = 12.0
    codes, scales = act_planes(tk, 8, INTER)
    out = sentinel_plane((8, HIDDEN), torch.int16)
    op = tk.Nvfp4DownOp(ctx)
    w, s, xd = dev(wc), dev(wsc), dev(x.view(np.int16))
    launch = lambda: op.launch(None, batch, xd, w, s, F.NVFP4_WEIGHT_SCALE_DIVISOR, out,
                               activation_codes=codes, activation_scales=scales,
                               input_global_divisor=divisor)
    launch()
    torch.cuda.synchronize()
    check_quantiser(oracle, x, divisor, codes, scales, batch)
    exp = oracle.nvfp4_a16_dot(x[:batch], wc, wsc, F.NVFP4_WEIGHT_SCALE_DIVISOR)
    for row in (0, 1, 127, 128, HIDDEN - 1):
        assert exp[0, row] == pytest.approx(F.nvfp4_closed_form_dot(x, 0, row, wc, wsc, INTER), rel=1e-12)
    check_close(_u16(out)[:batch], exp, 0.25, 0.025, "NVFP4 down")
    assert_inactive_untouched(out, batch)
    eager = host(out.view(torch.uint8)).copy()
    g = graph_replay(launch)
    out.view(torch.uint8).fill_(0xA5)
    g.replay()
    g.replay()
    torch.cuda.synchronize()
    assert np.array_equal(host(out.view(torch.uint8)), eager)
    assert ctx.device_status() == 0


_FIXTURES = {}


def cached_fixture(kind):
    if kind not in _FIXTURES:
        if kind == "gate_up":
            _FIXTURES[kind] = F.nvfp4_weights(2 * INTER, HIDDEN, gate_up_split=INTER)
        else:
            _FIXTURES[kind] = F.nvfp4_weights(HIDDEN, INTER, gate_up_split=None)
    return _FIXTURES[kind]


@pytest.mark.parametrize("rows", [1, 32, 100, 256])
def test_synthetic_mlp_small_geometry(tk, oracle, rows):
    """Random N(0,1) activations and N(0,0.02) weights on a small geometry (hidden 1024,
    intermediate 512) where the whole W4A4 oracle is cheap: gate_up+SwiGLU, re-quantise,
    down; max relative error 1e-2 at every step against the oracle run on the device's own
    quantised operands."""
    from tuiskollm_b200 import synth

    hidden, inter = 1024, 512
    ctx = tk.Context(device=0, hidden=hidden, intermediate=inter, max_rows=512)
    xb = synth.normal_bf16(4, rows, (rows, hidden))
    gu_codes, gu_scales, gu_div = synth.nvfp4_weights(4, 1, 2 * inter, hidden)
    dn_codes, dn_scales, dn_div = synth.nvfp4_weights(4, 2, hidden, inter)
    a_div = float(np.float32(448.0 * 6.0 / 5.0))  # calibration: |x| stays below ~5
    codes, scales = act_planes(tk, rows + 1, hidden)
    mid = sentinel_plane((rows + 1, inter), torch.int16)
    tk.Nvfp4SwiGluOp(ctx).launch(None, rows, dev(xb.view(np.int16)), dev(gu_codes), dev(gu_scales),
                                 float(gu_div), mid, activation_codes=codes,
                                 activation_scales=scales, input_global_divisor=a_div)
    torch.cuda.synchronize()
    oc, osc = check_quantiser(oracle, xb, a_div, codes, scales, rows)
    dots = oracle.nvfp4_w4a4_dot(oc, osc, a_div, gu_codes, gu_scales, float(gu_div))
    exp_mid = oracle.silu_mul(dots[:, :inter], dots[:, inter:])
    got_mid = _u16(mid)[:rows]
    scale_mid = float(np.abs(exp_mid).mean())
    assert max_relative_error(got_mid, exp_mid, 4 * scale_mid) <= 1e-2
    check_close(got_mid, exp_mid, 0.25, 0.025, "gate_up")
    assert_inactive_untouched(mid, rows)
    # down projection from the device's own intermediate
    m_div = float(np.float32(448.0 * 6.0) / max(np.abs(oracle.bf16_to_f32(got_mid)).max(), 1e-6))
    codes2, scales2 = act_planes(tk, rows + 1, inter)
    out = sentinel_plane((rows + 1, hidden), torch.int16)
    tk.Nvfp4DownOp(ctx).launch(None, rows, mid, dev(dn_codes), dev(dn_scales), float(dn_div), out,
                               activation_codes=codes2, activation_scales=scales2,
                               input_global_divisor=m_div)
    torch.cuda.synchronize()
    oc2, osc2 = check_quantiser(oracle, got_mid, m_div, codes2, scales2, rows)
    exp_out = oracle.nvfp4_w4a4_dot(oc2, osc2, m_div, dn_codes, dn_scales, float(dn_div))
    got_out = _u16(out)[:rows]
    assert max_relative_error(got_out, exp_out, 4 * float(np.abs(exp_out).mean())) <= 1e-2
    assert_inactive_untouched(out, rows)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("rows", [256, 300, 512])
def test_pair_route_small_geometry(tk, oracle, rows, monkeypatch):
    """The CTA-pair (cta_group::2) prefill route forced on at small sizes: gate_up + SwiGLU
    (gate CTA / up CTA exchange halves over distributed shared memory) and down, ragged token
    counts included, against the W4A4 oracle and against the one-CTA route."""
    from tuiskollm_b200 import synth

    hidden, inter = 1024, 512
    xb = synth.normal_bf16(14, rows, (rows, hidden))
    gu_codes, gu_scales, gu_div = synth.nvfp4_weights(14, 1, 2 * inter, hidden)
    dn_codes, dn_scales, dn_div = synth.nvfp4_weights(14, 2, hidden, inter)
    a_div = float(np.float32(448.0 * 6.0 / 5.0))
    results = {}
    for route, min_rows in (("pair", "1"), ("single", "1000000")):
        monkeypatch.setenv("TK100_PAIR_MIN_ROWS", min_rows)
        monkeypatch.setenv("TK100_PAIR", "2")  # gate_up on pairs too (off by default)
        ctx = tk.Context(device=0, hidden=hidden, intermediate=inter, max_rows=512)
        codes, scales = act_planes(tk, rows + 1, hidden)
        mid = sentinel_plane((rows + 1, inter), torch.int16)
        tk.Nvfp4SwiGluOp(ctx).launch(None, rows, dev(xb.view(np.int16)), dev(gu_codes), dev(gu_scales),
                                     float(gu_div), mid, activation_codes=codes,
                                     activation_scales=scales, input_global_divisor=a_div)
        torch.cuda.synchronize()
        got_mid = _u16(mid)[:rows].copy()
        assert_inactive_untouched(mid, rows)
        m_div = float(np.float32(448.0 * 6.0 / 8.0))
        codes2, scales2 = act_planes(tk, rows + 1, inter)
        out = sentinel_plane((rows + 1, hidden), torch.int16)
        tk.Nvfp4DownOp(ctx).launch(None, rows, mid, dev(dn_codes), dev(dn_scales), float(dn_div), out,
                                   activation_codes=codes2, activation_scales=scales2,
                                   input_global_divisor=m_div)
        torch.cuda.synchronize()
        assert_inactive_untouched(out, rows)
        assert ctx.device_status() == 0, route
        results[route] = (got_mid, _u16(out)[:rows].copy(), host(codes)[:rows].copy(), host(scales).copy(),
                          host(codes2)[:rows].copy(), host(scales2).copy())
    oc, osc = oracle.nvfp4_quantize(xb, a_div)
    dots = oracle.nvfp4_w4a4_dot(oc, osc, a_div, gu_codes, gu_scales, float(gu_div))
    exp_mid = oracle.silu_mul(dots[:, :inter], dots[:, inter:])
    for route in ("pair", "single"):
        got_mid, got_out, _, _, c2, s2 = results[route]
        assert max_relative_error(got_mid, exp_mid, 4 * float(np.abs(exp_mid).mean())) <= 1e-2, route
        oc2, osc2 = oracle.nvfp4_quantize(got_mid, float(np.float32(448.0 * 6.0 / 8.0)))
        assert np.array_equal(c2, oc2)
        exp_out = oracle.nvfp4_w4a4_dot(oc2, osc2, float(np.float32(448.0 * 6.0 / 8.0)), dn_codes, dn_scales, float(dn_div))
        assert max_relative_error(got_out, exp_out, 4 * float(np.abs(exp_out).mean())) <= 1e-2, route
    # same products, same fp32 accumulation order per output: the two routes agree to the bit
    assert np.array_equal(results["pair"][0], results["single"][0])


@pytest.mark.parametrize("rows", [1, 7, 32, 33, 130, 256])
def test_gate_up_cluster_pairs_and_fused_kernel_agree(tk, oracle, rows, monkeypatch):
    """gate_up + SwiGLU on its two routes, ragged token counts included: clusters of a gate CTA
    and an up CTA that swap accumulator halves over distributed shared memory (the default), and
    one CTA that holds both tiles (TK100_SWIGLU_PAIRS=0).  Both against the W4A4 oracle; the
    two agree to the bit (same products, same fp32 accumulation order per output)."""
    from tuiskollm_b200 import synth

    hidden, inter = 1024, 512
    xb = synth.normal_bf16(15, rows, (rows, hidden))
    gu_codes, gu_scales, gu_div = synth.nvfp4_weights(15, 1, 2 * inter, hidden)
    a_div = float(np.float32(448.0 * 6.0 / 5.0))
    results = {}
    for route, env in (("pairs", "1"), ("fused", "0")):
        monkeypatch.setenv("TK100_SWIGLU_PAIRS", env)
        ctx = tk.Context(device=0, hidden=hidden, intermediate=inter, max_rows=512)
        codes, scales = act_planes(tk, rows + 1, hidden)
        mid = sentinel_plane((rows + 1, inter), torch.int16)
        tk.Nvfp4SwiGluOp(ctx).launch(None, rows, dev(xb.view(np.int16)), dev(gu_codes), dev(gu_scales),
                                     float(gu_div), mid, activation_codes=codes,
                                     activation_scales=scales, input_global_divisor=a_div)
        torch.cuda.synchronize()
        assert_inactive_untouched(mid, rows)
        assert ctx.device_status() == 0, route
        results[route] = _u16(mid)[:rows].copy()
    oc, osc = oracle.nvfp4_quantize(xb, a_div)
    dots = oracle.nvfp4_w4a4_dot(oc, osc, a_div, gu_codes, gu_scales, float(gu_div))
    exp_mid = oracle.silu_mul(dots[:, :inter], dots[:, inter:])
    for route, got in results.items():
        assert max_relative_error(got, exp_mid, 4 * float(np.abs(exp_mid).mean())) <= 1e-2, route
    assert np.array_equal(results["pairs"], results["fused"])


def test_activation_quantiser_rounding_ties(tk, oracle):
    """Values that sit exactly on the E2M1 rounding midpoints after the quantiser's IEEE divide
    (ties go to the even code), one BF16 step beside them, and beyond the largest magnitude must
    come out as the oracle's divide-then-round does."""
    k = 64
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    mid_bits = mids.view(np.uint32) >> 16
    above = ((mid_bits + 1) << 16).astype(np.uint32).view(np.float32)  # next BF16 value up
    below = ((mid_bits - 1) << 16).astype(np.uint32).view(np.float32)  # next BF16 value down
    g0 = np.concatenate([[6.0], mids, -mids, [-6.0]]).astype(np.float32)            # scale 1
    g1 = (2.0 * g0).astype(np.float32)                                               # scale 2
    g2 = (1.5 * g0).astype(np.float32)                                               # scale 1.5
    g3 = np.concatenate([[6.0], above, -below, [7.0]]).astype(np.float32)  # beside the ties
    rows = np.stack([np.concatenate([g0, g1, g2, g3]),
                     np.concatenate([g3, -g2, g1 * np.float32(0.5), -g0]),
                     np.concatenate([g0 * np.float32(2.0 ** -12), np.zeros(16, np.float32), -np.zeros(16, np.float32) - 0.0, g0 * np.float32(40.0)])])
    bits = (rows.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    assert np.array_equal((bits.astype(np.uint32) << 16).view(np.float32), rows), "values must be BF16-exact"
    ctx = tk.Context(device=0, hidden=1024, intermediate=512, max_rows=512)
    for divisor in (1.0, 2.0, 0.5):
        codes, scales = act_planes(tk, rows.shape[0] + 1, k)
        tk.Nvfp4DownOp(ctx).quantize(None, rows.shape[0], k, dev(bits.view(np.int16)), divisor, codes, scales)
        torch.cuda.synchronize()
        check_quantiser(oracle, bits, divisor, codes, scales, rows.shape[0])
    assert ctx.device_status() == 0


@pytest.mark.parametrize("rows", [1, 20, 33, 129, 300])
def test_gate_up_epilogue_quantisation_equals_the_quantiser(tk, oracle, rows, monkeypatch):
    """tk100_nvfp4_gate_up_swiglu_quantize: the codes and block scales it leaves for the down
    projection equal, bit for bit, what the stand-alone quantiser (and the oracle) make of its
    BF16 output, whether they come from the projection's epilogue (up to 32 rows on the cluster
    route) or from the quantiser launch behind it; inactive rows stay untouched."""
    from tuiskollm_b200 import ops, synth

    hidden, inter = 1024, 512
    xb = synth.normal_bf16(16, rows, (rows, hidden))
    gu_codes, gu_scales, gu_div = synth.nvfp4_weights(16, 1, 2 * inter, hidden)
    a_div = float(np.float32(448.0 * 6.0 / 5.0))
    m_div = float(np.float32(448.0 * 6.0 / 8.0))
    planes = {}
    for route, env in (("pairs", "1"), ("fused", "0")):
        monkeypatch.setenv("TK100_SWIGLU_PAIRS", env)
        ctx = tk.Context(device=0, hidden=hidden, intermediate=inter, max_rows=512)
        codes, scales = act_planes(tk, rows + 1, hidden)
        mid = sentinel_plane((rows + 1, inter), torch.int16)
        q_codes = sentinel_plane((rows + 1, inter // 2), torch.uint8)
        q_scales = sentinel_plane((ops.nvfp4_scale_plane_bytes(rows, inter),), torch.uint8)
        launches = ctx.launch_count
        tk.Nvfp4SwiGluOp(ctx).launch_quantize(
            None, rows, dev(xb.view(np.int16)), dev(gu_codes), dev(gu_scales), float(gu_div), mid,
            activation_codes=codes, activation_scales=scales, input_global_divisor=a_div,
            output_global_divisor=m_div, output_codes=q_codes, output_scales=q_scales)
        torch.cuda.synchronize()
        assert ctx.device_status() == 0, route
        # input quantiser + projection, + the output quantiser where the epilogue does not do it
        in_epilogue = route == "pairs" and rows <= 32
        assert ctx.launch_count - launches == (2 if in_epilogue else 3), route
        assert_inactive_untouched(mid, rows)
        got_mid = _u16(mid)[:rows].copy()
        check_quantiser(oracle, got_mid, m_div, q_codes, q_scales, rows)
        planes[route] = (host(q_codes)[:rows].copy(), got_mid)
    assert np.array_equal(planes["pairs"][1], planes["fused"][1])
    assert np.array_equal(planes["pairs"][0], planes["fused"][0])


@pytest.mark.parametrize("world,rows", [(2, 5), (8, 40), (8, 200)])
def test_row_parallel_down_shards_sum_to_the_full_projection(tk, oracle, world, rows):
    """Tensor-parallel down projection emulated on one GPU: every rank's reduction shard
    (at world 8 the shard is 384 columns = one full 256-column stage + a 128-column tail)
    produces fp32 partial sums; their sum, rounded once, matches the W4A4 oracle on the whole
    reduction and the single-rank kernel."""
    from tuiskollm_b200 import ops, synth

    hidden, inter = 1024, 3072
    xb = synth.normal_bf16(6, rows, (rows, inter))
    w_codes, w_scales, w_div = synth.nvfp4_weights(6, 1, hidden, inter)
    a_div = float(np.float32(448.0 * 6.0 / 5.0))
    full_ctx = tk.Context(device=0, hidden=hidden, intermediate=inter, max_rows=256)
    codes, scales = act_planes(tk, rows, inter)
    full = sentinel_plane((rows, hidden), torch.int16)
    tk.Nvfp4DownOp(full_ctx).launch(None, rows, dev(xb.view(np.int16)), dev(w_codes), dev(w_scales),
                                    float(w_div), full, activation_codes=codes,
                                    activation_scales=scales, input_global_divisor=a_div)
    torch.cuda.synchronize()
    oc, osc = oracle.nvfp4_quantize(xb, a_div)
    exp = oracle.nvfp4_w4a4_dot(oc, osc, a_div, w_codes, w_scales, float(w_div))
    ks = inter // world
    shard_ctx = tk.Context(device=0, hidden=hidden, intermediate=ks, max_rows=256)
    total = np.zeros((rows, hidden), np.float64)
    for r in range(world):
        wc_r, ws_r = synth.nvfp4_reduction_shard(w_codes, w_scales, inter, world, r)
        x_r = np.ascontiguousarray(xb[:, r * ks:(r + 1) * ks])
        c_r, s_r = act_planes(tk, rows, ks)
        part = sentinel_plane((rows + 1, hidden), torch.float32)
        tk.Nvfp4DownOp(shard_ctx).launch_partial(None, rows, dev(x_r.view(np.int16)), dev(wc_r),
                                                 dev(ws_r), float(w_div), part, activation_codes=c_r,
                                                 activation_scales=s_r, input_global_divisor=a_div)
        torch.cuda.synchronize()
        # block-local quantisation: the shard's codes are the matching columns of the full plane
        assert np.array_equal(host(c_r)[:rows], oc[:, r * ks // 2:(r + 1) * ks // 2])
        assert_inactive_untouched(part, rows)
        total += host(part)[:rows].astype(np.float64)
    floor = 4 * float(np.abs(exp).mean())
    assert (np.abs(total - exp) / np.maximum(np.abs(exp), floor)).max() <= 2e-3
    summed = torch.from_numpy(total.astype(np.float32)).cuda()
    rounded = sentinel_plane((rows, hidden), torch.int16)
    ops.f32_to_bf16(shard_ctx, None, rows * hidden, summed, rounded)
    torch.cuda.synchronize()
    assert np.array_equal(_u16(rounded), oracle.f32_to_bf16(total.astype(np.float32)))
    assert max_relative_error(_u16(rounded), exp, floor) <= 1e-2
    assert max_relative_error(_u16(full), exp, floor) <= 1e-2
    assert shard_ctx.device_status() == 0 and full_ctx.device_status() == 0


def test_full_size_prefill_sampled_tiles(tk, ctx, oracle):
    """Configuration 4 (M = 2048, gate_up 34816 x 5120, down 5120 x 17408): too large for the
    CPU oracle as a whole, so whole 128-row tiles are sampled -- first, last and two inner
    weight tiles x first and last token tiles -- and checked against the W4A4 oracle."""
    from tuiskollm_b200 import ops, synth

    rows = 2048
    x = synth.torch_normal_bf16(12, 1, (rows, HIDDEN), "cuda")
    gu_codes, gu_scales, gu_div = synth.torch_nvfp4_weights(12, 2, 2 * INTER, HIDDEN, "cuda")
    a_div = float(np.float32(448.0 * 6.0 / 6.0))
    codes, scales = act_planes(tk, rows, HIDDEN)
    mid = sentinel_plane((rows, INTER), torch.int16)
    tk.Nvfp4SwiGluOp(ctx).launch(None, rows, x, gu_codes, gu_scales, gu_div, mid,
                                 activation_codes=codes, activation_scales=scales,
                                 input_global_divisor=a_div)
    torch.cuda.synchronize()
    g_in, g_w = HIDDEN // 16, HIDDEN // 16
    tok_tiles, w_tiles = [0, rows // 128 - 1], [0, 57, 100, INTER // 128 - 1]

    def tile_slice(plane, tile, groups):
        return plane[tile * 128 * groups:(tile + 1) * 128 * groups]

    xb = _u16(x.view(torch.int16))
    for tt in tok_tiles:
        oc, osc = oracle.nvfp4_quantize(xb[tt * 128:(tt + 1) * 128], a_div)
        assert np.array_equal(host(codes[tt * 128:(tt + 1) * 128]), oc)
        assert np.array_equal(host(tile_slice(scales, tt, g_in)), osc)
        for wt in w_tiles:
            rows_g = slice(wt * 128, (wt + 1) * 128)
            rows_u = slice(INTER + wt * 128, INTER + (wt + 1) * 128)
            wc = np.concatenate([host(gu_codes[rows_g]), host(gu_codes[rows_u])])
            ws = np.concatenate([host(tile_slice(gu_scales, wt, g_w)),
                                 host(tile_slice(gu_scales, INTER // 128 + wt, g_w))])
            dots = oracle.nvfp4_w4a4_dot(oc, osc, a_div, wc, ws, gu_div)
            exp = oracle.silu_mul(dots[:, :128], dots[:, 128:])
            got = _u16(mid)[tt * 128:(tt + 1) * 128, rows_g]
            assert max_relative_error(got, exp, 4 * float(np.abs(exp).mean())) <= 1e-2
    assert ctx.device_status() == 0


@pytest.mark.parametrize("rows", [1, 8, 32, 200])
def test_reduction_routes_of_the_mlp_agree_bit_for_bit(tk, oracle, rows, monkeypatch):
    """Gate/up pairs and the split-K down projection with their partial tiles pushed into the
    finishing CTA's shared memory (TK100_CLUSTER=2; by default only the pairs at 128-token tiles
    push) against the two-barrier cluster exchange (1) and, for down, the global-scratch
    reduction (0): same bits in the intermediate, in its NVFP4 form and in the output, at the full
    MLP geometry."""
    from tuiskollm_b200 import ops, synth

    x = synth.torch_normal_bf16(17, rows, (rows, HIDDEN), "cuda")
    gu = synth.torch_nvfp4_weights(17, 1, 2 * INTER, HIDDEN, "cuda")
    dn = synth.torch_nvfp4_weights(17, 2, HIDDEN, INTER, "cuda")
    a_div, m_div = float(np.float32(448.0)), float(np.float32(448.0 * 6.0 / 8.0))
    got, routes = {}, {}
    for mode in ("2", "1", "0"):
        monkeypatch.setenv("TK100_CLUSTER", mode)
        c = tk.Context(device=0)
        a_codes, a_scales = act_planes(tk, rows + 1, HIDDEN)
        m_codes, m_scales = act_planes(tk, rows + 1, INTER)
        mid = sentinel_plane((rows + 1, INTER), torch.int16)
        out = sentinel_plane((rows + 1, HIDDEN), torch.int16)
        tk.Nvfp4SwiGluOp(c).launch_quantize(None, rows, x, gu[0], gu[1], gu[2], mid,
                                            activation_codes=a_codes, activation_scales=a_scales,
                                            input_global_divisor=a_div, output_global_divisor=m_div,
                                            output_codes=m_codes, output_scales=m_scales)
        r_gu = c.last_kernel
        tk.Nvfp4DownOp(c).launch(None, rows, None, dn[0], dn[1], dn[2], out, activation_codes=m_codes,
                                 activation_scales=m_scales, input_global_divisor=m_div)
        torch.cuda.synchronize()
        routes[mode] = (r_gu, c.last_kernel)
        assert c.device_status() == 0, mode
        for pl in (mid, out, m_codes):
            assert_inactive_untouched(pl, rows)
        got[mode] = (_u16(mid)[:rows].copy(), host(m_codes)[:rows].copy(), _u16(out)[:rows].copy())
    assert "cluster-leader" in routes["2"][0] and "cluster-leader" not in routes["1"][0], routes
    if rows <= 32:
        assert "cluster-leader" in routes["2"][1], routes
    for mode in ("1", "0"):
        for a, b in zip(got["2"], got[mode]):
            assert np.array_equal(a, b), (mode, routes)
    # and the values are the W4A4 oracle's on a sample of the outputs
    xb = _u16(x.view(torch.int16))
    oc, osc = oracle.nvfp4_quantize(xb, a_div)
    g = HIDDEN // 16
    wc = np.concatenate([host(gu[0][:128]), host(gu[0][INTER:INTER + 128])])
    ws = np.concatenate([host(gu[1][:128 * g]), host(gu[1][(INTER // 128) * 128 * g:(INTER // 128 + 1) * 128 * g])])
    dots = oracle.nvfp4_w4a4_dot(oc, osc, a_div, wc, ws, gu[2])
    exp = oracle.silu_mul(dots[:, :128], dots[:, 128:])
    assert max_relative_error(got["2"][0][:, :128], exp, 4 * float(np.abs(exp).mean())) <= 1e-2


@pytest.mark.parametrize("rows", [256, 300, 700, 1030])
def test_persistent_pair_route_matches_plain_route_and_oracle(tk, oracle, rows, monkeypatch):
    """Prefill token counts run on persistent CTA pairs (256-row x 256-token pair tiles, each pair
    walking several tiles, gate/up halves exchanged through the partner's shared memory).  On a
    small geometry with ragged token counts: every output within tolerance of the W4A4 oracle,
    inactive rows untouched, and the same bits as the one-CTA kernels (TK100_PERSIST=0) -- both
    add the K blocks in order into one fp32 accumulator."""
    from tuiskollm_b200 import synth

    hidden, inter = 1024, 1536
    xb = synth.normal_bf16(18, rows, (rows, hidden))
    gu_codes, gu_scales, gu_div = synth.nvfp4_weights(18, 1, 2 * inter, hidden)
    dn_codes, dn_scales, dn_div = synth.nvfp4_weights(18, 2, hidden, inter)
    a_div, m_div = float(np.float32(448.0 * 6.0 / 5.0)), float(np.float32(448.0 * 6.0 / 8.0))
    got = {}
    for route, env in (("persistent", "1"), ("plain", "0")):
        monkeypatch.setenv("TK100_PERSIST", env)
        monkeypatch.setenv("TK100_PERSIST_MIN_ROWS", "256")
        c = tk.Context(device=0, hidden=hidden, intermediate=inter, max_rows=2048)
        a_codes, a_scales = act_planes(tk, rows + 1, hidden)
        m_codes, m_scales = act_planes(tk, rows + 1, inter)
        mid = sentinel_plane((rows + 1, inter), torch.int16)
        out = sentinel_plane((rows + 1, hidden), torch.int16)
        part = sentinel_plane((rows + 1, hidden), torch.float32)
        tk.Nvfp4SwiGluOp(c).launch_quantize(None, rows, dev(xb.view(np.int16)), dev(gu_codes), dev(gu_scales),
                                            float(gu_div), mid, activation_codes=a_codes,
                                            activation_scales=a_scales, input_global_divisor=a_div,
                                            output_global_divisor=m_div, output_codes=m_codes,
                                            output_scales=m_scales)
        r_gu = c.last_kernel
        tk.Nvfp4DownOp(c).launch(None, rows, None, dev(dn_codes), dev(dn_scales), float(dn_div), out,
                                 activation_codes=m_codes, activation_scales=m_scales,
                                 input_global_divisor=m_div)
        r_dn = c.last_kernel
        tk.Nvfp4DownOp(c).launch_partial(None, rows, None, dev(dn_codes), dev(dn_scales), float(dn_div),
                                         part, activation_codes=m_codes, activation_scales=m_scales,
                                         input_global_divisor=m_div)
        torch.cuda.synchronize()
        assert c.device_status() == 0, route
        assert r_gu.startswith("nvfp4_persist_kernel") == (route == "persistent"), (route, r_gu)
        assert r_dn.startswith("nvfp4_persist_kernel") == (route == "persistent"), (route, r_dn)
        for pl in (mid, out, part):
            assert_inactive_untouched(pl, rows)
        got[route] = (_u16(mid)[:rows].copy(), _u16(out)[:rows].copy(), host(part)[:rows].copy())
    oc, osc = oracle.nvfp4_quantize(xb, a_div)
    dots = oracle.nvfp4_w4a4_dot(oc, osc, a_div, gu_codes, gu_scales, float(gu_div))
    exp_mid = oracle.silu_mul(dots[:, :inter], dots[:, inter:])
    assert max_relative_error(got["persistent"][0], exp_mid, 4 * float(np.abs(exp_mid).mean())) <= 1e-2
    mc, msc = oracle.nvfp4_quantize(got["persistent"][0], m_div)
    exp_out = oracle.nvfp4_w4a4_dot(mc, msc, m_div, dn_codes, dn_scales, float(dn_div))
    floor = 4 * float(np.abs(exp_out).mean())
    assert max_relative_error(got["persistent"][1], exp_out, floor) <= 1e-2
    assert (np.abs(got["persistent"][2] - exp_out) / np.maximum(np.abs(exp_out), floor)).max() <= 2e-3
    assert np.array_equal(oracle.f32_to_bf16(got["persistent"][2]), got["persistent"][1])
    for a, b in zip(got["persistent"], got["plain"]):
        assert np.array_equal(a, b)


def test_full_size_prefill_down_sampled_tiles(tk, ctx, oracle):
    """Configuration 4's down projection at full size (M = 2048, 5120 x 17408: unsplit 128-token
    tiles over 68 k-blocks): first, last and two inner weight tiles x first and last token tile
    against the W4A4 oracle, the activation quantiser bit for bit on those token tiles."""
    from tuiskollm_b200 import synth

    rows = 2048
    x = synth.torch_normal_bf16(13, 1, (rows, INTER), "cuda")
    dn_codes, dn_scales, dn_div = synth.torch_nvfp4_weights(13, 2, HIDDEN, INTER, "cuda")
    a_div = float(np.float32(448.0 * 6.0 / 6.0))
    codes, scales = act_planes(tk, rows, INTER)
    out = sentinel_plane((rows, HIDDEN), torch.int16)
    tk.Nvfp4DownOp(ctx).launch(None, rows, x, dn_codes, dn_scales, dn_div, out,
                               activation_codes=codes, activation_scales=scales,
                               input_global_divisor=a_div)
    torch.cuda.synchronize()
    groups = INTER // 16
    xb = _u16(x.view(torch.int16))
    got = _u16(out)
    for tt in (0, rows // 128 - 1):
        ts = slice(tt * 128, (tt + 1) * 128)
        oc, osc = oracle.nvfp4_quantize(xb[ts], a_div)
        assert np.array_equal(host(codes[ts]), oc)
        assert np.array_equal(host(scales[tt * 128 * groups:(tt + 1) * 128 * groups]), osc)
        for wt in (0, 13, 22, HIDDEN // 128 - 1):
            rs = slice(wt * 128, (wt + 1) * 128)
            exp = oracle.nvfp4_w4a4_dot(oc, osc, a_div, host(dn_codes[rs]),
                                        host(dn_scales[wt * 128 * groups:(wt + 1) * 128 * groups]), dn_div)
            assert max_relative_error(got[ts, rs], exp, 4 * float(np.abs(exp).mean())) <= 1e-2, (tt, wt)
    assert ctx.device_status() == 0


def test_rejected_launches(tk, ctx):
    codes, scales = act_planes(tk, 8, HIDDEN)
    x = torch.zeros((8, HIDDEN), dtype=torch.int16, device="cuda")
    w = torch.zeros((2 * INTER, HIDDEN // 2), dtype=torch.uint8, device="cuda")
    s = torch.zeros((2 * INTER * HIDDEN // 16,), dtype=torch.uint8, device="cuda")
    out = torch.zeros((8, INTER), dtype=torch.int16, device="cuda")
    op = tk.Nvfp4SwiGluOp(ctx)
    kw = dict(activation_codes=codes, activation_scales=scales, input_global_divisor=1.0)
    for bad in (0.0, -1.0, float("inf"), float("nan")):
        with pytest.raises(tk.GpuError) as info:
            op.launch(None, 1, x, w, s, bad, out, **kw)
        assert info.value.code == "gpu.launch"
        assert "weight scale divisor must be finite and positive" in str(info.value)
    with pytest.raises(tk.GpuError) as info:
        op.launch(None, 0, x, w, s, 1.0, out, **kw)
    assert "NVFP4 SwiGLU row count" in str(info.value)
    with pytest.raises(tk.GpuError) as info:
        op.launch(None, 1, x, w, s, 1.0, out, activation_codes=codes, activation_scales=scales,
                  input_global_divisor=0.0)
    assert "input scale divisor" in str(info.value)
    torch.cuda.synchronize()


@pytest.mark.parametrize("rows", [256, 300, 700])
def test_wide_tile_route_matches_plain_route_bit_for_bit(tk, rows, monkeypatch):
    """TK100_NVFP4_WIDE=2 runs prefill shapes on 256-token tiles (one CTA per SM, a second
    activation scale tile per stage): same K order into one fp32 accumulator as the 128-token
    tiles, so the same bits -- also with a ragged last tile whose second scale tile does not exist."""
    from tuiskollm_b200 import synth

    hidden, inter = 1024, 1536
    xb = synth.normal_bf16(19, rows, (rows, hidden))
    gu_codes, gu_scales, gu_div = synth.nvfp4_weights(19, 1, 2 * inter, hidden)
    dn_codes, dn_scales, dn_div = synth.nvfp4_weights(19, 2, hidden, inter)
    a_div, m_div = float(np.float32(448.0 * 6.0 / 5.0)), float(np.float32(448.0 * 6.0 / 8.0))
    got = {}
    for route, env in (("wide", "2"), ("plain", "0")):
        monkeypatch.setenv("TK100_NVFP4_WIDE", env)
        monkeypatch.setenv("TK100_NVFP4_WIDE_MIN_ROWS", "256")
        c = tk.Context(device=0, hidden=hidden, intermediate=inter, max_rows=2048)
        a_codes, a_scales = act_planes(tk, rows + 1, hidden)
        m_codes, m_scales = act_planes(tk, rows + 1, inter)
        mid = sentinel_plane((rows + 1, inter), torch.int16)
        out = sentinel_plane((rows + 1, hidden), torch.int16)
        tk.Nvfp4SwiGluOp(c).launch_quantize(None, rows, dev(xb.view(np.int16)), dev(gu_codes), dev(gu_scales),
                                            float(gu_div), mid, activation_codes=a_codes,
                                            activation_scales=a_scales, input_global_divisor=a_div,
                                            output_global_divisor=m_div, output_codes=m_codes,
                                            output_scales=m_scales)
        r_gu = c.last_kernel
        tk.Nvfp4DownOp(c).launch(None, rows, None, dev(dn_codes), dev(dn_scales), float(dn_div), out,
                                 activation_codes=m_codes, activation_scales=m_scales,
                                 input_global_divisor=m_div)
        r_dn = c.last_kernel
        torch.cuda.synchronize()
        assert c.device_status() == 0, route
        assert r_gu.startswith("nvfp4_gemm_kernel<256") == (route == "wide"), (route, r_gu)
        assert r_dn.startswith("nvfp4_gemm_kernel<256") == (route == "wide"), (route, r_dn)
        for pl in (mid, out):
            assert_inactive_untouched(pl, rows)
        got[route] = (_u16(mid)[:rows].copy(), _u16(out)[:rows].copy())
    assert np.array_equal(got["wide"][0], got["plain"][0]), "gate/up + SwiGLU"
    assert np.array_equal(got["wide"][1], got["plain"][1]), "down"
