"""GPU parity: FP8 QKV / GDN-input projections through the C ABI against the CPU oracle,
following qual/src/fp8_qkv.rs and qual/src/fp8_gdn_input.rs (bit-exact codes and scales,
outputs within tolerance, sentinels, eager == graph replay)."""
import os

import numpy as np
import pytest
import torch

import fixtures_ref as F
from gpu_util import (assert_inactive_untouched, check_close, dev, graph_replay, host,
                      max_relative_error, sentinel_plane)

pytestmark = pytest.mark.gpu


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
    def __init__(self, max_rows, hidden, out_rows):
        self.codes = sentinel_plane((max_rows, hidden), torch.uint8)
        self.scales = sentinel_plane((max_rows,), torch.float32)
        self.out = sentinel_plane((max_rows, out_rows), torch.int16)

    def reset(self):
        for p in (self.codes, self.scales, self.out):
            p.view(torch.uint8).fill_(0xA5)

    def check_inactive(self, rows):
        for p in (self.codes, self.scales, self.out):
            assert_inactive_untouched(p, rows)


def check_projection(oracle, xb, wc, ws, planes, rows, floor):
    oc, os_ = oracle.quantize_e4m3(xb[:rows])
    assert np.array_equal(host(planes.codes)[:rows], oc), "activation codes"
    assert np.array_equal(host(planes.scales)[:rows].view(np.uint32), os_.view(np.uint32)), "activation scales"
    exp = oracle.fp8_projection(oc, os_, wc, ws)
    got = _u16(planes.out)[:rows]
    # reference tolerance max(1/16, 1 %) (qual/src/fp8_qkv.rs:289) ...
    check_close(got, exp, 1 / 16, 0.01, "projection")
    # ... and the tighter benchmark contract: max relative error 1e-2
    rel = max_relative_error(got, exp, floor)
    assert rel <= 1e-2, rel
    planes.check_inactive(rows)
    return rel


@pytest.mark.parametrize("rows", [1, 2, 3, 4, 5, 6, 7, 8, 16])
def test_reference_fixture_qkv_exact_routes(tk, ctx, oracle, rows):
    """qual/src/fp8_qkv.rs: structured fixture, N = 14336 (the reference's QKV rows), every
    exact route 1..8 and 16; closed-form expectation represented_sum * w * a_scale * w_scale."""
    hidden, out_rows, max_rows = 5120, 14336, 16
    xb = F.fp8_input(max_rows, hidden)
    wc, ws = F.fp8_weights(out_rows, hidden)
    op = tk.FullAttentionQkvOp(ctx, out_rows)
    planes = Planes(max_rows, hidden, out_rows)
    x, w, s = dev(xb.view(np.int16)), dev(wc), dev(ws.view(np.int16))
    launch = lambda: op.launch(None, rows, x, planes.codes, planes.scales, w, s, planes.out)
    launch()
    torch.cuda.synchronize()
    got = _u16(planes.out)
    for t in range(rows):
        c, sc, rsum = oracle.quantize_e4m3_token(xb[t], search=True)
        assert np.array_equal(host(planes.codes)[t], c)
        assert host(planes.scales)[t] == sc
        check_close(got[t], F.fp8_expected(rsum, sc, out_rows), 1 / 16, 0.01, f"token {t}")
    planes.check_inactive(rows)
    eager = [host(p.view(torch.uint8)).copy() for p in (planes.codes, planes.scales, planes.out)]
    g = graph_replay(launch)
    planes.reset()
    g.replay()
    g.replay()
    torch.cuda.synchronize()
    for e, p in zip(eager, (planes.codes, planes.scales, planes.out)):
        assert np.array_equal(host(p.view(torch.uint8)), e)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("kind,out_rows,rows", [
    ("qkv", 8192, 1), ("qkv", 8192, 8), ("gdn", 12288, 1), ("gdn", 12288, 8), ("gdn", 12288, 32),
    ("gdn", 16384, 4), ("qkv", 8192, 100), ("qkv", 8192, 256), ("gdn", 12288, 300),
])
def test_synthetic_configs_match_oracle(tk, ctx, oracle, kind, out_rows, rows):
    """BASELINE shapes with ~N(0,1) activations and ~N(0,0.02) weights; ragged token counts
    exercise the zero-filled tile tails."""
    from tuiskollm_b200 import synth

    hidden = 5120
    xb = synth.normal_bf16(42, 10 + rows, (rows, hidden))
    wc, ws = synth.fp8_weights(42, out_rows, out_rows, hidden)
    op = (tk.FullAttentionQkvOp if kind == "qkv" else tk.GdnInputProjectionOp)(ctx, out_rows)
    planes = Planes(rows + 2, hidden, out_rows)
    op.launch(None, rows, dev(xb.view(np.int16)), planes.codes, planes.scales, dev(wc),
              dev(ws.view(np.int16)), planes.out)
    torch.cuda.synchronize()
    # typical |output| is ~1.4 (sqrt(5120) * 0.02); relative error is judged above 0.25
    check_projection(oracle, xb, wc, ws, planes, rows, floor=0.25)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("out_rows,rows", [(512, 512), (768, 700), (256, 1030), (5120, 600)])
def test_pair_route_matches_oracle_and_one_cta_route(tk, oracle, out_rows, rows, monkeypatch):
    """Prefill token counts take the CTA-pair kernel (cta_group::2, 256-row x 256-token pair
    tiles); ragged token counts exercise the zero-filled tails.  Against the oracle, and against
    the one-CTA kernel, which splits K at these small sizes: the two may differ by one BF16
    rounding step, no more."""
    from tuiskollm_b200 import synth

    hidden = 1024
    xb = synth.normal_bf16(43, rows, (rows, hidden))
    wc, ws = synth.fp8_weights(43, out_rows, out_rows, hidden)
    outs = {}
    for route, env in (("pair", "2"), ("single", "0")):  # "2": also for launches of few CTAs
        monkeypatch.setenv("TK100_FP8_PAIR", env)
        ctx = tk.Context(device=0, hidden=hidden, max_rows=2048)
        planes = Planes(rows + 2, hidden, out_rows)
        launches = ctx.launch_count
        tk.GdnInputProjectionOp(ctx, out_rows).launch(
            None, rows, dev(xb.view(np.int16)), planes.codes, planes.scales, dev(wc),
            dev(ws.view(np.int16)), planes.out)
        torch.cuda.synchronize()
        assert ctx.launch_count - launches == 2, route  # quantiser + one projection kernel
        check_projection(oracle, xb, wc, ws, planes, rows, floor=0.25 * (hidden / 5120) ** 0.5)
        assert ctx.device_status() == 0, route
        outs[route] = _u16(planes.out)[:rows].copy()
    a = (outs["pair"].astype(np.uint32) << 16).view(np.float32)
    b = (outs["single"].astype(np.uint32) << 16).view(np.float32)
    assert np.all(np.abs(a - b) <= np.maximum(np.abs(a), np.abs(b)) * 2.0 ** -7 + 1e-4)


@pytest.mark.parametrize("out_rows,rows", [(8192, 512), (8192, 2048), (12288, 512), (12288, 2048)])
def test_benchmarked_prefill_shapes_sampled_tiles(tk, ctx, oracle, out_rows, rows):
    """The prefill shapes the benchmark times (K = 5120, M = 512 / 2048, N = 8192 / 12288) run on
    the CTA-pair kernel; the f64 oracle cannot do the whole product in seconds, so whole
    128 x 128 tiles are sampled -- first, last and two inner weight tiles x first, an inner and
    the last token tile -- after the activation codes and scales of ALL rows are checked bit for
    bit."""
    from tuiskollm_b200 import synth

    hidden = 5120
    x = synth.torch_normal_bf16(44, rows, (rows, hidden), "cuda")
    w, s = synth.torch_fp8_weights(44, out_rows, out_rows, hidden, "cuda")
    planes = Planes(rows + 1, hidden, out_rows)
    tk.GdnInputProjectionOp(ctx, out_rows).launch(None, rows, x, planes.codes, planes.scales, w, s,
                                                  planes.out)
    torch.cuda.synchronize()
    assert ctx.last_kernel.startswith(("fp8_pair_kernel", "fp8_pair_persist_kernel")), ctx.last_kernel
    xb = _u16(x)
    oc, os_ = oracle.quantize_e4m3(xb)
    assert np.array_equal(host(planes.codes)[:rows], oc)
    assert np.array_equal(host(planes.scales)[:rows].view(np.uint32), os_.view(np.uint32))
    got = _u16(planes.out)
    n_tiles, m_tiles = out_rows // 128, rows // 128
    for tt in sorted({0, m_tiles // 2 + 1, m_tiles - 1}):
        ts = slice(tt * 128, (tt + 1) * 128)
        for wt in sorted({0, 1, n_tiles // 2, n_tiles - 1}):
            rs = slice(wt * 128, (wt + 1) * 128)
            exp = oracle.fp8_projection(oc[ts], os_[ts], host(w[rs]), _u16(s[rs]))
            check_close(got[ts, rs], exp, 1 / 16, 0.01, f"tile ({tt}, {wt})")
            assert max_relative_error(got[ts, rs], exp, 0.25) <= 1e-2
    planes.check_inactive(rows)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("splits", [1, 2, 3, 8])
@pytest.mark.parametrize("block_tok", [0, 64])
def test_split_k_is_exact_and_deterministic(tk, oracle, splits, block_tok):
    """Forced K splits: same values within tolerance, and bit-identical from launch to launch
    and under graph replay (fixed-order reduction)."""
    from tuiskollm_b200 import synth

    os.environ["TK100_SPLITS"] = str(splits)
    os.environ["TK100_BLOCK_TOK"] = str(block_tok)
    try:
        ctx = tk.Context(device=0)
    finally:
        del os.environ["TK100_SPLITS"], os.environ["TK100_BLOCK_TOK"]
    hidden, out_rows, rows = 5120, 1040, 5  # 1040 = 8 tiles + a 16-row tail
    xb = synth.normal_bf16(3, 1, (rows, hidden))
    wc, ws = synth.fp8_weights(3, 2, out_rows, hidden)
    op = tk.GdnInputProjectionOp(ctx, out_rows)
    planes = Planes(rows + 1, hidden, out_rows)
    x, w, s = dev(xb.view(np.int16)), dev(wc), dev(ws.view(np.int16))
    launch = lambda: op.launch(None, rows, x, planes.codes, planes.scales, w, s, planes.out)
    launch()
    torch.cuda.synchronize()
    check_projection(oracle, xb, wc, ws, planes, rows, floor=0.25)
    first = host(planes.out.view(torch.uint8)).copy()
    for _ in range(3):
        planes.reset()
        launch()
        torch.cuda.synchronize()
        assert np.array_equal(host(planes.out.view(torch.uint8)), first)
    g = graph_replay(launch)
    planes.reset()
    g.replay()
    g.replay()
    torch.cuda.synchronize()
    assert np.array_equal(host(planes.out.view(torch.uint8)), first)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("rows", [1, 8, 16, 32])
def test_split_k_reduction_routes_agree_bit_for_bit(tk, oracle, rows, monkeypatch):
    """The three split-K reductions -- partial tiles pushed into a leader CTA's shared memory
    (TK100_CLUSTER=2, an experiment switch), the symmetric two-barrier cluster reduction (1, what
    the default takes) and fp32 tiles in global scratch behind a ticket (0) -- add the same partials in the same
    order: every output bit must agree, at the decode shape of the QKV plane (N = 8192: six splits),
    eagerly and under graph replay."""
    from tuiskollm_b200 import synth

    hidden, out_rows = 5120, 8192
    xb = synth.normal_bf16(45, rows, (rows, hidden))
    w, s = synth.torch_fp8_weights(45, 1, out_rows, hidden, "cuda")
    x = dev(xb.view(np.int16))
    outs, routes = {}, {}
    for mode in ("2", "1", "0"):
        monkeypatch.setenv("TK100_CLUSTER", mode)
        c = tk.Context(device=0)
        planes = Planes(rows + 1, hidden, out_rows)
        op = tk.FullAttentionQkvOp(c, out_rows)
        launch = lambda: op.launch(None, rows, x, planes.codes, planes.scales, w, s, planes.out)
        launch()
        torch.cuda.synchronize()
        routes[mode] = c.last_kernel
        eager = _u16(planes.out).copy()
        g = graph_replay(launch)
        planes.reset()
        g.replay()
        g.replay()
        torch.cuda.synchronize()
        assert np.array_equal(_u16(planes.out), eager), mode
        planes.check_inactive(rows)
        assert c.device_status() == 0, mode
        outs[mode] = eager[:rows]
    assert "splits=6" in routes["2"], routes
    assert ("cluster-leader" in routes["2"]) == (rows <= 16), routes  # 32 rows x 5 tiles exceed the ring
    monkeypatch.delenv("TK100_CLUSTER")
    c = tk.Context(device=0)
    planes = Planes(rows + 1, hidden, out_rows)
    tk.FullAttentionQkvOp(c, out_rows).launch(None, rows, x, planes.codes, planes.scales, w, s, planes.out)
    torch.cuda.synchronize()
    assert c.last_kernel == routes["1"], (c.last_kernel, routes)
    assert np.array_equal(_u16(planes.out)[:rows], outs["1"])
    assert "cluster-leader" not in routes["1"] and "cluster" in routes["1"] and "cluster" not in routes["0"]
    assert np.array_equal(outs["2"], outs["1"]) and np.array_equal(outs["2"], outs["0"])
    oc, os_ = oracle.quantize_e4m3(xb)
    sample = np.r_[0:256, 4000:4128, out_rows - 128:out_rows]
    exp = oracle.fp8_projection(oc, os_, host(w)[sample], _u16(s)[sample])
    assert max_relative_error(outs["2"][:, sample], exp, 0.25) <= 1e-2


def test_fused_producer_feeds_projection(tk, ctx, oracle):
    """Decode slice of the first benchmark configuration: residual add + RMSNorm + quantise in
    one kernel, then the QKV projection reads the codes it wrote (input == NULL)."""
    from tuiskollm_b200 import synth

    hidden, out_rows, rows = 5120, 8192, 1
    xb = synth.normal_bf16(1, 1, (rows, hidden))
    bb = synth.normal_bf16(1, 2, (rows, hidden))
    nb = synth.normal_bf16(1, 3, (hidden,), std=0.1)
    wc, ws = synth.fp8_weights(1, 4, out_rows, hidden)
    planes = Planes(rows + 1, hidden, out_rows)
    res = sentinel_plane((rows + 1, hidden), torch.int16)
    norm = sentinel_plane((rows + 1, hidden), torch.int16)
    tk.ResidualNormOp(ctx).launch_quantize(None, rows, dev(xb.view(np.int16)), dev(bb.view(np.int16)),
                                           dev(nb.view(np.int16)), res, norm, planes.codes, planes.scales)
    tk.FullAttentionQkvOp(ctx, out_rows).launch(None, rows, None, planes.codes, planes.scales,
                                                dev(wc), dev(ws.view(np.int16)), planes.out)
    torch.cuda.synchronize()
    res_o, _ = oracle.residual_rms_norm(xb, bb, nb, 1e-6)
    assert np.array_equal(_u16(res)[:rows], res_o)
    check_projection(oracle, _u16(norm)[:rows], wc, ws, planes, rows, floor=0.25)


def test_generic_reduction_lengths(tk, ctx, oracle):
    """K = 6144 (GDN output plane) and K = 17408 (dense-FP8 down plane)."""
    from tuiskollm_b200 import synth

    for k, out_rows, rows in ((6144, 5120, 3), (17408, 640, 2), (128, 16, 1)):
        xb = synth.normal_bf16(8, k, (rows, k))
        wc, ws = synth.fp8_weights(8, k + 1, out_rows, k)
        planes = Planes(rows + 1, k, out_rows)
        tk.Fp8ProjectionOp(ctx).launch(None, rows, out_rows, k, dev(xb.view(np.int16)), planes.codes,
                                       planes.scales, dev(wc), dev(ws.view(np.int16)), planes.out)
        torch.cuda.synchronize()
        check_projection(oracle, xb, wc, ws, planes, rows, floor=0.25 * (k / 5120) ** 0.5)
    assert ctx.device_status() == 0


def test_rejected_launches(tk, ctx):
    hidden, out_rows = 5120, 256
    x = torch.zeros((4, hidden), dtype=torch.int16, device="cuda")
    codes = torch.zeros((4, hidden), dtype=torch.uint8, device="cuda")
    scales = torch.zeros((4,), dtype=torch.float32, device="cuda")
    w = torch.zeros((out_rows, hidden), dtype=torch.uint8, device="cuda")
    ws = torch.zeros((out_rows,), dtype=torch.int16, device="cuda")
    out = torch.zeros((4, out_rows), dtype=torch.int16, device="cuda")
    op = tk.FullAttentionQkvOp(ctx, out_rows)
    for rows in (0, 2049):
        with pytest.raises(tk.GpuError) as info:
            op.launch(None, rows, x, codes, scales, w, ws, out)
        assert info.value.code == "gpu.launch" and "FP8 QKV row count" in str(info.value)
    with pytest.raises(tk.GpuError) as info:
        op.launch(None, 1, x, codes, scales, w.data_ptr() + 16, ws, out)
    assert "128-byte aligned" in str(info.value)
    with pytest.raises(tk.GpuError) as info:
        tk.FullAttentionQkvOp(ctx, 250).launch(None, 1, x, codes, scales, w, ws, out)
    assert "multiple of 16" in str(info.value)
    with pytest.raises(tk.GpuError) as info:
        tk.Fp8ProjectionOp(ctx).launch(None, 1, out_rows, 5000, x, codes, scales, w, ws, out)
    assert "multiple of 128" in str(info.value)
    torch.cuda.synchronize()


def test_registered_plane_is_not_encoded_again(tk, ctx, oracle):
    """A plane declared with tk100_register_plane gets its tensor map at load time: its launches add
    no weight map to the lazy cache (only the activation plane's), and the result is the one an
    undeclared plane gives."""
    import tuiskollm_b200.synth as synth
    rows, n, k = 3, 1024, 5120
    w, s = synth.fp8_weights(7, 61, n, k)
    x = synth.normal_bf16(7, 62, (rows, k))
    wd, sd, xd = dev(w), dev(s.view(np.int16)), dev(x.view(np.int16))
    wd2 = wd.clone()
    codes = torch.empty((rows, k), dtype=torch.uint8, device="cuda")
    scales = torch.empty((rows,), dtype=torch.float32, device="cuda")
    out_a = torch.empty((rows, n), dtype=torch.int16, device="cuda")
    out_b = torch.empty_like(out_a)
    op = tk.FullAttentionQkvOp(ctx, n)
    registered0, _ = ctx.tensor_map_counts
    ctx.register_plane(wd)
    registered1, transient1 = ctx.tensor_map_counts
    assert registered1 == registered0 + 1
    op.launch(None, rows, xd, codes, scales, wd, sd, out_a)
    _, transient2 = ctx.tensor_map_counts
    assert transient2 <= transient1 + 1            # the activation plane only
    op.launch(None, rows, xd, codes, scales, wd2, sd, out_b)   # undeclared copy of the same plane
    _, transient3 = ctx.tensor_map_counts
    assert transient3 == transient2 + 1            # its weight map is encoded on first use
    torch.cuda.synchronize()
    assert torch.equal(out_a, out_b)
    with pytest.raises(tk.GpuError, match="register plane"):
        ctx.register_plane(wd.view(-1)[1:1 + 1024 * 64].view(1024, 64))   # not 128-byte aligned


@pytest.mark.parametrize("out_rows,rows", [(1024, 700), (4096, 1300), (4096, 2600)])
def test_persistent_pair_route_matches_pair_route_bit_for_bit(tk, oracle, out_rows, rows, monkeypatch):
    """TK100_FP8_PERSIST: resident CTA pairs walk the pair tiles with two TMEM accumulators in
    rotation.  (4096, 1300) gives some pairs a second tile, (4096, 2600) a third (the first
    accumulator is reused, so the issuer has to wait for its epilogue).  Same K order into one fp32
    accumulator as the one-tile-per-pair kernel: the same bits, ragged token tails included; the
    first case is also checked against the oracle."""
    from tuiskollm_b200 import synth

    hidden = 1024
    xb = synth.normal_bf16(47, rows, (rows, hidden))
    wc, ws = synth.fp8_weights(47, out_rows, out_rows, hidden)
    outs = {}
    for route, env in (("persistent", "2"), ("pair", "0")):
        monkeypatch.setenv("TK100_FP8_PAIR", "2")
        monkeypatch.setenv("TK100_FP8_PERSIST", env)
        c = tk.Context(device=0, hidden=hidden, max_rows=4096)
        planes = Planes(rows + 2, hidden, out_rows)
        tk.GdnInputProjectionOp(c, out_rows).launch(
            None, rows, dev(xb.view(np.int16)), planes.codes, planes.scales, dev(wc),
            dev(ws.view(np.int16)), planes.out)
        torch.cuda.synchronize()
        assert c.device_status() == 0, route
        assert c.last_kernel.startswith("fp8_pair_persist_kernel") == (route == "persistent"), c.last_kernel
        planes.check_inactive(rows)
        if out_rows == 1024:
            check_projection(oracle, xb, wc, ws, planes, rows, floor=0.25 * (hidden / 5120) ** 0.5)
        outs[route] = _u16(planes.out)[:rows].copy()
    assert np.array_equal(outs["persistent"], outs["pair"])


@pytest.mark.parametrize("out_rows,hidden,rows", [(1024, 1024, 256), (1024, 2048, 700), (4096, 1024, 1300),
                                                  (5120, 6144, 256), (8192, 5120, 300)])
def test_stream_k_pair_route(tk, oracle, out_rows, hidden, rows, monkeypatch):
    """TK100_FP8_STREAMK=1: the resident pairs share the launch's tiles x K steps evenly; a tile
    whose K range is cut meets in fp32 scratch under a ticket and is summed in K order by whichever
    CTA arrives last.  The result is the oracle's within the projection tolerance (a split sum is
    not the unsplit sum's bits, so the pair route is compared within one BF16 step, and tiles that
    no range cuts bit for bit by construction), ragged token tails included; launches repeat bit
    for bit, eagerly and as graph replays, and scratch counters re-arm (three launches)."""
    from tuiskollm_b200 import synth

    xb = synth.normal_bf16(53, rows, (rows, hidden))
    wc, ws = synth.fp8_weights(53, out_rows + hidden, out_rows, hidden)
    outs = {}
    for route, env in (("stream_k", "1"), ("pair", "0")):
        monkeypatch.setenv("TK100_FP8_PAIR", "2")
        monkeypatch.setenv("TK100_FP8_STREAMK", env)
        c = tk.Context(device=0, hidden=hidden, max_rows=4096)
        planes = Planes(rows + 2, hidden, out_rows)
        op = tk.GdnInputProjectionOp(c, out_rows)
        x, w, s = dev(xb.view(np.int16)), dev(wc), dev(ws.view(np.int16))
        launch = lambda: op.launch(None, rows, x, planes.codes, planes.scales, w, s, planes.out)
        launch()
        torch.cuda.synchronize()
        assert c.device_status() == 0, route
        assert c.last_kernel.startswith("fp8_pair_stream_k_kernel") == (route == "stream_k"), c.last_kernel
        planes.check_inactive(rows)
        first = _u16(planes.out)[:rows].copy()
        if route == "stream_k":
            if out_rows * rows <= 1024 * 700:
                check_projection(oracle, xb, wc, ws, planes, rows, floor=0.25 * (hidden / 5120) ** 0.5)
            for _ in range(2):
                planes.out.fill_(0x5A5A)
                launch()
                torch.cuda.synchronize()
                assert np.array_equal(_u16(planes.out)[:rows], first)
            g = graph_replay(launch)
            planes.out.fill_(0x5A5A)
            g.replay()
            g.replay()
            torch.cuda.synchronize()
            assert np.array_equal(_u16(planes.out)[:rows], first)
            assert c.device_status() == 0
        outs[route] = first
    a = oracle.bf16_to_f32(outs["stream_k"].reshape(-1)).astype(np.float64)
    b = oracle.bf16_to_f32(outs["pair"].reshape(-1)).astype(np.float64)
    # one BF16 step of the larger magnitude, plus the cancellation floor of a split fp32 sum
    assert np.all(np.abs(a - b) <= np.maximum(np.abs(a), np.abs(b)) * 2.0 ** -7 + 1e-3), np.abs(a - b).max()
    assert (outs["stream_k"] == outs["pair"]).mean() > 0.9
