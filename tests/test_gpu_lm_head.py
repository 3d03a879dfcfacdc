"""GPU parity: FP8 LM head with the fused greedy argmax (qual/src/fp8_lm_head.rs for the
projection, tuisko-engine/src/sampling.rs:162-173 for the selection rule), on one GPU and
as vocabulary shards merged with the first-maximum rule."""
import numpy as np
import pytest
import torch

import fixtures_ref as F
from gpu_util import (assert_inactive_untouched, check_close, dev, graph_replay, host,
                      max_relative_error, sentinel_plane)

pytestmark = pytest.mark.gpu

PAIR = np.dtype([("value", np.float32), ("index", np.int32)])


@pytest.fixture(scope="module")
def tk():
    import tuiskollm_b200 as tk
    return tk


@pytest.fixture(scope="module")
def ctx(tk):
    return tk.Context(device=0)


def _u16(t):
    return host(t.view(torch.int16)).view(np.uint16)


def lm_head(tk, ctx, x, w, s, rows, vocab_rows, vocab_offset, max_rows, hidden, f32=True):
    op = tk.LmHeadOp(ctx, vocab_rows, vocab_offset)
    p = dict(codes=sentinel_plane((max_rows, hidden), torch.uint8),
             scales=sentinel_plane((max_rows,), torch.float32),
             out=sentinel_plane((max_rows, vocab_rows), torch.int16),
             f32=sentinel_plane((max_rows, vocab_rows), torch.float32) if f32 else None,
             pairs=sentinel_plane((max_rows, 2), torch.int32))
    scratch = torch.zeros((max_rows,), dtype=torch.int64, device="cuda")
    launch = lambda: op.launch(None, rows, x, p["codes"], p["scales"], w, s, p["out"], p["f32"],
                               scratch, p["pairs"])
    return op, p, scratch, launch


def pairs_of(t, rows):
    return host(t)[:rows].copy().view(PAIR).reshape(rows)


@pytest.mark.parametrize("rows", [1, 4, 32])
def test_lm_head_matches_oracle_and_greedy_rule(tk, ctx, oracle, rows):
    from tuiskollm_b200 import synth

    hidden, vocab = 5120, 4096 + 64  # 32 full tiles + a 64-row tail tile (the 8-way shard shape)
    xb = synth.normal_bf16(77, rows, (rows, hidden))
    wc, ws = synth.fp8_weights(77, 100, vocab, hidden)
    x, w, s = dev(xb.view(np.int16)), dev(wc), dev(ws.view(np.int16))
    op, p, scratch, launch = lm_head(tk, ctx, x, w, s, rows, vocab, 0, rows + 1, hidden)
    launch()
    torch.cuda.synchronize()
    oc, os_ = oracle.quantize_e4m3(xb)
    assert np.array_equal(host(p["codes"])[:rows], oc)
    assert np.array_equal(host(p["scales"])[:rows].view(np.uint32), os_.view(np.uint32))
    exp = oracle.fp8_projection(oc, os_, wc, ws)
    logits = _u16(p["out"])[:rows]
    check_close(logits, exp, 1 / 16, 0.01, "BF16 logits")
    assert max_relative_error(logits, exp, 0.25) <= 1e-2
    f32 = host(p["f32"])[:rows]
    assert np.abs(f32 - exp).max() <= 1e-3 * max(1.0, np.abs(exp).max())
    # the BF16 plane is the rounding of the fp32 plane
    assert np.array_equal(oracle.f32_to_bf16(f32), logits)
    got = pairs_of(p["pairs"], rows)
    for t in range(rows):
        g = oracle.greedy_index(logits[t])
        assert got["index"][t] == g
        assert got["value"][t] == oracle.bf16_to_f32(logits[t, g:g + 1])[0]
        # identical to the f64 oracle's choice wherever its top-2 gap exceeds the tolerance
        order = np.argsort(exp[t])
        top, second = exp[t, order[-1]], exp[t, order[-2]]
        if top - second > 1e-2 * abs(top):
            assert g == order[-1]
    for name in ("codes", "scales", "out", "f32", "pairs"):
        assert_inactive_untouched(p[name], rows)
    assert int(scratch.abs().sum()) == 0, "argmax scratch must be left zero"
    # replays are idempotent and bit-identical
    eager = {k: host(v.view(torch.uint8)).copy() for k, v in p.items()}
    g = graph_replay(launch)
    for v in p.values():
        v.view(torch.uint8).fill_(0xA5)
    g.replay()
    g.replay()
    torch.cuda.synchronize()
    for k, v in p.items():
        assert np.array_equal(host(v.view(torch.uint8)), eager[k]), k
    assert ctx.device_status() == 0


@pytest.mark.parametrize("rows", [1, 3, 4, 5])
def test_fused_quantiser_and_tail_equal_the_separate_launches(tk, oracle, rows, monkeypatch):
    """With TK100_FUSED_QUANT=1 the projection kernel quantises up to 4 hidden rows in its prologue
    (off by default), and by default its last CTA unpacks the maxima; TK100_FUSED_QUANT=0 /
    TK100_FUSED_TAIL=0 keep the quantiser and the finalizer as launches of their own.  Every plane must come out bit-identical on both routes,
    eagerly and as graph replays, with and without split K (the 4160-row plane is unsplit with the
    longer ring, the 1040-row plane splits K eight ways)."""
    from tuiskollm_b200 import synth

    hidden = 5120
    for vocab in (4096 + 64, 1040):
        xb = synth.normal_bf16(78, rows, (rows, hidden))
        wc, ws = synth.fp8_weights(78, 100 + vocab, vocab, hidden)
        x, w, s = dev(xb.view(np.int16)), dev(wc), dev(ws.view(np.int16))
        planes = {}
        for route, (fq, ft) in (("fused", ("1", "1")), ("separate", ("0", "0"))):
            monkeypatch.setenv("TK100_FUSED_QUANT", fq)
            monkeypatch.setenv("TK100_FUSED_TAIL", ft)
            c = tk.Context(device=0)
            launches = c.launch_count
            op, p, scratch, launch = lm_head(tk, c, x, w, s, rows, vocab, 0, rows + 1, hidden)
            launch()
            torch.cuda.synchronize()
            expect_launches = 1 if (route == "fused" and rows <= 4) else (2 if route == "fused" else 3)
            assert c.launch_count - launches == expect_launches, (route, rows)
            for name in ("codes", "scales", "out", "f32", "pairs"):
                assert_inactive_untouched(p[name], rows)
            assert int(scratch.abs().sum()) == 0, "argmax scratch must be left zero"
            eager = {k: host(v.view(torch.uint8)).copy() for k, v in p.items()}
            g = graph_replay(launch)
            for v in p.values():
                v.view(torch.uint8).fill_(0xA5)
            g.replay()
            g.replay()
            torch.cuda.synchronize()
            for k, v in p.items():
                assert np.array_equal(host(v.view(torch.uint8)), eager[k]), (route, k)
            assert c.device_status() == 0
            planes[route] = eager
        for k in planes["fused"]:
            assert np.array_equal(planes["fused"][k], planes["separate"][k]), (vocab, k)
        oc, os_ = oracle.quantize_e4m3(xb)
        assert np.array_equal(planes["fused"]["codes"][:rows], oc)
        assert np.array_equal(planes["fused"]["scales"][: 4 * rows].view(np.uint32), os_.view(np.uint32))


@pytest.mark.parametrize("vocab", [112, 640, 1040, 4096 + 64])
def test_spread_maxima_equal_direct_keys(tk, oracle, vocab, monkeypatch):
    """Up to 32 tokens the CTAs collect their maxima in per-group keys and draw per-group tickets
    (TK100_ARGMAX_SPREAD=0: straight into the caller's keys).  Same pairs and planes on both
    routes, launch after launch on one context (keys and tickets re-arm themselves), for fewer
    tiles than groups (112 and 640 rows), split K (1040) and uneven groups (4160), at token counts
    that take the per-token and the batched maxima of 16- and 32-token tiles; 33 tokens are past
    the spread plane and use the direct keys on both."""
    from tuiskollm_b200 import synth

    hidden = 5120
    wc, ws = synth.fp8_weights(81, 300 + vocab, vocab, hidden)
    w, s = dev(wc), dev(ws.view(np.int16))
    results = {}
    for spread in ("1", "0"):
        monkeypatch.setenv("TK100_ARGMAX_SPREAD", spread)
        c = tk.Context(device=0)
        for rows in (1, 3, 4, 16, 17, 32, 33, 2):
            xb = synth.normal_bf16(81, rows, (rows, hidden))
            x = dev(xb.view(np.int16))
            op, p, scratch, launch = lm_head(tk, c, x, w, s, rows, vocab, 0, rows + 1, hidden)
            launch()
            launch()
            torch.cuda.synchronize()
            assert c.device_status() == 0
            assert int(scratch.abs().sum()) == 0, "argmax scratch must be left zero"
            got = pairs_of(p["pairs"], rows)
            logits = _u16(p["out"])[:rows]
            for t in range(rows):
                assert got["index"][t] == oracle.greedy_index(logits[t]), (spread, rows, t)
            assert_inactive_untouched(p["pairs"], rows)
            results[(spread, rows)] = {k: host(v.view(torch.uint8)).copy() for k, v in p.items()}
    for (spread, rows), planes in results.items():
        if spread == "1":
            for k, v in planes.items():
                assert np.array_equal(v, results[("0", rows)][k]), (rows, k)


def test_sharded_entry_on_one_rank_equals_the_plain_entry(tk, ctx, oracle):
    """tk100_fp8_lm_head_sharded with world = 1 (its own buffer list empty) gives the pairs of
    tk100_fp8_lm_head, step after step, and leaves the scratch zero."""
    from tuiskollm_b200 import synth

    hidden, vocab, rows = 5120, 2048 + 64, 2
    wc, ws = synth.fp8_weights(79, 2, vocab, hidden)
    w, s = dev(wc), dev(ws.view(np.int16))
    for step in range(3):
        xb = synth.normal_bf16(79, 10 + step, (rows, hidden))
        x = dev(xb.view(np.int16))
        op, p, scratch, launch = lm_head(tk, ctx, x, w, s, rows, vocab, 0, rows, hidden, f32=False)
        launch()
        merged = sentinel_plane((rows, 2), torch.int32)
        op.launch_sharded(None, rows, x, p["codes"], p["scales"], w, s, p["out"], None, scratch, 1, 0,
                          None, merged)
        torch.cuda.synchronize()
        a, b = pairs_of(merged, rows), pairs_of(p["pairs"], rows)
        assert np.array_equal(a["index"], b["index"]) and np.array_equal(a["value"], b["value"])
        assert a["index"][0] == oracle.greedy_index(_u16(p["out"])[0])
        assert int(scratch.abs().sum()) == 0
    assert ctx.device_status() == 0


def test_first_maximum_wins_and_total_order(tk, ctx, oracle):
    """Duplicate weight rows give equal logits: the lowest index must win, across tiles and
    inside one tile (tuisko-engine/src/sampling.rs:313-335)."""
    from tuiskollm_b200 import synth

    hidden, vocab, rows = 5120, 1024, 2
    xb = synth.normal_bf16(5, 1, (rows, hidden))
    wc, ws = synth.fp8_weights(5, 2, vocab, hidden)
    oc, os_ = oracle.quantize_e4m3(xb)
    exp = oracle.fp8_projection(oc, os_, wc, ws)
    best = int(np.argmax(exp[0]))
    for dup in (best + 1 if best + 1 < vocab else best - 1, (best + 517) % vocab, (best + 130) % vocab):
        wc2, ws2 = wc.copy(), ws.copy()
        wc2[dup], ws2[dup] = wc[best], ws[best]
        op, p, scratch, launch = lm_head(tk, ctx, dev(xb.view(np.int16)), dev(wc2), dev(ws2.view(np.int16)),
                                         rows, vocab, 0, rows, hidden, f32=False)
        launch()
        torch.cuda.synchronize()
        got = pairs_of(p["pairs"], rows)
        logits = _u16(p["out"])
        assert logits[0, dup] == logits[0, best]
        assert got["index"][0] == min(best, dup) == oracle.greedy_index(logits[0])
        assert got["index"][1] == oracle.greedy_index(logits[1])
    # all logits zero: +0 beats -0, then the first index
    z = np.zeros((rows, hidden), np.uint16)
    op, p, scratch, launch = lm_head(tk, ctx, dev(z.view(np.int16)), dev(wc), dev(ws.view(np.int16)),
                                     rows, vocab, 0, rows, hidden, f32=False)
    launch()
    torch.cuda.synchronize()
    logits = _u16(p["out"])
    got = pairs_of(p["pairs"], rows)
    assert got["index"][0] == oracle.greedy_index(logits[0])


def test_non_finite_logit_is_reported(tk, ctx, oracle):
    """A non-finite logit is an error for the host sampler (sampling.rs:233-242, NaN at token
    37 in its test); the device reports it through the status word."""
    from tuiskollm_b200 import synth, _lib

    hidden, vocab, rows = 5120, 256, 1
    xb = synth.normal_bf16(6, 1, (rows, hidden))
    wc, ws = synth.fp8_weights(6, 2, vocab, hidden)
    ws = ws.copy()
    ws[37] = 0x7F80  # +inf row scale
    op, p, scratch, launch = lm_head(tk, ctx, dev(xb.view(np.int16)), dev(wc), dev(ws.view(np.int16)),
                                     rows, vocab, 0, rows, hidden, f32=False)
    assert ctx.device_status() == 0
    launch()
    assert ctx.device_status() & _lib.DEVICE_NONFINITE_LOGIT
    assert ctx.device_status() == 0  # reading clears it
    with pytest.raises(ValueError, match="token 37"):
        oracle.greedy_index(_u16(p["out"])[0])


@pytest.mark.parametrize("shards", [2, 4, 8])
def test_vocab_shards_merge_to_the_single_gpu_answer(tk, ctx, oracle, shards):
    """Each shard is launched as its own LM head with a vocabulary offset; the gathered
    (max, index) pairs reduce to exactly the unsharded selection."""
    from tuiskollm_b200 import synth

    hidden, rows = 5120, 4
    vocab = 8 * (128 * 3 + 64)  # per-shard row counts that are not multiples of 128
    xb = synth.normal_bf16(9, 1, (rows, hidden))
    wc, ws = synth.fp8_weights(9, 2, vocab, hidden)
    # make one token's maximum a cross-shard tie
    oc, os_ = oracle.quantize_e4m3(xb)
    exp = oracle.fp8_projection(oc, os_, wc, ws)
    b = int(np.argmax(exp[1]))
    other = (b + vocab // 2) % vocab
    wc[other], ws[other] = wc[b], ws[b]
    x, w, s = dev(xb.view(np.int16)), dev(wc), dev(ws.view(np.int16))
    _, full, _, launch = lm_head(tk, ctx, x, w, s, rows, vocab, 0, rows, hidden, f32=False)
    launch()
    per = vocab // shards
    gathered = torch.zeros((shards, rows, 2), dtype=torch.int32, device="cuda")
    logits = np.zeros((rows, vocab), np.uint16)
    op = None
    for r in range(shards):
        ws_r = s[r * per:(r + 1) * per].clone()  # own allocation: alignment as a shard would have
        wc_r = w[r * per:(r + 1) * per].clone()
        op, p, _, l = lm_head(tk, ctx, x, wc_r, ws_r, rows, per, r * per, rows, hidden, f32=False)
        l()
        gathered[r] = p["pairs"]
        logits[:, r * per:(r + 1) * per] = _u16(p["out"])
    merged = torch.zeros((rows, 2), dtype=torch.int32, device="cuda")
    op.merge(None, rows, shards, gathered, merged)
    torch.cuda.synchronize()
    single = pairs_of(full["pairs"], rows)
    got = pairs_of(merged, rows)
    assert np.array_equal(logits, _u16(full["out"]))
    assert np.array_equal(got["index"], single["index"]) and np.array_equal(got["value"], single["value"])
    for t in range(rows):
        assert got["index"][t] == oracle.greedy_index(logits[t])
    assert got["index"][1] == min(b, other)


@pytest.mark.parametrize("rows", [1, 4, 32])
def test_full_vocabulary_properties(tk, ctx, oracle, rows):
    """Full LM-head size (248320 x 5120, M = 1, 4, 32: the 16- and 32-token epilogues): too large
    for the CPU oracle as a whole, so check (1) for every token the device argmax equals
    greedy_index over the BF16 plane it wrote, (2) a sample of 512 rows (including both ends and
    the last tile) against the f64 oracle, for all tokens."""
    from tuiskollm_b200 import synth

    hidden, vocab = 5120, 248320
    wc, ws = synth.torch_fp8_weights(11, 1, vocab, hidden, "cuda")
    xb = synth.normal_bf16(11, 2, (rows, hidden))
    _, p, scratch, launch = lm_head(tk, ctx, dev(xb.view(np.int16)), wc, ws.view(torch.int16), rows,
                                    vocab, 0, rows, hidden, f32=True)
    launch()
    torch.cuda.synchronize()
    logits = _u16(p["out"])
    got = pairs_of(p["pairs"], rows)
    for t in range(rows):
        assert got["index"][t] == oracle.greedy_index(logits[t]), t
    assert np.array_equal(oracle.f32_to_bf16(host(p["f32"])[:rows]), logits)
    rng = np.random.default_rng(0)
    sample = np.unique(np.concatenate([rng.integers(0, vocab, 500), [0, 1, 127, 128, vocab - 129, vocab - 128, vocab - 1]]))
    idx = torch.from_numpy(sample).cuda()
    wsel = host(wc[idx])
    ssel = host(ws.view(torch.int16)[idx]).view(np.uint16)
    oc, os_ = oracle.quantize_e4m3(xb)
    exp = oracle.fp8_projection(oc, os_, wsel, ssel)
    check_close(logits[:, sample], exp, 1 / 16, 0.01, "sampled logits")
    assert max_relative_error(logits[:, sample], exp, 0.25) <= 1e-2
    assert ctx.device_status() == 0


def test_peer_exchange_single_rank_and_bounded_wait(tk, ctx, oracle):
    """The fused exchange kernel with world = 1 (its own buffer is the only peer) must give the
    same pairs as the finalize route; with a second 'rank' whose flag never arrives the
    bounded wait runs out and reports TK100_DEVICE_WAIT_TIMEOUT instead of hanging."""
    from tuiskollm_b200 import _lib, ops, synth

    hidden, vocab, rows = 5120, 1024, 3
    xb = synth.normal_bf16(15, 1, (rows, hidden))
    wc, ws = synth.fp8_weights(15, 2, vocab, hidden)
    x, w, s = dev(xb.view(np.int16)), dev(wc), dev(ws.view(np.int16))
    op, p, scratch, launch = lm_head(tk, ctx, x, w, s, rows, vocab, 0, rows, hidden, f32=False)
    launch()
    torch.cuda.synchronize()
    expect = pairs_of(p["pairs"], rows)
    buf = torch.zeros((ops.exchange_bytes(rows, 1) + 7) // 8, dtype=torch.int64, device="cuda")
    merged = sentinel_plane((rows, 2), torch.int32)
    for _ in range(3):  # steps alternate parity; the keys are cleared every time
        op.launch(None, rows, x, p["codes"], p["scales"], w, s, p["out"], None, scratch, None)
        assert int(scratch.abs().sum()) != 0, "packed maxima must stay in the scratch"
        op.exchange(None, rows, 1, 0, scratch, [buf.data_ptr()], merged)
        torch.cuda.synchronize()
        got = pairs_of(merged, rows)
        assert np.array_equal(got["index"], expect["index"]) and np.array_equal(got["value"], expect["value"])
        assert int(scratch.abs().sum()) == 0
    assert ctx.device_status() == 0
    # world = 2 on one GPU: rank 1 does not exist, its flag never comes
    buf2 = torch.zeros((2, (ops.exchange_bytes(rows, 2) + 7) // 8), dtype=torch.int64, device="cuda")
    op.launch(None, rows, x, p["codes"], p["scales"], w, s, p["out"], None, scratch, None)
    op.exchange(None, rows, 2, 0, scratch, [buf2[0].data_ptr(), buf2[1].data_ptr()], merged)
    assert ctx.device_status() & _lib.DEVICE_WAIT_TIMEOUT
    assert ctx.device_status() == 0
    # the context is usable again: reading a timed-out status word re-arms tickets and keys
    scratch.zero_()
    launch()
    torch.cuda.synchronize()
    again = pairs_of(p["pairs"], rows)
    assert np.array_equal(again["index"], expect["index"]) and np.array_equal(again["value"], expect["value"])
    assert ctx.device_status() == 0
    with pytest.raises(tk.GpuError):
        op.exchange(None, rows, 9, 0, scratch, [buf.data_ptr()] * 9, merged)
