"""GPU parity of the device sampler through the C ABI: the reference's own known answers
(tuisko-engine/src/sampling.rs:263-483) and seeded random rows against the CPU oracle -- the
surviving top-k list bit for bit (values, indices, order), the sampled token, the stop mark and the
generator state after every draw."""
import numpy as np
import pytest
import torch

from gpu_util import dev, graph_replay, host
from test_oracle_sampler import STOP_IDS, VOCAB, bf16, flat_row, lcg_row

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tk():
    import tuiskollm_b200 as tk
    return tk


@pytest.fixture(scope="module")
def ctx(tk):
    return tk.Context(device=0)


def rows_to_device(rows):
    return dev(np.stack(rows).view(np.int16))


def decisions(sampler):
    torch.cuda.synchronize()
    return [tuple(int(v) for v in d) for d in host(sampler.decisions)]


def states(sampler):
    torch.cuda.synchronize()
    return [int(v) & (2 ** 64 - 1) for v in host(sampler.rng_state)]


def test_reference_known_answers(tk, ctx):
    first = flat_row(); first[17] = bf16(3.0); first[STOP_IDS[0]] = bf16(3.0)
    second = flat_row(); second[17] = bf16(3.0); second[STOP_IDS[0]] = bf16(4.0)
    pinned = flat_row(); pinned[3] = bf16(2.0); pinned[5] = bf16(1.0)
    options = [tk.SamplingOptions.greedy(), tk.SamplingOptions.greedy(),
               tk.SamplingOptions(temperature=1.0, top_p=1.0, top_k=2, seed=7)]
    sampler = tk.Sampler(ctx, VOCAB, options, [STOP_IDS] * 3)
    sampler.sample(None, rows_to_device([first, second, pinned]))
    assert decisions(sampler) == [(17, 0), (STOP_IDS[0], 1), (5, 0)]
    assert ctx.device_status(None) == 0


def test_top_k_matches_the_full_sort_of_the_reference_row(tk, ctx, oracle):
    row = lcg_row()
    sampler = tk.Sampler(ctx, row.size, [tk.SamplingOptions(top_k=20, seed=1)], [(1, 2)])
    sampler.sample(None, rows_to_device([row]), want_top=True)
    torch.cuda.synchronize()
    top = host(sampler.top)[0, :20]
    index, value = oracle.top_k_select(row, 20)
    assert list(top[:, 1].view(np.uint32)) == list(index)
    assert np.array_equal(top[:, 0].copy().view(np.float32), value)


def test_sampled_route_never_leaves_top_k(tk, ctx, oracle):
    row = flat_row(); row[3] = bf16(3.0); row[5] = bf16(2.0); row[7] = bf16(1.0)
    logits = rows_to_device([row] * 8)
    for base in range(0, 64, 8):
        options = [tk.SamplingOptions(temperature=1.0, top_p=1.0, top_k=2, seed=base + i) for i in range(8)]
        sampler = tk.Sampler(ctx, VOCAB, options, [STOP_IDS] * 8)
        sampler.sample(None, logits)
        got = decisions(sampler)
        for i, (token, stopped) in enumerate(got):
            want = oracle.Sampler(1.0, 1.0, 2, base + i, STOP_IDS).sample(row)
            assert token in (3, 5) and (token, bool(stopped)) == want


@pytest.mark.parametrize("vocab", [VOCAB, 4096, 50_000])
def test_random_rows_follow_the_oracle_draw_by_draw(tk, ctx, oracle, vocab):
    """Eight requests with different controls, six consecutive draws each on fresh logits: token,
    stop mark and generator state equal the oracle's after every draw."""
    rng = np.random.default_rng(4242 + vocab)
    controls = [(1.0, 0.95, 20), (0.7, 0.9, 20), (1.3, 1.0, 32), (1.0, 0.5, 8), (0.0, 0.95, 20),
                (1.0, 0.95, 1), (2.0, 0.99, 5), (0.3, 0.0, 20)]
    stops = [(int(rng.integers(0, vocab // 2)), int(rng.integers(vocab // 2, vocab))) for _ in controls]
    options = [tk.SamplingOptions(t, p, k, seed=100 + i) for i, (t, p, k) in enumerate(controls)]
    sampler = tk.Sampler(ctx, vocab, options, stops)
    refs = [oracle.Sampler(t, p, k, 100 + i, stops[i]) for i, (t, p, k) in enumerate(controls)]
    for draw in range(6):
        values = rng.normal(0.0, 3.0, (8, vocab)).astype(np.float32)
        values[:, rng.integers(0, vocab, 40)] += 6.0          # a few clear candidates
        values[3, 11] = values[3, 4000]                        # an exact tie inside one row
        rows = [oracle.f32_to_bf16(values[i]) for i in range(8)]
        if draw == 2:
            rows[6][stops[6][0]] = bf16(60.0)                  # a stop token wins
        sampler.sample(None, rows_to_device(rows), want_top=True)
        got = decisions(sampler)
        top = host(sampler.top)
        for i, ref in enumerate(refs):
            want_token, want_stop = ref.sample(rows[i])
            assert got[i] == (want_token, int(want_stop)), f"draw {draw}, request {i}"
            index, value = oracle.top_k_select(rows[i], controls[i][2])
            assert list(top[i, :controls[i][2], 1].view(np.uint32)) == list(index)
            assert np.array_equal(top[i, :controls[i][2], 0].copy().view(np.float32), value)
        assert states(sampler) == [r.state.value for r in refs]
    assert ctx.device_status(None) == 0


def test_graph_replay_advances_the_generator_like_eager_calls(tk, ctx, oracle):
    rng = np.random.default_rng(9)
    rows = [oracle.f32_to_bf16(rng.normal(0, 2.0, VOCAB).astype(np.float32)) for _ in range(2)]
    logits = rows_to_device(rows)
    options = [tk.SamplingOptions(seed=5), tk.SamplingOptions(temperature=0.8, seed=6)]
    sampler = tk.Sampler(ctx, VOCAB, options, [STOP_IDS] * 2)
    refs = [oracle.Sampler(1.0, 0.95, 20, 5, STOP_IDS), oracle.Sampler(0.8, 0.95, 20, 6, STOP_IDS)]
    graph = graph_replay(lambda: sampler.sample(None, logits))   # one warm-up call + capture
    for r, row in zip(refs, rows):
        r.sample(row)
    for _ in range(3):
        graph.replay()
        want = [r.sample(row) for r, row in zip(refs, rows)]
        assert decisions(sampler) == [(t, int(s)) for t, s in want]
    assert states(sampler) == [r.state.value for r in refs]


def test_non_finite_logit_sets_the_status_bit(tk, ctx):
    from tuiskollm_b200 import _lib
    row = flat_row(); row[37] = 0x7FC0
    sampler = tk.Sampler(ctx, VOCAB, [tk.SamplingOptions()], [STOP_IDS])
    sampler.sample(None, rows_to_device([row]))
    assert ctx.device_status(None) & _lib.DEVICE_NONFINITE_LOGIT


def test_invalid_options_are_refused_before_any_launch(tk, ctx):
    """sampling.rs:415-468: the reference's bad-option table, plus the device limit on top_k."""
    logits = rows_to_device([flat_row()])
    before = ctx.launch_count
    bad = [dict(temperature=float("nan")), dict(temperature=-1.0), dict(top_p=1.1), dict(top_p=float("nan")),
           dict(top_k=0), dict(top_k=VOCAB + 1), dict(top_k=33)]
    for kw in bad:
        with pytest.raises(tk.GpuError, match=r"engine\.sampling"):
            tk.Sampler(ctx, VOCAB, [tk.SamplingOptions(**kw)], [STOP_IDS]).sample(None, logits)
    for stops in ((1, 1), (0, VOCAB)):
        with pytest.raises(tk.GpuError, match=r"engine\.sampling"):
            tk.Sampler(ctx, VOCAB, [tk.SamplingOptions()], [stops]).sample(None, logits)
    assert ctx.launch_count == before
