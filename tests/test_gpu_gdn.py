"""GPU parity of the gated-delta-net decode steps through the C ABI, on the reference's own
fixtures and tolerances: qual/src/gdn_prepare.rs (controls and convolution within 0.002 of the FP64
formula, history bit-exact, sentinels beyond the active batch, eager == graph replay) and
qual/src/gdn_recurrence.rs (state within max(2e-4, 0.2 %), outputs within max(1/64, 1 %), unmapped
state rows untouched), plus seeded random planes against the same oracle."""
import numpy as np
import pytest
import torch

import fixtures_ref as F
from gpu_util import assert_inactive_untouched, bf16_bits_to_f64, dev, graph_replay, host, sentinel_plane
from oracle import gdn_oracle as G

pytestmark = pytest.mark.gpu

MAX_BATCH = 8


@pytest.fixture(scope="module")
def tk():
    import tuiskollm_b200 as tk
    return tk


@pytest.fixture(scope="module")
def ctx(tk):
    return tk.Context(device=0)


def _i16(a):
    return dev(np.ascontiguousarray(a).view(np.int16))


def _u16(t):
    return host(t.view(torch.int16)).view(np.uint16)


class PreparePlanes:
    def __init__(self, f):
        self.f = f
        self.input = _i16(f["input"])
        self.control_weights = _i16(f["control_weights"])
        self.a_log = _i16(f["a_log"])
        self.dt_bias = _i16(f["dt_bias"])
        self.projected = _i16(f["projected"])
        self.convolution_weights = _i16(f["convolution_weights"])
        self.state_rows = dev(f["state_rows"].view(np.int32))
        self.history = _i16(f["history"])
        self.log_decay = sentinel_plane((MAX_BATCH, 48), torch.float32)
        self.beta = sentinel_plane((MAX_BATCH, 48), torch.float32)
        self.convolved = sentinel_plane((MAX_BATCH, 10240), torch.int16)

    def reset(self):
        self.history.copy_(_i16(self.f["history"]))
        for p in (self.log_decay, self.beta, self.convolved):
            p.view(torch.uint8).fill_(0xA5)

    def launch(self, op, batch):
        op.launch(None, batch, self.input, self.control_weights, self.a_log, self.dt_bias, self.projected,
                  self.convolution_weights, self.state_rows, self.history, self.log_decay, self.beta,
                  self.convolved)

    def observe(self):
        torch.cuda.synchronize()
        return (host(self.log_decay).copy(), host(self.beta).copy(), _u16(self.convolved).copy(),
                _u16(self.history).copy())


def check_prepare(f, batch, observed):
    log_decay, beta, convolved, history = observed
    want_decay, want_beta = G.gdn_controls(f["input"][:batch], f["control_weights"], f["a_log"], f["dt_bias"])
    # qual/src/gdn_prepare.rs:362: absolute error <= 0.002
    assert np.abs(log_decay[:batch].astype(np.float64) - want_decay).max() <= 0.002
    assert np.abs(beta[:batch].astype(np.float64) - want_beta).max() <= 0.002
    want_conv, want_history = G.gdn_convolution(f["projected"][:batch], f["convolution_weights"],
                                                f["state_rows"], f["history"])
    # qual/src/gdn_prepare.rs:406
    assert np.abs(bf16_bits_to_f64(convolved[:batch]) - want_conv).max() <= 0.002
    assert np.array_equal(history, want_history), "history after the shift"


@pytest.mark.parametrize("batch", list(range(1, MAX_BATCH + 1)))
def test_prepare_reference_fixture(tk, ctx, batch):
    f = F.gdn_prepare_fixture()
    planes = PreparePlanes(f)
    op = tk.GdnPrepareOp(ctx)
    planes.reset()
    planes.launch(op, batch)
    eager = planes.observe()
    check_prepare(f, batch, eager)
    for p in (planes.log_decay, planes.beta, planes.convolved):
        assert_inactive_untouched(p, batch)
    # graph replay reproduces the eager launch bit for bit (qual/src/gdn_prepare.rs:117-124)
    graph = graph_replay(lambda: planes.launch(op, batch))
    planes.reset()
    graph.replay()
    replay = planes.observe()
    for a, b in zip(eager, replay):
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8))
    for p in (planes.log_decay, planes.beta, planes.convolved):
        assert_inactive_untouched(p, batch)
    assert ctx.device_status(None) == 0


def test_prepare_random_planes(tk, ctx):
    rng = np.random.default_rng(20260)
    from oracle import tuisko_oracle as O
    f = dict(
        input=O.f32_to_bf16(rng.normal(0, 1.0, (MAX_BATCH, 5120)).astype(np.float32)).reshape(MAX_BATCH, 5120),
        control_weights=O.f32_to_bf16(rng.normal(0, 0.02, (96, 5120)).astype(np.float32)).reshape(96, 5120),
        a_log=O.f32_to_bf16(rng.uniform(-3, 1, 48).astype(np.float32)),
        dt_bias=O.f32_to_bf16(rng.normal(0, 1, 48).astype(np.float32)),
        projected=O.f32_to_bf16(rng.normal(0, 1.5, (MAX_BATCH, 16384)).astype(np.float32)).reshape(MAX_BATCH, 16384),
        convolution_weights=O.f32_to_bf16(rng.normal(0, 0.5, (10240, 4)).astype(np.float32)).reshape(10240, 4),
        history=O.f32_to_bf16(rng.normal(0, 1.5, (MAX_BATCH, 10240, 3)).astype(np.float32)).reshape(MAX_BATCH, 10240, 3),
        state_rows=np.array([3, 6, 0, 7, 1, 5, 2, 4], dtype=np.uint32))
    planes = PreparePlanes(f)
    op = tk.GdnPrepareOp(ctx)
    for batch in (1, 5, 8):
        planes.reset()
        planes.launch(op, batch)
        log_decay, beta, convolved, history = planes.observe()
        want_decay, want_beta = G.gdn_controls(f["input"][:batch], f["control_weights"], f["a_log"], f["dt_bias"])
        # fp32 accumulation of 5120 products of O(1) x O(0.02) values and ex2/lg2.approx: the
        # reference's bound scaled by the magnitude of the result
        assert (np.abs(log_decay[:batch] - want_decay) <= 0.002 * np.maximum(1.0, np.abs(want_decay))).all()
        assert np.abs(beta[:batch] - want_beta).max() <= 0.002
        want_conv, want_history = G.gdn_convolution(f["projected"][:batch], f["convolution_weights"],
                                                    f["state_rows"], f["history"])
        got = bf16_bits_to_f64(convolved[:batch])
        # BF16 rounding of the output: half an ulp = 2^-9 relative
        assert (np.abs(got - want_conv) <= np.maximum(0.002, np.abs(want_conv) * 2.0 ** -8)).all()
        assert np.array_equal(history, want_history)


class RecurrencePlanes:
    def __init__(self, f):
        self.f = f
        self.qkv = _i16(f["qkv"])
        self.projected = _i16(f["projected"])
        self.log_decay = dev(f["log_decay"])
        self.beta = dev(f["beta"])
        self.norm_weight = _i16(f["norm_weight"])
        self.state_rows = dev(f["state_rows"].view(np.int32))
        self.state = dev(f["state"])
        self.output = sentinel_plane((MAX_BATCH, 6144), torch.int16)

    def reset(self):
        self.state.copy_(dev(self.f["state"]))
        self.output.view(torch.uint8).fill_(0xA5)

    def launch(self, op, batch):
        op.launch(None, batch, self.qkv, self.projected, self.log_decay, self.beta, self.norm_weight,
                  self.state_rows, self.state, self.output)

    def observe(self):
        torch.cuda.synchronize()
        return host(self.state).copy(), _u16(self.output).copy()


def check_recurrence(f, batch, observed):
    state, output = observed
    want_state, want_output = G.gdn_recurrence(f["qkv"][:batch], f["projected"][:batch], f["log_decay"],
                                               f["beta"], f["norm_weight"], f["state_rows"], f["state"])
    err = np.abs(state.astype(np.float64) - want_state)
    # qual/src/gdn_recurrence.rs:349
    assert (err <= np.maximum(2.0e-4, np.abs(want_state) * 0.002)).all(), f"state, worst {err.max()}"
    idle = [r for r in range(MAX_BATCH) if r not in list(f["state_rows"][:batch])]
    assert np.array_equal(state[idle], f["state"][idle]), "state rows no token maps to"
    err = np.abs(bf16_bits_to_f64(output[:batch]) - want_output)
    # qual/src/gdn_recurrence.rs:364
    assert (err <= np.maximum(0.015625, np.abs(want_output) * 0.01)).all(), f"output, worst {err.max()}"
    return float(err.max())


@pytest.mark.parametrize("batch", list(range(1, MAX_BATCH + 1)))
def test_recurrence_reference_fixture(tk, ctx, batch):
    f = F.gdn_recurrence_fixture()
    planes = RecurrencePlanes(f)
    op = tk.GdnRecurrenceOp(ctx)
    planes.reset()
    planes.launch(op, batch)
    eager = planes.observe()
    check_recurrence(f, batch, eager)
    assert_inactive_untouched(planes.output, batch)
    graph = graph_replay(lambda: planes.launch(op, batch))
    planes.reset()
    graph.replay()
    replay = planes.observe()
    assert np.array_equal(eager[0].view(np.uint32), replay[0].view(np.uint32))
    assert np.array_equal(eager[1], replay[1])
    assert ctx.device_status(None) == 0


def test_recurrence_random_planes_two_steps(tk, ctx):
    """Seeded random planes; two consecutive steps on the same state (the second step reads what
    the first wrote)."""
    rng = np.random.default_rng(777)
    from oracle import tuisko_oracle as O
    f = dict(
        qkv=O.f32_to_bf16(rng.normal(0, 1.0, (MAX_BATCH, 10240)).astype(np.float32)).reshape(MAX_BATCH, 10240),
        projected=O.f32_to_bf16(rng.normal(0, 1.0, (MAX_BATCH, 16384)).astype(np.float32)).reshape(MAX_BATCH, 16384),
        log_decay=(-rng.uniform(0.01, 2.0, (MAX_BATCH, 48))).astype(np.float32),
        beta=rng.uniform(0.05, 0.95, (MAX_BATCH, 48)).astype(np.float32),
        norm_weight=O.f32_to_bf16(rng.uniform(0.5, 1.5, 128).astype(np.float32)),
        state=rng.normal(0, 0.05, (MAX_BATCH, 48, 128, 128)).astype(np.float32),
        state_rows=np.array([2, 4, 6, 0, 1, 3, 5, 7], dtype=np.uint32))
    planes = RecurrencePlanes(f)
    op = tk.GdnRecurrenceOp(ctx)
    batch = 6
    planes.reset()
    planes.launch(op, batch)
    first = planes.observe()
    check_recurrence(f, batch, first)
    planes.launch(op, batch)
    second = planes.observe()
    g = dict(f)
    g["state"] = first[0]
    check_recurrence(g, batch, second)


def test_batch_outside_the_admitted_range_is_refused(tk, ctx):
    """tuisko-kernels-sm120/src/gdn/prepare.rs:13-24 and its test :296-308: 0, 9 and 16 are refused."""
    f = F.gdn_recurrence_fixture()
    planes = RecurrencePlanes(f)
    op = tk.GdnRecurrenceOp(ctx)
    for batch in (0, 9, 16):
        with pytest.raises(tk.GpuError, match="outside the admitted range"):
            planes.launch(op, batch)
    prep = PreparePlanes(F.gdn_prepare_fixture())
    for batch in (0, 9):
        with pytest.raises(tk.GpuError, match="outside the admitted range"):
            prep.launch(tk.GdnPrepareOp(ctx), batch)

