"""CPU checks of the gated-delta-net oracle: the vectorised FP64 restatement
(oracle/gdn_oracle.py) against a scalar pure-Python evaluation of the same formulas
(qual/src/gdn_prepare.rs:333-431, qual/src/gdn_recurrence.rs:274-335) on sampled elements of the
reference's fixtures, and the fixture generators against values computed by hand from the
reference's constants."""
import math

import numpy as np

import fixtures_ref as F
from oracle import gdn_oracle as G
from oracle import tuisko_oracle as O


def _f(bits):
    return float(O.bf16_to_f32(np.array([bits], dtype=np.uint16))[0])


def test_fixture_generators_follow_the_reference_constants():
    f = F.gdn_prepare_fixture()
    # token 2, column 5: INPUT_PATTERN[(2*5120 + 5 + 2) & 7] * (1 + 2/8)
    assert _f(f["input"][2, 5]) == float(F.GDN_INPUT_PATTERN[7] * np.float32(1.25))
    assert _f(f["input"][3, 1]) == float(O.bf16_to_f32(O.f32_to_bf16(
        np.array([F.GDN_INPUT_PATTERN[(3 * 5120 + 1 + 3) & 7] * np.float32(1.375)], dtype=np.float32)))[0])
    # control weight row 50, column 9: WEIGHT_PATTERN[(9 + 150) & 7]
    assert _f(f["control_weights"][50, 9]) == float(O.bf16_to_f32(O.f32_to_bf16(
        np.array([F.GDN_WEIGHT_PATTERN[(9 + 150) & 7]], dtype=np.float32)))[0])
    assert _f(f["a_log"][6]) == -2.0 + 2 * 0.125
    assert _f(f["dt_bias"][0]) == _f(int(O.f32_to_bf16(np.array([-23.5 / 256.0], dtype=np.float32))[0]))
    assert _f(f["convolution_weights"][77, 2]) == 0.125
    # history word (row 1, channel 3, tap 2): index = (1*10240 + 3)*3 + 2
    i = (10240 + 3) * 3 + 2
    assert _f(f["history"][1, 3, 2]) == float(F.GDN_INPUT_PATTERN[(5 * i + i // 3) & 7]) * 0.5
    assert list(f["state_rows"]) == [7, 0, 5, 2, 6, 1, 4, 3]

    r = F.gdn_recurrence_fixture()
    assert _f(r["qkv"][3, 10]) == [0.75, -0.625, 0.5, -0.375, 0.25, -0.1875, 0.125, -0.0625][(10 + 3) & 7]
    assert _f(r["qkv"][1, 2048 + 4]) == [0.75, -0.625, 0.5, -0.375, 0.25, -0.1875, 0.125, -0.0625][(12 + 2) & 7]
    assert _f(r["projected"][2, 10240 + 130]) == [-1.0, -0.5, -0.25, 0.0, 0.25, 0.5, 0.75, 1.0][(130 + 1 + 2) & 7]
    assert r["log_decay"][1, 3] == np.float32(-0.125 - ((48 + 3) & 7) * 0.03125)
    assert r["beta"][0, 2] == np.float32(0.5)
    idx = (2 * 48 * 128 * 128 + 5)
    assert r["state"].reshape(-1)[idx] == np.float32((((idx * 13) & 31) - 15.5) / 2048.0)


def test_controls_match_a_scalar_evaluation():
    f = F.gdn_prepare_fixture()
    log_decay, beta = G.gdn_controls(f["input"][:3], f["control_weights"], f["a_log"], f["dt_bias"])
    x = O.bf16_to_f32(f["input"]).astype(np.float64)
    w = O.bf16_to_f32(f["control_weights"]).astype(np.float64)
    for token, row in [(0, 0), (1, 17), (2, 47), (0, 48), (2, 95)]:
        total = math.fsum(float(a) * float(b) for a, b in zip(x[token], w[row]))
        if row < 48:
            control = total + _f(f["dt_bias"][row])
            want = -math.exp(_f(f["a_log"][row])) * math.log(1.0 + math.exp(control))
            assert abs(log_decay[token, row] - want) < 1e-12
        else:
            assert abs(beta[token, row - 48] - 1.0 / (1.0 + math.exp(-total))) < 1e-12


def test_convolution_matches_a_scalar_evaluation_and_shifts_history():
    f = F.gdn_prepare_fixture()
    batch = 3
    out, history = G.gdn_convolution(f["projected"][:batch], f["convolution_weights"], f["state_rows"],
                                     f["history"])
    for token, channel in [(0, 0), (1, 4099), (2, 10239)]:
        row = int(f["state_rows"][token])
        taps = [_f(f["history"][row, channel, t]) for t in range(3)] + [_f(f["projected"][token, channel])]
        total = math.fsum(_f(f["convolution_weights"][channel, t]) * taps[t] for t in range(4))
        assert abs(out[token, channel] - total / (1.0 + math.exp(-total))) < 1e-12
        assert list(history[row, channel]) == [f["history"][row, channel, 1], f["history"][row, channel, 2],
                                               f["projected"][token, channel]]
    untouched = [r for r in range(8) if r not in list(f["state_rows"][:batch])]
    assert np.array_equal(history[untouched], f["history"][untouched])


def test_recurrence_matches_a_scalar_evaluation():
    r = F.gdn_recurrence_fixture()
    batch = 2
    state, output = G.gdn_recurrence(r["qkv"][:batch], r["projected"][:batch], r["log_decay"], r["beta"],
                                     r["norm_weight"], r["state_rows"], r["state"])
    qkv = O.bf16_to_f32(r["qkv"]).astype(np.float64)
    token, head = 1, 31
    key_head = head // 3
    row_index = int(r["state_rows"][token])
    q = qkv[token, key_head * 128:(key_head + 1) * 128]
    k = qkv[token, 2048 + key_head * 128:2048 + (key_head + 1) * 128]
    q = [v / math.sqrt(math.fsum(a * a for a in q) + 1e-6) for v in q]
    k = [v / math.sqrt(math.fsum(a * a for a in k) + 1e-6) for v in k]
    decay = math.exp(float(r["log_decay"][token, head]))
    beta = float(r["beta"][token, head])
    old = r["state"][row_index, head].astype(np.float64)
    recurrent = []
    for row in range(128):
        state_key = math.fsum(old[row, c] * k[c] for c in range(128))
        update = beta * (qkv[token, 4096 + head * 128 + row] - decay * state_key)
        new = [decay * old[row, c] + update * k[c] for c in range(128)]
        if row in (0, 77, 127):
            assert np.allclose(state[row_index, head, row], new, rtol=0, atol=1e-13)
        recurrent.append(math.fsum(new[c] * q[c] for c in range(128)) * 0.088_388_35)
    rms = math.sqrt(math.fsum(v * v for v in recurrent) / 128 + 1e-6)
    for row in (0, 5, 127):
        gate = _f(r["projected"][token, 10240 + head * 128 + row])
        want = recurrent[row] / rms * _f(r["norm_weight"][row]) * gate / (1.0 + math.exp(-gate))
        assert abs(output[token, head * 128 + row] - want) < 1e-12
    # state rows no token maps to stay as they were
    idle = [x for x in range(8) if x not in list(r["state_rows"][:batch])]
    assert np.array_equal(state[idle], r["state"][idle].astype(np.float64))
