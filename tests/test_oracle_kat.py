"""Pins the CPU oracle against every known-answer value the reference's own unit
tests hold for the quantized projection path (CPU only)."""
import math

import numpy as np
import pytest

import fixtures_ref as F


def test_bf16_rounding_pins(oracle):
    # qual/src/fp8_projection_oracle.rs:111-114, qual/src/residual_norm.rs:395-402
    L = oracle.lib()
    assert L.tko_f32_to_bf16(1.0 + 0.00390625) == 0x3F80
    assert L.tko_f32_to_bf16(L.tko_bf16_to_f32(0x3F81) + 0.00390625) == 0x3F82
    assert oracle.f32_to_bf16(np.array([1.0 + 0.00390625], np.float32))[0] == 0x3F80


def test_e4m3_codec_pins(oracle):
    # qual/src/fp8_projection_oracle.rs:115-118
    tab = oracle.e4m3_decode_table()
    for search in (True, False):
        assert oracle.e4m3_encode(1.0, search) == 0x38
        assert oracle.e4m3_encode(-0.5, search) == 0xB0
    assert tab[0x7E] == 448.0
    assert math.isnan(tab[0x7F]) and math.isnan(tab[0xFF])
    # signed zero and saturation (qual/src/fp8_projection_oracle.rs:56-61)
    assert oracle.e4m3_encode(-0.0) == 0x80 and oracle.e4m3_encode(0.0) == 0x00
    assert oracle.e4m3_encode(1e9) == 0x7E and oracle.e4m3_encode(-1e9) == 0xFE
    assert oracle.e4m3_encode(float("nan")) == -1
    # tiny negatives keep their sign: they round to 0x80, not 0x00
    assert oracle.e4m3_encode(-1e-8, True) == 0x80 and oracle.e4m3_encode(-1e-8) == 0x80


def test_fixture_weight_codes_decode_to_stated_values(oracle):
    # qual/src/fp8_projection_oracle.rs:6-7
    tab = oracle.e4m3_decode_table()
    assert np.array_equal(tab[F.WEIGHT_CODES], F.WEIGHT_VALUES)


def test_arithmetic_encoder_equals_reference_search_encoder(oracle):
    """Every finite BF16 value (all 65536 patterns) divided by a sweep of scales: both
    encoders agree."""
    import ctypes as C
    L = oracle.lib()
    rng = np.random.default_rng(3)
    scales = np.concatenate([
        np.array([1.0, 1.0 / 448.0, 3.7 / 448.0, 0.013, 2.5e-3, 7.25, 1.0 / 3.0, 448.0, 2.0 ** -20], np.float32),
        (np.abs(rng.standard_normal(24)).astype(np.float32) * np.float32(4.0) / np.float32(448.0)),
        (np.float32(2.0) ** rng.integers(-12, 6, 8).astype(np.float32)) * np.float32(1.1),
    ])
    for s in scales:
        first = C.c_uint32(0)
        bad = L.tko_e4m3_encoder_disagreements(C.c_float(float(s)), C.byref(first))
        assert bad == 0, (float(s), hex(first.value))
    # all midpoints and neighbours of every code
    tab = oracle.e4m3_decode_table()
    pos = np.sort(tab[:0x7F])
    for a, b in zip(pos[:-1], pos[1:]):
        mid = np.float32((np.float64(a) + np.float64(b)) / 2)
        for v in (mid, np.nextafter(mid, np.float32(0)), np.nextafter(mid, np.float32(1e9))):
            for sgn in (1.0, -1.0):
                x = float(sgn * v)
                assert L.tko_e4m3_encode(C.c_float(x)) == L.tko_e4m3_encode_search(C.c_float(x)), x


def test_nvfp4_codec_and_swizzle_pins(oracle):
    # qual/src/nvfp4_swiglu.rs:421-431, qual/src/nvfp4_down.rs:412-422
    assert oracle.e2m1_decode(0x07) == 6.0 and oracle.e2m1_decode(0x0F) == -6.0
    tab = oracle.e4m3_decode_table()
    assert tab[0x01] == 2.0 ** -9 and tab[0x38] == 1.0 and tab[0x40] == 2.0
    g = 5120 // 16
    assert oracle.nvfp4_scale_offset(0, 0, g) == 0
    assert oracle.nvfp4_scale_offset(32, 0, g) == 4
    assert oracle.nvfp4_scale_offset(127, 319, g) == 40_959
    assert oracle.nvfp4_scale_offset(128, 0, g) == 40_960
    g = 17408 // 16
    assert oracle.nvfp4_scale_offset(127, 1087, g) == 139_263
    assert oracle.nvfp4_scale_offset(128, 0, g) == 139_264
    # the vectorised table equals the scalar function and is a permutation
    offs = oracle.nvfp4_scale_offsets(256, 320)
    assert offs[127, 319] == 40_959 and offs[128, 0] == 40_960
    assert np.array_equal(np.sort(offs.reshape(-1)), np.arange(256 * 320))


def test_e2m1_encode_round_trip_and_ties(oracle):
    mags = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for c, m in enumerate(mags):
        assert oracle.e2m1_encode(m) == c and oracle.e2m1_encode(-m) == (c | 8)
    # ties go to the even code; saturation at 6
    assert oracle.e2m1_encode(0.25) == 0 and oracle.e2m1_encode(0.75) == 2
    assert oracle.e2m1_encode(1.25) == 2 and oracle.e2m1_encode(1.75) == 4
    assert oracle.e2m1_encode(2.5) == 4 and oracle.e2m1_encode(3.5) == 6
    assert oracle.e2m1_encode(5.0) == 6 and oracle.e2m1_encode(100.0) == 7
    assert oracle.e2m1_encode(-100.0) == 15


def test_fp8_structured_fixture_matches_closed_form(oracle):
    """qual/src/fp8_qkv.rs:249-295: codes/scale of the fixture tokens and the closed-form
    output; the general dot-product oracle must reproduce the closed form exactly."""
    hidden, out_rows, rows = 5120, 64, 16
    x = F.fp8_input(rows, hidden)
    w, ws = F.fp8_weights(out_rows, hidden)
    codes_s, scales_s = oracle.quantize_e4m3(x, search=True)
    codes_a, scales_a = oracle.quantize_e4m3(x, search=False)
    assert np.array_equal(codes_s, codes_a) and np.array_equal(scales_s, scales_a)
    out = oracle.fp8_projection(codes_a, scales_a, w, ws)
    for t in range(rows):
        c, s, rsum = oracle.quantize_e4m3_token(x[t])
        assert np.array_equal(c, codes_a[t]) and s == scales_a[t]
        # token amax is 0.875*|factor| -> scale = amax/448, the largest code is +-448
        assert s == np.float32(abs(0.875 * F.FP8_TOKEN_FACTORS[t])) / np.float32(448.0)
        assert set(np.unique(c[np.abs(oracle.bf16_to_f32(x[t])) == np.abs(oracle.bf16_to_f32(x[t])).max()])) <= {0x7E, 0xFE}
        exp = F.fp8_expected(rsum, s, out_rows)
        np.testing.assert_allclose(out[t], exp, rtol=1e-12, atol=1e-12)


def test_quantize_zero_row_has_unit_scale(oracle):
    # qual/src/fp8_projection_oracle.rs:32-36
    x = np.zeros((1, 1024), np.uint16)
    x[0, 5] = 0x8000  # -0.0
    codes, scales = oracle.quantize_e4m3(x)
    assert scales[0] == 1.0 and codes[0, 5] == 0x80 and codes.sum() == 0x80


def test_quantize_rejects_non_finite(oracle):
    x = np.zeros((1, 64), np.uint16)
    x[0, 3] = 0x7FC0
    with pytest.raises(ValueError):
        oracle.quantize_e4m3(x)


def test_residual_norm_oracle_properties(oracle):
    """qual/src/residual_norm.rs:228-232,328-348 on the reference's own input patterns."""
    rows, hidden = 8, 5120
    x, b, w = F.norm_fixture(rows, hidden)
    res, norm = oracle.residual_rms_norm(x, b, w, 1e-6)
    # residual is the BF16 sum, bit exact, independently recomputed
    exp_res = oracle.f32_to_bf16(oracle.bf16_to_f32(x) + oracle.bf16_to_f32(b))
    assert np.array_equal(res, exp_res)
    # independent numpy f64 restatement of the norm
    rf = oracle.bf16_to_f32(res).astype(np.float64)
    inv = 1.0 / np.sqrt((rf * rf).sum(axis=1, keepdims=True) / hidden + np.float64(np.float32(1e-6)))
    exp = oracle.f32_to_bf16((rf * inv * (1.0 + oracle.bf16_to_f32(w).astype(np.float64))).astype(np.float32))
    assert np.array_equal(norm, exp)
    _, plain = oracle.residual_rms_norm(x, None, w, 1e-6)
    assert plain.shape == x.shape and not np.array_equal(plain, norm)


def test_greedy_index_contract(oracle):
    # tuisko-engine/src/sampling.rs:313-335 (first maximum wins), :450-454 (NaN at token 37)
    bf = lambda v: int(np.array([v], np.float32).view(np.uint32)[0] >> 16)
    row = np.full(248_320, bf(-4.0), np.uint16)
    row[17] = bf(3.0)
    row[248_044] = bf(3.0)
    assert oracle.greedy_index(row) == 17
    row[248_044] = bf(4.0)
    assert oracle.greedy_index(row) == 248_044
    bad = np.full(248_320, bf(-4.0), np.uint16)
    bad[37] = 0x7FC0
    with pytest.raises(ValueError, match="token 37"):
        oracle.greedy_index(bad)
    # total order: +0 beats -0, and the first of equal values stays
    z = np.array([0x8000, 0x0000, 0x0000, 0x8000], np.uint16)
    assert oracle.greedy_index(z) == 1
    assert oracle.greedy_index(np.array([bf(-1.0), bf(-2.0)], np.uint16)) == 0


@pytest.mark.parametrize("kind", ["gate_up", "down"])
def test_nvfp4_structured_fixture_matches_closed_form(oracle, kind):
    """qual/src/nvfp4_swiglu.rs:306-353 / qual/src/nvfp4_down.rs:300-340: the general A16 dot
    oracle reproduces the fixtures' closed form (one exceptional group per row)."""
    if kind == "gate_up":
        k, out_rows = 5120, 256
        codes, scales = F.nvfp4_weights(2 * out_rows, k, gate_up_split=out_rows)
    else:
        k, out_rows = 17408, 256
        codes, scales = F.nvfp4_weights(out_rows, k, gate_up_split=None)
    x = F.nvfp4_input(8, k)
    dots = oracle.nvfp4_a16_dot(x, codes, scales, F.NVFP4_WEIGHT_SCALE_DIVISOR)
    for token in (0, 3, 7):
        for row in (0, 1, 127, 128, out_rows - 1, codes.shape[0] - 1):
            exp = F.nvfp4_closed_form_dot(x, token, row, codes, scales, k)
            assert dots[token, row] == pytest.approx(exp, rel=1e-12, abs=1e-12)
    if kind == "gate_up":
        out = oracle.silu_mul(dots[:, :out_rows], dots[:, out_rows:])
        g, u = dots[2, 5], dots[2, 5 + out_rows]
        assert out[2, 5] == pytest.approx(oracle.lib().tko_silu_mul(g, u), rel=1e-15)
        assert np.isfinite(out).all()


def test_nvfp4_fixture_exceptional_group_differs(oracle):
    # qual/src/nvfp4_swiglu.rs:433-458
    k, out_rows = 5120, 256
    codes, scales = F.nvfp4_weights(2 * out_rows, k, gate_up_split=out_rows)
    g = k // 16
    for row in (0, 1, 127, 128, out_rows - 1, out_rows):
        eg = F.nvfp4_exceptional_group(row, g)
        og = (eg + 1) % g
        assert not np.array_equal(codes[row, eg * 8:eg * 8 + 8], codes[row, og * 8:og * 8 + 8])
        assert scales[oracle.nvfp4_scale_offset(row, eg, g)] != scales[oracle.nvfp4_scale_offset(row, og, g)]


def test_nvfp4_activation_quantiser_definition(oracle):
    """Own definition (parity unpinned): round trip and block-local scales."""
    rng = np.random.default_rng(7)
    k = 256
    x = oracle.f32_to_bf16(rng.standard_normal((5, k)).astype(np.float32))
    x[3, :16] = 0  # an all-zero block
    x[3, 3] = 0x8000
    div = 448.0 * 6.0 / 4.5
    codes, scales = oracle.nvfp4_quantize(x, div)
    tab = oracle.e4m3_decode_table()
    xf = oracle.bf16_to_f32(x)
    for r in range(5):
        for g in range(k // 16):
            sc = scales[oracle.nvfp4_scale_offset(r, g, k // 16)]
            assert sc < 0x7F
            blk = xf[r, g * 16:(g + 1) * 16]
            s = tab[sc]
            if np.abs(blk).max() == 0:
                assert sc == 0
                continue
            deq = np.array([oracle.e2m1_decode(int(codes[r, g * 8 + c // 2] >> (4 * (c & 1))) & 15)
                            for c in range(16)], np.float64) * s / div
            # half a code step (<= 1 in the scaled domain at the top binade) plus scale rounding
            assert np.abs(deq - blk).max() <= 0.5 * np.abs(blk).max() * (1 / 3 + 1 / 8) + 1e-6
    assert codes[3, 1] >> 4 == 8  # -0.0 keeps its sign in an all-zero block
    # W4A4 dot over represented values equals an independent numpy evaluation
    wq, ws = oracle.nvfp4_quantize(oracle.f32_to_bf16((rng.standard_normal((128, k)) * 0.02).astype(np.float32)), 448.0 * 6.0 / 0.08)
    out = oracle.nvfp4_w4a4_dot(codes, scales, div, wq, ws, 448.0 * 6.0 / 0.08)

    def deq_plane(c, s, rows, d):
        vals = np.empty((rows, k))
        for r in range(rows):
            for col in range(k):
                code = (int(c[r, col // 2]) >> (4 * (col & 1))) & 15
                vals[r, col] = oracle.e2m1_decode(code) * float(tab[s[oracle.nvfp4_scale_offset(r, col // 16, k // 16)]])
        return vals / d

    ref = deq_plane(codes, scales, 5, np.float64(np.float32(div))) @ deq_plane(wq, ws, 128, np.float64(np.float32(448.0 * 6.0 / 0.08))).T
    np.testing.assert_allclose(out, ref, rtol=1e-9, atol=1e-12)
