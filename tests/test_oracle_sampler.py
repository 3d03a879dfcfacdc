"""CPU checks of the sampler oracle against the known answers the reference's own tests hold
(tuisko-engine/src/sampling.rs:263-483): routes, first-maximum greedy choice with stop marks,
top-k against an independent full sort of the reference's generated row, the token pinned by
seed 7, the draws of seeds 0..64 staying inside the top-k, the unit interval of the generator."""
import numpy as np
import pytest

from oracle import tuisko_oracle as O

VOCAB = 248_320
STOP_IDS = (248_046, 248_044)


def bf16(value) -> np.uint16:
    return np.uint16(np.float32(value).view(np.uint32) >> 16)


def flat_row():
    return np.full(VOCAB, bf16(-4.0), dtype=np.uint16)


def lcg_row():
    """sampling.rs:339-346: 4096 values from the test's linear congruential generator."""
    seed, values = 0x8B8B_8B8B_8B8B_8B8B, []
    for _ in range(4096):
        seed = (seed * 6_364_136_223_846_793_005 + 1_442_695_040_888_963_407) & (2 ** 64 - 1)
        values.append(bf16(np.float32((seed >> 40) - 32_768) / np.float32(1024.0)))
    return np.array(values, dtype=np.uint16)


def test_greedy_keeps_the_first_maximum_and_marks_stop_tokens():
    row = flat_row()
    row[17] = bf16(3.0)
    row[STOP_IDS[0]] = bf16(3.0)
    sampler = O.Sampler(temperature=0.0, top_p=1.0, top_k=1, seed=0, stop_ids=STOP_IDS)
    assert sampler.sample(row) == (17, False)
    row[STOP_IDS[0]] = bf16(4.0)
    assert sampler.sample(row) == (STOP_IDS[0], True)


def test_top_k_matches_an_independent_full_sort():
    row = lcg_row()
    index, value = O.top_k_select(row, 20)
    values = O.bf16_to_f32(row)
    order = sorted(range(row.size), key=lambda t: (-float(values[t]), t))[:20]
    assert list(index) == order
    assert list(value) == [values[t] for t in order]


def test_tie_order_follows_the_total_order():
    # sampling.rs:470-482: (1, 1.0), (2, 1.0), (4, 0.0), (3, -0.0)
    row = np.full(32, bf16(-9.0), dtype=np.uint16)
    row[2], row[1], row[3], row[4] = bf16(1.0), bf16(1.0), np.uint16(0x8000), bf16(0.0)
    index, _ = O.top_k_select(row, 4)
    assert list(index) == [1, 2, 4, 3]


def test_sampled_route_never_leaves_top_k():
    row = flat_row()
    row[3], row[5], row[7] = bf16(3.0), bf16(2.0), bf16(1.0)
    for seed in range(64):
        token, _ = O.Sampler(temperature=1.0, top_p=1.0, top_k=2, seed=seed, stop_ids=STOP_IDS).sample(row)
        assert token in (3, 5)


def test_deterministic_seed_pins_the_sampled_token():
    row = flat_row()
    row[3], row[5] = bf16(2.0), bf16(1.0)
    sampler = O.Sampler(temperature=1.0, top_p=1.0, top_k=2, seed=7, stop_ids=STOP_IDS)
    assert sampler.sample(row)[0] == 5


def test_greedy_route_draws_no_random_number():
    row = flat_row()
    row[9] = bf16(1.0)
    for temperature, top_k in ((0.0, 20), (1.0, 1)):
        sampler = O.Sampler(temperature=temperature, top_p=0.95, top_k=top_k, seed=3, stop_ids=STOP_IDS)
        before = sampler.state.value
        assert sampler.sample(row)[0] == 9
        assert sampler.state.value == before


def test_random_draw_stays_in_the_unit_interval():
    import ctypes as C
    lib = O.lib()
    state = C.c_uint64(lib.tko_xorshift_new(9))
    for _ in range(1024):
        value = lib.tko_xorshift_unit(C.byref(state))
        assert 0.0 <= value < 1.0
    formerly_zero = C.c_uint64(lib.tko_xorshift_new(0x9E37_79B9_7F4A_7C15))
    assert lib.tko_xorshift_unit(C.byref(formerly_zero)) > 0.0


def test_non_finite_logit_is_reported_with_its_token():
    row = flat_row()
    row[37] = 0x7FC0
    with pytest.raises(ValueError, match="token 37"):
        O.top_k_select(row, 20)
