"""GPU parity of the device-side weight materialisation through the C ABI, on the cases of the
reference's own tests (tuisko-model/src/materialize.rs:441-723): the fused QKV gather keeps every
source byte, the NVFP4 scale planes are only permuted (checked against the reference test's
independent tile walk and against the offset formula of the oracle), weights stay untouched, bad
geometry and bad scale codes are refused with the reference's messages."""
import numpy as np
import pytest
import torch

from gpu_util import dev, host

pytestmark = pytest.mark.gpu

ROWS, GROUPS = 128, 8


@pytest.fixture(scope="module")
def tk():
    import tuiskollm_b200 as tk
    return tk


@pytest.fixture(scope="module")
def ctx(tk):
    return tk.Context(device=0)


def scale_codes(seed, rows=ROWS, groups=GROUPS):
    """materialize.rs:483-487."""
    return ((np.arange(rows * groups) * 37 + seed) % 0x7F).astype(np.uint8).reshape(rows, groups)


def block_scale_oracle(source, rows, groups):
    """materialize.rs:489-507: the test's own walk over tiles, independent of the offset formula."""
    source = source.reshape(rows, groups)
    out = []
    for row_tile in range(rows // 128):
        for group_tile in range(groups // 4):
            for row_mod32 in range(32):
                for quartile in range(4):
                    for lane in range(4):
                        out.append(source[row_tile * 128 + quartile * 32 + row_mod32, group_tile * 4 + lane])
    return np.array(out, dtype=np.uint8)


def test_full_attention_qkv_gathers_exact_source_words(tk, ctx):
    """materialize.rs:510-566: shapes [4,3] / [1,3] / [1,3], scales as BF16 words."""
    m = tk.Materializer(ctx)
    qw = np.arange(0x10, 0x1C, dtype=np.uint8).reshape(4, 3)
    kw = np.arange(0x30, 0x33, dtype=np.uint8).reshape(1, 3)
    vw = np.arange(0x50, 0x53, dtype=np.uint8).reshape(1, 3)
    qs = np.array([0x3F80, 0x4000, 0x4040, 0x4080], dtype=np.uint16).reshape(4, 1)
    ks = np.array([0x40A0], dtype=np.uint16).reshape(1, 1)
    vs = np.array([0x40C0], dtype=np.uint16).reshape(1, 1)
    to = lambda a: dev(a.view(np.int16)) if a.dtype == np.uint16 else dev(a)
    weight, scale = m.full_attention_qkv(None, (to(qw), to(qs)), (to(kw), to(ks)), (to(vw), to(vs)))
    torch.cuda.synchronize()
    assert tuple(weight.shape) == (6, 3)
    assert np.array_equal(host(weight), np.concatenate([qw, kw, vw]))
    assert np.array_equal(host(scale).view(np.uint16), np.concatenate([qs, ks, vs]))
    # incompatible shapes (materialize.rs:568-598)
    bad_key = dev(np.full((1, 2), 0x20, dtype=np.uint8))
    with pytest.raises(tk.GpuError, match="incompatible shapes"):
        m.full_attention_qkv(None, (to(qw), to(qs)), (bad_key, to(ks)), (to(vw), to(vs)))


def test_full_size_qkv_gather_is_lossless(tk, ctx):
    """The model's planes: 6144 + 1024 + 1024 rows of 5120 E4M3 codes, BF16 row scales."""
    rng = np.random.default_rng(5)
    planes = [rng.integers(0, 256, (rows, 5120), dtype=np.uint8) for rows in (6144, 1024, 1024)]
    scales = [rng.integers(0, 65536, (rows, 1), dtype=np.uint16) for rows in (6144, 1024, 1024)]
    m = tk.Materializer(ctx)
    weight, scale = m.full_attention_qkv(None, *[(dev(w), dev(s.view(np.int16))) for w, s in zip(planes, scales)])
    torch.cuda.synchronize()
    assert np.array_equal(host(weight), np.concatenate(planes))
    assert np.array_equal(host(scale).view(np.uint16), np.concatenate(scales))


def test_gate_up_and_down_scales_are_only_permuted(tk, ctx, oracle):
    """materialize.rs:600-686."""
    m = tk.Materializer(ctx)
    gate, up = scale_codes(3), scale_codes(11)
    out = m.nvfp4_scales(None, [dev(gate), dev(up)])
    want = block_scale_oracle(np.concatenate([gate, up]), 2 * ROWS, GROUPS)
    assert np.array_equal(host(out), want)
    down = scale_codes(19)
    assert np.array_equal(host(m.nvfp4_scales(None, [dev(down)])), block_scale_oracle(down, ROWS, GROUPS))


@pytest.mark.parametrize("rows,groups,planes", [(17408, 320, 2), (5120, 1088, 1), (256, 20, 1), (128, 4, 2)])
def test_scale_layout_follows_the_offset_formula(tk, ctx, oracle, rows, groups, planes):
    """Model-sized planes (gate/up 2 x 17408 x 320, down 5120 x 1088) and ragged tile counts against
    nvfp4_scale_offset (materialize.rs:410-422, restated in the oracle)."""
    rng = np.random.default_rng(rows + groups)
    sources = [rng.integers(0, 0x7F, (rows, groups), dtype=np.uint8) for _ in range(planes)]
    m = tk.Materializer(ctx)
    out = host(m.nvfp4_scales(None, [dev(s) for s in sources]))
    fused = np.concatenate(sources)
    offsets = oracle.nvfp4_scale_offsets(planes * rows, groups)
    want = np.zeros(fused.size, dtype=np.uint8)
    want[offsets.reshape(-1)] = fused.reshape(-1)
    assert np.array_equal(out, want)


def test_bad_geometry_and_bad_codes_are_refused(tk, ctx):
    """materialize.rs:688-710 and bindings.rs:1105-1120."""
    m = tk.Materializer(ctx)
    with pytest.raises(tk.GpuError, match="scale rows 127 are not tiled by 128"):
        m.nvfp4_scales(None, [dev(np.zeros((127, 8), dtype=np.uint8))])
    with pytest.raises(tk.GpuError, match="scale groups 6 are not tiled by 4"):
        m.nvfp4_scales(None, [dev(np.zeros((128, 6), dtype=np.uint8))])
    for bad in (0x80, 0x7F, 0xFF):
        codes = scale_codes(1)
        codes[77, 5] = bad
        with pytest.raises(tk.GpuError, match="negative or NaN E4M3FN code"):
            m.nvfp4_scales(None, [dev(codes)])
    # the status word was read and cleared by the failing calls
    assert ctx.device_status(None) == 0
