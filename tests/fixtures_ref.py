"""Structured fixtures of the reference's own device qualification tests, rebuilt
from the constants those tests state (they are data, not code).  Each builder
names the reference test it follows; sizes are parameters so that the same
patterns can be used on small planes."""
import numpy as np

from oracle import tuisko_oracle as O

# qual/src/fp8_projection_oracle.rs:6-8
WEIGHT_CODES = np.array([0x38, 0xB0, 0x30, 0x28], dtype=np.uint8)
WEIGHT_VALUES = np.array([1.0, -0.5, 0.5, 0.25], dtype=np.float32)
SCALE_VALUES = np.array([1.0, 0.5, 0.25, 2.0], dtype=np.float32)
# qual/src/fp8_qkv.rs:23-30
FP8_INPUT_PATTERN = np.array([0.875, -0.875, 0.5, -0.5, 0.25, -0.25, 0.125, -0.125, 0.0625,
                              -0.0625, 0.03125, -0.03125, 0.0, 0.5, -0.25, 0.125], dtype=np.float32)
FP8_TOKEN_FACTORS = np.array([1.0, 0.5, 0.25, 0.125, -1.0, -0.5, -0.25, -0.125, 0.75, -0.75,
                              0.375, -0.375, 0.1875, -0.1875, 0.09375, -0.09375], dtype=np.float32)
# qual/src/residual_norm.rs:12-19
NORM_INPUT_PATTERN = np.array([0.875, -0.75, 0.625, -0.5, 0.375, -0.25, 0.125, -0.0625, -0.875,
                               0.75, -0.625, 0.5, -0.375, 0.25, -0.125, 0.0625], dtype=np.float32)
NORM_BRANCH_PATTERN = np.array([0.25, -0.125, 0.0625, -0.03125, -0.25, 0.125, -0.0625, 0.03125],
                               dtype=np.float32)
NORM_WEIGHT_PATTERN = np.array([-0.25, -0.125, -0.0625, 0.0, 0.0625, 0.125, 0.1875, 0.25],
                               dtype=np.float32)
# qual/src/nvfp4_swiglu.rs:16-23,196-199
NVFP4_WEIGHT_SCALE_DIVISOR = 0.125
NVFP4_INPUT_PATTERN = np.array([0.5, -0.5, 0.25, -0.25, 0.125, -0.125, 0.0, 0.5, -0.5, 0.25, -0.25,
                                0.125, -0.125, 0.0, 0.5, -0.5], dtype=np.float32)
NVFP4_TOKEN_FACTORS = np.array([1.0, 0.5, 0.25, 0.125, 1.0, 0.5, 0.25, 0.125], dtype=np.float32)
NVFP4_BASE = np.array([0xF7, 0xD5, 0xB3, 0x70, 0x5F, 0x3D, 0x0B, 0xF7], dtype=np.uint8)
NVFP4_SPARSE = np.array([0x01, 0, 0, 0, 0, 0, 0, 0], dtype=np.uint8)
NVFP4_SCALE_CODES = np.array([0x38, 0x01, 0x40, 0x01], dtype=np.uint8)


def fp8_input(rows: int, hidden: int) -> np.ndarray:
    """qual/src/fp8_qkv.rs:169-177 (make_input): BF16 bits [rows, hidden]."""
    idx = np.arange(rows * hidden)
    vals = FP8_INPUT_PATTERN[idx & 15] * FP8_TOKEN_FACTORS[(idx // hidden) % 16]
    return O.f32_to_bf16(vals).reshape(rows, hidden)


def fp8_weights(out_rows: int, hidden: int):
    """qual/src/fp8_qkv.rs:179-195 (make_weights): constant code per row, BF16 row scales."""
    rows = np.arange(out_rows)
    codes = np.repeat(WEIGHT_CODES[rows & 3][:, None], hidden, axis=1).astype(np.uint8)
    scales = O.f32_to_bf16(SCALE_VALUES[rows & 3])
    return np.ascontiguousarray(codes), scales


def fp8_expected(represented_sum: float, scale: np.float32, out_rows: int) -> np.ndarray:
    """qual/src/fp8_qkv.rs:281-285 closed form, f64 [out_rows]."""
    rows = np.arange(out_rows)
    return (represented_sum * WEIGHT_VALUES[rows & 3].astype(np.float64) * np.float64(scale)
            * SCALE_VALUES[rows & 3].astype(np.float64))


def norm_fixture(rows: int, hidden: int):
    """qual/src/residual_norm.rs:80-94: (input, branch, weight) BF16 bit planes."""
    idx = np.arange(rows * hidden)
    tok = idx // hidden
    x = NORM_INPUT_PATTERN[(idx + tok) & 15] * (np.float32(1.0) - tok.astype(np.float32) * np.float32(0.03125))
    b = NORM_BRANCH_PATTERN[(idx * 3 + tok) & 7]
    w = NORM_WEIGHT_PATTERN[np.arange(hidden) & 7]
    return (O.f32_to_bf16(x).reshape(rows, hidden), O.f32_to_bf16(b).reshape(rows, hidden),
            O.f32_to_bf16(w))


def nvfp4_input(rows: int, k: int) -> np.ndarray:
    """qual/src/nvfp4_swiglu.rs:173-180 (make_fixture input)."""
    idx = np.arange(rows * k)
    vals = NVFP4_INPUT_PATTERN[idx & 15] * NVFP4_TOKEN_FACTORS[(idx // k) % 8]
    return O.f32_to_bf16(vals).reshape(rows, k)


def nvfp4_exceptional_group(row, groups):
    """qual/src/nvfp4_swiglu.rs:355-357."""
    return (row * 17 + row // 128 * 13) % groups


def nvfp4_weights(rows_w: int, k: int, gate_up_split: int | None):
    """qual/src/nvfp4_swiglu.rs:196-234 (gate_up_split = OUTPUT_ROWS) and
    qual/src/nvfp4_down.rs:196-230 (gate_up_split = None).  Returns (codes [rows_w,k/2],
    swizzled scale plane)."""
    groups = k // 16
    negative = NVFP4_BASE ^ 0x88
    codes = np.zeros((rows_w, groups, 8), dtype=np.uint8)
    scales = np.zeros(rows_w * groups, dtype=np.uint8)
    offs = O.nvfp4_scale_offsets(rows_w, groups)
    for row in range(rows_w):
        base_is_base = (row & 1) == 0
        if gate_up_split is None:
            base = NVFP4_BASE if base_is_base else negative
        elif row < gate_up_split and row & 1:
            base = NVFP4_SPARSE
        elif row >= gate_up_split and row & 1:
            base = negative
        else:
            base = NVFP4_BASE
        exceptional = NVFP4_SPARSE if base_is_base else NVFP4_BASE
        eg = nvfp4_exceptional_group(row, groups)
        codes[row, :, :] = base
        codes[row, eg, :] = exceptional
        sc = np.full(groups, NVFP4_SCALE_CODES[row & 3], dtype=np.uint8)
        sc[eg] = NVFP4_SCALE_CODES[(row + 1) & 3]
        scales[offs[row]] = sc
    return codes.reshape(rows_w, k // 2), scales


def nvfp4_closed_form_dot(x_bits: np.ndarray, token: int, row: int, codes, scales, k: int) -> float:
    """qual/src/nvfp4_swiglu.rs:317-353 (dot_oracle + group_dot): the fixture's closed form."""
    groups = k // 16
    eg = nvfp4_exceptional_group(row, groups)
    og = (eg + 1) % groups
    xf = O.bf16_to_f32(x_bits[token]).astype(np.float64)
    tab = O.e4m3_decode_table().astype(np.float64)

    def group_dot(g):
        s = 0.0
        for c in range(16):
            packed = int(codes[row, g * 8 + c // 2])
            code = (packed >> 4) if (c & 1) else (packed & 15)
            s += xf[g * 16 + c] * O.e2m1_decode(code)
        return s

    so = tab[scales[O.nvfp4_scale_offset(row, og, groups)]]
    se = tab[scales[O.nvfp4_scale_offset(row, eg, groups)]]
    return ((groups - 1) * group_dot(og) * so + group_dot(eg) * se) / NVFP4_WEIGHT_SCALE_DIVISOR


# ------------------------------------------------ dense-FP8 MLP and GDN output (torch builders)
# qual/src/fp8_swiglu.rs:13-20, qual/src/fp8_down.rs:13-20, qual/src/gdn_output.rs:13-16
MLP_TOKEN_FACTORS = np.array([1.0, 0.5, 0.25, 0.125, -1.0, -0.5, -0.25, -0.125], dtype=np.float32)
GDN_OUT_INPUT_PATTERN = np.array([0.875, -0.75, 0.625, -0.5, 0.375, -0.25, 0.125, -0.0625],
                                 dtype=np.float32)
FP8_SWIGLU_ROUTES = (1, 2, 3, 4, 5, 6, 7, 8, 32, 64, 128)  # qual/src/fp8_swiglu.rs:14


def mlp_input(rows: int, columns: int, pattern=FP8_INPUT_PATTERN) -> np.ndarray:
    """make_input of qual/src/fp8_swiglu.rs:165-173 / fp8_down.rs:169-176 / gdn_output.rs:141-148:
    BF16 bits [rows, columns], pattern by flat index, factor by token & 7."""
    idx = np.arange(rows * columns)
    vals = pattern[idx & (len(pattern) - 1)] * MLP_TOKEN_FACTORS[(idx // columns) & 7]
    return O.f32_to_bf16(vals).reshape(rows, columns)


def fp8_swiglu_weights(intermediate: int, hidden: int, device):
    """make_weights of qual/src/fp8_swiglu.rs:175-191: one code per source row,
    WEIGHT_CODES[(row + (row >= I)) & 3]; BF16 scales SCALE_VALUES[row & 3].  Torch tensors."""
    import torch

    rows = torch.arange(2 * intermediate, device=device)
    sel = (rows + (rows >= intermediate).long()) & 3
    codes = torch.from_numpy(WEIGHT_CODES).to(device)[sel][:, None].expand(-1, hidden).contiguous()
    scales = torch.from_numpy(O.f32_to_bf16(SCALE_VALUES).view(np.int16)).to(device)[rows & 3].contiguous()
    return codes, scales


def fp8_swiglu_expected(represented_sum: float, scale: np.float32, intermediate: int) -> np.ndarray:
    """Closed form of qual/src/fp8_swiglu.rs:268-281, f64 [intermediate]."""
    row = np.arange(intermediate)
    up_src = row + intermediate
    base = represented_sum * np.float64(scale)
    gate = base * WEIGHT_VALUES[row & 3].astype(np.float64) * SCALE_VALUES[row & 3].astype(np.float64)
    up = base * WEIGHT_VALUES[(up_src + 1) & 3].astype(np.float64) * SCALE_VALUES[up_src & 3].astype(np.float64)
    return gate / (1.0 + np.exp(-gate)) * up


def fp8_down_weights(hidden: int, intermediate: int, device):
    """make_weights of qual/src/fp8_down.rs:178-194: WEIGHT_CODES[(row + column) & 3]."""
    import torch

    r = torch.arange(hidden, device=device)[:, None]
    c = torch.arange(intermediate, device=device)[None, :]
    codes = torch.from_numpy(WEIGHT_CODES).to(device)[(r + c) & 3].contiguous()
    scales = torch.from_numpy(O.f32_to_bf16(SCALE_VALUES).view(np.int16)).to(device)[r[:, 0] & 3].contiguous()
    return codes, scales


def gdn_output_weights(hidden: int, columns: int, device):
    """make_weights of qual/src/gdn_output.rs:150-166: WEIGHT_CODES[row & 3] along the whole row."""
    import torch

    r = torch.arange(hidden, device=device)
    codes = torch.from_numpy(WEIGHT_CODES).to(device)[r & 3][:, None].expand(-1, columns).contiguous()
    scales = torch.from_numpy(O.f32_to_bf16(SCALE_VALUES).view(np.int16)).to(device)[r & 3].contiguous()
    return codes, scales


# ----------------------------------------------------------------- gated delta net
# qual/src/gdn_prepare.rs:10-29 and qual/src/gdn_recurrence.rs:10-20
GDN_MAX_BATCH = 8
GDN_STATE_ROWS = np.array([7, 0, 5, 2, 6, 1, 4, 3], dtype=np.uint32)
GDN_INPUT_PATTERN = np.array([0.25, -0.125, 0.0625, -0.03125, 0.1875, -0.09375, 0.046875, 0.0],
                             dtype=np.float32)
GDN_WEIGHT_PATTERN = np.array([0.00390625, -0.001953125, 0.0009765625, 0.001953125, -0.00390625,
                               0.00048828125, 0.0014648438, -0.0009765625], dtype=np.float32)
GDN_CONV_PATTERN = np.array([0.5, -0.25, 0.125, 0.25], dtype=np.float32)


def gdn_prepare_fixture(hidden=5120, control_rows=48, qkv_rows=10240, input_rows=16384):
    """qual/src/gdn_prepare.rs:187-230 (fixture): every plane for the maximum batch, BF16 bits."""
    batch = GDN_MAX_BATCH
    idx = np.arange(batch * hidden)
    token = idx // hidden
    inp = O.f32_to_bf16(GDN_INPUT_PATTERN[(idx + token) & 7]
                        * (np.float32(1.0) + token.astype(np.float32) / np.float32(8.0)))
    idx = np.arange(2 * control_rows * hidden)
    row, column = idx // hidden, idx % hidden
    control_weights = O.f32_to_bf16(GDN_WEIGHT_PATTERN[(column + 3 * row) & 7])
    rows = np.arange(control_rows)
    a_log = O.f32_to_bf16(np.float32(-2.0) + (rows & 3).astype(np.float32) * np.float32(0.125))
    dt_bias = O.f32_to_bf16((rows.astype(np.float32) - np.float32(23.5)) / np.float32(256.0))
    idx = np.arange(batch * input_rows)
    token = idx // input_rows
    projected = O.f32_to_bf16(GDN_INPUT_PATTERN[(3 * idx + token) & 7]
                              * (np.float32(1.0) + token.astype(np.float32) / np.float32(16.0)))
    convolution_weights = O.f32_to_bf16(GDN_CONV_PATTERN[np.arange(qkv_rows * 4) & 3])
    idx = np.arange(batch * qkv_rows * 3)
    history = O.f32_to_bf16(GDN_INPUT_PATTERN[(5 * idx + idx // 3) & 7] * np.float32(0.5))
    return dict(input=inp.reshape(batch, hidden),
                control_weights=control_weights.reshape(2 * control_rows, hidden),
                a_log=a_log, dt_bias=dt_bias, projected=projected.reshape(batch, input_rows),
                convolution_weights=convolution_weights.reshape(qkv_rows, 4),
                history=history.reshape(batch, qkv_rows, 3), state_rows=GDN_STATE_ROWS.copy())


def gdn_recurrence_fixture():
    """qual/src/gdn_recurrence.rs:158-198 (fixture)."""
    qk = np.array([0.75, -0.625, 0.5, -0.375, 0.25, -0.1875, 0.125, -0.0625], dtype=np.float32)
    value = np.array([0.5, -0.375, 0.25, -0.125, 0.0625, -0.03125, 0.1875, -0.25], dtype=np.float32)
    gate = np.array([-1.0, -0.5, -0.25, 0.0, 0.25, 0.5, 0.75, 1.0], dtype=np.float32)
    norm = np.array([0.75, 0.875, 1.0, 1.125, 0.625, 1.25, 0.5, 1.5], dtype=np.float32)
    batch, head, heads_k, heads_v = GDN_MAX_BATCH, 128, 16, 48
    qk_width, value_width = heads_k * head, heads_v * head
    qkv_rows, input_rows = 2 * qk_width + value_width, 2 * qk_width + 2 * value_width
    qkv = np.zeros((batch, qkv_rows), dtype=np.uint16)
    projected = np.zeros((batch, input_rows), dtype=np.uint16)
    iq, iv = np.arange(qk_width), np.arange(value_width)
    for token in range(batch):
        qkv[token, :qk_width] = O.f32_to_bf16(qk[(iq + token) & 7])
        qkv[token, qk_width:2 * qk_width] = O.f32_to_bf16(qk[(3 * iq + token + 1) & 7])
        qkv[token, 2 * qk_width:] = O.f32_to_bf16(value[(5 * iv + token) & 7])
        projected[token, qkv_rows:] = O.f32_to_bf16(gate[(iv + iv // head + token) & 7])
    ic = np.arange(batch * heads_v)
    log_decay = (np.float32(-0.125) - (ic & 7).astype(np.float32) * np.float32(0.03125)).astype(np.float32)
    beta = (np.float32(0.25) + (ic & 3).astype(np.float32) * np.float32(0.125)).astype(np.float32)
    norm_weight = O.f32_to_bf16(norm[np.arange(head) & 7])
    istate = np.arange(batch * heads_v * head * head, dtype=np.uint64)
    state = ((((istate * 13) & 31).astype(np.float32) - np.float32(15.5)) / np.float32(2048.0))
    return dict(qkv=qkv, projected=projected, log_decay=log_decay.reshape(batch, heads_v),
                beta=beta.reshape(batch, heads_v), norm_weight=norm_weight,
                state=state.astype(np.float32).reshape(batch, heads_v, head, head),
                state_rows=GDN_STATE_ROWS.copy())
