"""Seeded synthetic tensors with the shapes and distributions of the benchmark
configurations (no model checkpoint is involved anywhere in this package).

* activations / residual / branch: BF16 ~ N(0, 1)
* RMSNorm weight: stored zero-centred, BF16 ~ N(0, 0.1) (applied as 1 + w)
* FP8 weights: draw ~ N(0, 0.02), one BF16 scale per output row = bf16(amax_row / 448),
  codes = e4m3_rne_sat(w / scale) against the *represented* BF16 scale
* NVFP4 weights: draw ~ N(0, 0.02), global divisor = 448 * 6 / amax_tensor, one E4M3
  scale per 16 columns = e4m3_rne(divisor * amax_block / 6), codes = e2m1_rne_sat,
  scales stored in 128-row x 4-group tiles (tuisko-model/src/materialize.rs:410-422)

numpy builders serve the parity tests (CPU-side copies feed the oracle); the torch
builders make full-size planes directly on the GPU for the benchmark.
"""
from __future__ import annotations

import numpy as np

# BASELINE configurations (d = 5120 everywhere)
HIDDEN = 5120
INTERMEDIATE = 17408
VOCAB = 248320
QKV_ROWS = 8192          # 24 q heads x 256 + 2 x 4 kv heads x 256
QKV_ROWS_REF = 14336     # the reference's fused query+gate layout
GDN_ROWS = 12288
GDN_ROWS_REF = 16384
EPS = 1e-6


# ----------------------------------------------------------------- numpy codecs

def f32_to_bf16_bits(values) -> np.ndarray:
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFFFFFF) >> 16).astype(np.uint16)


def bf16_bits_to_f32(bits) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def e4m3_encode(values) -> np.ndarray:
    """Vectorised round-to-nearest-even E4M3FN encoder, saturating to +-448."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    sign = np.where(np.signbit(v), 0x80, 0).astype(np.int32)
    a = np.minimum(np.abs(v), np.float32(448.0)).astype(np.float32)
    _, e = np.frexp(a)
    exp2 = np.maximum(e.astype(np.int32) - 1, -6)
    step = np.ldexp(np.float32(1.0), exp2 - 3).astype(np.float32)
    n = np.rint(a / step).astype(np.int32)
    sub = (exp2 == -6) & (n < 8)
    carry = n == 16
    ebits = exp2 + 7 + carry.astype(np.int32)
    n = np.where(carry, 8, n)
    code = np.where(sub, n, (ebits << 3) | (n - 8))
    code = np.where(a == 0, 0, np.minimum(code, 0x7E))
    return (sign | code).astype(np.uint8)


_E4M3_TABLE = None


def e4m3_table() -> np.ndarray:
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        c = np.arange(256)
        e, f = (c >> 3) & 15, c & 7
        mag = np.where(e == 0, f * 2.0 ** -9, (1 + f / 8.0) * 2.0 ** (e - 7.0))
        mag = np.where((e == 15) & (f == 7), np.nan, mag)
        _E4M3_TABLE = np.where(c & 0x80, -mag, mag).astype(np.float32)
    return _E4M3_TABLE


E2M1_MAGNITUDES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def e2m1_encode(values) -> np.ndarray:
    """Nearest-even E2M1 codes (4 bits, bit 3 = sign), saturating to +-6."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    a = np.abs(v)
    mids = (E2M1_MAGNITUDES[:-1] + E2M1_MAGNITUDES[1:]) / 2
    code = np.full(a.shape, 7, dtype=np.int32)
    for c in range(6, -1, -1):
        take = (a < mids[c]) | ((a == mids[c]) & (c % 2 == 0))
        code = np.where(take, c, code)
    return (code | np.where(np.signbit(v), 8, 0)).astype(np.uint8)


def nvfp4_scale_offsets(rows: int, groups: int) -> np.ndarray:
    r = np.arange(rows, dtype=np.int64)[:, None]
    g = np.arange(groups, dtype=np.int64)[None, :]
    return ((r // 128) * (groups // 4) + g // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4


def nvfp4_swizzle(scale_matrix: np.ndarray) -> np.ndarray:
    """[rows, groups] E4M3 scale bytes -> the 128-row x 4-group tile plane."""
    rows, groups = scale_matrix.shape
    plane = np.zeros(((rows + 127) // 128) * 128 * groups, dtype=np.uint8)
    plane[nvfp4_scale_offsets(rows, groups)] = scale_matrix
    return plane


def nvfp4_unswizzle(plane: np.ndarray, rows: int, groups: int) -> np.ndarray:
    return np.asarray(plane)[nvfp4_scale_offsets(rows, groups)]


def nvfp4_reduction_shard(codes: np.ndarray, plane: np.ndarray, k: int, world: int, rank: int):
    """Row-parallel (reduction) shard of an NVFP4 weight plane: the rank's columns of the code
    matrix and a scale plane re-tiled for the narrower matrix."""
    rows = codes.shape[0]
    ks = k // world
    assert ks % 64 == 0
    sc = nvfp4_unswizzle(plane, rows, k // 16)[:, rank * ks // 16:(rank + 1) * ks // 16]
    return (np.ascontiguousarray(codes[:, rank * ks // 2:(rank + 1) * ks // 2]),
            nvfp4_swizzle(np.ascontiguousarray(sc)))


# --------------------------------------------------------------- numpy builders

def rng_for(seed: int, stream: int) -> np.random.Generator:
    """One seed, one counter-based (Philox) stream per tensor."""
    return np.random.Generator(np.random.Philox(key=[seed & 0xFFFFFFFFFFFFFFFF, stream]))


def normal_bf16(seed: int, stream: int, shape, std: float = 1.0) -> np.ndarray:
    x = rng_for(seed, stream).standard_normal(shape, dtype=np.float32) * np.float32(std)
    return f32_to_bf16_bits(x).reshape(shape)


def fp8_weights(seed: int, stream: int, out_rows: int, k: int, std: float = 0.02):
    """(codes u8 [out_rows, k], scales BF16 bits [out_rows])."""
    w = rng_for(seed, stream).standard_normal((out_rows, k), dtype=np.float32) * np.float32(std)
    amax = np.abs(w).max(axis=1)
    scale_bits = f32_to_bf16_bits(np.where(amax == 0, 1.0, amax / np.float32(448.0)))
    scale = bf16_bits_to_f32(scale_bits)
    codes = e4m3_encode(w / scale[:, None])
    return codes, scale_bits


def nvfp4_quantize_weights(w: np.ndarray):
    """fp32 [rows, k] -> (codes u8 [rows, k/2], swizzled E4M3 scales u8, global divisor f32)."""
    rows, k = w.shape
    groups = k // 16
    amax_t = np.float32(np.abs(w).max())
    divisor = np.float32(448.0 * 6.0) / amax_t if amax_t > 0 else np.float32(1.0)
    blocks = w.reshape(rows, groups, 16).astype(np.float32)
    amax_b = np.abs(blocks).max(axis=2)
    sc = e4m3_encode((amax_b * divisor) / np.float32(6.0))
    s = e4m3_table()[sc]
    safe = np.where(s == 0, np.float32(1.0), s)
    q = (blocks * divisor) / safe[:, :, None]
    nib = e2m1_encode(np.where(s[:, :, None] == 0, np.copysign(np.float32(0), blocks), q))
    nib = nib.reshape(rows, k)
    codes = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    plane = np.zeros(((rows + 127) // 128) * 128 * groups, dtype=np.uint8)
    plane[nvfp4_scale_offsets(rows, groups)] = sc
    return codes, plane, np.float32(divisor)


def nvfp4_weights(seed: int, stream: int, rows: int, k: int, std: float = 0.02):
    w = rng_for(seed, stream).standard_normal((rows, k), dtype=np.float32) * np.float32(std)
    return nvfp4_quantize_weights(w)


# --------------------------------------------------------------- torch builders

def torch_normal_bf16(seed: int, stream: int, shape, device, std: float = 1.0):
    import torch

    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + stream) & 0x7FFFFFFFFFFFFFFF)
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)


def torch_fp8_weights(seed: int, stream: int, out_rows: int, k: int, device, std: float = 0.02,
                      chunk_rows: int = 8192):
    """Full-size FP8 plane built on the GPU in row chunks: (codes uint8 [out_rows, k],
    scales bfloat16 [out_rows]).  Same recipe as :func:`fp8_weights`."""
    import torch

    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + stream) & 0x7FFFFFFFFFFFFFFF)
    codes = torch.empty((out_rows, k), dtype=torch.uint8, device=device)
    scales = torch.empty((out_rows,), dtype=torch.bfloat16, device=device)
    for r0 in range(0, out_rows, chunk_rows):
        r1 = min(out_rows, r0 + chunk_rows)
        w = torch.randn((r1 - r0, k), generator=g, device=device, dtype=torch.float32) * std
        amax = w.abs().amax(dim=1)
        s = torch.where(amax == 0, torch.ones_like(amax), amax / 448.0).to(torch.bfloat16)
        q = (w / s.float()[:, None]).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn)
        codes[r0:r1] = q.view(torch.uint8)
        scales[r0:r1] = s
    return codes, scales


def torch_nvfp4_quantize(w):
    """fp32 CUDA tensor [rows, k] -> (codes uint8 [rows, k/2], swizzled scales uint8 [plane],
    divisor float).  Same recipe as :func:`nvfp4_quantize_weights`, on the GPU."""
    import torch

    rows, k = w.shape
    groups = k // 16
    dev = w.device
    amax_t = w.abs().max()
    divisor = (torch.tensor(448.0 * 6.0, dtype=torch.float32, device=dev) / amax_t).float()
    blocks = w.reshape(rows, groups, 16)
    amax_b = blocks.abs().amax(dim=2)
    raw = (amax_b * divisor) / 6.0
    sc8 = raw.clamp(max=448.0).to(torch.float8_e4m3fn)
    s = sc8.float()
    safe = torch.where(s == 0, torch.ones_like(s), s)
    q = (blocks * divisor) / safe[:, :, None]
    a = q.abs()
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=torch.float32, device=dev)
    odd = torch.tensor([0, 1, 0, 1, 0, 1, 0], dtype=torch.bool, device=dev)
    code = torch.zeros_like(a, dtype=torch.uint8)
    for c in range(7):
        up = (a > mids[c]) | ((a == mids[c]) & odd[c])
        code += up.to(torch.uint8)
    code = torch.where((s == 0)[:, :, None], torch.zeros_like(code), code)
    sign = (torch.signbit(blocks).to(torch.uint8) << 3)
    nib = (code | sign).reshape(rows, k)
    codes = (nib[:, 0::2] | (nib[:, 1::2] << 4)).contiguous()
    padded = ((rows + 127) // 128) * 128
    plane = torch.zeros((padded // 128, groups // 4, 32, 4, 4), dtype=torch.uint8, device=dev)
    sc = sc8.view(torch.uint8)
    if padded != rows:
        sc = torch.cat([sc, torch.zeros((padded - rows, groups), dtype=torch.uint8, device=dev)])
    # [tile, quartile, row%32, group/4, group%4] -> [tile, group/4, row%32, quartile, group%4]
    plane.copy_(sc.reshape(padded // 128, 4, 32, groups // 4, 4).permute(0, 3, 2, 1, 4))
    return codes, plane.reshape(-1), float(divisor.item())


def torch_nvfp4_weights(seed: int, stream: int, rows: int, k: int, device, std: float = 0.02):
    import torch

    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + stream) & 0x7FFFFFFFFFFFFFFF)
    w = torch.randn((rows, k), generator=g, device=device, dtype=torch.float32) * std
    return torch_nvfp4_quantize(w)
