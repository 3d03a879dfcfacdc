// Shared device helpers: BF16 / E4M3 / E2M1 conversions with the exact rounding the
// qualification oracles pin, and small block-wide reductions with a fixed order.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tk100 {

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}

// Low half = element 2j, high half = element 2j+1 of a packed BF16 pair.
__device__ __forceinline__ float bf16x2_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16x2_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Round-to-nearest-even f32 -> BF16 bits (cvt.rn.bf16.f32).
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float v) {
  return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(v)));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  return f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16);
}

// Two f32 -> two E4M3FN codes, round-to-nearest-even, saturating to +-448
// (cvt.rn.satfinite.e4m3x2.f32); `lo` lands in the low byte.
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {
  return static_cast<uint32_t>(
      __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}

// One E4M3FN code -> f32 (exact).
__device__ __forceinline__ float e4m3_to_f32(uint32_t code) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(code), __NV_E4M3);
  return __half2float(__half(h));
}

// Two f32 -> two E2M1 codes in one byte, nearest-even, saturating to +-6
// (cvt.rn.satfinite.e2m1x2.f32); `lo` lands in the low nibble.
__device__ __forceinline__ uint32_t f32x2_to_e2m1x2(float lo, float hi) {
  return static_cast<uint32_t>(
      __nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum / max with a fixed evaluation order (bit-reproducible across
// launches): butterfly inside each warp, then every thread folds the per-warp
// values in warp order.  `scratch` holds one float per warp.
template <bool IS_MAX>
__device__ __forceinline__ float block_reduce(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
  for (int i = 1; i < warps; ++i) r = IS_MAX ? fmaxf(r, scratch[i]) : r + scratch[i];
  return r;
}

}  // namespace tk100
