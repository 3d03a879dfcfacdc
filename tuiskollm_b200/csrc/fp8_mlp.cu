// Dense-FP8 MLP, first half: gate/up projection + SwiGLU in one kernel,
//   out[m, r] = bf16( silu(gate) * up ),
//   gate = (sum_k a[m,k] * w[r,k])     * a_scale[m] * w_scale[r],
//   up   = (sum_k a[m,k] * w[I + r,k]) * a_scale[m] * w_scale[I + r],
// on the weight plane the reference's operator takes: E4M3 codes [2 * I, K], gate rows first, one
// BF16 scale per row (tuisko-kernels-sm120/src/fp8/swiglu.rs:366-376; device bodies
// device/fp8_swiglu.rs:67-197 for decode, :398-658 for its 32/64/128-token mma.sync routes).
// SiLU in that path's form, v / (1 + ex2(-v * log2 e)) (device/fp8_swiglu.rs:13-15).
//
// Same swap-AB tcgen05 skeleton as the FP8 projection (fp8_proj.cu): a CTA owns the gate tile
// (rows r .. r+127) AND the up tile (rows I + r ..) of the same 128 outputs, so a stage is two
// 128-row x 128-byte weight tiles plus the token tile, two TMEM accumulators share the token
// operand, and the epilogue needs no exchange.  One CTA per SM (136 tiles for I = 17 408): decode
// shapes are one wave of weight streaming, 16 KB + 16 KB in flight per stage.
// The second half of the MLP (per-token E4M3 quantisation of the 17 408-wide intermediate and the
// down projection, fp8/down.rs:197-207) is the generic FP8 projection with K = I.
#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tk100 {

namespace {

constexpr int kRows = 128;       // outputs per CTA (gate rows and up rows each)
constexpr int kTileKBytes = 128; // K bytes per stage (one 128-byte swizzle row)
constexpr int kWTile = kRows * kTileKBytes;
constexpr int kEpilogueWarps = 8;  // two per TMEM lane quadrant, alternate 16-token chunks
constexpr int kThreads = 64 + 32 * kEpilogueWarps;

// Ring depth.  32-token tiles: 5 stages of 36 KB.  128-token tiles: 4 stages of 48 KB when the
// launch is one token tile deep (136 CTAs, one per SM: the deep ring carries the stream), 2 stages
// when it has several token tiles -- then two CTAs share an SM (96 KB each, their two accumulators
// fill the 512 TMEM columns) and one runs its ramp or its SwiGLU epilogue under the other's K loop
// (M = 256: 57.8 -> 48.9 us, M = 512: 97.3 -> 87.0 us, M = 2048: 357.7 -> 315.0 us; a single
// token tile on the shallow ring: 30.9 -> 42.6 us, hence both).
__host__ __device__ constexpr int sw_stages(int block_tok, bool shallow) {
  return block_tok <= 32 ? 5 : (shallow ? 2 : 4);
}
__host__ __device__ constexpr int sw_stage_bytes(int block_tok) { return 2 * kWTile + block_tok * kTileKBytes; }

template <int BLOCK_TOK, bool SHALLOW>
struct SwControl {
  uint64_t full[sw_stages(BLOCK_TOK, SHALLOW)];
  uint64_t empty[sw_stages(BLOCK_TOK, SHALLOW)];
  uint64_t tmem_full;
  float a_scale[BLOCK_TOK];
  uint32_t tmem_base;
  uint32_t pad;
};

template <int BLOCK_TOK, bool SHALLOW>
constexpr size_t sw_smem_bytes() {
  return 1024 + static_cast<size_t>(sw_stages(BLOCK_TOK, SHALLOW)) * sw_stage_bytes(BLOCK_TOK) +
         sizeof(SwControl<BLOCK_TOK, SHALLOW>);
}

__device__ __forceinline__ float silu_fp8_path(float v) {
  float ex;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(-v * 1.4426950408889634f));
  return __fdividef(v, 1.0f + ex);
}

template <int BLOCK_TOK, bool SHALLOW>
__global__ void __launch_bounds__(kThreads, SHALLOW ? 2 : 1)
    fp8_swiglu_kernel(const __grid_constant__ CUtensorMap tmap_w,
                      const __grid_constant__ CUtensorMap tmap_a, const Fp8SwigluParams p) {
  constexpr int STAGES = sw_stages(BLOCK_TOK, SHALLOW);
  constexpr int STAGE_BYTES = sw_stage_bytes(BLOCK_TOK);
  constexpr uint32_t TMEM_COLS = 2 * BLOCK_TOK;  // 64 or 256: gate accumulator, then up
  constexpr uint32_t IDESC = umma_idesc_e4m3(kRows, BLOCK_TOK);
  using Ctl = SwControl<BLOCK_TOK, SHALLOW>;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  Ctl* ctl = reinterpret_cast<Ctl*>(smem + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // token tiles vary fastest so that the CTAs sharing a weight tile run together (L2 reuse)
  const int tile_m = blockIdx.x, tile_n = blockIdx.y;
  const int nkb = p.k / kTileKBytes;
  const int tok0 = tile_m * BLOCK_TOK;
  const int up_row0 = p.intermediate + tile_n * kRows;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    mbar_init(&ctl->tmem_full, 1);
    fence_mbar_init();
    prefetch_tensormap(&tmap_w);
    prefetch_tensormap(&tmap_a);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_base;
  pdl_trigger();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // weights are streamed once when there is a single token tile, shared otherwise
      const uint64_t pol_a = l2_policy_evict_last();
      const uint64_t pol_w = gridDim.x == 1 ? l2_policy_evict_first() : pol_a;
      // weights of the first ring pass do not depend on the predecessor kernel
      const int pre = nkb < STAGES ? nkb : STAGES;
      for (int i = 0; i < pre; ++i) {
        uint8_t* stage = smem + i * STAGE_BYTES;
        mbar_arrive_expect_tx(&ctl->full[i], STAGE_BYTES);
        tma_load_2d(stage, &tmap_w, &ctl->full[i], i * kTileKBytes, tile_n * kRows, pol_w);
        tma_load_2d(stage + kWTile, &tmap_w, &ctl->full[i], i * kTileKBytes, up_row0, pol_w);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) {
        tma_load_2d(smem + i * STAGE_BYTES + 2 * kWTile, &tmap_a, &ctl->full[i], i * kTileKBytes, tok0, pol_a);
      }
      bool ok = true;
      for (int i = pre; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(&ctl->empty[s], ((i / STAGES) & 1) ^ 1, p.status);
        if (!ok) break;
        uint8_t* stage = smem + s * STAGE_BYTES;
        mbar_arrive_expect_tx(&ctl->full[s], STAGE_BYTES);
        tma_load_2d(stage, &tmap_w, &ctl->full[s], i * kTileKBytes, tile_n * kRows, pol_w);
        tma_load_2d(stage + kWTile, &tmap_w, &ctl->full[s], i * kTileKBytes, up_row0, pol_w);
        tma_load_2d(stage + 2 * kWTile, &tmap_a, &ctl->full[s], i * kTileKBytes, tok0, pol_a);
      }
      if (!ok) {
        // Give copies already in flight time to land before shared memory is released.
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- UMMA issuer
    if (lane == 0) {
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(&ctl->full[s], (i / STAGES) & 1, p.status);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t base = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t desc_g = umma_desc_sw128(base);
        const uint64_t desc_u = umma_desc_sw128(base + kWTile);
        const uint64_t desc_a = umma_desc_sw128(base + 2 * kWTile);
#pragma unroll
        for (int k4 = 0; k4 < kTileKBytes / 32; ++k4) {
          // +2 in the address field = +32 bytes along K inside the swizzled row
          umma_f8f6f4(tmem, desc_g + 2 * k4, desc_a + 2 * k4, IDESC, (i | k4) != 0);
          umma_f8f6f4(tmem + BLOCK_TOK, desc_u + 2 * k4, desc_a + 2 * k4, IDESC, (i | k4) != 0);
        }
        umma_commit(&ctl->empty[s]);
      }
      umma_commit(&ctl->tmem_full);  // accumulators complete (also releases the epilogue on error)
    }
  } else {
    // ----------------------------------------------------------------- epilogue
    const int et = threadIdx.x - 64;
    const int quad = warp & 3;         // TMEM lane quadrant of this warp
    const int half = (warp - 2) >> 2;  // which of the two warps of the quadrant
    const int row_in_tile = quad * 32 + lane;
    const int n = tile_n * kRows + row_in_tile;
    const bool row_ok = n < p.intermediate;
    const int valid_tok = min(BLOCK_TOK, p.rows - tok0);

    pdl_wait();  // activation scales and the output plane belong to the predecessor until now
    for (int j = et; j < BLOCK_TOK; j += 32 * kEpilogueWarps) {
      ctl->a_scale[j] = j < valid_tok ? p.act_scales[tok0 + j] : 0.0f;
    }
    const float ws_gate = row_ok ? bf16_bits_to_f32(p.w_scales[n]) : 0.0f;
    const float ws_up = row_ok ? bf16_bits_to_f32(p.w_scales[p.intermediate + n]) : 0.0f;
    asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpilogueWarps) : "memory");

    mbar_wait(&ctl->tmem_full, 0, p.status);
    tc_fence_after_sync();
    const uint32_t taddr = tmem + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
    for (int c0 = half * 16; c0 < BLOCK_TOK; c0 += 32) {
      if (c0 >= valid_tok) break;  // warp-uniform
      uint32_t g[16], u[16];
      tmem_ld16(taddr + c0, g);
      tmem_ld16(taddr + BLOCK_TOK + c0, u);
      tmem_ld_wait();
      // all 16 results first, branch-free, so that their ex2 / rcp chains overlap
      uint32_t bits[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float a = ctl->a_scale[c0 + j];
        const float gate = __fmul_rn(__fmul_rn(__uint_as_float(g[j]), a), ws_gate);
        const float up = __fmul_rn(__fmul_rn(__uint_as_float(u[j]), a), ws_up);
        bits[j] = f32_to_bf16_bits(__fmul_rn(silu_fp8_path(gate), up));
      }
      if (row_ok) {
        uint16_t* dst = p.out + static_cast<size_t>(tok0 + c0) * p.intermediate + n;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c0 + j < valid_tok) dst[static_cast<size_t>(j) * p.intermediate] = static_cast<uint16_t>(bits[j]);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <int BLOCK_TOK, bool SHALLOW>
cudaError_t sw_launch(cudaStream_t stream, const CUtensorMap& tmap_w, const CUtensorMap& tmap_a,
                      const Fp8SwigluParams& p) {
  dim3 grid((p.rows + BLOCK_TOK - 1) / BLOCK_TOK, (p.intermediate + kRows - 1) / kRows, 1);
  return launch_kernel(fp8_swiglu_kernel<BLOCK_TOK, SHALLOW>, grid, dim3(kThreads),
                       sw_smem_bytes<BLOCK_TOK, SHALLOW>(), stream, tmap_w, tmap_a, p);
}

template <int BLOCK_TOK, bool SHALLOW>
cudaError_t sw_prepare() {
  return cudaFuncSetAttribute(fp8_swiglu_kernel<BLOCK_TOK, SHALLOW>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(sw_smem_bytes<BLOCK_TOK, SHALLOW>()));
}

}  // namespace

cudaError_t fp8_swiglu_prepare() {
  cudaError_t e = sw_prepare<32, false>();
  if (e != cudaSuccess) return e;
  if ((e = sw_prepare<128, false>()) != cudaSuccess) return e;
  return sw_prepare<128, true>();
}

cudaError_t launch_fp8_swiglu(cudaStream_t stream, int block_tok, const CUtensorMap& tmap_w,
                              const CUtensorMap& tmap_a, const Fp8SwigluParams& p) {
  if (block_tok == 32) return sw_launch<32, false>(stream, tmap_w, tmap_a, p);
  if (block_tok == 128) {
    // several token tiles: the shallow ring, two CTAs per SM
    return p.rows > 128 ? sw_launch<128, true>(stream, tmap_w, tmap_a, p)
                        : sw_launch<128, false>(stream, tmap_w, tmap_a, p);
  }
  return cudaErrorInvalidValue;
}

}  // namespace tk100
