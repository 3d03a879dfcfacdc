// NVFP4 MLP projections on the block-scaled tcgen05 tensor cores (W4A4).
//
// Weights are the reference's planes unchanged: E2M1 codes [rows_w, K/2] (low nibble = even
// column), one E4M3 scale per 16 columns in 128-row x 4-group tiles
// (tuisko-model/src/materialize.rs:410-422) and an fp32 global divisor, value =
// e2m1 * e4m3(scale) / divisor (tuisko-kernels-sm89/src/nvfp4/swiglu.rs:211-212).  The
// reference multiplies them with BF16 activations on CUDA cores (A16,
// tuisko-kernels-sm89/src/nvfp4/swiglu.rs:166-320, nvfp4/down.rs:158-305); here the
// activations are quantised to the same format per 16-column block (definition in
// nvfp4_quantize_kernel below; the reference has no counterpart for that step) so that
// tcgen05.mma kind::mxf4nvf4.block_scale consumes both operands and their scale tiles
// directly.  That 128 x 4 tile order is exactly what tcgen05.cp.32x128b.warpx4 moves into
// TMEM as a scale-factor operand, so the weight scale plane is streamed as is.
//
// Kernel shape (swap-AB, as the FP8 projection): a CTA owns 128 weight rows x BLOCK_TOK
// tokens; a stage is 256 K-elements: 128 rows x 128 bytes of codes per weight tile, the
// token tile, and 2 KB of scales per tile.  With GATE_UP the CTA holds the gate tile
// (rows r) and the up tile (rows I + r) of the same outputs in two TMEM accumulators and
// the epilogue writes bf16(silu(gate) * up) -- the fusion the reference has
// (nvfp4/swiglu.rs:300-320), now after a tensor-core contraction.
#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tk100 {

namespace {

constexpr int kRows = 128;           // weight rows per tile (UMMA M)
constexpr int kStageKBytes = 128;    // code bytes per row per stage = 256 elements
constexpr int kStageK = 256;         // elements
constexpr int kWTile = kRows * kStageKBytes;  // 16 KB
constexpr int kSfChunk = 512;        // scales of 128 rows x 4 groups (one UMMA K = 64)
constexpr int kSfStage = 4 * kSfChunk;  // 2 KB: 128 rows x 16 groups
constexpr int kThreads = 320;        // warp 0: TMA, warp 1: UMMA + TMEM, warps 2-9: epilogue
// The fused gate/up epilogue at 128 tokens is latency-bound math (ex2, rcp) with one CTA per SM:
// four warps per TMEM lane quadrant instead of two.
__host__ __device__ constexpr int nv_threads(int block_tok, bool gate_up) {
  return (gate_up && block_tok >= 128) ? 576 : kThreads;
}
constexpr int kEpilogueThreads = 256; // two warps per TMEM lane quadrant, alternate 16-column chunks
constexpr int kSfSlots = 8;          // TMEM scale slots in rotation
constexpr int kSfSlotCols = 16;      // columns per slot: SFA0 [0,4) SFA1 [4,8) SFB [8,12)

__host__ __device__ constexpr int nv_stages(int block_tok, bool gate_up) {
  // plain projection: 4 stages (98 KB) at <= 32 tokens and 3 stages (108 KB) at 128, so that
  // two CTAs share an SM (one runs its epilogue or split reduction under the other's loop)
  // 256-token tiles: 4 stages of 54 KB, one CTA per SM
  return gate_up ? (block_tok <= 32 ? 5 : 4) : (block_tok <= 32 ? 4 : block_tok <= 128 ? 3 : 4);
}

__host__ __device__ constexpr int nv_stage_bytes(int block_tok, bool gate_up) {
  // activation scales: one 128-token scale tile per 128 tokens of the tile
  return (gate_up ? 2 : 1) * (kWTile + kSfStage) + block_tok * kStageKBytes +
         (block_tok > 128 ? 2 : 1) * kSfStage;
}

template <int STAGES, int BLOCK_TOK>
struct NvControl {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full;
  uint64_t go;    // a cluster peer's ring is free: this CTA may store into the peer's shared memory
  uint64_t done;  // the peers' stores into this CTA's shared memory have landed
  uint32_t tmem_base;
  uint32_t flag;
};

template <int BLOCK_TOK, bool GATE_UP>
__host__ __device__ constexpr size_t nv_smem_bytes() {
  return 1024 + static_cast<size_t>(nv_stages(BLOCK_TOK, GATE_UP)) *
                    nv_stage_bytes(BLOCK_TOK, GATE_UP) +
         sizeof(NvControl<nv_stages(BLOCK_TOK, GATE_UP), BLOCK_TOK>);
}

__device__ __forceinline__ void nv_epilogue_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
}

// silu(v) in the sign-stable form of the reference's NVFP4 route
// (tuisko-kernels-sm89/src/nvfp4/swiglu.rs:142-155), ex2.approx for the exponential.
__device__ __forceinline__ float silu_stable(float v) {
  const float e = -fabsf(v) * 1.4426950408889634f;
  float ex;  // .ftz: 2^e below the normal range reads as 0, as the e < -126 cut-off did
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(e));
  return __fdividef(v >= 0.0f ? v : v * ex, 1.0f + ex);
}

// One value per lane, a 16-column block = 16 consecutive lanes: the block's E4M3 scale code
// (bits 8..15 of the result) and this lane's E2M1 code (bits 0..3), as nvfp4_quantize_kernel
// defines them.  Kept out of line so that the sixteen calls of an epilogue chunk do not interleave
// (the surrounding kernel runs at its register limit).
static __device__ __noinline__ uint32_t nvfp4_code_of_lane(uint32_t bf16_bits, float divisor) {
  const float v = __uint_as_float(bf16_bits << 16);
  float amax = fmaxf(0.0f, fabsf(v));
#pragma unroll
  for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const uint32_t sc = f32x2_to_e4m3x2(__fdiv_rn(__fmul_rn(amax, divisor), 6.0f), 0.0f) & 0xffu;
  const float sf = e4m3_to_f32(sc);
  const uint32_t nib = sf == 0.0f ? (signbit(v) ? 0x8u : 0u)
                                  : (f32x2_to_e2m1x2(__fdiv_rn(__fmul_rn(v, divisor), sf), 0.0f) & 0xfu);
  return nib | (sc << 8);
}

template <int BLOCK_TOK, bool GATE_UP>
__global__ void __launch_bounds__(nv_threads(BLOCK_TOK, GATE_UP), (GATE_UP || BLOCK_TOK > 128) ? 1 : 2)
    nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w,
                      const __grid_constant__ CUtensorMap tmap_a, const Nvfp4Params p) {
  constexpr int STAGES = nv_stages(BLOCK_TOK, GATE_UP);
  constexpr int STAGE_BYTES = nv_stage_bytes(BLOCK_TOK, GATE_UP);
  constexpr int NW = GATE_UP ? 2 : 1;
  // stage layout: [W0][W1?][A][SFA0][SFA1?][SFB]
  constexpr int OFF_A = NW * kWTile;
  constexpr int OFF_SFA = OFF_A + BLOCK_TOK * kStageKBytes;
  constexpr int OFF_SFB = OFF_SFA + NW * kSfStage;
  constexpr uint32_t ACC_COLS = NW * BLOCK_TOK;
  constexpr uint32_t NEED_COLS = ACC_COLS + kSfSlots * kSfSlotCols;
  constexpr uint32_t TMEM_COLS = NEED_COLS <= 32 ? 32 : NEED_COLS <= 64 ? 64 : NEED_COLS <= 128 ? 128 : NEED_COLS <= 256 ? 256 : 512;
  constexpr uint32_t IDESC = umma_idesc_nvfp4(kRows, BLOCK_TOK);
  using Ctl = NvControl<STAGES, BLOCK_TOK>;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  Ctl* ctl = reinterpret_cast<Ctl*>(smem + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // token tiles vary fastest so that the CTAs sharing a weight tile run together (L2 reuse)
  const int tile_m = blockIdx.x, tile_n = blockIdx.y, split = blockIdx.z;
  const int tiles_m = gridDim.x, tiles_n = gridDim.y;
  // gate/up as a cluster of two plain tiles: CTA 0 = gate tile `pair`, CTA 1 = up tile `pair`
  const bool pair_swiglu = !GATE_UP && p.pair_swiglu != 0;
  const uint32_t pair_rank = pair_swiglu ? cluster_cta_rank() : 0u;
  const int out_tile = pair_swiglu ? tile_n >> 1 : tile_n;
  const int w_tile = pair_swiglu ? (pair_rank == 0 ? out_tile : p.up_row_offset / kRows + out_tile) : tile_n;
  // K is a multiple of 64 (one UMMA K); the last 256-element stage may hold 1..4 such steps.
  const int kb_total = (p.k + kStageK - 1) / kStageK;
  const int kb_begin = static_cast<int>(static_cast<long long>(split) * kb_total / p.splits);
  const int kb_end = static_cast<int>(static_cast<long long>(split + 1) * kb_total / p.splits);
  const int nkb = kb_end - kb_begin;
  const int tok0 = tile_m * BLOCK_TOK;

  // A short weight stream (decode shapes) is queued at L2 whole before anything else: it does
  // not depend on the predecessor kernel, and HBM then works through that kernel's tail and
  // this one's set-up.
  if (warp == 2 && p.l2_prefetch > 0) {
    const int ahead = nkb < p.l2_prefetch ? nkb : p.l2_prefetch;
    const size_t chunks_per_tile = static_cast<size_t>(p.k / 64);
    for (int i = lane; i < ahead; i += 32) {
      const int kb = kb_begin + i;
      const uint32_t sf_bytes = static_cast<uint32_t>(min(4, (p.k - kb * kStageK) / 64)) * kSfChunk;
      tma_prefetch_l2_2d(&tmap_w, kb * kStageKBytes, w_tile * kRows);
      bulk_prefetch_l2(p.w_scales + (static_cast<size_t>(w_tile) * chunks_per_tile) * kSfChunk +
                           static_cast<size_t>(kb) * kSfStage,
                       sf_bytes);
      if (GATE_UP) {
        tma_prefetch_l2_2d(&tmap_w, kb * kStageKBytes, p.up_row_offset + tile_n * kRows);
        bulk_prefetch_l2(p.w_scales +
                             (static_cast<size_t>(p.up_row_offset / kRows + tile_n) * chunks_per_tile) * kSfChunk +
                             static_cast<size_t>(kb) * kSfStage,
                         sf_bytes);
      }
    }
  }

  const bool clustered = !GATE_UP && p.cluster != 0 && p.splits > 1;
  // p.cluster == 2: partial tiles are pushed into a peer's shared memory and summed there (split K:
  // into the leader, which finishes every token; gate/up pairs: each CTA sends the half of its
  // accumulator that the partner finishes), one-way stores and barrier arrivals instead of two
  // cluster barriers around remote loads.
  const bool pushed = !GATE_UP && p.cluster == 2 && (clustered || pair_swiglu);

  // The producer's loads (thread 0 issues all of them).
  const uint64_t pol_a = l2_policy_evict_last();
  // weights are streamed once when there is a single token tile, shared otherwise
  const uint64_t pol_w = tiles_m == 1 ? l2_policy_evict_first() : pol_a;
  // Scale tiles: chunk (tile, kb) of a plane with G = K/16 groups per row starts at
  // ((tile * G/4) + 4 * kb) * 512 bytes and is 2 KB long (4 consecutive 512-byte chunks).
  const size_t chunks_per_tile = static_cast<size_t>(p.k / 64);
  const uint8_t* sfa0 = p.w_scales + (static_cast<size_t>(w_tile) * chunks_per_tile) * kSfChunk;
  const uint8_t* sfa1 =
      p.w_scales + (static_cast<size_t>(p.up_row_offset / kRows + tile_n) * chunks_per_tile) * kSfChunk;
  const uint8_t* sfb = p.a_scales + (static_cast<size_t>(tok0 / kRows) * chunks_per_tile) * kSfChunk;
  auto load_weights = [&](int i, int s) {
    uint8_t* stage = smem + s * STAGE_BYTES;
    const int kb = kb_begin + i;
    const int kbyte = kb * kStageKBytes;
    const size_t sf_off = static_cast<size_t>(kb) * kSfStage;
    // scale bytes of this stage: 512 per 64-element step that exists (the code tiles always
    // arrive as full boxes, zero-filled beyond the end of the row)
    const uint32_t sf_bytes = static_cast<uint32_t>(min(4, (p.k - kb * kStageK) / 64)) * kSfChunk;
    const uint32_t code_bytes = NW * kWTile + BLOCK_TOK * kStageKBytes;
    // a 256-token tile brings a second activation scale tile, when its tokens exist
    const uint32_t sfb_tiles = (BLOCK_TOK > 128 && tok0 + kRows < p.rows) ? 2u : 1u;
    mbar_arrive_expect_tx(&ctl->full[s],
                          TK100_DBG(p, DBG_NO_ACT)
                              ? NW * (kWTile + sf_bytes)
                              : code_bytes + (NW + sfb_tiles) * sf_bytes);
    tma_load_2d(stage, &tmap_w, &ctl->full[s], kbyte, w_tile * kRows, pol_w);
    bulk_load_1d(stage + OFF_SFA, sfa0 + sf_off, sf_bytes, &ctl->full[s], pol_w);
    if (GATE_UP) {
      tma_load_2d(stage + kWTile, &tmap_w, &ctl->full[s], kbyte,
                  p.up_row_offset + tile_n * kRows, pol_w);
      bulk_load_1d(stage + OFF_SFA + kSfStage, sfa1 + sf_off, sf_bytes, &ctl->full[s], pol_w);
    }
  };
  auto load_activations = [&](int i, int s) {
    if (TK100_DBG(p, DBG_NO_ACT)) return;
    uint8_t* stage = smem + s * STAGE_BYTES;
    const int kb = kb_begin + i;
    tma_load_2d(stage + OFF_A, &tmap_a, &ctl->full[s], kb * kStageKBytes, tok0, pol_a);
    const uint32_t sf_bytes = static_cast<uint32_t>(min(4, (p.k - kb * kStageK) / 64)) * kSfChunk;
    bulk_load_1d(stage + OFF_SFB, sfb + static_cast<size_t>(kb) * kSfStage, sf_bytes,
                 &ctl->full[s], pol_a);
    if (BLOCK_TOK > 128 && tok0 + kRows < p.rows) {
      bulk_load_1d(stage + OFF_SFB + kSfStage,
                   sfb + chunks_per_tile * kSfChunk + static_cast<size_t>(kb) * kSfStage, sf_bytes,
                   &ctl->full[s], pol_a);
    }
  };
  const int pre = nkb < STAGES ? nkb : STAGES;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    mbar_init(&ctl->tmem_full, 1);
    mbar_init(&ctl->go, 1);
    // arrivals: one per epilogue warp of every sending CTA
    mbar_init(&ctl->done, pushed ? static_cast<uint32_t>(pair_swiglu ? 1 : p.splits - 1) * (kEpilogueThreads / 32) : 1u);
    ctl->flag = 0u;
    fence_mbar_init();
    // Weights of the first ring pass leave now, ahead of the TMEM allocation and the CTA barrier:
    // they depend on nothing (the activation operands follow after pdl_wait()).
    for (int i = 0; i < pre; ++i) load_weights(i, i);
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
  // the cluster's barriers exist from here on; the matching wait comes just before the first
  // access to a peer's shared memory
  if (pushed) cluster_arrive();

  if (warp == 0) {
    if (lane == 0) {
      // the weights of the first ring pass were requested during set-up
      pdl_wait();
      for (int i = 0; i < pre; ++i) load_activations(i, i);
      bool ok = true;
      for (int i = pre; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (i / STAGES) & 1;
        ok = mbar_wait(&ctl->empty[s], phase ^ 1, p.status);
        if (!ok) break;
        load_weights(i, s);
        load_activations(i, s);
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t sf_base = tmem + ACC_COLS;
      // a BLOCK_TOK < 128 tile sits in one 32-row quartile of its 128-row scale tile:
      // quartile q of the chunk lands in TMEM column q
      const uint32_t sfb_quartile = static_cast<uint32_t>((tok0 % kRows) / 32);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (i / STAGES) & 1;
        ok = mbar_wait(&ctl->full[s], phase, p.status);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t base = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t desc_w0 = umma_desc_sw128(base);
        const uint64_t desc_w1 = umma_desc_sw128(base + kWTile);
        const uint64_t desc_a = umma_desc_sw128(base + OFF_A);
        const int steps = min(4, (p.k - (kb_begin + i) * kStageK) / 64);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          if (k4 >= steps || TK100_DBG(p, DBG_NO_MMA)) break;
          const uint32_t slot = sf_base + static_cast<uint32_t>(((i * 4 + k4) % kSfSlots) * kSfSlotCols);
          tmem_cp_32x128b_warpx4(slot, umma_desc_noswizzle_rows16(base + OFF_SFA + k4 * kSfChunk));
          if (GATE_UP) {
            tmem_cp_32x128b_warpx4(
                slot + 4, umma_desc_noswizzle_rows16(base + OFF_SFA + kSfStage + k4 * kSfChunk));
          }
          tmem_cp_32x128b_warpx4(slot + 8, umma_desc_noswizzle_rows16(base + OFF_SFB + k4 * kSfChunk));
          if (BLOCK_TOK > 128) {  // tokens [128, 256): the next four scale columns
            tmem_cp_32x128b_warpx4(slot + 12,
                                   umma_desc_noswizzle_rows16(base + OFF_SFB + kSfStage + k4 * kSfChunk));
          }
          const uint32_t acc = (i | k4) != 0;
          umma_nvfp4(tmem, desc_w0 + 2 * k4, desc_a + 2 * k4, IDESC, slot, slot + 8 + sfb_quartile, acc);
          if (GATE_UP) {
            umma_nvfp4(tmem + BLOCK_TOK, desc_w1 + 2 * k4, desc_a + 2 * k4, IDESC, slot + 4,
                       slot + 8 + sfb_quartile, acc);
          }
        }
        umma_commit(&ctl->empty[s]);
      }
      umma_commit(&ctl->tmem_full);
    }
  } else {
    const int et = threadIdx.x - 64;   // 0..255
    const int quad = warp & 3;         // TMEM lane quadrant of this warp
    const int half = (warp - 2) >> 2;  // which of the warps of the quadrant
    constexpr int kChunkStride = 16 * ((nv_threads(BLOCK_TOK, GATE_UP) - 64) / 128);
    const int row_in_tile = quad * 32 + lane;
    const int n = out_tile * kRows + row_in_tile;
    const bool row_ok = n < p.out_rows;
    const int valid_tok = min(BLOCK_TOK, p.rows - tok0);
    const float s = p.out_scale;

    pdl_wait();  // scratch and outputs belong to the predecessor until now
    mbar_wait(&ctl->tmem_full, 0, p.status);
    tc_fence_after_sync();
    const uint32_t taddr = tmem + (static_cast<uint32_t>(quad * 32) << 16);

    if (TK100_DBG(p, DBG_NO_EPILOGUE)) {
      // experiment: accumulators left unread
    } else if (GATE_UP) {
#pragma unroll 1
      for (int c0 = half * 16; c0 < BLOCK_TOK; c0 += kChunkStride) {
        if (c0 >= valid_tok) break;
        uint32_t g[16], u[16];
        tmem_ld16(taddr + c0, g);
        tmem_ld16(taddr + BLOCK_TOK + c0, u);
        tmem_ld_wait();
        // all 16 results first, branch-free, so that their ex2/rcp chains overlap
        uint32_t bits[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float gate = __fmul_rn(__uint_as_float(g[j]), s);
          const float up = __fmul_rn(__uint_as_float(u[j]), s);
          bits[j] = f32_to_bf16_bits(__fmul_rn(silu_stable(gate), up));
        }
        uint16_t* dst = p.out + static_cast<size_t>(tok0 + c0) * p.out_rows + n;
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j < valid_tok) dst[static_cast<size_t>(j) * p.out_rows] = static_cast<uint16_t>(bits[j]);
          }
        }
      }
    } else if (pair_swiglu && pushed) {
      // Each CTA finishes half of the token tile: the gate CTA tokens [0, H), the up CTA [H, 2H).
      // It sends the other half of its accumulator straight into the partner's shared memory
      // ([token][row] fp32 over the partner's ring, once the partner says its ring is free).
      constexpr int H = BLOCK_TOK / 2;
      const int send0 = pair_rank == 0 ? H : 0;
      cluster_wait();  // both CTAs have initialised their barriers
      if (et == 0) mbar_arrive_remote(mapa_u32(smem_u32(&ctl->go), pair_rank ^ 1u));  // my ring is free
      mbar_wait_cluster(&ctl->go, 0, p.status);
      const uint32_t slot = mapa_u32(smem_u32(reinterpret_cast<float*>(smem) + row_in_tile), pair_rank ^ 1u);
#pragma unroll 1
      for (int c = half * 16; c < H; c += 32) {
        if (send0 + c >= valid_tok) break;
        uint32_t r[16];
        tmem_ld16(taddr + send0 + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) st_dsmem_f32(slot + static_cast<uint32_t>(c + j) * kRows * 4, __uint_as_float(r[j]));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(mapa_u32(smem_u32(&ctl->done), pair_rank ^ 1u));
    } else if (pair_swiglu) {
      // Each CTA finishes half of the token tile: the gate CTA tokens [0, H), the up CTA
      // [H, 2H).  Here it parks the other half of its accumulator ([token][row] fp32 over the
      // ring, free once tmem_full has fired) for the partner.
      constexpr int H = BLOCK_TOK / 2;
      const int park0 = pair_rank == 0 ? H : 0;
      float* mine = reinterpret_cast<float*>(smem) + row_in_tile;
#pragma unroll 1
      for (int c = half * 16; c < H; c += 32) {
        if (park0 + c >= valid_tok) break;
        uint32_t r[16];
        tmem_ld16(taddr + park0 + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) mine[(c + j) * kRows] = __uint_as_float(r[j]);
      }
    } else if (p.splits == 1) {
#pragma unroll 1
      for (int c0 = half * 16; c0 < BLOCK_TOK; c0 += 32) {
        if (c0 >= valid_tok) break;
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c0 + j < valid_tok && row_ok) {
            const size_t o = static_cast<size_t>(tok0 + c0 + j) * p.out_rows + n;
            const float v = __fmul_rn(__uint_as_float(r[j]), s);
            if (p.out_f32) p.out_f32[o] = v;
            else p.out[o] = static_cast<uint16_t>(f32_to_bf16_bits(v));
          }
        }
      }
    } else if (BLOCK_TOK > 128) {
      // 256-token tiles are launched unsplit only
    } else if (clustered && pushed) {
      const uint32_t rank = cluster_cta_rank();  // = split
      cluster_wait();
      float* land = reinterpret_cast<float*>(smem);  // leader: [split - 1][token][row] over its ring
      if (rank == 0) {
        if (et == 0) {
          for (int r = 1; r < p.splits; ++r) mbar_arrive_remote(mapa_u32(smem_u32(&ctl->go), r));
        }
        mbar_wait_cluster(&ctl->done, 0, p.status);
#pragma unroll 1
        for (int c0 = half * 16; c0 < BLOCK_TOK; c0 += 32) {
          if (c0 >= valid_tok) break;
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j0 = 0; j0 < 16; j0 += 4) {
            if (c0 + j0 < valid_tok) {  // warp-uniform
              float v[8][4];
#pragma unroll
              for (int sp = 1; sp < 8; ++sp) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  v[sp][j] = (sp < p.splits && c0 + j0 + j < valid_tok)
                                 ? land[(static_cast<size_t>(sp - 1) * valid_tok + c0 + j0 + j) * kRows + row_in_tile]
                                 : 0.0f;
                }
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float acc = __fadd_rn(0.0f, __uint_as_float(r[j0 + j]));  // split 0 = this CTA
#pragma unroll
                for (int sp = 1; sp < 8; ++sp) {
                  if (sp < p.splits) acc = __fadd_rn(acc, v[sp][j]);  // fixed split order
                }
                if (c0 + j0 + j < valid_tok && row_ok) {
                  const size_t o = static_cast<size_t>(tok0 + c0 + j0 + j) * p.out_rows + n;
                  const float val = __fmul_rn(acc, s);
                  if (p.out_f32) p.out_f32[o] = val;
                  else p.out[o] = static_cast<uint16_t>(f32_to_bf16_bits(val));
                }
              }
            }
          }
        }
      } else {
        mbar_wait_cluster(&ctl->go, 0, p.status);
        const uint32_t slot = mapa_u32(smem_u32(land + static_cast<size_t>(rank - 1) * valid_tok * kRows + row_in_tile), 0);
#pragma unroll 1
        for (int c0 = half * 16; c0 < BLOCK_TOK; c0 += 32) {
          if (c0 >= valid_tok) break;
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j < valid_tok) st_dsmem_f32(slot + static_cast<uint32_t>(c0 + j) * kRows * 4, __uint_as_float(r[j]));
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(mapa_u32(smem_u32(&ctl->done), 0));
      }
    } else if (clustered) {
      // split-K inside a thread-block cluster: park the partial tile in this CTA's shared
      // memory ([token][row] fp32 over the ring, free once tmem_full has fired)
      float* mine = reinterpret_cast<float*>(smem) + row_in_tile;
#pragma unroll 1
      for (int c0 = half * 16; c0 < BLOCK_TOK; c0 += 32) {
        if (c0 >= valid_tok) break;
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c0 + j < valid_tok) mine[(c0 + j) * kRows] = __uint_as_float(r[j]);
        }
      }
    } else {
      // split-K: fixed-order sum of fp32 partial tiles by the last CTA to arrive
      const size_t tile_elems = static_cast<size_t>(BLOCK_TOK) * kRows;
      const size_t tile_index = (static_cast<size_t>(split) * tiles_m + tile_m) * tiles_n + tile_n;
      float* mine = p.partials + tile_index * tile_elems + row_in_tile;
#pragma unroll 1
      for (int c0 = half * 16; c0 < BLOCK_TOK; c0 += 32) {
        if (c0 >= valid_tok) break;
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c0 + j < valid_tok) __stcg(mine + (c0 + j) * kRows, __uint_as_float(r[j]));
        }
      }
      __threadfence();
      nv_epilogue_barrier();
      if (et == 0) {
        unsigned int* counter = p.counters + tile_m * tiles_n + tile_n;
        const unsigned int ticket = atomicAdd(counter, 1u);
        const bool last = ticket == static_cast<unsigned int>(p.splits - 1);
        if (last) *counter = 0u;
        ctl->flag = last ? 1u : 0u;
      }
      nv_epilogue_barrier();
      if (ctl->flag) {
        __threadfence();
        const size_t split_stride = static_cast<size_t>(tiles_m) * tiles_n * tile_elems;
        const float* base =
            p.partials + (static_cast<size_t>(tile_m) * tiles_n + tile_n) * tile_elems + row_in_tile;
#pragma unroll 1
        for (int j0 = half * 8; j0 < valid_tok; j0 += 16) {
          float v[8][8];  // [split][token]: every load of the batch is issued before the adds
#pragma unroll
          for (int sp = 0; sp < 8; ++sp) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              v[sp][j] = (sp < p.splits && j0 + j < valid_tok)
                             ? __ldcg(base + sp * split_stride + (j0 + j) * kRows)
                             : 0.0f;
            }
          }
          float acc[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc[j] = 0.0f;
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) {
              if (sp < p.splits) acc[j] = __fadd_rn(acc[j], v[sp][j]);  // fixed split order
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (j0 + j < valid_tok && row_ok) {
              const size_t o = static_cast<size_t>(tok0 + j0 + j) * p.out_rows + n;
              const float v = __fmul_rn(acc[j], s);
              if (p.out_f32) p.out_f32[o] = v;
              else p.out[o] = static_cast<uint16_t>(f32_to_bf16_bits(v));
            }
          }
        }
      }
    }
  }

  if (pair_swiglu) {
    if (pushed) {
      if (warp >= 2) mbar_wait_cluster(&ctl->done, 0, p.status);  // the partner's half has landed here
    } else {
      cluster_arrive();
      cluster_wait();
    }
    if (warp >= 2 && !TK100_DBG(p, DBG_NO_EPILOGUE)) {
      constexpr int H = BLOCK_TOK / 2;
      const int quad = warp & 3;
      const int half = (warp - 2) >> 2;
      const int row_in_tile = quad * 32 + lane;
      const int n = out_tile * kRows + row_in_tile;
      const bool row_ok = n < p.out_rows;
      const int valid_tok = min(BLOCK_TOK, p.rows - tok0);
      const int keep0 = pair_rank == 0 ? 0 : H;
      const uint32_t taddr = tmem + (static_cast<uint32_t>(quad * 32) << 16);
      const uint32_t other_addr = smem_u32(reinterpret_cast<float*>(smem) + row_in_tile);
#pragma unroll 1
      for (int c = half * 16; c < H; c += 32) {
        const int c0 = keep0 + c;
        if (c0 >= valid_tok) break;
        uint32_t own[16];
        tmem_ld16(taddr + c0, own);
        float oth[16];
        if (pushed) {  // the partner stored its half into this CTA's shared memory
          const float* landed = reinterpret_cast<const float*>(smem) + row_in_tile;
#pragma unroll
          for (int j = 0; j < 16; ++j) oth[j] = landed[(c + j) * kRows];
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) oth[j] = ld_dsmem_f32(other_addr + (c + j) * kRows * 4, pair_rank ^ 1u);
        }
        tmem_ld_wait();
        uint32_t bits[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float mine_v = __fmul_rn(__uint_as_float(own[j]), p.out_scale);
          const float oth_v = __fmul_rn(oth[j], p.out_scale);
          const float gate = pair_rank == 0 ? mine_v : oth_v;
          const float up = pair_rank == 0 ? oth_v : mine_v;
          bits[j] = f32_to_bf16_bits(__fmul_rn(silu_stable(gate), up));
        }
        if (row_ok && p.out) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j < valid_tok) {
              p.out[static_cast<size_t>(tok0 + c0 + j) * p.out_rows + n] = static_cast<uint16_t>(bits[j]);
            }
          }
        }
        if (BLOCK_TOK == 32 && p.q_codes) {
          // NVFP4 form of the rounded outputs, as nvfp4_quantize_kernel defines it: a block is 16
          // consecutive outputs of a token = 16 lanes of this warp (out_rows is a multiple of
          // 128, so every lane holds a valid row).
          const int groups = p.out_rows >> 4;
          const int g = n >> 4;
          auto store_q = [&](int j, uint32_t nib, uint32_t other, uint32_t scale_code) {
            const int r = tok0 + c0 + j;
            if (!(lane & 1)) {
              p.q_codes[static_cast<size_t>(r) * (p.out_rows >> 1) + (n >> 1)] =
                  static_cast<uint8_t>(nib | (other << 4));
            }
            if (!(lane & 15)) {
              const size_t off = (static_cast<size_t>(r >> 7) * (groups >> 2) + (g >> 2)) * 512 +
                                 static_cast<size_t>(r & 31) * 16 + ((r & 127) >> 5) * 4 + (g & 3);
              p.q_scales[off] = static_cast<uint8_t>(scale_code);
            }
          };
          // decode shapes only (the operator sends larger launches through the quantiser
          // kernel, which is faster there): the valid tokens one after the other
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j < valid_tok) {  // warp-uniform
              const uint32_t packed = nvfp4_code_of_lane(bits[j], p.q_divisor);
              const uint32_t nib = packed & 0xfu;
              store_q(j, nib, __shfl_xor_sync(0xffffffffu, nib, 1), packed >> 8);
            }
          }
        }
      }
    }
    if (pushed) {
      if (warp < 2) cluster_wait();  // completes the barrier every thread arrived on after set-up
    } else {
      cluster_arrive_relaxed();  // both CTAs keep their shared memory until the partner has read it
      cluster_wait_relaxed();
    }
  }

  if (clustered && pushed) {
    if (warp < 2) cluster_wait();  // completes the barrier every thread arrived on after set-up
  } else if (clustered) {
    // CTA `rank` of the cluster finishes tokens rank, rank + S, ...: partials come from the
    // peers' shared memory and are added in split order (fixed => bit-reproducible).
    cluster_arrive();
    cluster_wait();
    if (warp >= 2 && !TK100_DBG(p, DBG_NO_EPILOGUE)) {
      const int quad = warp & 3;
      const int half = (warp - 2) >> 2;
      const int row_in_tile = quad * 32 + lane;
      const int n = tile_n * kRows + row_in_tile;
      const bool row_ok = n < p.out_rows;
      const int valid_tok = min(BLOCK_TOK, p.rows - tok0);
      const uint32_t rank = cluster_cta_rank();
      const uint32_t my_addr = smem_u32(reinterpret_cast<float*>(smem) + row_in_tile);
#pragma unroll 1
      for (int j = static_cast<int>(rank) + half * p.splits; j < valid_tok; j += 2 * p.splits) {
        float v[8];
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) {
          v[sp] = sp < p.splits ? ld_dsmem_f32(my_addr + j * kRows * 4, static_cast<uint32_t>(sp)) : 0.0f;
        }
        float acc = 0.0f;
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) {
          if (sp < p.splits) acc = __fadd_rn(acc, v[sp]);
        }
        if (row_ok) {
          const size_t o = static_cast<size_t>(tok0 + j) * p.out_rows + n;
          const float val = __fmul_rn(acc, p.out_scale);
          if (p.out_f32) p.out_f32[o] = val;
          else p.out[o] = static_cast<uint16_t>(f32_to_bf16_bits(val));
        }
      }
    }
    cluster_arrive_relaxed();  // no CTA's shared memory may go away while a peer still reads it
    cluster_wait_relaxed();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// Activation quantiser, one thread per 16-column block.  This build's own definition (the
// reference never quantises NVFP4 activations), all steps IEEE fp32:
//   amax   = max |x|                              s_code = e4m3_rne_sat((amax * divisor) / 6)
//   s      = decode(s_code)                       code_j = e2m1_rne_sat((x_j * divisor) / s)
// and signed zeros when s == 0.  Scales go to the 128-row x 4-group tile order with
// row = token; entries of rows >= `rows` are left untouched.
__global__ void __launch_bounds__(256)
    nvfp4_quantize_kernel(const uint16_t* __restrict__ x, int rows, int k, float divisor,
                          uint8_t* __restrict__ codes, uint8_t* __restrict__ scales) {
  pdl_trigger();
  pdl_wait();
  const int groups = k >> 4;
  const long long total = static_cast<long long>(rows) * groups;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(idx / groups);
    const int g = static_cast<int>(idx - static_cast<long long>(r) * groups);
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * k + g * 16);
    const uint4 a = src[0], b = src[1];
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float v[16];
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[2 * j] = bf16x2_lo(w[j]);
      v[2 * j + 1] = bf16x2_hi(w[j]);
      amax = fmaxf(amax, fmaxf(fabsf(v[2 * j]), fabsf(v[2 * j + 1])));
    }
    const float raw = __fdiv_rn(__fmul_rn(amax, divisor), 6.0f);
    const uint32_t sc = f32x2_to_e4m3x2(raw, 0.0f) & 0xffu;
    const float s = e4m3_to_f32(sc);
    uint32_t packed[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint32_t byte;
      if (s == 0.0f) {
        byte = (signbit(v[2 * j]) ? 0x08u : 0u) | (signbit(v[2 * j + 1]) ? 0x80u : 0u);
      } else {
        byte = f32x2_to_e2m1x2(__fdiv_rn(__fmul_rn(v[2 * j], divisor), s),
                               __fdiv_rn(__fmul_rn(v[2 * j + 1], divisor), s)) & 0xffu;
      }
      packed[j >> 2] |= byte << (8 * (j & 3));
    }
    *reinterpret_cast<uint2*>(codes + static_cast<size_t>(r) * (k >> 1) + g * 8) =
        make_uint2(packed[0], packed[1]);
    const size_t off = (static_cast<size_t>(r >> 7) * (groups >> 2) + (g >> 2)) * 512 +
                       static_cast<size_t>(r & 31) * 16 + ((r & 127) >> 5) * 4 + (g & 3);
    scales[off] = static_cast<uint8_t>(sc);
  }
}

// fp32 -> BF16 (round to nearest even), 4 values per thread; n is a multiple of 4.
__global__ void __launch_bounds__(256)
    f32_to_bf16_kernel(const float4* __restrict__ in, uint2* __restrict__ out, long long n4) {
  pdl_trigger();
  pdl_wait();
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = in[i];
    out[i] = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
  }
}

template <int BLOCK_TOK, bool GATE_UP>
cudaError_t nv_launch(cudaStream_t stream, const CUtensorMap& tmap_w, const CUtensorMap& tmap_a,
                      const Nvfp4Params& p) {
  const bool pair_swiglu = !GATE_UP && p.pair_swiglu;
  dim3 grid((p.rows + BLOCK_TOK - 1) / BLOCK_TOK,
            (p.out_rows + kRows - 1) / kRows * (pair_swiglu ? 2 : 1), p.splits);
  dim3 cluster(1, 1, 1);
  if (pair_swiglu) cluster = dim3(1, 2, 1);
  else if (!GATE_UP && p.cluster && p.splits > 1) cluster = dim3(1, 1, p.splits);
  return launch_kernel_cluster(nvfp4_gemm_kernel<BLOCK_TOK, GATE_UP>, grid,
                               dim3(nv_threads(BLOCK_TOK, GATE_UP)),
                               nv_smem_bytes<BLOCK_TOK, GATE_UP>(), stream, cluster, tmap_w, tmap_a, p);
}

template <int BLOCK_TOK, bool GATE_UP>
cudaError_t nv_prepare() {
  return cudaFuncSetAttribute(nvfp4_gemm_kernel<BLOCK_TOK, GATE_UP>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(nv_smem_bytes<BLOCK_TOK, GATE_UP>()));
}

}  // namespace

size_t nvfp4_ring_bytes(int block_tok) {
  const int tile = block_tok <= 32 ? 32 : block_tok <= 128 ? 128 : 256;
  return static_cast<size_t>(nv_stages(tile, false)) * nv_stage_bytes(tile, false);
}

cudaError_t nvfp4_prepare() {
  cudaError_t e;
  if ((e = nv_prepare<32, true>()) != cudaSuccess) return e;
  if ((e = nv_prepare<128, true>()) != cudaSuccess) return e;
  if ((e = nv_prepare<32, false>()) != cudaSuccess) return e;
  if ((e = nv_prepare<256, false>()) != cudaSuccess) return e;
  return nv_prepare<128, false>();
}

cudaError_t launch_nvfp4_gemm(cudaStream_t stream, int block_tok, bool gate_up,
                              const CUtensorMap& tmap_w, const CUtensorMap& tmap_a,
                              const Nvfp4Params& p) {
  if (block_tok == 32) {
    return gate_up ? nv_launch<32, true>(stream, tmap_w, tmap_a, p)
                   : nv_launch<32, false>(stream, tmap_w, tmap_a, p);
  }
  if (block_tok == 128) {
    return gate_up ? nv_launch<128, true>(stream, tmap_w, tmap_a, p)
                   : nv_launch<128, false>(stream, tmap_w, tmap_a, p);
  }
  if (block_tok == 256 && !gate_up) return nv_launch<256, false>(stream, tmap_w, tmap_a, p);
  return cudaErrorInvalidValue;
}

cudaError_t launch_f32_to_bf16(cudaStream_t stream, long long n, const float* in, uint16_t* out) {
  const long long n4 = n / 4;
  long long blocks = (n4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  return launch_kernel(f32_to_bf16_kernel, dim3(static_cast<unsigned int>(blocks)), dim3(256), 0,
                       stream, reinterpret_cast<const float4*>(in), reinterpret_cast<uint2*>(out), n4);
}

cudaError_t launch_nvfp4_quantize(cudaStream_t stream, int rows, int k, const uint16_t* x,
                                  float divisor, uint8_t* codes, uint8_t* scales) {
  const long long total = static_cast<long long>(rows) * (k / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_kernel(nvfp4_quantize_kernel, dim3(static_cast<unsigned int>(blocks)), dim3(256), 0,
                       stream, x, rows, k, divisor, codes, scales);
}

}  // namespace tk100
