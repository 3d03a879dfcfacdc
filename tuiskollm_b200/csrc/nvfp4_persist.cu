// NVFP4 projections for prefill shapes: persistent CTA pairs (tcgen05 cta_group::2).
//
// What bounds the block-scaled contraction at 2048 tokens is operand delivery from L2 into
// shared memory: a 128-row x 128-token tile moves 36 KB per 4.2 M MACs through the SM's L2 port.
// Here the two CTAs of a cluster form one UMMA unit on a 256-row x 256-token pair tile; each CTA
// loads only ITS 128 weight rows and ITS 128 tokens (38 KB with the scale tiles per 8.4 M MACs),
// holds the accumulator of its 128 rows x 256 tokens in 256 TMEM columns and finishes it itself.
// The wide tile also halves the cost of the scale copies per MAC: three tcgen05.cp per
// 128 x 256 x 64 MMA instead of two per 128 x 128 x 64.
//
// One pair per two SMs stays resident and walks its share of the tiles (token tiles fastest, so
// that the pairs running at the same time read the same weight rows from L2):
//   * warp 0: TMA producer, runs ahead across tile boundaries through one ring;
//   * warp 1 (even CTA): issues the scale copies and the MMAs of both CTAs;
//   * eight epilogue warps: a warp pulls its 128 accumulator columns into registers, hands the
//     accumulator back (the next tile's MMAs start at once) and only then converts and stores.
// No load is shared through multicast: every CTA fetches its own operands.
//
// GATE_UP: the pair is (gate tile r, up tile r) of the same 128 outputs; the gate CTA finishes
// tokens 0-127 of the pair tile, the up CTA tokens 128-255.  The halves the partner finishes are
// stored straight into the partner's exchange buffer (distributed shared memory, one-way stores
// followed by an mbarrier arrival): output bf16(silu(gate * s) * up * s), as the one-CTA kernel
// writes it (tuisko-kernels-sm89/src/nvfp4/swiglu.rs:142-155, 300-320 for the formula).
//
// Barriers (all waits bounded): `full[s]` of the even CTA counts both CTAs' TMA bytes; `empty[s]`
// and `tmem_full` exist in both CTAs and are arrived by tcgen05.commit; `acc_empty` of the even
// CTA takes one arrival per epilogue warp of both CTAs; `xchg_full` / `xchg_empty` pace the
// exchange buffer.
#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tk100 {

namespace {

constexpr int kRows = 128;         // weight rows per CTA
constexpr int kTok = 256;          // tokens per pair tile
constexpr int kTokHalf = 128;      // tokens whose codes one CTA loads
constexpr int kStageKBytes = 128;  // 256 K elements
constexpr int kStageK = 256;
constexpr int kWTile = kRows * kStageKBytes;     // 16 KB
constexpr int kATile = kTokHalf * kStageKBytes;  // 16 KB
constexpr int kSfChunk = 512;
constexpr int kSfTile = 4 * kSfChunk;  // 2 KB: 128 rows x 16 groups
constexpr int kStageBytes = kWTile + kATile + kSfTile /*SFA*/ + 2 * kSfTile /*SFB, 256 tokens*/;
constexpr int kOffA = kWTile;
constexpr int kOffSfa = kOffA + kATile;
constexpr int kOffSfb = kOffSfa + kSfTile;
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;  // warp 0 TMA, warp 1 UMMA/TMEM, 8 epilogue warps
constexpr int kSfSlots = 8;
constexpr int kSfSlotCols = 16;  // SFA [0,4), SFB [4,12)
constexpr uint32_t kAccCols = kTok;
constexpr uint32_t kTmemCols = 512;  // 256 accumulator + 128 scale columns -> next power of two
constexpr int kXchgBytes = kTokHalf * kRows * 4;  // gate/up exchange buffer: [token][row] fp32

__host__ __device__ constexpr int stages_for(bool gate_up) { return gate_up ? 4 : 5; }

template <int STAGES>
struct PersistControl {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full;
  uint64_t acc_empty;
  uint64_t xchg_full;
  uint64_t xchg_empty;
  uint32_t tmem_base;
  uint32_t pad;
};

template <bool GATE_UP>
constexpr size_t persist_smem_bytes() {
  return 1024 + static_cast<size_t>(stages_for(GATE_UP)) * kStageBytes + (GATE_UP ? kXchgBytes : 0) +
         sizeof(PersistControl<stages_for(GATE_UP)>);
}

__device__ __forceinline__ float silu_stable_persist(float v) {
  const float e = -fabsf(v) * 1.4426950408889634f;
  float ex;  // .ftz: 2^e below the normal range reads as 0
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(e));
  return __fdividef(v >= 0.0f ? v : v * ex, 1.0f + ex);
}

// Ten warps: up to 168 registers per thread, 128 of them the accumulator values a warp keeps
// while it finishes them.
template <bool GATE_UP>
__global__ void __launch_bounds__(kThreads, 1)
    nvfp4_persist_kernel(const __grid_constant__ CUtensorMap tmap_w,
                         const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_wsf,
                         const __grid_constant__ CUtensorMap tmap_asf, const Nvfp4Params p) {
  constexpr int STAGES = stages_for(GATE_UP);
  constexpr uint32_t IDESC = umma_idesc_nvfp4(2 * kRows, kTok);
  using Ctl = PersistControl<STAGES>;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  float* xchg = reinterpret_cast<float*>(smem + STAGES * kStageBytes);
  Ctl* ctl = reinterpret_cast<Ctl*>(smem + STAGES * kStageBytes + (GATE_UP ? kXchgBytes : 0));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();  // 0 = even CTA (issues the MMAs), 1 = odd
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int tiles_m = (p.rows + kTok - 1) / kTok;
  const int row_units = GATE_UP ? p.out_rows / kRows : p.out_rows / (2 * kRows);
  const int tiles = tiles_m * row_units;
  const int nkb = (p.k + kStageK - 1) / kStageK;
  const int chunks_per_tile = p.k / 64;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    mbar_init(&ctl->tmem_full, 1);
    mbar_init(&ctl->acc_empty, 2 * kEpilogueWarps);
    mbar_init(&ctl->xchg_full, kEpilogueWarps / 2);   // the partner's four sending warps
    mbar_init(&ctl->xchg_empty, kEpilogueWarps / 2);  // the partner's four finishing warps
    fence_mbar_init();
    prefetch_tensormap(&tmap_w);
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_wsf);
    prefetch_tensormap(&tmap_asf);
  }
  if (warp == 1) {
    tmem_alloc_pair(&ctl->tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  // both CTAs' barriers exist before either touches the other's
  cluster_arrive();
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_base;
  pdl_trigger();

  // tile t = unit * tiles_m + token tile: token tiles vary fastest

#ifdef TK100_EXPERIMENT
  // experiment builds: cycles a role spent waiting, written at exit to stamps[cta * 8 + k]
  // (k: 0 kernel cycles, 1 producer on empty[], 2 issuer on full[], 3 issuer on acc_empty,
  //  4 epilogue warp 0 on tmem_full, 5 epilogue warp 0 busy, 6 epilogue on the exchange)
  long long wait_cycles = 0, wait_cycles2 = 0, busy_cycles = 0;
  const long long kernel_t0 = clock64();
#define TK100_TIMED(acc, expr) do { const long long _t = clock64(); expr; acc += clock64() - _t; } while (0)
#else
#define TK100_TIMED(acc, expr) do { expr; } while (0)
#endif
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol = l2_policy_evict_last();
      bool ok = true;
      pdl_wait();
      int it = 0;  // stages issued so far, across tiles
      for (int t = pair; t < tiles && ok; t += pairs) {
        const int unit = t / tiles_m;
        const int tok0 = (t - unit * tiles_m) * kTok;
        const int w_tile = GATE_UP ? (rank == 0 ? unit : p.up_row_offset / kRows + unit)
                                   : 2 * unit + static_cast<int>(rank);
        for (int i = 0; i < nkb && ok; ++i, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (TK100_DBG(p, 8)) continue;  // experiment: no loads at all (the MMAs run on stale shared memory)
          TK100_TIMED(wait_cycles, ok = mbar_wait(&ctl->empty[s], phase ^ 1, p.status));
          if (!ok) break;
          uint8_t* stage = smem + s * kStageBytes;
          // bytes both CTAs deliver to the even CTA's barrier for this stage (every box counts in
          // full, zero-filled where it reaches past the end of a plane)
          if (rank == 0) mbar_arrive_expect_tx(&ctl->full[s], 2u * kStageBytes);
          const uint32_t bar = mapa_u32(smem_u32(&ctl->full[s]), 0);
          const int kbyte = i * kStageKBytes;
          tma_load_2d_pair(stage, &tmap_w, bar, kbyte, w_tile * kRows, pol);
          tma_load_2d_pair(stage + kOffA, &tmap_a, bar, kbyte, tok0 + static_cast<int>(rank) * kTokHalf, pol);
          // scale planes as [chunk, 128 x u32]: four consecutive 512-byte chunks per 128-row tile
          const int chunk0 = i * 4;
          tma_load_2d_pair(stage + kOffSfa, &tmap_wsf, bar, 0, w_tile * chunks_per_tile + chunk0, pol);
          tma_load_2d_pair(stage + kOffSfb, &tmap_asf, bar, 0, (tok0 / kRows) * chunks_per_tile + chunk0, pol);
          tma_load_2d_pair(stage + kOffSfb + kSfTile, &tmap_asf, bar, 0,
                           (tok0 / kRows + 1) * chunks_per_tile + chunk0, pol);
        }
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- UMMA issuer
    if (lane == 0 && rank == 0) {
      const uint32_t sf_base = tmem + kAccCols;
      bool ok = true;
      int it = 0, round = 0;
      for (int t = pair; t < tiles && ok; t += pairs, ++round) {
        if (round > 0) {
          // the epilogue warps of both CTAs have pulled the previous tile out of TMEM
          TK100_TIMED(wait_cycles2, ok = mbar_wait_cluster(&ctl->acc_empty, (round - 1) & 1, p.status));
          if (!ok) break;
          tc_fence_after_sync();
        }
        for (int i = 0; i < nkb && ok; ++i, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!TK100_DBG(p, 8)) TK100_TIMED(wait_cycles, ok = mbar_wait(&ctl->full[s], phase, p.status));
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t base = smem_u32(smem + s * kStageBytes);
          const uint64_t desc_w = umma_desc_sw128(base);
          const uint64_t desc_a = umma_desc_sw128(base + kOffA);
          const int steps = min(4, (p.k - i * kStageK) / 64);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            if (k4 >= steps) break;
            // Per 64-element step: three scale copies (this CTA's weight rows, the two 128-token
            // scale tiles) into a rotating TMEM slot, then the MMA that reads them.
            const uint32_t slot = sf_base + static_cast<uint32_t>(((it * 4 + k4) % kSfSlots) * kSfSlotCols);
            if (!TK100_DBG(p, 16)) {  // experiment switch: MMAs without the scale copies
              tmem_cp_32x128b_warpx4_pair(slot, umma_desc_noswizzle_rows16(base + kOffSfa + k4 * kSfChunk));
              tmem_cp_32x128b_warpx4_pair(slot + 4, umma_desc_noswizzle_rows16(base + kOffSfb + k4 * kSfChunk));
              tmem_cp_32x128b_warpx4_pair(slot + 8,
                                          umma_desc_noswizzle_rows16(base + kOffSfb + kSfTile + k4 * kSfChunk));
            }
            if (!TK100_DBG(p, DBG_NO_MMA)) {
              umma_nvfp4_pair(tmem, desc_w + 2 * k4, desc_a + 2 * k4, IDESC, slot, slot + 4, (i | k4) != 0);
            }
          }
          umma_commit_pair(&ctl->empty[s]);
        }
        umma_commit_pair(&ctl->tmem_full);  // also releases both epilogues after a failed wait
      }
    }
  } else {
    // ----------------------------------------------------------------- epilogue
    const int ew = warp - 2;    // 0..7
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int part = ew >> 2;   // which 128 of the tile's 256 tokens
    const int row_in_tile = quad * 32 + lane;
    const float s = p.out_scale;
    // GATE_UP: this CTA finishes tokens [mine0, mine0 + 128) of the pair tile and sends the rest
    const int mine0 = rank == 0 ? 0 : kTokHalf;
    const bool sender = GATE_UP && ((part == 1) == (rank == 0));
    pdl_wait();
    int round = 0;
    for (int t = pair; t < tiles; t += pairs, ++round) {
      const int unit = t / tiles_m;
      const int tok0 = (t - unit * tiles_m) * kTok;
      const int out_row0 = GATE_UP ? unit * kRows : (2 * unit + static_cast<int>(rank)) * kRows;
      const int n = out_row0 + row_in_tile;
      const bool row_ok = n < p.out_rows;
      bool got = false;
      if (TK100_DBG(p, 32)) {  // experiment: sleep between looks instead of spinning
        while (!mbar_try_wait(&ctl->tmem_full, round & 1)) __nanosleep(500);
      }
      TK100_TIMED(wait_cycles, got = mbar_wait(&ctl->tmem_full, round & 1, p.status));
      if (!got) break;
#ifdef TK100_EXPERIMENT
      const long long busy_t0 = clock64();
#endif
      tc_fence_after_sync();
      // this warp's 128 columns -> registers, then the accumulator goes back to the MMA thread
      uint32_t r[8][16];
      {
        const uint32_t taddr = ctl->tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                               static_cast<uint32_t>(part * kTokHalf);
#pragma unroll
        for (int c = 0; c < 8; ++c) tmem_ld16(taddr + c * 16, r[c]);
      }
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(mapa_u32(smem_u32(&ctl->acc_empty), 0));

      if (!GATE_UP) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int tokc = tok0 + part * kTokHalf + c * 16;
          if (tokc >= p.rows) break;  // warp-uniform
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (tokc + j < p.rows && row_ok) {
              const size_t o = static_cast<size_t>(tokc + j) * p.out_rows + n;
              const float v = __fmul_rn(__uint_as_float(r[c][j]), s);
              if (p.out_f32) p.out_f32[o] = v;
              else p.out[o] = static_cast<uint16_t>(f32_to_bf16_bits(v));
            }
          }
        }
      } else if (sender) {
        // the partner finishes these 128 tokens: straight into its exchange buffer, once the
        // partner has read the previous tile's values out of it
        bool free_ = true;
        if (round > 0) TK100_TIMED(wait_cycles2, free_ = mbar_wait_cluster(&ctl->xchg_empty, (round - 1) & 1, p.status));
        if (!free_) break;
        const uint32_t dst = mapa_u32(smem_u32(xchg + row_in_tile), rank ^ 1u);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            st_dsmem_f32(dst + static_cast<uint32_t>(c * 16 + j) * kRows * 4, __uint_as_float(r[c][j]));
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(mapa_u32(smem_u32(&ctl->xchg_full), rank ^ 1u));
      } else {
        // finisher: own 128 columns in registers, the partner's values for the same tokens from the
        // exchange buffer
        bool landed_ = false;
        TK100_TIMED(wait_cycles2, landed_ = mbar_wait_cluster(&ctl->xchg_full, round & 1, p.status));
        if (!landed_) break;
        const uint32_t other = smem_u32(xchg + row_in_tile);
        uint16_t* out_col = p.out + static_cast<size_t>(tok0 + mine0) * p.out_rows + n;
        const int live = p.rows - (tok0 + mine0);  // tokens of this half that exist
#pragma unroll
        for (int c = 0; c < 8; ++c) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float landed;
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(landed) : "r"(other + static_cast<uint32_t>((c * 16 + j) * kRows * 4)));
            const float own = __fmul_rn(__uint_as_float(r[c][j]), s);
            const float oth = __fmul_rn(landed, s);
            // the gate CTA holds gate values and receives up values, the up CTA the reverse
            const float v = rank == 0 ? __fmul_rn(silu_stable_persist(own), oth) : __fmul_rn(silu_stable_persist(oth), own);
            if (row_ok && c * 16 + j < live) out_col[static_cast<size_t>(c * 16 + j) * p.out_rows] = static_cast<uint16_t>(f32_to_bf16_bits(v));
          }
        }
        // the exchange buffer may be overwritten by the partner's next tile
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(mapa_u32(smem_u32(&ctl->xchg_empty), rank ^ 1u));
      }
#ifdef TK100_EXPERIMENT
      busy_cycles += clock64() - busy_t0;
#endif
    }
  }
#ifdef TK100_EXPERIMENT
  if (p.stamps && lane == 0) {
    unsigned long long* out = p.stamps + static_cast<size_t>(blockIdx.x) * 8;
    if (warp == 0) { out[0] = clock64() - kernel_t0; out[1] = wait_cycles; }
    if (warp == 1 && rank == 0) { out[2] = wait_cycles; out[3] = wait_cycles2; }
    if (warp == 2) { out[4] = wait_cycles; out[5] = busy_cycles; out[6] = wait_cycles2; }
    if (warp == 6) { out[7] = busy_cycles; }
  }
#endif

  // Neither CTA may release shared memory or TMEM while the pair still works on it (execution
  // order only: nothing here waits for the epilogue's global stores).
  tc_fence_before_sync();
  cluster_arrive_relaxed();
  cluster_wait_relaxed();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc_pair(tmem, kTmemCols);
  }
}

template <bool GATE_UP>
cudaError_t persist_launch(cudaStream_t stream, int pairs, const CUtensorMap& tmap_w,
                           const CUtensorMap& tmap_a, const CUtensorMap& tmap_wsf,
                           const CUtensorMap& tmap_asf, const Nvfp4Params& p) {
  return launch_kernel_cluster(nvfp4_persist_kernel<GATE_UP>, dim3(2 * pairs, 1, 1), dim3(kThreads),
                               persist_smem_bytes<GATE_UP>(), stream, dim3(2, 1, 1), tmap_w, tmap_a,
                               tmap_wsf, tmap_asf, p);
}

}  // namespace

cudaError_t nvfp4_persist_prepare(int* max_pairs) {
  cudaError_t e = cudaFuncSetAttribute(nvfp4_persist_kernel<false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(persist_smem_bytes<false>()));
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(nvfp4_persist_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(persist_smem_bytes<true>()));
  if (e != cudaSuccess) return e;
  // pairs that can be resident at once (clusters of two, one CTA per SM)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 1024, 1, 1);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = persist_smem_bytes<true>();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  e = cudaOccupancyMaxActiveClusters(&clusters, nvfp4_persist_kernel<true>, &cfg);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    clusters = 0;
  }
  if (clusters <= 0) {  // no answer: one pair per two SMs (pairs that do not fit at once simply run later)
    int device = 0, sms = 0;
    if ((e = cudaGetDevice(&device)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return e;
    clusters = sms / 2;
  }
  *max_pairs = clusters;
  return cudaSuccess;
}

cudaError_t launch_nvfp4_persist(cudaStream_t stream, bool gate_up, int pairs, const CUtensorMap& tmap_w,
                                 const CUtensorMap& tmap_a, const CUtensorMap& tmap_wsf,
                                 const CUtensorMap& tmap_asf, const Nvfp4Params& p) {
  return gate_up ? persist_launch<true>(stream, pairs, tmap_w, tmap_a, tmap_wsf, tmap_asf, p)
                 : persist_launch<false>(stream, pairs, tmap_w, tmap_a, tmap_wsf, tmap_asf, p);
}

}  // namespace tk100
