// FP8 projections for prefill shapes on CTA pairs (tcgen05 cta_group::2).
//
// At 512 tokens and more the one-CTA kernel (fp8_proj.cu, 128-row x 128-token tiles) is bound
// by operand delivery L2 -> shared memory: 32 KB per 2.1 M MACs.  Here two CTAs of a cluster
// form one UMMA unit on a 256-row x 256-token pair tile; each CTA loads only ITS 128 weight
// rows and ITS 128 tokens (32 KB per 4.2 M MACs, half the bytes per MAC), keeps the accumulator
// of its 128 rows x 256 tokens in 256 TMEM columns and runs its own epilogue.  A CTA needs
// 97 KB of shared memory and half of TMEM, so two CTAs (of different pairs) share an SM and one
// pair's epilogue runs under the other's main loop.  No load is shared through multicast:
// every CTA fetches its own operands.
//
// Barrier protocol per stage s, as in the NVFP4 pair kernel: `full[s]` of the EVEN CTA counts
// the bytes of both CTAs' loads (the odd CTA's TMA names that barrier through its
// shared::cluster address) and the even CTA's UMMA thread waits on it; `empty[s]` exists in
// both CTAs and is arrived by two tcgen05.commit (one per CTA) once the MMAs that read the
// stage are done.
//
// Same arithmetic as the one-CTA kernel (reference: tuisko-kernels-sm89/src/fp8/projection.rs
// :25-140): fp32 accumulation over K in order, times the token's fp32 scale, times the row's
// BF16 scale, rounded to BF16 once.
#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tk100 {

namespace {

constexpr int kRows = 128;        // weight rows per CTA
constexpr int kTok = 256;         // tokens per pair tile
constexpr int kTokHalf = 128;     // tokens whose codes one CTA loads
constexpr int kTileKBytes = 128;  // K bytes (= elements) per stage
constexpr int kWTile = kRows * kTileKBytes;     // 16 KB
constexpr int kATile = kTokHalf * kTileKBytes;  // 16 KB
constexpr int kStageBytes = kWTile + kATile;
// 3 stages (97 KB): two CTAs share an SM.  6 stages (193 KB) for launches with at most one
// CTA per SM anyway, where a 3-stage ring alone cannot cover the load latency.
constexpr int kThreads = 320;          // warp 0 TMA, warp 1 UMMA/TMEM, warps 2-9 epilogue
constexpr int kEpilogueThreads = 256;  // two warps per TMEM lane quadrant
constexpr uint32_t kTmemCols = 256;    // 128 lanes x 256 fp32 columns

template <int kStages>
struct PairControl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full;
  uint32_t tmem_base;
  uint32_t pad;
  float a_scale[kTok];
};

template <int kStages>
constexpr size_t pair_smem_bytes() {
  return 1024 + static_cast<size_t>(kStages) * kStageBytes + sizeof(PairControl<kStages>);
}

__device__ __forceinline__ void pair_epilogue_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
}

template <int kStages>
__global__ void __launch_bounds__(kThreads, kStages <= 3 ? 2 : 1)
    fp8_pair_kernel(const __grid_constant__ CUtensorMap tmap_w,
                    const __grid_constant__ CUtensorMap tmap_a, const Fp8ProjParams p) {
  constexpr uint32_t IDESC = umma_idesc_e4m3(2 * kRows, kTok);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  PairControl<kStages>* ctl = reinterpret_cast<PairControl<kStages>*>(smem + kStages * kStageBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();  // 0 = even CTA (issues the MMAs), 1 = odd
  const int tile_m = blockIdx.x >> 1;        // 256-token tile; token tiles of a row pair run together
  const int pair = blockIdx.y;               // pair of 128-row weight tiles
  const int tok0 = tile_m * kTok;
  const int row0 = (2 * pair + static_cast<int>(rank)) * kRows;  // this CTA's weight rows
  const int nkb = p.k / kTileKBytes;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    mbar_init(&ctl->tmem_full, 1);
    fence_mbar_init();
    prefetch_tensormap(&tmap_w);
    prefetch_tensormap(&tmap_a);
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_last();  // re-read by the other token tiles
      const uint64_t pol_a = l2_policy_evict_last();
      const uint32_t bar0 = mapa_u32(smem_u32(&ctl->full[0]), 0);  // the even CTA's full[0]
      auto bar_of = [&](int s) { return bar0 + static_cast<uint32_t>(s * sizeof(uint64_t)); };
      // First pass over the ring: weights do not depend on the predecessor kernel and are
      // requested before pdl_wait(); the activation codes of the same stages follow it.
      const int pre = nkb < kStages ? nkb : kStages;
      for (int i = 0; i < pre; ++i) {
        if (rank == 0) mbar_arrive_expect_tx(&ctl->full[i], 2u * kStageBytes);
        tma_load_2d_pair(smem + i * kStageBytes, &tmap_w, bar_of(i), i * kTileKBytes, row0, pol_w);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) {
        tma_load_2d_pair(smem + i * kStageBytes + kWTile, &tmap_a, bar_of(i), i * kTileKBytes,
                         tok0 + static_cast<int>(rank) * kTokHalf, pol_a);
      }
      bool ok = true;
      for (int i = pre; i < nkb && ok; ++i) {
        const int s = i % kStages;
        const uint32_t phase = (i / kStages) & 1;
        ok = mbar_wait(&ctl->empty[s], phase ^ 1, p.status);
        if (!ok) break;
        uint8_t* stage = smem + s * kStageBytes;
        if (rank == 0) mbar_arrive_expect_tx(&ctl->full[s], 2u * kStageBytes);
        tma_load_2d_pair(stage, &tmap_w, bar_of(s), i * kTileKBytes, row0, pol_w);
        tma_load_2d_pair(stage + kWTile, &tmap_a, bar_of(s), i * kTileKBytes,
                         tok0 + static_cast<int>(rank) * kTokHalf, pol_a);
      }
      if (!ok) {
        // Give copies already in flight time to land before shared memory is released.
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- UMMA issuer
    if (lane == 0 && rank == 0) {
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % kStages;
        const uint32_t phase = (i / kStages) & 1;
        ok = mbar_wait(&ctl->full[s], phase, p.status);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t base = smem_u32(smem + s * kStageBytes);
        const uint64_t desc_w = umma_desc_sw128(base);
        const uint64_t desc_a = umma_desc_sw128(base + kWTile);
#pragma unroll
        for (int k4 = 0; k4 < kTileKBytes / 32; ++k4) {
          if (TK100_DBG(p, DBG_NO_MMA)) break;
          umma_f8f6f4_pair(tmem, desc_w + 2 * k4, desc_a + 2 * k4, IDESC, (i | k4) != 0);
        }
        umma_commit_pair(&ctl->empty[s]);
      }
      umma_commit_pair(&ctl->tmem_full);  // also releases both epilogues after a failed wait
    }
  } else {
    // ----------------------------------------------------------------- epilogue
    const int et = threadIdx.x - 64;   // 0..255
    const int quad = warp & 3;         // TMEM lane quadrant this warp may read
    const int part = (warp - 2) >> 2;  // which of the two warps of the quadrant
    const int n = row0 + quad * 32 + lane;
    const bool row_ok = n < p.out_rows;

    pdl_wait();  // activation scales and the output plane belong to the predecessor until now
    {
      const int tok = tok0 + et;
      ctl->a_scale[et] = tok < p.rows ? p.act_scales[tok] : 0.0f;
    }
    const float w_scale = row_ok ? bf16_bits_to_f32(p.w_scales[n]) : 0.0f;
    pair_epilogue_barrier();

    mbar_wait(&ctl->tmem_full, 0, p.status);
    tc_fence_after_sync();
    const uint32_t taddr = tmem + (static_cast<uint32_t>(quad * 32) << 16);

    if (!TK100_DBG(p, DBG_NO_EPILOGUE)) {
#pragma unroll 1
      for (int c0 = part * 16; c0 < kTok; c0 += 32) {
        if (tok0 + c0 >= p.rows) break;  // warp-uniform
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        tmem_ld_wait();
        uint32_t bits[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          bits[j] = f32_to_bf16_bits(
              __fmul_rn(__fmul_rn(__uint_as_float(r[j]), ctl->a_scale[c0 + j]), w_scale));
        }
        if (row_ok) {
          uint16_t* dst = p.out + static_cast<size_t>(tok0 + c0) * p.out_rows + n;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (tok0 + c0 + j < p.rows) dst[static_cast<size_t>(j) * p.out_rows] = static_cast<uint16_t>(bits[j]);
          }
        }
      }
    }
  }

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

}  // namespace

cudaError_t fp8_pair_prepare() {
  cudaError_t e = cudaFuncSetAttribute(fp8_pair_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(pair_smem_bytes<3>()));
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(fp8_pair_kernel<6>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(pair_smem_bytes<6>()));
}

cudaError_t launch_fp8_pair(cudaStream_t stream, const CUtensorMap& tmap_w, const CUtensorMap& tmap_a,
                            const Fp8ProjParams& p) {
  const unsigned int tiles_m = (p.rows + kTok - 1) / kTok;
  const unsigned int pairs = p.out_rows / (2 * kRows);
  if (p.deep_ring) {
    return launch_kernel_cluster(fp8_pair_kernel<6>, dim3(2 * tiles_m, pairs, 1), dim3(kThreads),
                                 pair_smem_bytes<6>(), stream, dim3(2, 1, 1), tmap_w, tmap_a, p);
  }
  return launch_kernel_cluster(fp8_pair_kernel<3>, dim3(2 * tiles_m, pairs, 1), dim3(kThreads),
                               pair_smem_bytes<3>(), stream, dim3(2, 1, 1), tmap_w, tmap_a, p);
}

}  // namespace tk100
