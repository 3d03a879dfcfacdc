// NVFP4 projections for prefill shapes on CTA pairs (tcgen05 cta_group::2).
//
// The one-CTA kernel (nvfp4.cu) is bound by operand delivery L2 -> shared memory: a 128-row x
// 128-token tile re-reads too many bytes per MAC.  Here two CTAs of a cluster form one UMMA
// unit: a 256-row x 256-token pair tile in which each CTA loads only ITS 128 weight rows and
// ITS 128 tokens (plus the small scale tiles), i.e. 38 KB per stage for the MACs the one-CTA
// kernel needs 72 KB for.  The even CTA issues tcgen05.mma.cta_group::2 for both; each CTA
// keeps the accumulator of its own 128 rows x 256 tokens in its own TMEM and runs its own
// epilogue.  No load is shared through multicast: every CTA fetches its own operands.
//
//   GATE_UP: the pair is (gate tile r, up tile r) of the same 128 outputs.  After the main
//   loop CTA 0 holds gate[128 x 256], CTA 1 holds up[128 x 256]; each parks the half the
//   other needs in shared memory, one cluster barrier, and CTA 0 finishes tokens 0-127,
//   CTA 1 tokens 128-255 reading the partner's values over distributed shared memory.
//
// Barrier protocol per stage s: `full[s]` of the EVEN CTA counts the bytes of both CTAs'
// loads (the odd CTA's TMA names that barrier through its shared::cluster address); the even
// CTA's UMMA thread waits on it.  `empty[s]` exists in both CTAs and is arrived by two
// tcgen05.commit (one per CTA) once the MMAs that read the stage are done.
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
constexpr int kWTile = kRows * kStageKBytes;      // 16 KB
constexpr int kATile = kTokHalf * kStageKBytes;   // 16 KB
constexpr int kSfChunk = 512;
constexpr int kSfTile = 4 * kSfChunk;             // 2 KB: 128 rows x 16 groups
constexpr int kStageBytes = kWTile + kATile + kSfTile /*SFA*/ + 2 * kSfTile /*SFB, 256 tokens*/;
constexpr int kStages = 5;
constexpr int kThreads = 320;  // warp 0 TMA, warp 1 UMMA/TMEM, warps 2-9 epilogue
constexpr int kOffA = kWTile;
constexpr int kOffSfa = kOffA + kATile;
constexpr int kOffSfb = kOffSfa + kSfTile;
constexpr int kSfSlots = 8;
constexpr int kSfSlotCols = 16;  // SFA [0,4), SFB [4,12)
constexpr uint32_t kAccCols = kTok;
constexpr uint32_t kTmemCols = 512;  // 256 accumulator + 128 scale columns -> next power of two

struct PairControl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full;
  uint32_t tmem_base;
  uint32_t flag;
};

constexpr size_t kSmemBytes = 1024 + static_cast<size_t>(kStages) * kStageBytes + sizeof(PairControl);

__device__ __forceinline__ float silu_stable_pair(float v) {
  const float e = -fabsf(v) * 1.4426950408889634f;
  float ex;  // .ftz: 2^e below the normal range reads as 0
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(e));
  return __fdividef(v >= 0.0f ? v : v * ex, 1.0f + ex);
}

template <bool GATE_UP>
__global__ void __launch_bounds__(kThreads, 1)
    nvfp4_pair_kernel(const __grid_constant__ CUtensorMap tmap_w,
                      const __grid_constant__ CUtensorMap tmap_a,
                      const __grid_constant__ CUtensorMap tmap_wsf,
                      const __grid_constant__ CUtensorMap tmap_asf, const Nvfp4Params p) {
  constexpr uint32_t IDESC = umma_idesc_nvfp4(2 * kRows, kTok);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  PairControl* ctl = reinterpret_cast<PairControl*>(smem + kStages * kStageBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();  // 0 = even CTA (issues the MMAs), 1 = odd
  const int tile_m = blockIdx.x >> 1;        // 256-token tile
  const int pair = blockIdx.y;               // pair of weight tiles
  const int tok0 = tile_m * kTok;
  // weight tile (128 rows) of this CTA, in units of 128-row tiles of the weight plane
  const int w_tile = GATE_UP ? (rank == 0 ? pair : p.up_row_offset / kRows + pair) : 2 * pair + static_cast<int>(rank);
  // first output row this CTA's accumulator lanes stand for
  const int out_row0 = GATE_UP ? pair * kRows : w_tile * kRows;
  const int nkb = (p.k + kStageK - 1) / kStageK;
  const int chunks_per_tile = p.k / 64;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    mbar_init(&ctl->tmem_full, 1);
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

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol = l2_policy_evict_last();
      bool ok = true;
      pdl_wait();
      for (int i = 0; i < nkb && ok; ++i) {
        if (TK100_DBG(p, 8)) break;  // experiment: no loads at all (the MMAs run on stale shared memory)
        const int s = i % kStages;
        const uint32_t phase = (i / kStages) & 1;
        ok = mbar_wait(&ctl->empty[s], phase ^ 1, p.status);
        if (!ok) break;
        uint8_t* stage = smem + s * kStageBytes;
        // bytes both CTAs deliver to the even CTA's barrier for this stage (every box counts in
        // full, zero-filled where it reaches past the end of a plane)
        if (rank == 0) mbar_arrive_expect_tx(&ctl->full[s], 2u * kStageBytes);
        const uint32_t bar = mapa_u32(smem_u32(&ctl->full[s]), 0);
        const int kbyte = i * kStageKBytes;
        tma_load_2d_pair(stage, &tmap_w, bar, kbyte, w_tile * kRows, pol);
        tma_load_2d_pair(stage + kOffA, &tmap_a, bar, kbyte, tok0 + static_cast<int>(rank) * kTokHalf, pol);
        // scale planes as [chunk, 128 x u32]: `steps` consecutive 512-byte chunks per 128-row tile
        const int chunk0 = i * 4;
        tma_load_2d_pair(stage + kOffSfa, &tmap_wsf, bar, 0, w_tile * chunks_per_tile + chunk0, pol);
        tma_load_2d_pair(stage + kOffSfb, &tmap_asf, bar, 0, (tok0 / kRows) * chunks_per_tile + chunk0, pol);
        tma_load_2d_pair(stage + kOffSfb + kSfTile, &tmap_asf, bar, 0,
                         (tok0 / kRows + 1) * chunks_per_tile + chunk0, pol);
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t sf_base = tmem + kAccCols;
      // Per 64-element step: three scale copies (this CTA's weight rows, the two 128-token
      // scale tiles) into a rotating TMEM slot, then the MMA that reads them.  (Queueing a whole
      // stage's copies ahead of the previous stage's MMAs was measured and is slower: the
      // copies take tensor-pipe time of their own, about 60 cycles each.)
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % kStages;
        const uint32_t phase = (i / kStages) & 1;
        if (!TK100_DBG(p, 8)) ok = mbar_wait(&ctl->full[s], phase, p.status);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t base = smem_u32(smem + s * kStageBytes);
        const uint64_t desc_w = umma_desc_sw128(base);
        const uint64_t desc_a = umma_desc_sw128(base + kOffA);
        const int steps = min(4, (p.k - i * kStageK) / 64);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          if (k4 >= steps || TK100_DBG(p, DBG_NO_MMA)) break;
          const uint32_t slot = sf_base + static_cast<uint32_t>(((i * 4 + k4) % kSfSlots) * kSfSlotCols);
          if (!TK100_DBG(p, 16)) {  // experiment switch: MMAs without the scale copies
            tmem_cp_32x128b_warpx4_pair(slot, umma_desc_noswizzle_rows16(base + kOffSfa + k4 * kSfChunk));
            tmem_cp_32x128b_warpx4_pair(slot + 4, umma_desc_noswizzle_rows16(base + kOffSfb + k4 * kSfChunk));
            tmem_cp_32x128b_warpx4_pair(slot + 8,
                                        umma_desc_noswizzle_rows16(base + kOffSfb + kSfTile + k4 * kSfChunk));
          }
          umma_nvfp4_pair(tmem, desc_w + 2 * k4, desc_a + 2 * k4, IDESC, slot, slot + 4, (i | k4) != 0);
        }
        umma_commit_pair(&ctl->empty[s]);
      }
      umma_commit_pair(&ctl->tmem_full);
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row_in_tile = quad * 32 + lane;
    const int n = out_row0 + row_in_tile;
    const bool row_ok = n < p.out_rows;
    const float s = p.out_scale;
    pdl_wait();
    mbar_wait(&ctl->tmem_full, 0, p.status);
    tc_fence_after_sync();
    const uint32_t taddr = tmem + (static_cast<uint32_t>(quad * 32) << 16);

    if (TK100_DBG(p, DBG_NO_EPILOGUE)) {
      // experiment: accumulator left unread
    } else if (!GATE_UP) {
#pragma unroll 1
      for (int c0 = half * 16; c0 < kTok; c0 += 32) {
        if (tok0 + c0 >= p.rows) break;
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int tok = tok0 + c0 + j;
          if (tok < p.rows && row_ok) {
            const size_t o = static_cast<size_t>(tok) * p.out_rows + n;
            const float v = __fmul_rn(__uint_as_float(r[j]), s);
            if (p.out_f32) p.out_f32[o] = v;
            else p.out[o] = static_cast<uint16_t>(f32_to_bf16_bits(v));
          }
        }
      }
    } else {
      // Park the half the partner finishes: CTA 0 (gate) parks tokens 128-255, CTA 1 (up) parks
      // tokens 0-127, as [token][row] fp32 over the (now free) ring.
      float* park = reinterpret_cast<float*>(smem) + row_in_tile;
      const int foreign0 = rank == 0 ? kTokHalf : 0;
#pragma unroll 1
      for (int c0 = half * 16; c0 < kTokHalf; c0 += 32) {
        uint32_t r[16];
        tmem_ld16(taddr + foreign0 + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) park[(c0 + j) * kRows] = __uint_as_float(r[j]);
      }
    }
  }

  if (GATE_UP) {
    cluster_arrive();
    cluster_wait();
    if (warp >= 2 && !TK100_DBG(p, DBG_NO_EPILOGUE)) {
      const int quad = warp & 3;
      const int half = (warp - 2) >> 2;
      const int row_in_tile = quad * 32 + lane;
      const int n = out_row0 + row_in_tile;
      const bool row_ok = n < p.out_rows;
      const float s = p.out_scale;
      const uint32_t taddr = tmem + (static_cast<uint32_t>(quad * 32) << 16);
      const int mine0 = rank == 0 ? 0 : kTokHalf;  // tokens this CTA finishes
      const uint32_t park_addr = smem_u32(reinterpret_cast<float*>(smem) + row_in_tile);
#pragma unroll 1
      for (int c0 = half * 16; c0 < kTokHalf; c0 += 32) {
        if (tok0 + mine0 + c0 >= p.rows) break;
        uint32_t r[16];
        tmem_ld16(taddr + mine0 + c0, r);
        float other[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) other[j] = ld_dsmem_f32(park_addr + (c0 + j) * kRows * 4, rank ^ 1u);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int tok = tok0 + mine0 + c0 + j;
          if (tok < p.rows && row_ok) {
            const float own = __fmul_rn(__uint_as_float(r[j]), s);
            const float oth = __fmul_rn(other[j], s);
            const float gate = rank == 0 ? own : oth;
            const float up = rank == 0 ? oth : own;
            p.out[static_cast<size_t>(tok) * p.out_rows + n] =
                static_cast<uint16_t>(f32_to_bf16_bits(__fmul_rn(silu_stable_pair(gate), up)));
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

size_t nvfp4_pair_smem_bytes() { return kSmemBytes; }

cudaError_t nvfp4_pair_prepare() {
  cudaError_t e = cudaFuncSetAttribute(nvfp4_pair_kernel<false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kSmemBytes));
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(nvfp4_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(kSmemBytes));
}

cudaError_t launch_nvfp4_pair(cudaStream_t stream, bool gate_up, const CUtensorMap& tmap_w,
                              const CUtensorMap& tmap_a, const CUtensorMap& tmap_wsf,
                              const CUtensorMap& tmap_asf, const Nvfp4Params& p) {
  const unsigned int tiles_m = (p.rows + kTok - 1) / kTok;
  const unsigned int pairs = gate_up ? p.out_rows / kRows : p.out_rows / (2 * kRows);
  dim3 grid(2 * tiles_m, pairs, 1);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned int n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  attr[n].id = cudaLaunchAttributeClusterDimension;
  attr[n].val.clusterDim.x = 2;
  attr[n].val.clusterDim.y = 1;
  attr[n].val.clusterDim.z = 1;
  ++n;
  cfg.attrs = attr;
  cfg.numAttrs = n;
  if (gate_up) {
    return cudaLaunchKernelEx(&cfg, nvfp4_pair_kernel<true>, tmap_w, tmap_a, tmap_wsf, tmap_asf, p);
  }
  return cudaLaunchKernelEx(&cfg, nvfp4_pair_kernel<false>, tmap_w, tmap_a, tmap_wsf, tmap_asf, p);
}

}  // namespace tk100
