// FP8 projections for prefill shapes: persistent CTA pairs (tcgen05 cta_group::2) with two
// accumulators in rotation.
//
// The one-tile-per-pair kernel (fp8_pair.cu) pays, per 256-row x 256-token pair tile, a launch
// ramp, an epilogue and -- when the tiles do not fill whole waves -- idle slots: at 2048 tokens
// 512 CTAs run on 296 slots.  Here one pair per two SMs stays resident and walks the tiles (token
// tiles fastest, so that the pairs working on one weight tile run together): the K loop of tile
// j + 1 accumulates into TMEM columns [256, 512) while the epilogue warps still read tile j from
// [0, 256), the ring never drains between tiles, and no slot idles until the last round.  FP8
// needs no scale slots in TMEM, so both 256-column accumulators fit.
//
// Barriers: `full[s]` of the even CTA counts both CTAs' bytes; `empty[s]` and `tmem_full[b]` exist
// in both CTAs and are arrived by tcgen05.commit (to both); `acc_empty[b]` of the even CTA takes
// one arrival per epilogue warp of BOTH CTAs once tile j has left accumulator b.  Every wait is
// bounded.  No load is shared through multicast.
//
// Same arithmetic as the other FP8 kernels: fp32 accumulation over K in order, times the token's
// fp32 scale, times the row's BF16 scale, rounded to BF16 once -- bit-identical to them.
//
// STREAM_K: the launch's work is the sequence of all (tile, K step) pairs, cut into one contiguous
// range per resident pair, so every pair streams the same number of K steps whatever the tile
// count (32 pair tiles of a 256-token QKV launch keep 74 pairs busy instead of 32).  A range
// covers the tail of one tile, whole tiles, and the head of another.  A CTA that holds only part
// of a tile's K range writes its fp32 accumulator ([token][row], its own slot of the context's
// scratch) and takes a ticket on the tile's counter; the CTA that draws the last ticket adds the
// slots in K order (fixed, so launches repeat bit for bit; a split sum is not the unsplit sum's
// bits) and finishes the tile.  Nobody waits for anybody: no spin, and the counters re-arm.
// Measured, it does not pay on this part and stays a switch: with the exchange compiled out the
// even schedule alone is within 6 % of the one-tile-per-pair kernel at 256 tokens (8192 x 5120:
// 19.5 against 20.7 us) and slower at 2048 (92 against 67 us: pairs on consecutive tiles no longer
// read the same weight tile at the same time), and the exchange costs 20-30 us on top.
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
constexpr int kStages = 6;
constexpr int kThreads = 320;          // warp 0 TMA, warp 1 UMMA/TMEM, warps 2-9 epilogue
constexpr int kEpilogueWarps = 8;      // two per TMEM lane quadrant
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr uint32_t kAccCols = 256;     // one accumulator: 128 lanes x 256 fp32 columns
constexpr uint32_t kTmemCols = 512;    // two of them

struct PersistControl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t is_last;
  float a_scale[2][kTok];
};

// One piece of a pair's work: K steps [k0, k1) of pair tile `tile`.
struct Segment {
  int tile, k0, k1;
};

// The segments of pair `pair` of `pairs`: whole tiles pair, pair + pairs, ... or, STREAM_K, the
// pieces of its contiguous range of the launch's tiles x nkb steps.
template <bool STREAM_K>
struct Walk {
  long long g, g_end;
  int nkb, stride;
  __device__ Walk(int pair, int pairs, int tiles, int nkb_) : nkb(nkb_), stride(pairs) {
    if (STREAM_K) {
      const long long steps = static_cast<long long>(tiles) * nkb;
      g = steps * pair / pairs;
      g_end = steps * (pair + 1) / pairs;
    } else {
      g = pair;
      g_end = tiles;
    }
  }
  __device__ bool next(Segment& s) {
    if (g >= g_end) return false;
    if (STREAM_K) {
      s.tile = static_cast<int>(g / nkb);
      s.k0 = static_cast<int>(g - static_cast<long long>(s.tile) * nkb);
      const long long left = g_end - g;
      s.k1 = (nkb - s.k0 <= left) ? nkb : s.k0 + static_cast<int>(left);
      g += s.k1 - s.k0;
    } else {
      s.tile = static_cast<int>(g);
      s.k0 = 0;
      s.k1 = nkb;
      g += stride;
    }
    return true;
  }
};

// The pair whose range holds step `step`: the p with steps * p / pairs <= step < steps * (p + 1) / pairs.
__device__ __forceinline__ int pair_of_step(long long step, long long steps, int pairs) {
  int q = static_cast<int>(step * pairs / steps);
  while (q + 1 < pairs && steps * (q + 1) / pairs <= step) ++q;
  while (q > 0 && steps * q / pairs > step) --q;
  return q;
}

constexpr size_t persist_smem_bytes() {
  return 1024 + static_cast<size_t>(kStages) * kStageBytes + sizeof(PersistControl);
}

__device__ __forceinline__ void epilogue_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
}

template <bool STREAM_K>
__global__ void __launch_bounds__(kThreads, 1)
    fp8_pair_persist_kernel(const __grid_constant__ CUtensorMap tmap_w,
                            const __grid_constant__ CUtensorMap tmap_a, const Fp8ProjParams p) {
  constexpr uint32_t IDESC = umma_idesc_e4m3(2 * kRows, kTok);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  PersistControl* ctl = reinterpret_cast<PersistControl*>(smem + kStages * kStageBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();  // 0 = even CTA (issues the MMAs), 1 = odd
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int tiles_m = (p.rows + kTok - 1) / kTok;
  const int tiles = tiles_m * (p.out_rows / (2 * kRows));
  const int nkb = p.k / kTileKBytes;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&ctl->tmem_full[b], 1);
      mbar_init(&ctl->acc_empty[b], 2 * kEpilogueWarps);
    }
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

  // tile t = row pair * tiles_m + token tile: token tiles vary fastest
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol = l2_policy_evict_last();  // weight tiles are re-read by the other token tiles
      const uint32_t bar0 = mapa_u32(smem_u32(&ctl->full[0]), 0);  // the even CTA's full[0]
      bool ok = true;
      pdl_wait();
      int it = 0;  // stages issued so far, across tiles
      Walk<STREAM_K> walk(pair, pairs, tiles, nkb);
      Segment seg;
      while (ok && walk.next(seg)) {
        const int unit = seg.tile / tiles_m;
        const int tok0 = (seg.tile - unit * tiles_m) * kTok;
        const int row0 = (2 * unit + static_cast<int>(rank)) * kRows;
        for (int i = seg.k0; i < seg.k1 && ok; ++i, ++it) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1;
          ok = mbar_wait(&ctl->empty[s], phase ^ 1, p.status);
          if (!ok) break;
          uint8_t* stage = smem + s * kStageBytes;
          const uint32_t bar = bar0 + static_cast<uint32_t>(s * sizeof(uint64_t));
          if (rank == 0) mbar_arrive_expect_tx(&ctl->full[s], 2u * kStageBytes);
          tma_load_2d_pair(stage, &tmap_w, bar, i * kTileKBytes, row0, pol);
          tma_load_2d_pair(stage + kWTile, &tmap_a, bar, i * kTileKBytes,
                           tok0 + static_cast<int>(rank) * kTokHalf, pol);
        }
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
      int it = 0, round = 0;
      Walk<STREAM_K> walk(pair, pairs, tiles, nkb);
      Segment seg;
      for (; ok && walk.next(seg); ++round) {
        const int b = round & 1;
        if (round >= 2) {
          // the epilogue warps of both CTAs have read segment (round - 2) out of this accumulator
          ok = mbar_wait_cluster(&ctl->acc_empty[b], ((round >> 1) - 1) & 1, p.status);
          if (!ok) break;
          tc_fence_after_sync();
        }
        const uint32_t acc = tmem + static_cast<uint32_t>(b) * kAccCols;
        for (int i = seg.k0; i < seg.k1 && ok; ++i, ++it) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1;
          ok = mbar_wait(&ctl->full[s], phase, p.status);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t base = smem_u32(smem + s * kStageBytes);
          const uint64_t desc_w = umma_desc_sw128(base);
          const uint64_t desc_a = umma_desc_sw128(base + kWTile);
#pragma unroll
          for (int k4 = 0; k4 < kTileKBytes / 32; ++k4) {
            umma_f8f6f4_pair(acc, desc_w + 2 * k4, desc_a + 2 * k4, IDESC, i != seg.k0 || k4 != 0);
          }
          umma_commit_pair(&ctl->empty[s]);
        }
        umma_commit_pair(&ctl->tmem_full[b]);  // also releases both epilogues after a failed wait
      }
      // after a failed wait the epilogues of tiles never issued give up by themselves: their
      // waits are bounded and the status word is already set
    }
  } else {
    // ----------------------------------------------------------------- epilogue
    const int et = threadIdx.x - 64;   // 0..255
    const int quad = warp & 3;         // TMEM lane quadrant this warp may read
    const int part = (warp - 2) >> 2;  // which of the two warps of the quadrant
    const uint32_t acc_empty0 = mapa_u32(smem_u32(&ctl->acc_empty[0]), 0);  // in the even CTA

    pdl_wait();  // activation scales and the output plane belong to the predecessor until now
    int round = 0;
    Walk<STREAM_K> walk(pair, pairs, tiles, nkb);
    Segment seg;
    const long long steps = static_cast<long long>(tiles) * nkb;
    for (; walk.next(seg); ++round) {
      const int b = round & 1;
      const int t = seg.tile;
      const int unit = t / tiles_m;
      const int tok0 = (t - unit * tiles_m) * kTok;
      const int row = quad * 32 + lane;
      const int n = (2 * unit + static_cast<int>(rank)) * kRows + row;
      const bool row_ok = n < p.out_rows;
      const bool whole = !STREAM_K || (seg.k0 == 0 && seg.k1 == nkb);
      {
        const int tok = tok0 + et;
        ctl->a_scale[b][et] = tok < p.rows ? p.act_scales[tok] : 0.0f;
      }
      const float w_scale = row_ok ? bf16_bits_to_f32(p.w_scales[n]) : 0.0f;
      epilogue_barrier();

      const bool got = mbar_wait(&ctl->tmem_full[b], (round >> 1) & 1, p.status);
      tc_fence_after_sync();
      const uint32_t taddr = tmem + static_cast<uint32_t>(b) * kAccCols + (static_cast<uint32_t>(quad * 32) << 16);
      // Scales, rounds and stores 16 tokens of this thread's row.
      auto finish = [&](int c0, const float (&acc)[16]) {
        uint32_t bits[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          bits[j] = f32_to_bf16_bits(__fmul_rn(__fmul_rn(acc[j], ctl->a_scale[b][c0 + j]), w_scale));
        }
        if (row_ok) {
          uint16_t* dst = p.out + static_cast<size_t>(tok0 + c0) * p.out_rows + n;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (tok0 + c0 + j < p.rows) dst[static_cast<size_t>(j) * p.out_rows] = static_cast<uint16_t>(bits[j]);
          }
        }
      };
      // this pair's slot for the piece: 0 for the first segment of its range, 1 for the last
      float* mine = nullptr;
      if (STREAM_K && !whole) {
        mine = p.partials +
               ((static_cast<size_t>(pair) * 2 + (round == 0 ? 0 : 1)) * 2 + rank) * (kRows * kTok) + row * 16;
      }
      if (got) {
#pragma unroll 1
        for (int c0 = part * 16; c0 < kTok; c0 += 32) {
          if (tok0 + c0 >= p.rows) break;  // warp-uniform
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
          if (whole) {
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = __uint_as_float(r[j]);
            finish(c0, acc);
          } else {
            // slot layout [16-token chunk][row][16 tokens]: 64 contiguous bytes per thread
            float4* dst = reinterpret_cast<float4*>(mine + static_cast<size_t>(c0 / 16) * (kRows * 16));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __stcg(dst + j, make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                          __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
            }
          }
        }
      }
      // this warp has read its share of accumulator b
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(acc_empty0 + static_cast<uint32_t>(b * sizeof(uint64_t)));
      // After a wait that ran out the loop goes on (every later wait gives up at its first look):
      // leaving here would strand the other epilogue warps at the named barriers.
      if (STREAM_K && !whole) {
        // The pieces of this CTA's half of the tile: one per pair whose range meets the tile.
        const long long tile_step0 = static_cast<long long>(t) * nkb;
        const int first = pair_of_step(tile_step0, steps, pairs);
        const int last = pair_of_step(tile_step0 + nkb - 1, steps, pairs);
        __threadfence();
        epilogue_barrier();
        if (et == 0) {
          unsigned int* counter = p.counters + 2 * t + rank;
          const unsigned int ticket = atomicAdd(counter, 1u);
          const bool closes = ticket == static_cast<unsigned int>(last - first);
          if (closes) *counter = 0u;  // re-armed for the next launch
          ctl->is_last = closes ? 1u : 0u;
        }
        epilogue_barrier();
        const bool closes = ctl->is_last != 0u;
        if (closes) {
          __threadfence();
          // 16 tokens at a time, up to four pieces side by side: 16 loads of 16 bytes in flight
#pragma unroll 1
          for (int c0 = part * 16; c0 < kTok; c0 += 32) {
            if (tok0 + c0 >= p.rows) break;
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
#pragma unroll 1
            for (int q0 = first; q0 <= last; q0 += 4) {  // K order
              float4 v[4][4];
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                const int q = q0 + w <= last ? q0 + w : last;  // a missing piece: read again, not added
                const bool heads_here = static_cast<int>((steps * q / pairs) / nkb) == t;
                const float4* src = reinterpret_cast<const float4*>(
                    p.partials + ((static_cast<size_t>(q) * 2 + (heads_here ? 0 : 1)) * 2 + rank) * (kRows * kTok) +
                    static_cast<size_t>(c0 / 16) * (kRows * 16) + row * 16);
#pragma unroll
                for (int j = 0; j < 4; ++j) v[w][j] = __ldcg(src + j);
              }
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                if (q0 + w <= last) {
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    acc[4 * j] = __fadd_rn(acc[4 * j], v[w][j].x);
                    acc[4 * j + 1] = __fadd_rn(acc[4 * j + 1], v[w][j].y);
                    acc[4 * j + 2] = __fadd_rn(acc[4 * j + 2], v[w][j].z);
                    acc[4 * j + 3] = __fadd_rn(acc[4 * j + 3], v[w][j].w);
                  }
                }
              }
            }
            finish(c0, acc);
          }
        }
      }
    }
  }

  // Neither CTA may release shared memory or TMEM while the pair still works on it.
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive_relaxed();  // execution order only: nothing here waits for the epilogue's global stores
  cluster_wait_relaxed();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc_pair(tmem, kTmemCols);
  }
}

}  // namespace

cudaError_t fp8_pair_persist_prepare() {
  cudaError_t e = cudaFuncSetAttribute(fp8_pair_persist_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(persist_smem_bytes()));
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(fp8_pair_persist_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(persist_smem_bytes()));
}

size_t fp8_pair_stream_k_scratch_bytes(int pairs) {
  // two slots per pair (head and tail piece of its range), two CTAs, 128 rows x 256 tokens fp32
  return static_cast<size_t>(pairs) * 2 * 2 * kRows * kTok * sizeof(float);
}

cudaError_t launch_fp8_pair_persist(cudaStream_t stream, int pairs, const CUtensorMap& tmap_w,
                                    const CUtensorMap& tmap_a, const Fp8ProjParams& p, bool stream_k) {
  return stream_k ? launch_kernel_cluster(fp8_pair_persist_kernel<true>, dim3(2 * pairs, 1, 1), dim3(kThreads),
                                          persist_smem_bytes(), stream, dim3(2, 1, 1), tmap_w, tmap_a, p)
                  : launch_kernel_cluster(fp8_pair_persist_kernel<false>, dim3(2 * pairs, 1, 1), dim3(kThreads),
                                          persist_smem_bytes(), stream, dim3(2, 1, 1), tmap_w, tmap_a, p);
}

}  // namespace tk100
