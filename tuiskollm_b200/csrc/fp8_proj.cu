// FP8-E4M3 projection  out[m, n] = bf16( (sum_k a[m,k] * w[n,k]) * a_scale[m] * w_scale[n] )
// for the QKV, GDN-input and LM-head planes, any 1 <= M, on the tcgen05 tensor cores.
//
// The reference computes this on CUDA cores, one warp per two weight rows, decoding
// every weight byte in registers (tuisko-kernels-sm120/src/device/fp8_projection.rs:190-354)
// and has one mma.sync route for exactly 16 tokens (:394-603).  Here the weight plane is
// the 128-row UMMA operand ("swap-AB"): a CTA owns 128 weight rows x BLOCK_TOK tokens,
// TMA streams 128-row x 128-byte weight tiles (128-byte swizzle) and the matching
// activation-code tile through a shared-memory ring, one thread issues
// tcgen05.mma kind::f8f6f4 into a TMEM accumulator (lane = weight row, column = token)
// and four warps read it back with tcgen05.ld for the scale epilogue.  No CUDA core
// touches a weight byte, so decode shapes are bounded by HBM alone.
//
// Small planes do not fill 148 SMs with 128-row tiles, so K can be split over
// gridDim.z: every split writes its fp32 partial tile to scratch, the last CTA to
// arrive (ticket counter) adds the partials in split order -- a fixed order, so the
// result is bit-reproducible -- applies the epilogue and re-arms the counter.
//
// LM head: the same epilogue also folds a greedy argmax.  Key = the BF16-rounded
// logit in IEEE total order, ties to the lowest index, exactly the host rule at
// tuisko-engine/src/sampling.rs:162-173: 64-bit atomicMax on (key << 32 | ~index).
#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tk100 {

namespace {

constexpr int kTileRows = 128;   // weight rows per CTA (UMMA M)
constexpr int kTileKBytes = 128; // K bytes per stage (one 128-byte swizzle row)
constexpr int kWStageBytes = kTileRows * kTileKBytes;
constexpr int kThreads = 192;    // warp 0: TMA, warp 1: UMMA + TMEM, warps 2-5: epilogue
constexpr int kEpilogueThreads = 128;
constexpr int kMaxSplits = 8;     // upper bound of gridDim.z (the host never asks for more)

// DEEP: a longer ring for launches that put at most two CTAs on an SM anyway (few tiles):
// the same bytes in flight per SM with fewer CTAs.
// WIDE (ring 2, 16-token tiles only): a 3-stage ring so that four CTAs share an SM, for unsplit
// launches whose tile count lies between three and four CTAs per SM (a 4-way LM-head shard:
// 485 tiles) and would otherwise leave a short second wave.
__host__ __device__ constexpr int stages_for(int block_tok, int ring = 0) {
  if (ring == 2) return 3;
  if (ring == 1) return block_tok <= 16 ? 6 : block_tok <= 32 ? 5 : block_tok <= 64 ? 4 : block_tok <= 128 ? 6 : 4;
  // <= 32 tokens: three CTAs share an SM (a third slot lets the next kernel's CTAs start their
  // weight prefetch under this kernel's tail); 64 and 128: two (one CTA's epilogue runs under
  // the other's main loop); 256: one.
  return block_tok <= 16 ? 4 : block_tok <= 32 ? 3 : block_tok <= 64 ? 4 : block_tok <= 128 ? 3 : 4;
}

template <int BLOCK_TOK>
struct Control {
  uint64_t full[stages_for(BLOCK_TOK, 1)];
  uint64_t empty[stages_for(BLOCK_TOK, 1)];
  uint64_t tmem_full;
  uint64_t go;    // split-K on a leader: the leader's ring is free, peers may store into it
  uint64_t done;  // split-K on a leader: every peer's partial tile has landed (leader only)
  uint32_t red[BLOCK_TOK];  // per-token argmax keys of this CTA (local_key)
  float a_scale[BLOCK_TOK];
  float q_amax[4][kFusedQuantRows];  // fused quantiser: per-warp maxima of the epilogue warps
  uint32_t tmem_base;
  uint32_t is_last;
  uint32_t tail_last;                // fused tail: this CTA is the last of the launch
  uint32_t tail_step;
};

template <int BLOCK_TOK, int DEEP = 0>
__host__ __device__ constexpr size_t smem_bytes_for() {
  return 1024 /* alignment slack */ +
         static_cast<size_t>(stages_for(BLOCK_TOK, DEEP)) * (kWStageBytes + BLOCK_TOK * kTileKBytes) +
         sizeof(Control<BLOCK_TOK>);
}

__device__ __forceinline__ void epilogue_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
}

// IEEE total-order key of an f32 bit pattern: larger key <=> greater under total_cmp.
__device__ __forceinline__ uint32_t total_order_key(uint32_t bits) {
  return bits ^ ((bits & 0x80000000u) ? 0xffffffffu : 0x80000000u);
}

__device__ __forceinline__ ArgmaxPair unpack_key(unsigned long long packed) {
  const uint32_t key = static_cast<uint32_t>(packed >> 32);
  ArgmaxPair o;
  o.value = __uint_as_float(key ^ ((key & 0x80000000u) ? 0x80000000u : 0xffffffffu));
  o.index = packed == 0ull ? -1 : static_cast<int32_t>(0xffffffffu - static_cast<uint32_t>(packed));
  return o;
}

// Inside one CTA (128 consecutive weight rows) a candidate travels as 32 bits: the 16 significant
// bits of the BF16 logit's order key above 128 - row in tile (1..128, so a lower row wins a tie and
// 0 means "no candidate").  32-bit shuffles and native shared-memory maxima instead of 64-bit ones;
// global_key() widens the CTA's winner to the packed (order key, ~index) word the merge works on.
__device__ __forceinline__ uint32_t local_key(uint32_t bf16_bits, int row_in_tile) {
  return (total_order_key(bf16_bits << 16) & 0xffff0000u) | static_cast<uint32_t>(128 - row_in_tile);
}

__device__ __forceinline__ unsigned long long global_key(uint32_t local, uint32_t first_index) {
  const uint32_t high = local & 0xffff0000u;
  // low half of the order key of a value whose low 16 bits are zero: ones for a negative value
  // (top key bit clear), zeros otherwise
  const uint32_t order = high | ((high & 0x80000000u) ? 0u : 0xffffu);
  const uint32_t index = first_index + (128u - (local & 0xffffu));
  return (static_cast<unsigned long long>(order) << 32) |
         static_cast<unsigned long long>(0xffffffffu - index);
}

// Vocabulary-sharded greedy selection without a collective library call.  The calling threads
// (`tid` of `nthreads`, one CTA) unpack this rank's packed (max, index) keys, store them straight
// into every peer's exchange buffer over NVLink (plain peer stores), clear the keys, then wait --
// bounded -- for the pairs of all peers in this rank's own buffer and merge with the
// first-maximum rule.
// Every pair travels as two 8-byte words that carry the step number in their upper half:
// {step, value bits} and {step, index}.  An aligned 8-byte store is indivisible, so a word
// whose tag equals the current step IS the sender's data of this step: no fence, no separate
// flag and no second round trip (one NVLink write latency per exchange).
// Buffer layout on every rank (same offsets everywhere): [2 parities][world][rows][2] words.
// Steps alternate parity, and a rank can be at most one step ahead of its peers (finishing a
// step needs every peer's words of that step), so a fast rank's next step never overwrites what
// a slow rank is still waiting for.
__device__ __forceinline__ void exchange_and_merge(int tid, int nthreads, int rows, int world, int rank,
                                                   unsigned long long* keys, const ExchangePeers& peers,
                                                   unsigned int step, ArgmaxPair* out, uint32_t* status) {
  const unsigned long long tag = static_cast<unsigned long long>(step) << 32;
  const size_t parity_words = 2 * static_cast<size_t>(world) * rows;
  const size_t base = (step & 1u) * parity_words;
  for (int t = tid; t < rows; t += nthreads) {
    const unsigned long long packed = __ldcg(keys + t);
    keys[t] = 0ull;
    const uint32_t key = static_cast<uint32_t>(packed >> 32);
    const uint32_t value_bits = key ^ ((key & 0x80000000u) ? 0x80000000u : 0xffffffffu);
    const uint32_t index = packed == 0ull ? 0xffffffffu : 0xffffffffu - static_cast<uint32_t>(packed);
    for (int pr = 0; pr < world; ++pr) {
      volatile unsigned long long* dst = reinterpret_cast<volatile unsigned long long*>(peers.base[pr]) +
                                         base + 2 * (static_cast<size_t>(rank) * rows + t);
      dst[0] = tag | value_bits;
      dst[1] = tag | index;
    }
  }
  // every row: wait for each sender's two words of this step, merge as they are read
  const volatile unsigned long long* mine =
      reinterpret_cast<const volatile unsigned long long*>(peers.base[rank]) + base;
  const uint64_t start = global_timer_ns();
  for (int t = tid; t < rows; t += nthreads) {
    unsigned long long best = 0ull;
    bool ok = true;
    for (int sdr = 0; sdr < world && ok; ++sdr) {
      const volatile unsigned long long* slot = mine + 2 * (static_cast<size_t>(sdr) * rows + t);
      unsigned long long w0, w1;
      for (;;) {
        w0 = slot[0];
        w1 = slot[1];
        if ((w0 >> 32) == step && (w1 >> 32) == step) break;
        if (global_timer_ns() - start > 2000000000ull) {
          atomicOr(status, STATUS_WAIT_TIMEOUT);
          ok = false;
          break;
        }
      }
      if (!ok) break;
      const uint32_t vbits = static_cast<uint32_t>(w0);
      const uint32_t idx = static_cast<uint32_t>(w1);
      if (idx == 0xffffffffu) continue;  // the sender had no candidate
      const unsigned long long packed =
          (static_cast<unsigned long long>(total_order_key(vbits)) << 32) |
          static_cast<unsigned long long>(0xffffffffu - idx);
      best = packed > best ? packed : best;
    }
    if (!ok) continue;  // results are invalid; the status word says so
    out[t] = unpack_key(best);
  }
}

template <int BLOCK_TOK, int DEEP>  // DEEP: 0 normal ring, 1 deep, 2 wide
__global__ void __launch_bounds__(kThreads, BLOCK_TOK <= 32 ? (DEEP == 1 ? 2 : (DEEP == 2 ? 4 : 3))
                                                            : (BLOCK_TOK <= 128 ? 2 : 1))
    fp8_projection_kernel(const __grid_constant__ CUtensorMap tmap_w,
                          const __grid_constant__ CUtensorMap tmap_a, const Fp8ProjParams p) {
  constexpr int STAGES = stages_for(BLOCK_TOK, DEEP);
  constexpr int A_STAGE_BYTES = BLOCK_TOK * kTileKBytes;
  constexpr int STAGE_BYTES = kWStageBytes + A_STAGE_BYTES;
  constexpr uint32_t TMEM_COLS = BLOCK_TOK < 32 ? 32 : BLOCK_TOK;
  constexpr uint32_t IDESC = umma_idesc_e4m3(kTileRows, BLOCK_TOK);
  constexpr bool BATCHED16 = BLOCK_TOK == 16;  // 16-token tiles with more than three tokens: batched epilogue

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  Control<BLOCK_TOK>* ctl = reinterpret_cast<Control<BLOCK_TOK>*>(smem + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_n = blockIdx.x, tile_m = blockIdx.y, split = blockIdx.z;
  if (threadIdx.x == 0) TK100_STAMP(p, 0);
  const int kb_total = p.k / kTileKBytes;
  const int kb_begin = static_cast<int>(static_cast<long long>(split) * kb_total / p.splits);
  const int kb_end = static_cast<int>(static_cast<long long>(split + 1) * kb_total / p.splits);
  const int nkb = kb_end - kb_begin;

  // A short weight stream is queued at L2 whole, first thing: the weights do not depend on the
  // predecessor kernel, so HBM keeps working through the predecessor's tail and through this
  // kernel's own set-up, and the ring below then fills from L2.
  if (warp == 2 && p.l2_prefetch > 0) {
    const int ahead = nkb < p.l2_prefetch ? nkb : p.l2_prefetch;
    for (int i = lane; i < ahead; i += 32) {
      tma_prefetch_l2_2d(&tmap_w, (kb_begin + i) * kTileKBytes, tile_n * kTileRows);
    }
  }

  const bool clustered = p.cluster != 0 && p.splits > 1;
  // Split-K on a leader (p.cluster == 2): the peers store their partial tiles into the leader's
  // shared memory and leave; the leader adds them in split order and finishes every token.
  const bool on_leader = clustered && p.cluster == 2;

  // Fused activation quantiser (16-token tiles only): the epilogue warps make each stage's code
  // tile themselves, so a full[] barrier takes two arrivals: the weight TMA and that warp.
  bool fused_quant = false;
  if constexpr (BLOCK_TOK == 16) fused_quant = p.x_bf16 != nullptr;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], fused_quant ? 2 : 1);
      mbar_init(&ctl->empty[s], 1);
    }
    ctl->is_last = 0u;
    mbar_init(&ctl->tmem_full, 1);
    mbar_init(&ctl->go, 1);
    mbar_init(&ctl->done, on_leader ? static_cast<uint32_t>(p.splits - 1) * 4u : 1u);
    fence_mbar_init();
    // The first pass of weight tiles over the ring is requested here, before the TMEM allocation
    // and the CTA barrier below are through: the weights depend on nothing, and the sooner the
    // first request leaves the sooner the stream starts (the ramp is a third of a decode launch).
    {
      const uint64_t pol_w = l2_policy_evict_first();  // weights are streamed once
      const bool load_a = !TK100_DBG(p, DBG_NO_ACT) && !fused_quant;
      const uint32_t tx_bytes = load_a ? STAGE_BYTES : kWStageBytes;
      const int pre = nkb < STAGES ? nkb : STAGES;
      for (int i = 0; i < pre; ++i) {
        mbar_arrive_expect_tx(&ctl->full[i], tx_bytes);
        tma_load_2d(smem + i * STAGE_BYTES, &tmap_w, &ctl->full[i], (kb_begin + i) * kTileKBytes,
                    tile_n * kTileRows, pol_w);
      }
    }
    if (!fused_quant) prefetch_tensormap(&tmap_a);
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
  // access to a peer's shared memory, long after every CTA has passed this point
  if (on_leader) cluster_arrive();
  if (threadIdx.x == 0) TK100_STAMP(p, 1);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();  // weights are streamed once
      const uint64_t pol_a = l2_policy_evict_last();   // activation codes are re-read by every CTA
      // The weight tiles of the first pass over the ring are already on their way (requested
      // during set-up, they do not depend on the predecessor kernel); the activation-code tiles
      // of the same stages follow once the predecessor (the quantiser) is known to be complete.
      const bool load_a = !TK100_DBG(p, DBG_NO_ACT) && !fused_quant;
      const uint32_t tx_bytes = load_a ? STAGE_BYTES : kWStageBytes;
      const int pre = nkb < STAGES ? nkb : STAGES;
      pdl_wait();
      TK100_STAMP(p, 2);
      for (int i = 0; i < pre && load_a; ++i) {
        tma_load_2d(smem + i * STAGE_BYTES + kWStageBytes, &tmap_a, &ctl->full[i],
                    (kb_begin + i) * kTileKBytes, tile_m * BLOCK_TOK, pol_a);
      }
      bool ok = true;
      for (int i = pre; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t phase = (i / STAGES) & 1;
        ok = mbar_wait(&ctl->empty[s], phase ^ 1, p.status);
        if (!ok) break;
        uint8_t* stage = smem + s * STAGE_BYTES;
        mbar_arrive_expect_tx(&ctl->full[s], tx_bytes);
        const int kbyte = (kb_begin + i) * kTileKBytes;
        tma_load_2d(stage, &tmap_w, &ctl->full[s], kbyte, tile_n * kTileRows, pol_w);
        if (load_a) {
          tma_load_2d(stage + kWStageBytes, &tmap_a, &ctl->full[s], kbyte, tile_m * BLOCK_TOK, pol_a);
        }
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
        const uint32_t phase = (i / STAGES) & 1;
        ok = mbar_wait(&ctl->full[s], phase, p.status);
        if (!ok) break;
        if (i == 0) TK100_STAMP(p, 3);
        tc_fence_after_sync();
        const uint32_t w_addr = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t desc_w = umma_desc_sw128(w_addr);
        const uint64_t desc_a = umma_desc_sw128(w_addr + kWStageBytes);
#pragma unroll
        for (int k4 = 0; k4 < kTileKBytes / 32; ++k4) {
          if (TK100_DBG(p, DBG_NO_MMA)) break;
          // +2 in the address field = +32 bytes along K inside the swizzled row
          umma_f8f6f4(tmem, desc_w + 2 * k4, desc_a + 2 * k4, IDESC, (i | k4) != 0);
        }
        umma_commit(&ctl->empty[s]);  // frees the stage once these MMAs have read it
      }
      umma_commit(&ctl->tmem_full);  // accumulator complete (also releases the epilogue on error)
      TK100_STAMP(p, 4);
    }
  } else {
    // ----------------------------------------------------------------- epilogue
    const int et = threadIdx.x - 64;  // 0..127
    const int quad = warp & 3;        // TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    const int n = tile_n * kTileRows + row_in_tile;
    const bool row_ok = n < p.out_rows;
    const int tok0 = tile_m * BLOCK_TOK;
    const int valid_tok = min(BLOCK_TOK, p.rows - tok0);
    const bool want_argmax = p.argmax_keys != nullptr;

    pdl_wait();  // activation scales, scratch and outputs belong to the predecessor until now
    if constexpr (BLOCK_TOK == 16) {
      if (fused_quant) {
        // ---- per-token scale: amax over the whole BF16 row (all K, whatever this CTA's K range),
        // the four epilogue warps together; rows <= kFusedQuantRows
        const int chunks = p.k >> 3;  // 16-byte chunks per row
        float amax[kFusedQuantRows];
#pragma unroll
        for (int t = 0; t < kFusedQuantRows; ++t) amax[t] = 0.0f;
        for (int c = et; c < chunks; c += kEpilogueThreads) {
#pragma unroll
          for (int t = 0; t < kFusedQuantRows; ++t) {
            if (t < valid_tok) {
              const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.x_bf16 + static_cast<size_t>(tok0 + t) * p.k) + c);
              const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                amax[t] = fmaxf(amax[t], fmaxf(fabsf(bf16x2_lo(w4[q])), fabsf(bf16x2_hi(w4[q]))));
              }
            }
          }
        }
#pragma unroll
        for (int t = 0; t < kFusedQuantRows; ++t) {
          amax[t] = warp_max(amax[t]);
          if (lane == 0) ctl->q_amax[warp - 2][t] = amax[t];
        }
        epilogue_barrier();
        if (et < BLOCK_TOK) {
          float scale = 0.0f;
          if (et < valid_tok) {
            const float a = fmaxf(fmaxf(ctl->q_amax[0][et], ctl->q_amax[1][et]),
                                  fmaxf(ctl->q_amax[2][et], ctl->q_amax[3][et]));
            if (!(a <= 3.0e38f)) atomicOr(p.status, STATUS_NONFINITE_INPUT);
            scale = (a == 0.0f) ? 1.0f : __fdiv_rn(a, 448.0f);
            if (tile_n == 0 && split == 0 && p.scales_out) p.scales_out[tok0 + et] = scale;
          }
          ctl->a_scale[et] = scale;
          ctl->red[et] = 0u;
        }
        epilogue_barrier();
        // ---- each stage's code tile: epilogue warp w makes the k-blocks i = w, w + 4, ...; a lane
        // owns 4 consecutive columns of every token (8 bytes of BF16 in, 4 code bytes out, written
        // where the 128-byte swizzle of a TMA box would have put them)
        const int ew = warp - 2;
        const bool publish = tile_n == 0 && p.codes_out != nullptr;
        const int chunk = lane >> 2, within = (lane & 3) * 4;
        uint2 cur[kFusedQuantRows], nxt[kFusedQuantRows];
        auto fetch = [&](int i, uint2 (&dst)[kFusedQuantRows]) {
#pragma unroll
          for (int t = 0; t < kFusedQuantRows; ++t) {
            if (t < valid_tok && i < nkb) {
              dst[t] = __ldg(reinterpret_cast<const uint2*>(p.x_bf16 + static_cast<size_t>(tok0 + t) * p.k +
                                                           static_cast<size_t>(kb_begin + i) * kTileKBytes) + lane);
            } else {
              dst[t] = make_uint2(0u, 0u);
            }
          }
        };
        fetch(ew, cur);
        bool okq = true;
        for (int i = ew; i < nkb && okq; i += 4) {
          fetch(i + 4, nxt);
          const int s = i % STAGES;
          if (i >= STAGES) {
            okq = mbar_wait(&ctl->empty[s], ((i / STAGES) & 1) ^ 1, p.status);
            if (!okq) break;
          }
          uint8_t* a_tile = smem + s * STAGE_BYTES + kWStageBytes;
#pragma unroll
          for (int t = 0; t < kFusedQuantRows; ++t) {
            if (t < valid_tok) {
              const float sc = ctl->a_scale[t];
              const uint32_t lo = f32x2_to_e4m3x2(__fdiv_rn(bf16x2_lo(cur[t].x), sc), __fdiv_rn(bf16x2_hi(cur[t].x), sc));
              const uint32_t hi = f32x2_to_e4m3x2(__fdiv_rn(bf16x2_lo(cur[t].y), sc), __fdiv_rn(bf16x2_hi(cur[t].y), sc));
              const uint32_t word = lo | (hi << 16);
              *reinterpret_cast<uint32_t*>(a_tile + t * kTileKBytes + ((chunk ^ (t & 7)) << 4) + within) = word;
              if (publish) {
                *reinterpret_cast<uint32_t*>(p.codes_out + static_cast<size_t>(tok0 + t) * p.k +
                                             static_cast<size_t>(kb_begin + i) * kTileKBytes + lane * 4) = word;
              }
            }
          }
          fence_proxy_async_smem();  // generic-proxy writes -> visible to the UMMA reads
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->full[s]);
#pragma unroll
          for (int t = 0; t < kFusedQuantRows; ++t) cur[t] = nxt[t];
        }
      }
    }
    if (!fused_quant) {
      for (int j = et; j < BLOCK_TOK; j += kEpilogueThreads) {
        ctl->a_scale[j] = (j < valid_tok) ? p.act_scales[tok0 + j] : 0.0f;
        ctl->red[j] = 0u;
      }
    }
    const float w_scale = row_ok ? bf16_bits_to_f32(p.w_scales[n]) : 0.0f;
    epilogue_barrier();

    mbar_wait(&ctl->tmem_full, 0, p.status);
    if (et == 0) TK100_STAMP(p, 5);
    tc_fence_after_sync();
    const uint32_t taddr = tmem + (static_cast<uint32_t>(quad * 32) << 16);

    // Final value for (token tok0 + j, weight row n) from its fp32 accumulator.
    auto emit = [&](int j, float acc) {
      const float v = __fmul_rn(__fmul_rn(acc, ctl->a_scale[j]), w_scale);
      const uint32_t b = f32_to_bf16_bits(v);
      const size_t o = static_cast<size_t>(tok0 + j) * p.out_rows + n;
      if (row_ok) {
        if (p.out) p.out[o] = static_cast<uint16_t>(b);
        if (p.logits_f32) p.logits_f32[o] = v;
      }
      if (want_argmax) {
        uint32_t packed = 0u;
        if (row_ok) {
          if ((b & 0x7f80u) == 0x7f80u) atomicOr(p.status, STATUS_NONFINITE_LOGIT);
          packed = local_key(b, row_in_tile);
        }
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) packed = max(packed, __shfl_xor_sync(0xffffffffu, packed, o2));
        if (lane == 0) atomicMax(&ctl->red[j], packed);
      }
    };

    if (TK100_DBG(p, DBG_NO_EPILOGUE)) {
      // experiment: accumulator left unread
    } else if (p.splits == 1) {
#pragma unroll 1
      for (int c0 = 0; c0 < BLOCK_TOK; c0 += 16) {
        if (c0 >= valid_tok) break;  // warp-uniform
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        tmem_ld_wait();
        if (BLOCK_TOK >= 32 || (BATCHED16 && valid_tok > 3)) {
          // Several tokens per tile: the 16 tokens of a chunk go through scaling, rounding, stores
          // and the warp maxima side by side (one dependent chain per token would leave the few
          // epilogue warps waiting on latencies).  Same values; maxima commute.
          uint32_t b[16];
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            v[j] = __fmul_rn(__fmul_rn(__uint_as_float(r[j]), ctl->a_scale[c0 + j]), w_scale);
            b[j] = f32_to_bf16_bits(v[j]);
          }
          if (row_ok) {
            const size_t o0 = static_cast<size_t>(tok0 + c0) * p.out_rows + n;
            if (p.out) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (c0 + j < valid_tok) p.out[o0 + static_cast<size_t>(j) * p.out_rows] = static_cast<uint16_t>(b[j]);
              }
            }
            if (p.logits_f32) {
              // Many tokens: the fp32 logit plane ([tokens, vocab], one 512-byte piece per token per
              // CTA, the tokens' rows a megabyte apart) is stored with the evict_last policy, so
              // the lines wait in L2 for the end of the weight stream instead of interrupting it
              // with scattered DRAM writes (LM head, M = 32: 242 -> 232 us).
              if constexpr (BLOCK_TOK >= 32) {
                const uint64_t logits_policy = l2_policy_evict_last();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  if (c0 + j < valid_tok) {
                    st_global_f32_policy(p.logits_f32 + o0 + static_cast<size_t>(j) * p.out_rows, v[j], logits_policy);
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  if (c0 + j < valid_tok) p.logits_f32[o0 + static_cast<size_t>(j) * p.out_rows] = v[j];
                }
              }
            }
          }
          if (want_argmax) {
            uint32_t pk[16];
            uint32_t nonfinite = 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const bool live = row_ok && c0 + j < valid_tok;
              nonfinite |= (live && (b[j] & 0x7f80u) == 0x7f80u) ? 1u : 0u;
              pk[j] = live ? local_key(b[j], row_in_tile) : 0u;
            }
            if (nonfinite) atomicOr(p.status, STATUS_NONFINITE_LOGIT);
            // 16 tokens x 32 rows -> 16 maxima in 16 exchanges instead of 80: at each step a lane
            // hands half of its tokens to the partner and keeps the maximum of the other half, so
            // after offsets 16, 8, 4, 2 lane l holds token l >> 1 over 16 rows, and the exchange at
            // offset 1 completes it.  Integer maxima: any order gives the same key.
#pragma unroll
            for (int o2 = 16, count = 8; o2 > 1; o2 >>= 1, count >>= 1) {
              const bool upper = (lane & o2) != 0;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (j < count) {
                  const uint32_t give = upper ? pk[j] : pk[j + count];
                  const uint32_t keep = upper ? pk[j + count] : pk[j];
                  pk[j] = max(keep, __shfl_xor_sync(0xffffffffu, give, o2));
                }
              }
            }
            pk[0] = max(pk[0], __shfl_xor_sync(0xffffffffu, pk[0], 1));
            const int token = c0 + (lane >> 1);
            if ((lane & 1) == 0 && token < valid_tok && pk[0] != 0u) atomicMax(&ctl->red[token], pk[0]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j < valid_tok) emit(c0 + j, __uint_as_float(r[j]));
          }
        }
      }
    } else if (on_leader) {
      const uint32_t rank = cluster_cta_rank();  // = split: cluster dimension z covers the splits
      cluster_wait();  // every CTA of the cluster has initialised its barriers
      float* land = reinterpret_cast<float*>(smem);  // leader: [split - 1][token][row] over the ring
      if (rank == 0) {
        // the leader's MMAs have read the whole ring (tmem_full): the peers may store into it
        if (et == 0) {
          for (int r = 1; r < p.splits; ++r) mbar_arrive_remote(mapa_u32(smem_u32(&ctl->go), r));
        }
        mbar_wait_cluster(&ctl->done, 0, p.status);
#pragma unroll 1
        for (int c0 = 0; c0 < BLOCK_TOK; c0 += 16) {
          if (c0 >= valid_tok) break;
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j0 = 0; j0 < 16; j0 += 4) {
            if (c0 + j0 < valid_tok) {  // warp-uniform
              float v[kMaxSplits][4];
#pragma unroll
              for (int sidx = 1; sidx < kMaxSplits; ++sidx) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  v[sidx][j] = (sidx < p.splits && c0 + j0 + j < valid_tok)
                                   ? land[(static_cast<size_t>(sidx - 1) * valid_tok + c0 + j0 + j) * kTileRows + row_in_tile]
                                   : 0.0f;
                }
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float acc = __fadd_rn(0.0f, __uint_as_float(r[j0 + j]));  // split 0 = this CTA
#pragma unroll
                for (int sidx = 1; sidx < kMaxSplits; ++sidx) {
                  if (sidx < p.splits) acc = __fadd_rn(acc, v[sidx][j]);  // fixed split order
                }
                if (c0 + j0 + j < valid_tok) emit(c0 + j0 + j, acc);
              }
            }
          }
        }
      } else {
        mbar_wait_cluster(&ctl->go, 0, p.status);
        const uint32_t slot = mapa_u32(smem_u32(land + static_cast<size_t>(rank - 1) * valid_tok * kTileRows + row_in_tile), 0);
#pragma unroll 1
        for (int c0 = 0; c0 < BLOCK_TOK; c0 += 16) {
          if (c0 >= valid_tok) break;
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c0 + j < valid_tok) st_dsmem_f32(slot + static_cast<uint32_t>(c0 + j) * kTileRows * 4, __uint_as_float(r[j]));
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(mapa_u32(smem_u32(&ctl->done), 0));
      }
    } else if (clustered) {
      // Own partial tile -> own shared memory ([token][row] fp32, over ring stage 0, which
      // this CTA's MMAs have finished reading once tmem_full has fired).
      float* mine = reinterpret_cast<float*>(smem) + row_in_tile;
#pragma unroll 1
      for (int c0 = 0; c0 < BLOCK_TOK; c0 += 16) {
        if (c0 >= valid_tok) break;
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c0 + j < valid_tok) mine[(c0 + j) * kTileRows] = __uint_as_float(r[j]);
        }
      }
    } else {
      // Publish this split's partial tile: [split][tile_m][tile_n][token][row].
      const size_t tile_index =
          (static_cast<size_t>(split) * gridDim.y + tile_m) * gridDim.x + tile_n;
      float* mine = p.partials + tile_index * (BLOCK_TOK * kTileRows) + row_in_tile;
#pragma unroll 1
      for (int c0 = 0; c0 < BLOCK_TOK; c0 += 16) {
        if (c0 >= valid_tok) break;
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c0 + j < valid_tok && !TK100_DBG(p, 8)) __stcg(mine + (c0 + j) * kTileRows, __uint_as_float(r[j]));
        }
      }
      if (!TK100_DBG(p, 16)) __threadfence();
      epilogue_barrier();
      if (et == 0) {
        unsigned int* counter = p.counters + tile_m * gridDim.x + tile_n;
        const unsigned int ticket = atomicAdd(counter, 1u);
        const bool last = ticket == static_cast<unsigned int>(p.splits - 1);
        if (last) *counter = 0u;  // re-armed for the next launch
        ctl->is_last = last ? 1u : 0u;
      }
      epilogue_barrier();
      if (ctl->is_last && !TK100_DBG(p, 32)) {
        __threadfence();
        const size_t split_stride =
            static_cast<size_t>(gridDim.y) * gridDim.x * (BLOCK_TOK * kTileRows);
        const float* base = p.partials +
                            (static_cast<size_t>(tile_m) * gridDim.x + tile_n) *
                                (BLOCK_TOK * kTileRows) +
                            row_in_tile;
        // Four tokens at a time, every split's value of the batch requested before the
        // first add: one L2 round trip per batch instead of one per (token, split).
#pragma unroll 1
        for (int j0 = 0; j0 < valid_tok; j0 += 4) {
          float v[kMaxSplits][4];
#pragma unroll
          for (int s = 0; s < kMaxSplits; ++s) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              v[s][j] = (s < p.splits && j0 + j < valid_tok)
                            ? __ldcg(base + s * split_stride + (j0 + j) * kTileRows)
                            : 0.0f;
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float acc = 0.0f;
#pragma unroll
            for (int s = 0; s < kMaxSplits; ++s) {
              if (s < p.splits) acc = __fadd_rn(acc, v[s][j]);  // fixed split order
            }
            if (j0 + j < valid_tok) emit(j0 + j, acc);
          }
        }
      }
    }

    if (clustered && !on_leader) {
      // Every CTA of the cluster has published its tile after the first barrier; CTA `rank`
      // then finishes the tokens j = rank, rank + splits, ...: partials are read from the
      // peers' shared memory and added in split order (fixed, so bit-reproducible).
      cluster_arrive();
      cluster_wait();
      if (!TK100_DBG(p, DBG_NO_EPILOGUE)) {
        const uint32_t rank = cluster_cta_rank();
        const uint32_t my_addr = smem_u32(reinterpret_cast<float*>(smem) + row_in_tile);
#pragma unroll 1
        for (int j0 = static_cast<int>(rank); j0 < valid_tok; j0 += 2 * p.splits) {
          float v[2][kMaxSplits];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int j = j0 + u * p.splits;
#pragma unroll
            for (int s = 0; s < kMaxSplits; ++s) {
              v[u][s] = (j < valid_tok && s < p.splits)
                            ? ld_dsmem_f32(my_addr + j * kTileRows * 4, static_cast<uint32_t>(s))
                            : 0.0f;
            }
          }
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int j = j0 + u * p.splits;
            float acc = 0.0f;
#pragma unroll
            for (int s = 0; s < kMaxSplits; ++s) {
              if (s < p.splits) acc = __fadd_rn(acc, v[u][s]);
            }
            if (j < valid_tok) emit(j, acc);
          }
        }
      }
      cluster_arrive_relaxed();  // nobody's shared memory may go away while a peer still reads it
      cluster_wait_relaxed();
    }

    const bool spread = p.spread_keys != nullptr;
    const int group = tile_n % kArgmaxGroups;
    if (want_argmax && !TK100_DBG(p, DBG_NO_EPILOGUE) &&
        (p.splits == 1 || (clustered && !on_leader) || (on_leader && split == 0) || ctl->is_last)) {
      epilogue_barrier();
      for (int j = et; j < valid_tok; j += kEpilogueThreads) {
        const uint32_t local = ctl->red[j];
        if (local != 0u) {
          const unsigned long long best =
              global_key(local, static_cast<uint32_t>(p.vocab_offset + tile_n * kTileRows));
          // The value the atomic returns is stored to shared memory: the thread cannot pass the
          // barrier below before the atomic has been performed at L2, which orders it before the
          // ticket (no device-wide fence, which would also wait for this thread's logit stores).
          unsigned long long* key =
              spread ? p.spread_keys + (static_cast<size_t>(group) * kArgmaxSpreadRows + tok0 + j) * 16
                     : p.argmax_keys + tok0 + j;
          const unsigned long long before = atomicMax(key, best);
          if (p.tail_ticket != nullptr) ctl->red[j] = static_cast<uint32_t>(before >> 32);
        }
      }
    }
    if (p.tail_ticket != nullptr) {
      // Fused tail: every CTA takes a ticket once its maxima are in the global keys; the CTA that
      // draws the last one finalises (one GPU) or exchanges with the peers and merges.
      epilogue_barrier();
      if (et == 0) {
        bool last;
        if (spread) {
          // the group's ticket first; the last CTA of a group draws for the group
          const unsigned int groups = gridDim.x < kArgmaxGroups ? gridDim.x : kArgmaxGroups;
          const unsigned int members =
              (gridDim.x - group + kArgmaxGroups - 1) / kArgmaxGroups * gridDim.y * gridDim.z;
          unsigned int* group_ticket = p.spread_tickets + group * 32;
          last = atomicAdd(group_ticket, 1u) == members - 1;
          if (last) {
            *group_ticket = 0u;
            last = atomicAdd(p.tail_ticket, 1u) == groups - 1;
          }
        } else {
          const unsigned int total = gridDim.x * gridDim.y * gridDim.z;
          last = atomicAdd(p.tail_ticket, 1u) == total - 1;
        }
        unsigned int step = 0;
        if (last) {
          *p.tail_ticket = 0u;  // re-armed for the next launch
          if (p.world > 1) {
            step = *p.step_counter + 1u;
            if (step == 0u) step = 1u;  // 0 is what a zero-filled buffer holds
            *p.step_counter = step;
          }
        }
        ctl->tail_step = step;
        ctl->tail_last = last ? 1u : 0u;
      }
      epilogue_barrier();
      if (ctl->tail_last) {
        if (spread) {
          // fold the groups: all loads of a token first, then the maximum (any order: integer max)
          for (int t = et; t < p.rows; t += kEpilogueThreads) {
            unsigned long long k[kArgmaxGroups];
#pragma unroll
            for (int g = 0; g < kArgmaxGroups; ++g) {
              k[g] = __ldcg(p.spread_keys + (static_cast<size_t>(g) * kArgmaxSpreadRows + t) * 16);
            }
            unsigned long long best = 0ull;
#pragma unroll
            for (int g = 0; g < kArgmaxGroups; ++g) {
              if (k[g] != 0ull) p.spread_keys[(static_cast<size_t>(g) * kArgmaxSpreadRows + t) * 16] = 0ull;
              best = k[g] > best ? k[g] : best;
            }
            if (p.world > 1) {
              __stcg(p.argmax_keys + t, best);  // read back below by this same thread
            } else {
              p.pairs_out[t] = unpack_key(best);
            }
          }
        }
        if (p.world > 1) {
          exchange_and_merge(et, kEpilogueThreads, p.rows, p.world, p.rank, p.argmax_keys, p.peers,
                             ctl->tail_step, p.pairs_out, p.status);
        } else if (!spread) {
          for (int t = et; t < p.rows; t += kEpilogueThreads) {
            const unsigned long long packed = __ldcg(p.argmax_keys + t);
            p.argmax_keys[t] = 0ull;
            p.pairs_out[t] = unpack_key(packed);
          }
        }
      }
    }
  }
  if (threadIdx.x == 64) TK100_STAMP(p, 6);
  if (on_leader && warp < 2) {
    cluster_wait();  // completes the barrier every thread arrived on after set-up
  } else if (clustered && warp < 2) {
    // the TMA and UMMA warps take part in the two cluster barriers of the reduction
    cluster_arrive();
    cluster_wait();
    cluster_arrive_relaxed();
    cluster_wait_relaxed();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, TMEM_COLS);
  }
  if (threadIdx.x == 0) TK100_STAMP(p, 7);
}

__global__ void argmax_finalize_kernel(int rows, unsigned long long* keys, ArgmaxPair* pairs) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows) return;
  const unsigned long long packed = keys[t];
  keys[t] = 0ull;
  pairs[t] = unpack_key(packed);
}

__global__ void argmax_merge_kernel(int rows, int shards, const ArgmaxPair* gathered,
                                    ArgmaxPair* out) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows) return;
  unsigned long long best = 0ull;
  for (int s = 0; s < shards; ++s) {
    const ArgmaxPair c = gathered[static_cast<size_t>(s) * rows + t];
    if (c.index < 0) continue;
    const unsigned long long packed =
        (static_cast<unsigned long long>(total_order_key(__float_as_uint(c.value))) << 32) |
        static_cast<unsigned long long>(0xffffffffu - static_cast<uint32_t>(c.index));
    best = packed > best ? packed : best;
  }
  out[t] = unpack_key(best);
}

// The exchange as a launch of its own (one CTA per rank): see exchange_and_merge.
__global__ void __launch_bounds__(256)
    argmax_exchange_kernel(int rows, int world, int rank, unsigned long long* keys,
                           ExchangePeers peers, unsigned int* step_counter, ArgmaxPair* out,
                           uint32_t* status) {
  __shared__ unsigned int s_step;
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0) {
    s_step = *step_counter + 1u;
    if (s_step == 0u) s_step = 1u;  // 0 is what a zero-filled buffer holds
    *step_counter = s_step;
  }
  __syncthreads();
  exchange_and_merge(threadIdx.x, blockDim.x, rows, world, rank, keys, peers, s_step, out, status);
}

template <int BLOCK_TOK>
cudaError_t launch_one(cudaStream_t stream, const CUtensorMap& tmap_w, const CUtensorMap& tmap_a,
                       const Fp8ProjParams& p) {
  dim3 grid((p.out_rows + kTileRows - 1) / kTileRows, (p.rows + BLOCK_TOK - 1) / BLOCK_TOK,
            p.splits);
  const unsigned int cluster_z = (p.cluster && p.splits > 1) ? static_cast<unsigned int>(p.splits) : 1u;
  if (BLOCK_TOK <= 32 && p.deep_ring == 1) {
    return launch_kernel_cluster(fp8_projection_kernel<BLOCK_TOK, 1>, grid, dim3(kThreads),
                                 smem_bytes_for<BLOCK_TOK, 1>(), stream, dim3(1, 1, cluster_z), tmap_w,
                                 tmap_a, p);
  }
  if (BLOCK_TOK <= 16 && p.deep_ring == 2) {
    constexpr int BT = BLOCK_TOK <= 16 ? BLOCK_TOK : 16;  // only the 16-token tile has this variant
    return launch_kernel_cluster(fp8_projection_kernel<BT, 2>, grid, dim3(kThreads),
                                 smem_bytes_for<BT, 2>(), stream, dim3(1, 1, cluster_z), tmap_w, tmap_a, p);
  }
  return launch_kernel_cluster(fp8_projection_kernel<BLOCK_TOK, 0>, grid, dim3(kThreads),
                               smem_bytes_for<BLOCK_TOK, 0>(), stream, dim3(1, 1, cluster_z), tmap_w, tmap_a,
                               p);
}

template <int BLOCK_TOK>
cudaError_t prepare_one() {
  cudaError_t e = cudaFuncSetAttribute(fp8_projection_kernel<BLOCK_TOK, 0>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem_bytes_for<BLOCK_TOK, 0>()));
  if (e != cudaSuccess || BLOCK_TOK > 32) return e;
  e = cudaFuncSetAttribute(fp8_projection_kernel<BLOCK_TOK, 1>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem_bytes_for<BLOCK_TOK, 1>()));
  if (e != cudaSuccess || BLOCK_TOK > 16) return e;
  constexpr int BT = BLOCK_TOK <= 16 ? BLOCK_TOK : 16;
  return cudaFuncSetAttribute(fp8_projection_kernel<BT, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(smem_bytes_for<BT, 2>()));
}

}  // namespace

size_t fp8_projection_smem_bytes(int block_tok) {
  switch (block_tok) {
    case 16: return smem_bytes_for<16>();
    case 32: return smem_bytes_for<32>();
    case 64: return smem_bytes_for<64>();
    case 128: return smem_bytes_for<128>();
    default: return smem_bytes_for<256>();
  }
}

int fp8_projection_stages(int block_tok) { return stages_for(block_tok); }

cudaError_t fp8_projection_prepare() {
  cudaError_t e;
  if ((e = prepare_one<16>()) != cudaSuccess) return e;
  if ((e = prepare_one<32>()) != cudaSuccess) return e;
  if ((e = prepare_one<64>()) != cudaSuccess) return e;
  if ((e = prepare_one<128>()) != cudaSuccess) return e;
  return prepare_one<256>();
}

cudaError_t launch_fp8_projection(cudaStream_t stream, int block_tok, const CUtensorMap& tmap_w,
                                  const CUtensorMap& tmap_a, const Fp8ProjParams& p) {
  switch (block_tok) {
    case 16: return launch_one<16>(stream, tmap_w, tmap_a, p);
    case 32: return launch_one<32>(stream, tmap_w, tmap_a, p);
    case 64: return launch_one<64>(stream, tmap_w, tmap_a, p);
    case 128: return launch_one<128>(stream, tmap_w, tmap_a, p);
    case 256: return launch_one<256>(stream, tmap_w, tmap_a, p);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_argmax_finalize(cudaStream_t stream, int rows, unsigned long long* keys,
                                   ArgmaxPair* pairs) {
  return launch_kernel(argmax_finalize_kernel, dim3((rows + 127) / 128), dim3(128), 0, stream, rows,
                       keys, pairs);
}

cudaError_t launch_argmax_exchange(cudaStream_t stream, int rows, int world, int rank,
                                   unsigned long long* keys, const ExchangePeers& peers,
                                   unsigned int* step_counter, ArgmaxPair* out, uint32_t* status) {
  return launch_kernel(argmax_exchange_kernel, dim3(1), dim3(256), 0, stream, rows, world, rank,
                       keys, peers, step_counter, out, status);
}

cudaError_t launch_argmax_merge(cudaStream_t stream, int rows, int shards,
                                const ArgmaxPair* gathered, ArgmaxPair* out) {
  return launch_kernel(argmax_merge_kernel, dim3((rows + 127) / 128), dim3(128), 0, stream, rows,
                       shards, gathered, out);
}

}  // namespace tk100
