// Device-side token sampler: top-k / top-p selection with a per-request xorshift64 generator,
// replacing the host `Sampler` (tuisko-engine/src/sampling.rs:76-231) and the device -> host copy
// of a 248 320-wide logit row that feeds it.
//
// One launch for a decode batch of up to 8 rows.  A row of BF16 logits (0.5 MB) is cut into
// slices, one CTA each; every warp streams its share with 16-byte loads and keeps the 32 best
// (value, index) keys it has seen, one per lane, sorted -- a few candidates enter one by one (a
// ballot, a population count and one shuffle each), many at once through a bitonic sort and
// merge across the lanes.  Lists fold pairwise (warp -> CTA through shared memory); the CTAs leave
// theirs in a caller-owned scratch and take a ticket; the CTA that draws a row's last ticket
// merges them and runs the reference's scalar selection on the k survivors (same float / double
// operations in the same order), so no second launch and no host hop follow.
#include <math.h>

#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tk100 {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kList = 32;  // keys a warp keeps = the largest admitted top_k

// Larger key = earlier in the reference's order: value descending under the IEEE total order
// (+0 above -0), then index ascending (sampling.rs:219-224: only a strictly greater value
// displaces a retained one).
__device__ __forceinline__ uint64_t make_key(uint32_t bf16_bits, uint32_t index) {
  const uint32_t ord = (bf16_bits & 0x8000u) ? (~bf16_bits & 0xffffu) : (bf16_bits | 0x8000u);
  return (static_cast<uint64_t>(ord) << 32) | static_cast<uint64_t>(~index);
}
__device__ __forceinline__ uint32_t key_index(uint64_t key) { return ~static_cast<uint32_t>(key); }
__device__ __forceinline__ float key_value(uint64_t key) {
  const uint32_t ord = static_cast<uint32_t>(key >> 32);
  const uint32_t bits = (ord & 0x8000u) ? (ord & 0x7fffu) : (~ord & 0xffffu);
  return __uint_as_float(bits << 16);
}

// exp of a non-positive f32 argument as the f32 nearest to the exact value, returned as a double:
// the reference's `((v - max) / temperature).exp() as f64`.  Evaluated in double (argument
// reduction by ln 2 in two pieces, degree-13 Taylor polynomial on |r| <= 0.347: relative error
// below 1e-16), so the rounding to f32 is the correctly rounded result except within 1e-9 of a
// rounding boundary.  Written out here rather than calling the library exponential, whose slow
// path is a function call.
__device__ __forceinline__ double softmax_weight(float scaled) {
  const double x = static_cast<double>(scaled);
  if (!(x >= -104.0)) return 0.0;  // below half of the smallest f32 denormal (e^-103.97)
  const double n = rint(x * 1.4426950408889634);
  double r = fma(n, -6.93147180369123816490e-01, x);
  r = fma(n, -1.90821492927058770002e-10, r);
  double p = 1.0 / 6227020800.0;
  p = fma(p, r, 1.0 / 479001600.0);
  p = fma(p, r, 1.0 / 39916800.0);
  p = fma(p, r, 1.0 / 3628800.0);
  p = fma(p, r, 1.0 / 362880.0);
  p = fma(p, r, 1.0 / 40320.0);
  p = fma(p, r, 1.0 / 5040.0);
  p = fma(p, r, 1.0 / 720.0);
  p = fma(p, r, 1.0 / 120.0);
  p = fma(p, r, 1.0 / 24.0);
  p = fma(p, r, 1.0 / 6.0);
  p = fma(p, r, 0.5);
  p = fma(p, r, 1.0);
  p = fma(p, r, 1.0);
  const double scale = __longlong_as_double((static_cast<long long>(n) + 1023) << 52);  // 2^n, n >= -151
  return static_cast<double>(static_cast<float>(p * scale));
}

__device__ __forceinline__ uint64_t shfl64(uint64_t v, int src) {
  return __shfl_sync(0xffffffffu, v, src);
}

__device__ __forceinline__ uint64_t max64(uint64_t a, uint64_t b) { return a > b ? a : b; }
__device__ __forceinline__ uint64_t min64(uint64_t a, uint64_t b) { return a < b ? a : b; }

// Bitonic sort of one key per lane into descending order (lane 0 the largest): 15 exchanges.
__device__ __forceinline__ uint64_t sort_descending(uint64_t v, int lane) {
#pragma unroll
  for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      const uint64_t other = __shfl_xor_sync(0xffffffffu, v, j);
      const bool keep_max = ((lane & j) == 0) == ((lane & k) == 0);
      v = keep_max ? max64(v, other) : min64(v, other);
    }
  }
  return v;
}

// The 32 largest of two descending lists (one key per lane each), descending: reversing one list
// makes the lane-wise maxima a bitonic sequence of exactly those keys; 5 exchanges sort it.
__device__ __forceinline__ uint64_t merge_descending(uint64_t a, uint64_t b, int lane) {
  uint64_t v = max64(a, __shfl_sync(0xffffffffu, b, 31 - lane));
#pragma unroll
  for (int j = 16; j > 0; j >>= 1) {
    const uint64_t other = __shfl_xor_sync(0xffffffffu, v, j);
    v = ((lane & j) == 0) ? max64(v, other) : min64(v, other);
  }
  return v;
}

// The warp's sorted list lives one key per lane (`held`, lane 0 the best).  Offers `cand` of
// every lane whose `want` is set; `kth` is the key at position top_k - 1 (0 while the list is short).
// Many candidates at once (the first batches of a scan) go through a sort and a merge; a few
// enter one by one, each by a ballot, a population count and one shuffle.
__device__ __forceinline__ void offer(uint64_t& held, uint64_t& kth, uint64_t cand, bool want,
                                      int lane, int top_k) {
  unsigned pending = __ballot_sync(0xffffffffu, want);
  if (__popc(pending) >= 6) {
    held = merge_descending(held, sort_descending(want ? cand : 0ull, lane), lane);
    kth = shfl64(held, top_k - 1);
    return;
  }
  while (pending) {
    const int src = __ffs(pending) - 1;
    pending &= pending - 1;
    const uint64_t c = shfl64(cand, src);
    if (c > kth) {  // uniform across the warp: c and kth are
      const int pos = __popc(__ballot_sync(0xffffffffu, held > c));
      const uint64_t up = __shfl_up_sync(0xffffffffu, held, 1);
      if (lane > pos) held = up;
      else if (lane == pos) held = c;
      kth = shfl64(held, top_k - 1);
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1) sampler_kernel(SamplerParams p) {
  __shared__ uint64_t lists[kWarps][kList];
  __shared__ int is_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row = blockIdx.y, slice = blockIdx.x, slices = gridDim.x;
  const int top_k = p.top_k[row];
  const uint16_t* logits = p.logits + static_cast<size_t>(row) * p.vocab;
  uint64_t* row_scratch = p.scratch + static_cast<size_t>(row) * (slices * kList);
  unsigned int* ticket = reinterpret_cast<unsigned int*>(p.scratch + static_cast<size_t>(p.rows) * slices * kList) + row;

  pdl_wait();
  pdl_trigger();

  // 8-value chunks of the row, dealt to (slice, warp) in contiguous runs.
  const int chunks = p.vocab / 8;
  const int parts = slices * kWarps;
  const int part = slice * kWarps + warp;
  const int begin = static_cast<int>(static_cast<long long>(chunks) * part / parts);
  const int end = static_cast<int>(static_cast<long long>(chunks) * (part + 1) / parts);

  uint64_t held = 0, kth = 0;
  bool nonfinite = false;
  for (int base = begin; base < end; base += 32) {
    const int chunk = base + lane;
    uint32_t w[4] = {0, 0, 0, 0};
    const bool live = chunk < end;
    if (live) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(logits) + chunk);
      w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    }
    uint64_t cand[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t bits = (w[j >> 1] >> ((j & 1) * 16)) & 0xffffu;
      nonfinite |= live && (bits & 0x7f80u) == 0x7f80u;
      cand[j] = live ? make_key(bits, static_cast<uint32_t>(chunk * 8 + j)) : 0;
    }
    if (kth == 0) {
      // The list is not full yet (the first 256 values of the warp's share): sort the eight
      // batches side by side -- independent exchange chains hide each other's shuffle latency --
      // and fold them as a tree, instead of eight sort-and-merge rounds one after the other.
#pragma unroll
      for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
        for (int jj = k >> 1; jj > 0; jj >>= 1) {
          const bool keep_max = ((lane & jj) == 0) == ((lane & k) == 0);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint64_t other = __shfl_xor_sync(0xffffffffu, cand[j], jj);
            cand[j] = keep_max ? max64(cand[j], other) : min64(cand[j], other);
          }
        }
      }
#pragma unroll
      for (int span = 4; span > 0; span >>= 1) {
#pragma unroll
        for (int j = 0; j < span; ++j) cand[j] = merge_descending(cand[j], cand[j + span], lane);
      }
      held = merge_descending(held, cand[0], lane);
      kth = shfl64(held, top_k - 1);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) offer(held, kth, cand[j], cand[j] > kth, lane, top_k);
    }
  }
  if (nonfinite) atomicOr(p.status, STATUS_NONFINITE_LOGIT);

  // The CTA's eight lists fold into warp 0's as a tree of merges through shared memory.
  auto fold_warps = [&]() {
#pragma unroll
    for (int half = kWarps / 2; half > 0; half >>= 1) {
      if (warp >= half && warp < 2 * half) lists[warp][lane] = held;
      __syncthreads();
      if (warp < half) held = merge_descending(held, lists[warp + half][lane], lane);
      __syncthreads();
    }
  };
  fold_warps();
  if (warp == 0) {
    row_scratch[slice * kList + lane] = held;
    __threadfence();
    __syncwarp();
    if (lane == 0) is_last = atomicAdd(ticket, 1u) == static_cast<unsigned int>(slices - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();

  // The row's last CTA: every warp merges its share of the slices' lists, then the same tree.
  held = 0;
  {
    // at most 32 slices: four lists per warp, all requested before the first merge
    uint64_t other[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int s = warp + i * kWarps;
      other[i] = s < slices ? *reinterpret_cast<volatile uint64_t*>(row_scratch + s * kList + lane) : 0ull;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) held = merge_descending(held, other[i], lane);
  }
  fold_warps();
  if (warp != 0) return;
  if (lane == 0) *ticket = 0;  // ready for the next launch

  if (p.top_out != nullptr && lane < top_k) {
    p.top_out[(row * kList + lane) * 2] = __float_as_uint(key_value(held));
    p.top_out[(row * kList + lane) * 2 + 1] = key_index(held);
  }

  // sampling.rs:102-108: temperature 0 or top_k 1 is the greedy route and draws no random number.
  const float temperature = p.temperature[row];
  uint32_t token = key_index(shfl64(held, 0));
  if (!(temperature == 0.0f || top_k == 1)) {
    // sampling.rs:175-210, evaluated by every lane on the same values.
    // Lane i evaluates the weight of survivor i (the exponentials run side by side); the sums
    // below then walk the lanes in the reference's order.
    const float maximum = key_value(shfl64(held, 0));
    const float scaled = __fdiv_rn(key_value(held) - maximum, temperature);
    const double my_weight = lane < top_k ? softmax_weight(scaled) : 0.0;
    // Lane i ends with the running sum over survivors 0..i, added in survivor order (the
    // reference's three loops walk this same sequence).
    double running = 0.0;
#pragma unroll 1
    for (int i = 0; i < top_k; ++i) {
      const double w = __shfl_sync(0xffffffffu, my_weight, i);
      if (i <= lane) running += w;
    }
    const double total = __shfl_sync(0xffffffffu, running, top_k - 1);
    const double cutoff = static_cast<double>(fmaxf(p.top_p[row], 1.17549435e-38f)) * total;
    // first survivor whose running sum reaches the cut-off (all of them if none does)
    int retained = __popc(__ballot_sync(0xffffffffu, lane < top_k && !(running >= cutoff))) + 1;
    retained = retained > top_k ? top_k : retained;
    const double retained_total = __shfl_sync(0xffffffffu, running, retained - 1);
    // xorshift64 (sampling.rs:244-260); the state advances once per sampled token.
    uint64_t state = p.rng_state[row];
    state ^= state << 13;
    state ^= state >> 7;
    state ^= state << 17;
    const double unit = static_cast<double>(state >> 11) * (1.0 / 9007199254740992.0);
    const double threshold = unit * retained_total;
    int chosen = __popc(__ballot_sync(0xffffffffu, lane < retained && !(running >= threshold)));
    chosen = chosen >= retained ? retained - 1 : chosen;
    token = key_index(shfl64(held, chosen));
    if (lane == 0) p.rng_state[row] = state;
    if (!(retained_total > 0.0) || isinf(retained_total)) atomicOr(p.status, STATUS_NONFINITE_LOGIT);
  }
  if (lane == 0) {
    p.decisions[row * 2] = token;
    p.decisions[row * 2 + 1] = (token == p.stop_ids[row * 2] || token == p.stop_ids[row * 2 + 1]) ? 1u : 0u;
  }
}

}  // namespace

int sampler_slices(int vocab) {
  // About 1000 values per warp: 31 slices at the 248 320-wide vocabulary, fewer for small rows.
  int slices = (vocab + 8 * 1024 - 1) / (8 * 1024);
  return slices < 1 ? 1 : slices > 32 ? 32 : slices;
}

size_t sampler_scratch_bytes(int rows, int vocab) {
  return static_cast<size_t>(rows) * sampler_slices(vocab) * kList * sizeof(uint64_t) +
         static_cast<size_t>(rows) * sizeof(unsigned int) + 8;
}

cudaError_t launch_sampler(cudaStream_t stream, const SamplerParams& p) {
  return launch_kernel(sampler_kernel, dim3(sampler_slices(p.vocab), p.rows), dim3(kThreads), 0,
                       stream, p);
}

}  // namespace tk100
