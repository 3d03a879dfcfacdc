// Sum of the ranks' fp32 partial outputs over NVLink peer memory, rounded to BF16 once: the
// exchange step behind the row-parallel down projection of a tensor-parallel layer, done by
// this library's own kernel instead of a collective-library call plus a rounding kernel.
//
// Every rank owns an exchange buffer that all peers can address (plain peer stores and loads;
// no multicast object, no TMA).  Same layout on every rank:
//
//   [two-shot slots]  world x chunk fp32 partials as delivered by the senders
//   [one-shot slots]  2 parities x world x one-shot capacity fp32 partials
//   [results]         2 parities x BF16 sums of all chunks (two-shot form only)
//   [flags]           2 kinds x world step numbers (kind 0: partials delivered, 1: results delivered)
//
// Every region and every stride inside it is fixed by the buffer's CAPACITY, not by the size of
// the call at hand, and the one-shot and two-shot slots are disjoint: a rank that is one step
// ahead (a decode step of 5120 values behind a prefill chunk of 64 x 5120, say) can therefore
// never store into memory that a slower rank still reads for the step before.
//
// Small sums (up to kOneShotElems values) go ONE-SHOT: every rank stores its whole partial into
// every peer's slot [parity][sender], raises flag 0 there, waits for all senders' flags in its own
// buffer and adds the `world` partials in rank order.  One NVLink latency.
//
// Larger sums go TWO-SHOT: the values are cut into `world` chunks; rank d receives chunk d of
// every sender (slot [sender]), adds them in rank order, rounds, and stores the BF16 chunk into
// every peer's result region [parity]; after flag 1 from all ranks each rank copies the result
// region to its output.  Per rank (world - 1) / world of the fp32 values go out once and
// (world - 1) / world of the BF16 values once.
//
// The sum order is the rank order on every rank, so all ranks hold bit-identical outputs.
// A launch is `G <= SM count` CTAs that never wait for one another; the last CTA to finish a
// phase (ticket counter) raises that phase's flags.  Waits for peers are bounded (2 s) and end
// in STATUS_WAIT_TIMEOUT.  Steps are numbered by a device counter, so a captured graph can be
// replayed; the parities keep a fast rank's next step from overwriting what a slow rank still
// reads (a rank can be at most one step ahead: finishing a step needs every rank's flags).
#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tk100 {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Threads 0..world-1 wait until sender `threadIdx.x` has published `step`; false after 2 s.
__device__ __forceinline__ bool wait_flags(const unsigned int* flags, int world, unsigned int step,
                                           uint32_t* status, unsigned int* s_ok) {
  if (threadIdx.x < world) {
    const uint64_t start = global_timer_ns();
    for (;;) {
      if (static_cast<int>(ld_acquire_sys(flags + threadIdx.x) - step) >= 0) break;
      if (global_timer_ns() - start > 2000000000ull) {
        atomicOr(status, STATUS_WAIT_TIMEOUT);
        *s_ok = 0u;
        break;
      }
    }
  }
  __syncthreads();
  return *s_ok != 0u;
}

// True in exactly one CTA per phase: the last one to arrive.  Re-arms the ticket.
__device__ __forceinline__ bool last_cta(unsigned int* ticket, unsigned int* s_last) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(ticket, 1u);
    *s_last = t == gridDim.x - 1 ? 1u : 0u;
    if (*s_last) {
      *ticket = 0u;
      __threadfence_system();
    }
  }
  __syncthreads();
  return *s_last != 0u;
}

__global__ void __launch_bounds__(kThreads)
    peer_sum_kernel(PeerSumParams q, ExchangePeers peers) {
  __shared__ unsigned int s_step, s_ok, s_last;
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0) {
    s_step = *q.step_counter + 1u;  // stable for the whole launch: written back by the last CTA only
    s_ok = 1u;
  }
  __syncthreads();
  const unsigned int step = s_step;
  const unsigned int parity = step & 1u;
  const int world = q.world, rank = q.rank;
  const long long n = q.elems;           // multiple of 8
  const long long n4 = n >> 2;
  const long long tid = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * kThreads;
  unsigned char* mine = peers.base[rank];
  unsigned int* my_flags = reinterpret_cast<unsigned int*>(mine + q.flag_offset);
  const float4* src = reinterpret_cast<const float4*>(q.partial);

  if (q.one_shot) {
    // ---- deliver the whole partial to every rank's slot [parity][rank]
    for (int d = 0; d < world; ++d) {
      float4* dst = reinterpret_cast<float4*>(peers.base[d] + q.one_shot_offset) +
                    (static_cast<long long>(parity) * world + rank) * q.one_shot_stride4;
      for (long long i = tid; i < n4; i += stride) dst[i] = src[i];
    }
    if (last_cta(q.tickets + 0, &s_last) && threadIdx.x < world) {
      st_release_sys(reinterpret_cast<unsigned int*>(peers.base[threadIdx.x] + q.flag_offset) + rank, step);
    }
    if (!wait_flags(my_flags, world, step, q.status, &s_ok)) return;
    // ---- add the senders' partials in rank order, round once
    const float4* slots = reinterpret_cast<const float4*>(mine + q.one_shot_offset) +
                          static_cast<long long>(parity) * world * q.one_shot_stride4;
    for (long long i = tid; i < n4; i += stride) {
      float4 acc = __ldcv(slots + i);
      for (int s = 1; s < world; ++s) {
        const float4 v = __ldcv(slots + static_cast<long long>(s) * q.one_shot_stride4 + i);
        acc.x = __fadd_rn(acc.x, v.x);
        acc.y = __fadd_rn(acc.y, v.y);
        acc.z = __fadd_rn(acc.z, v.z);
        acc.w = __fadd_rn(acc.w, v.w);
      }
      reinterpret_cast<uint2*>(q.output)[i] = make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
    }
    if (last_cta(q.tickets + 2, &s_last) && threadIdx.x == 0) *q.step_counter = step;
    return;
  }

  // -------------------------------------------------------------------- two-shot
  const long long chunk4 = q.chunk >> 2;          // float4 per chunk of this call (chunk % 8 == 0)
  const long long slot4 = q.chunk_capacity >> 2;  // slot / result stride: the capacity's chunk
  // ---- chunk d of this rank's partial -> rank d, slot [rank]
  for (long long i = tid; i < n4; i += stride) {
    const long long d = i / chunk4, off = i - d * chunk4;
    reinterpret_cast<float4*>(peers.base[d])[static_cast<long long>(rank) * slot4 + off] = src[i];
  }
  if (last_cta(q.tickets + 0, &s_last) && threadIdx.x < world) {
    st_release_sys(reinterpret_cast<unsigned int*>(peers.base[threadIdx.x] + q.flag_offset) + rank, step);
  }
  if (!wait_flags(my_flags, world, step, q.status, &s_ok)) return;
  // ---- this rank's chunk: add the senders in rank order, round, publish to every rank
  {
    const long long begin4 = static_cast<long long>(rank) * chunk4;
    const long long len4 = max(0ll, min(chunk4, n4 - begin4));
    const float4* slots = reinterpret_cast<const float4*>(mine);
    for (long long i = tid; i < len4; i += stride) {
      float4 acc = __ldcv(slots + i);
      for (int s = 1; s < world; ++s) {
        const float4 v = __ldcv(slots + static_cast<long long>(s) * slot4 + i);
        acc.x = __fadd_rn(acc.x, v.x);
        acc.y = __fadd_rn(acc.y, v.y);
        acc.z = __fadd_rn(acc.z, v.z);
        acc.w = __fadd_rn(acc.w, v.w);
      }
      const uint2 r = make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
      for (int d = 0; d < world; ++d) {
        uint2* res = reinterpret_cast<uint2*>(peers.base[d] + q.result_offset) +
                     static_cast<long long>(parity) * world * slot4;
        res[begin4 + i] = r;
      }
    }
  }
  if (last_cta(q.tickets + 1, &s_last) && threadIdx.x < world) {
    st_release_sys(reinterpret_cast<unsigned int*>(peers.base[threadIdx.x] + q.flag_offset) + world + rank, step);
  }
  if (!wait_flags(my_flags + world, world, step, q.status, &s_ok)) return;
  // ---- all chunks are here: result region -> output
  {
    const uint2* res = reinterpret_cast<const uint2*>(mine + q.result_offset) +
                       static_cast<long long>(parity) * world * slot4;
    for (long long i = tid; i < n4; i += stride) reinterpret_cast<uint2*>(q.output)[i] = __ldcv(res + i);
  }
  if (last_cta(q.tickets + 2, &s_last) && threadIdx.x == 0) *q.step_counter = step;
}

}  // namespace

cudaError_t launch_peer_sum(cudaStream_t stream, int ctas, const PeerSumParams& q,
                            const ExchangePeers& peers) {
  return launch_kernel(peer_sum_kernel, dim3(static_cast<unsigned int>(ctas)), dim3(kThreads), 0, stream, q,
                       peers);
}

}  // namespace tk100
