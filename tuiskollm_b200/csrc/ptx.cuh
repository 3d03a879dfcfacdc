// Thin inline-PTX wrappers for the sm_100a features the projection kernels use:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM allocation, UMMA issue,
// commit, TMEM loads) and the shared-memory / instruction descriptors.
//
// Every wait is bounded: a spin that runs out records a code in the status word
// and returns false so that the caller can leave its loop, drain and exit
// instead of hanging the device.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tk100 {

// Bits of the device status word (ORed in by kernels, read back by the host).
enum : uint32_t {
  STATUS_WAIT_TIMEOUT = 1u << 0,     // a bounded mbarrier wait ran out
  STATUS_NONFINITE_LOGIT = 1u << 1,  // LM head produced a NaN/Inf logit
  STATUS_NONFINITE_INPUT = 1u << 2,  // quantiser met a NaN/Inf activation
  STATUS_BAD_ARGUMENT = 1u << 3,     // a kernel-side shape check failed
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-stream-serialisation attribute may start while
// its predecessor in the stream is still running.  pdl_wait() blocks until every
// predecessor grid has completed and its writes are visible; everything a kernel does
// before it must not depend on, or disturb, the predecessor (weight prefetch, barrier and
// TMEM set-up only).  pdl_trigger() lets the successor start launching.  Both are no-ops
// for a kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ------------------------------------------------------------ thread-block clusters
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// Cluster-wide barrier with release/acquire ordering of shared-memory writes; every thread
// of every CTA of the cluster must call both halves.
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// The same barrier without memory ordering: for "nobody leaves before everybody is done reading",
// where the reads have already returned their values.
__device__ __forceinline__ void cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_relaxed() {
  asm volatile("barrier.cluster.wait;" ::: "memory");
}

// shared::cluster address of the byte at local shared-memory address `local_smem_addr` in CTA
// `rank` of this cluster.
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
  return remote;
}

// fp32 load from the shared memory of CTA `rank` of this cluster, at the same offset as the
// local shared-memory address `local_smem_addr` (distributed shared memory).
__device__ __forceinline__ float ld_dsmem_f32(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// ------------------------------------------------------------------ mbarrier

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, UMMA).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: about two seconds of wall time, then STATUS_WAIT_TIMEOUT and false.  A wait that
// gave up earlier in this stream has already made the results invalid, so once the bit is set
// every later slow wait gives up at its first look instead of queueing more multi-second waits
// (no kernel reads the status word on its way in: that load sat on every CTA's critical path).
static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, uint32_t* status) {
  const uint64_t start = global_timer_ns();
  for (;;) {
    for (int i = 0; i < 1024; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (status && (*reinterpret_cast<volatile uint32_t*>(status) & STATUS_WAIT_TIMEOUT)) return false;
    if (global_timer_ns() - start > 2000000000ull) {
      if (status) atomicOr(status, STATUS_WAIT_TIMEOUT);
      return false;
    }
  }
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t* status) {
#pragma unroll 1
  for (int i = 0; i < 64; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return mbar_wait_slow(bar, parity, status);
}

// Cluster-scope forms for barriers that CTAs of the same cluster arrive on remotely
// (`cluster_addr` from mapa_u32): the arrive releases the arriving thread's prior writes --
// its stores into the owner's shared memory included -- and the owner's wait acquires them.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded like mbar_wait.
static __device__ __noinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, uint32_t* status) {
  const uint64_t start = global_timer_ns();
  for (;;) {
    for (int i = 0; i < 1024; ++i) {
      if (mbar_try_wait_cluster(bar, parity)) return true;
    }
    if (status && (*reinterpret_cast<volatile uint32_t*>(status) & STATUS_WAIT_TIMEOUT)) return false;
    if (global_timer_ns() - start > 2000000000ull) {
      if (status) atomicOr(status, STATUS_WAIT_TIMEOUT);
      return false;
    }
  }
}

// fp32 store into the shared memory of another CTA of this cluster (`cluster_addr` from mapa_u32).
__device__ __forceinline__ void st_dsmem_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}

// ----------------------------------------------------------------------- TMA

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// fp32 store with an L2 cache policy (e.g. evict_last: the line stays in L2 instead of being
// written back to DRAM in the middle of a read stream).
__device__ __forceinline__ void st_global_f32_policy(float* p, float v, uint64_t policy) {
  asm volatile("st.global.L2::cache_hint.f32 [%0], %1, %2;" ::"l"(p), "f"(v), "l"(policy) : "memory");
}

// 2-D tiled load, completion counted in bytes on `bar`.  c0 is the innermost
// coordinate; c0 * element size must be a multiple of 16 bytes.
// Asks L2 to fetch one box of a tiled tensor; nothing lands in shared memory and nothing is
// signalled.  Same 16-byte rule for x as a load.
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y)
               : "memory");
}

// Asks L2 to fetch `bytes` (a multiple of 16) from a 16-byte aligned global address.
__device__ __forceinline__ void bulk_prefetch_l2(const void* gptr, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<uint64_t>(gptr)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int32_t c0, int32_t c1, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1), "l"(policy)
      : "memory");
}

// 1-D bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                             uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes),
        "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// ------------------------------------------------------------------- tcgen05

// Allocates `cols` TMEM columns (power of two >= 32); one full warp must call it.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(cols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Arrives once on `bar` when every tcgen05 operation this thread issued so far is done.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], E4M3/E5M2/E2M1... operands (kind::f8f6f4), K = 32 bytes.
__device__ __forceinline__ void umma_f8f6f4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Block-scaled NVFP4: E2M1 operands, one UE4M3 scale per 16 elements, K = 64 elements.
__device__ __forceinline__ void umma_nvfp4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                           uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X"
      " [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb),
        "r"(accumulate)
      : "memory");
}

// Copies 32 rows x 16 bytes of shared memory into 4 TMEM columns, replicated to the
// four 32-lane quadrants (the layout block-scaled UMMA reads scale factors from).
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t tmem_dst, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(smem_desc)
               : "memory");
}

// 16 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------- tcgen05 with cta_group::2
// Two CTAs of a cluster (ranks 2k, 2k+1) work as one UMMA unit: each holds 128 rows of the
// "A" operand and half of the "B" columns in its own shared memory and 128 lanes of the
// accumulator in its own TMEM; the even CTA issues the instructions for both.

// Tiled load into this CTA's shared memory whose completion is counted on a barrier that may
// live in the pair's other CTA (`mbar_cluster_addr` is a shared::cluster address); the data
// itself goes to this CTA only.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map,
                                                 uint32_t mbar_cluster_addr, int32_t c0, int32_t c1,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(mbar_cluster_addr),
        "r"(c0), "r"(c1), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}

// Arrives on the barrier at this shared-memory offset in both CTAs of the pair when every
// tcgen05 operation issued so far by this thread has completed: one commit per CTA, the
// peer's barrier addressed through its shared::cluster address.  Issued by the even CTA.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint32_t mine = smem_u32(bar);
  const uint32_t peer = mapa_u32(mine, 1);
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   mine)
               : "memory");
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   peer)
               : "memory");
}

__device__ __forceinline__ void umma_nvfp4_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X"
      " [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb),
        "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_f8f6f4_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tmem_cp_32x128b_warpx4_pair(uint32_t tmem_dst, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(smem_desc)
               : "memory");
}

// Shared-memory matrix descriptor for a K-major operand stored as rows of 128 bytes
// with the 128-byte swizzle (what a TMA box of 128 bytes x R rows writes): groups of
// 8 rows are 1024 bytes apart; the tile base must be 1024-byte aligned.  Stepping
// along K inside the 128-byte row is done by adding the byte offset to `addr`.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);  // start address [0,14)
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused) [16,30)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset [32,46)
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                      // layout: 128-byte swizzle
  return d;
}

// Descriptor for an unswizzled block of 8-row x 16-byte core matrices stacked along
// rows (128 contiguous bytes per core matrix): used as the tcgen05.cp source for one
// 32-row x 16-byte scale-factor chunk.
__device__ __forceinline__ uint64_t umma_desc_noswizzle_rows16(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(0) << 16;          // leading byte offset (single 16-byte column)
  d |= static_cast<uint64_t>(128 >> 4) << 32;   // 8-row groups are 128 bytes apart
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// Instruction descriptor, kind::f8f6f4, E4M3 x E4M3 -> F32, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(uint32_t m, uint32_t n) {
  return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Instruction descriptor, kind::mxf4nvf4, E2M1 x E2M1 with UE4M3 block scales -> F32.
__host__ __device__ constexpr uint32_t umma_idesc_nvfp4(uint32_t m, uint32_t n) {
  return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (0u << 23) | ((m >> 4) << 24);
}

}  // namespace tk100
