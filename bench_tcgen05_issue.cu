// Micro-benchmark behind the NVFP4 kernels' design: how fast one thread can issue block-scaled
// tcgen05.mma together with the tcgen05.cp scale copies they need, with the operands already
// resident in shared memory (no loads).  One CTA per SM, clock64 around the loop, CUDA events
// around the launch.  Not linked into the library: `python bench.py --case issue` compiles it
// next to this file and runs it (the tensor-pipe ceiling of the instruction mix that the
// block-scaled FP4 roofline fractions are read against).  Every wait is bounded.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "tuiskollm_b200/csrc/ptx.cuh"

using namespace tk100;

constexpr int kIters = 4000;  // k-steps of 64

template <int N, int MODE>
__global__ void __launch_bounds__(128, 1) bench_kernel(long long* cycles, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t bar, bar2;
  __shared__ uint32_t tmem_base;
  // [W 16 KB][A N*128 B][SF 8 KB]
  for (int i = threadIdx.x; i < (16384 + N * 128 + 8192) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem)[i] = 0x38383838u;  // finite codes / scales
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init(&bar2, 1);
    fence_mbar_init();
  }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) {
    tmem_alloc(&tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base;
  if (threadIdx.x == 0) {
    const uint32_t base = smem_u32(smem);
    const uint64_t dw = umma_desc_sw128(base);
    const uint64_t da = umma_desc_sw128(base + 16384);
    const uint32_t sfsm = base + 16384 + N * 128;
    const uint32_t sf_base = tmem + 384;
    constexpr uint32_t IDESC = umma_idesc_nvfp4(128, N);
    const long long t0 = clock64();
    for (int it = 0; it < kIters; it += 4) {
      if (MODE == 2) {  // grouped: all copies of a 256-deep block first
        for (int k4 = 0; k4 < 4; ++k4) {
          const uint32_t slot = sf_base + ((it + k4) % 8) * 16;
          tmem_cp_32x128b_warpx4(slot, umma_desc_noswizzle_rows16(sfsm + k4 * 512));
          tmem_cp_32x128b_warpx4(slot + 8, umma_desc_noswizzle_rows16(sfsm + 2048 + k4 * 512));
          if (N == 256)
            tmem_cp_32x128b_warpx4(slot + 12, umma_desc_noswizzle_rows16(sfsm + 4096 + k4 * 512));
        }
      }
      for (int k4 = 0; k4 < 4; ++k4) {
        const uint32_t slot = sf_base + ((it + k4) % 8) * 16;
        if (MODE == 1 || MODE == 5) {  // interleaved
          tmem_cp_32x128b_warpx4(slot, umma_desc_noswizzle_rows16(sfsm + k4 * 512));
          tmem_cp_32x128b_warpx4(slot + 8, umma_desc_noswizzle_rows16(sfsm + 2048 + k4 * 512));
          if (N == 256)
            tmem_cp_32x128b_warpx4(slot + 12, umma_desc_noswizzle_rows16(sfsm + 4096 + k4 * 512));
        }
        if (MODE == 3) {  // copies only
          tmem_cp_32x128b_warpx4(slot, umma_desc_noswizzle_rows16(sfsm + k4 * 512));
          tmem_cp_32x128b_warpx4(slot + 8, umma_desc_noswizzle_rows16(sfsm + 2048 + k4 * 512));
        } else if (MODE == 4) {  // two MMAs (gate, up) sharing SFB, three copies
          tmem_cp_32x128b_warpx4(slot, umma_desc_noswizzle_rows16(sfsm + k4 * 512));
          tmem_cp_32x128b_warpx4(slot + 4, umma_desc_noswizzle_rows16(sfsm + 4096 + k4 * 512));
          tmem_cp_32x128b_warpx4(slot + 8, umma_desc_noswizzle_rows16(sfsm + 2048 + k4 * 512));
          umma_nvfp4(tmem, dw + 2 * k4, da + 2 * k4, IDESC, slot, slot + 8, 1u);
          umma_nvfp4(tmem + N, dw + 2 * k4, da + 2 * k4, IDESC, slot + 4, slot + 8, 1u);
        } else {
          umma_nvfp4(tmem, dw + 2 * k4, da + 2 * k4, IDESC, slot, slot + 8, 1u);
        }
      }
      // MODE 5 / 6: a commit after every 256-deep block, as a mainloop that frees a ring stage does
      // (it arrives on a barrier nobody waits for)
      if (MODE == 5 || MODE == 6) umma_commit(&bar2);
    }
    umma_commit(&bar);
    mbar_wait(&bar, 0, status);
    const long long t1 = clock64();
    cycles[blockIdx.x] = t1 - t0;
  }
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}

// CTA pairs (tcgen05 cta_group::2, M = 256, N = 256): the even CTA issues the MMAs for both.
//   PMODE 0: MMA only.
//   PMODE 1: per K step three cta_group::2 scale copies (SFA, two SFB tiles), then the MMA.
//   PMODE 5 / 6: PMODE 4 / 3 plus one commit (to both CTAs) after every 256-deep block.
//   PMODE 7: PMODE 2 on the ring, with the leader's commit per block and the odd CTA's own.
//   PMODE 2: every CTA issues its own three copies with cta_group::1 (the odd CTA's run beside
//            the even CTA's MMAs, unsynchronised: rate only), the even CTA the cta_group::2 MMA.
template <int PMODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1)
    pair_kernel(long long* cycles, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t bar, bar2, bar3;
  __shared__ uint32_t tmem_base;
  const uint32_t rank = cluster_cta_rank();
  // kPairStages x ([W 16 KB][A 16 KB (128 tokens)][SF 8 KB]); PMODE >= 3 walks the stages like a
  // ring (fresh operand addresses every K block of 256), PMODE < 3 stays on stage 0
  constexpr int kPairStages = 4, kPairStage = 16384 + 16384 + 8192;
  for (int i = threadIdx.x; i < kPairStages * kPairStage / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem)[i] = 0x38383838u;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init(&bar2, 1);
    mbar_init(&bar3, 1);
    fence_mbar_init();
  }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) {
    tmem_alloc_pair(&tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base;
  if (threadIdx.x == 0) {
    const uint32_t base0 = smem_u32(smem);
    const uint32_t sf_base = tmem + 256;
    constexpr uint32_t IDESC = umma_idesc_nvfp4(256, 256);
    const long long t0 = clock64();
    for (int it = 0; it < kIters; ++it) {
      const int k4 = it & 3;
      const uint32_t base = base0 + (PMODE >= 3 ? ((it >> 2) % kPairStages) * kPairStage : 0);
      const uint64_t dw = umma_desc_sw128(base);
      const uint64_t da = umma_desc_sw128(base + 16384);
      const uint32_t sfsm = base + 32768;
      const uint32_t slot = sf_base + (it % 8) * 16;
      if ((PMODE == 1 || PMODE == 4 || PMODE == 5) && rank == 0) {
        tmem_cp_32x128b_warpx4_pair(slot, umma_desc_noswizzle_rows16(sfsm + k4 * 512));
        tmem_cp_32x128b_warpx4_pair(slot + 4, umma_desc_noswizzle_rows16(sfsm + 2048 + k4 * 512));
        tmem_cp_32x128b_warpx4_pair(slot + 8, umma_desc_noswizzle_rows16(sfsm + 4096 + k4 * 512));
      }
      if (PMODE == 2 || PMODE == 7) {
        tmem_cp_32x128b_warpx4(slot, umma_desc_noswizzle_rows16(sfsm + k4 * 512));
        tmem_cp_32x128b_warpx4(slot + 4, umma_desc_noswizzle_rows16(sfsm + 2048 + k4 * 512));
        tmem_cp_32x128b_warpx4(slot + 8, umma_desc_noswizzle_rows16(sfsm + 4096 + k4 * 512));
      }
      if (rank == 0) umma_nvfp4_pair(tmem, dw + 2 * k4, da + 2 * k4, IDESC, slot, slot + 4, 1u);
      // PMODE 5 / 6: a commit (to both CTAs) after every 256-deep block
      if ((PMODE == 5 || PMODE == 6 || PMODE == 7) && rank == 0 && k4 == 3) umma_commit_pair(&bar2);
      // PMODE 7: the odd CTA reports its own copies of the block on a barrier of its own
      if (PMODE == 7 && rank == 1 && k4 == 3) umma_commit(&bar3);
    }
    if (rank == 0) {
      umma_commit_pair(&bar);
    } else if (PMODE == 2 || PMODE == 7) {
      umma_commit(&bar);  // the odd CTA's own copies
    }
    if (rank == 0 || PMODE == 2 || PMODE == 7) mbar_wait(&bar, 0, status);
    else mbar_wait(&bar, 0, status);  // the even CTA's commit arrives here too
    const long long t1 = clock64();
    cycles[blockIdx.x] = t1 - t0;
  }
  __syncthreads();
  tc_fence_before_sync();
  cluster_arrive();
  cluster_wait();
  if (threadIdx.x < 32) tmem_dealloc_pair(tmem, 512);
}

template <int PMODE>
void run_pair(const char* name, long long* d_cycles, uint32_t* d_status) {
  const size_t smem = 1024 + 4 * (16384 + 16384 + 8192);
  cudaFuncSetAttribute(pair_kernel<PMODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  cudaEvent_t a, b;
  cudaEventCreate(&a);
  cudaEventCreate(&b);
  pair_kernel<PMODE><<<148, 128, smem>>>(d_cycles, d_status);
  cudaDeviceSynchronize();
  cudaEventRecord(a);
  pair_kernel<PMODE><<<148, 128, smem>>>(d_cycles, d_status);
  cudaEventRecord(b);
  cudaError_t e = cudaDeviceSynchronize();
  float ms = 0;
  cudaEventElapsedTime(&ms, a, b);
  long long h[148];
  cudaMemcpy(h, d_cycles, sizeof(h), cudaMemcpyDeviceToHost);
  uint32_t st = 0;
  cudaMemcpy(&st, d_status, 4, cudaMemcpyDeviceToHost);
  const double flop = 2.0 * 256 * 256 * 64 * (double)kIters * 74;
  printf("%-34s pair M=256 N=256  %8.1f us  %7.1f cycles/k-step  %6.2f PF  (err %d status %u)\n", name,
         ms * 1e3, (double)h[0] / kIters, flop / (ms * 1e-3) / 1e15, (int)e, st);
}

template <int N, int MODE>
void run(const char* name, long long* d_cycles, uint32_t* d_status) {
  const size_t smem = 1024 + 16384 + N * 128 + 8192;
  cudaFuncSetAttribute(bench_kernel<N, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  cudaEvent_t a, b;
  cudaEventCreate(&a);
  cudaEventCreate(&b);
  bench_kernel<N, MODE><<<148, 128, smem>>>(d_cycles, d_status);
  cudaDeviceSynchronize();
  cudaEventRecord(a);
  bench_kernel<N, MODE><<<148, 128, smem>>>(d_cycles, d_status);
  cudaEventRecord(b);
  cudaError_t e = cudaDeviceSynchronize();
  float ms = 0;
  cudaEventElapsedTime(&ms, a, b);
  long long h[148];
  cudaMemcpy(h, d_cycles, sizeof(h), cudaMemcpyDeviceToHost);
  uint32_t st = 0;
  cudaMemcpy(&st, d_status, 4, cudaMemcpyDeviceToHost);
  const int mmas = MODE == 3 ? 0 : (MODE == 4 ? 2 : 1);
  const double flop = 2.0 * 128 * N * 64 * mmas * (double)kIters * 148;
  printf("%-34s N=%3d  %8.1f us  %7.1f cycles/k-step  %6.2f PF  (err %d status %u)\n", name, N,
         ms * 1e3, (double)h[0] / kIters, flop / (ms * 1e-3) / 1e15, (int)e, st);
}

int main() {
  long long* d_cycles;
  uint32_t* d_status;
  cudaMalloc(&d_cycles, 148 * sizeof(long long));
  cudaMalloc(&d_status, 4);
  cudaMemset(d_status, 0, 4);
  run<128, 0>("mma only", d_cycles, d_status);
  run<128, 1>("interleaved cpA cpB mma", d_cycles, d_status);
  run<128, 2>("grouped 8 cp then 4 mma", d_cycles, d_status);
  run<128, 3>("copies only (2 per step)", d_cycles, d_status);
  run<128, 4>("gate+up: 3 cp + 2 mma", d_cycles, d_status);
  run<256, 0>("mma only", d_cycles, d_status);
  run<256, 1>("interleaved cpA 2cpB mma", d_cycles, d_status);
  run<256, 2>("grouped 12 cp then 4 mma", d_cycles, d_status);
  run<64, 0>("mma only", d_cycles, d_status);
  run<64, 1>("interleaved", d_cycles, d_status);
  run_pair<0>("pair: mma only", d_cycles, d_status);
  run_pair<1>("pair: 3 cp.cg2 + mma", d_cycles, d_status);
  run_pair<2>("pair: 3 cp.cg1 per CTA + mma.cg2", d_cycles, d_status);
  run_pair<3>("pair: mma only, ring of 4 stages", d_cycles, d_status);
  run_pair<4>("pair: 3 cp.cg2 + mma, ring", d_cycles, d_status);
  run<128, 6>("mma only + commit per 4", d_cycles, d_status);
  run<128, 5>("interleaved + commit per 4", d_cycles, d_status);
  run_pair<6>("pair: mma only, ring, commit per 4", d_cycles, d_status);
  run_pair<5>("pair: 3 cp + mma, ring, commit/4", d_cycles, d_status);
  run_pair<7>("pair: own cg1 cps, ring, commit/4", d_cycles, d_status);
  return 0;
}
