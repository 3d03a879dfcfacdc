// Fused residual-add + zero-centred RMSNorm + per-token activation quantisation.
//
// One CTA owns one token row and keeps it in registers from the first load to the
// last store: x (+ branch) is read once, the rounded residual, the normalised row,
// the E4M3 codes and the fp32 scale are written once.  The reference runs this as
// three launches that each re-read the row from global memory
// (tuisko-kernels-sm120/src/residual_norm.rs:155-226 followed by
// tuisko-kernels-sm120/src/device/fp8_projection.rs:54-126).
//
// Numeric contract (bit-exact parts marked *):
//   res  = bf16_rn(f32(x) + f32(branch))                                  *
//   r    = 1/sqrt(sum(res^2)/H + eps), fp32, fixed summation order
//   y    = bf16_rn(res * r * (1 + w)), evaluated left to right in fp32
//   amax = max |y|; scale = amax == 0 ? 1 : amax / 448   (IEEE fp32 divide)   *
//   code = e4m3_rn_satfinite(y / scale)                  (IEEE fp32 divide)   *
// The starred results are bit-exact functions of their inputs; `codes`/`scale`
// are exact with respect to the normalised row this same kernel wrote.
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tk100 {

namespace {

constexpr int kMaxChunks = 4;  // 16-byte chunks (8 BF16) per thread

struct alignas(16) Chunk {
  uint32_t w[4];
};

// Optional NVFP4 side output of the fused producer (all null/zero when unused).
struct Nvfp4Out {
  uint8_t* codes;   // [rows, hidden/2]
  uint8_t* scales;  // 128-row x 4-group tiles, row = token
  float divisor;    // input global divisor
};

template <bool HAS_BRANCH, bool DO_NORM, bool DO_QUANT, int CHUNKS>
__global__ void __launch_bounds__(1024)
    resnorm_quant_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ branch,
                         const uint16_t* __restrict__ weight, uint16_t* __restrict__ residual_out,
                         uint16_t* __restrict__ normalized_out, uint8_t* __restrict__ codes,
                         float* __restrict__ scales, int hidden, float eps, uint32_t* status,
                         const Nvfp4Out nv) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();  // x / branch may be the predecessor's output
  const int row = blockIdx.x;
  const int chunks_per_row = hidden >> 3;
  const size_t row_off = static_cast<size_t>(row) * hidden;

  float v[CHUNKS][8];
  // The norm weight of this thread's columns is requested together with the row (one memory
  // latency less on the chain load -> reduce -> scale -> reduce -> store); with three or four
  // chunks per thread the registers do not allow it and the weight is loaded where it is used.
  constexpr bool EARLY_WEIGHT = DO_NORM && CHUNKS <= 2;
  Chunk wreg[EARLY_WEIGHT ? CHUNKS : 1];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < chunks_per_row) {
      if constexpr (EARLY_WEIGHT) wreg[i] = *reinterpret_cast<const Chunk*>(weight + c * 8);
      Chunk a = *reinterpret_cast<const Chunk*>(x + row_off + c * 8);
      if (HAS_BRANCH) {
        Chunk b = *reinterpret_cast<const Chunk*>(branch + row_off + c * 8);
        Chunk r;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = __fadd_rn(bf16x2_lo(a.w[j]), bf16x2_lo(b.w[j]));
          const float hi = __fadd_rn(bf16x2_hi(a.w[j]), bf16x2_hi(b.w[j]));
          r.w[j] = pack_bf16x2(lo, hi);
        }
        *reinterpret_cast<Chunk*>(residual_out + row_off + c * 8) = r;
        a = r;  // the norm consumes the rounded residual
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[i][2 * j] = bf16x2_lo(a.w[j]);
        v[i][2 * j + 1] = bf16x2_hi(a.w[j]);
      }
      if (DO_NORM) {
#pragma unroll
        for (int j = 0; j < 8; ++j) sum = __fmaf_rn(v[i][j], v[i][j], sum);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
    }
  }

  float amax = 0.0f;
  if (DO_NORM) {
    sum = block_reduce<false>(sum, scratch);
    const float mean = __fdiv_rn(sum, static_cast<float>(hidden));
    const float inv_rms = __frsqrt_rn(__fadd_rn(mean, eps));
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < chunks_per_row) {
        Chunk wv;
        if constexpr (EARLY_WEIGHT) wv = wreg[i];
        else wv = *reinterpret_cast<const Chunk*>(weight + c * 8);
        Chunk o;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = __fmul_rn(__fmul_rn(v[i][2 * j], inv_rms),
                                     __fadd_rn(1.0f, bf16x2_lo(wv.w[j])));
          const float hi = __fmul_rn(__fmul_rn(v[i][2 * j + 1], inv_rms),
                                     __fadd_rn(1.0f, bf16x2_hi(wv.w[j])));
          o.w[j] = pack_bf16x2(lo, hi);
          v[i][2 * j] = bf16x2_lo(o.w[j]);  // keep the rounded value for the quantiser
          v[i][2 * j + 1] = bf16x2_hi(o.w[j]);
        }
        *reinterpret_cast<Chunk*>(normalized_out + row_off + c * 8) = o;
      }
    }
  }

  if (nv.codes != nullptr) {
    // NVFP4 codes of the (rounded) row for the W4A4 MLP: a 16-column block is the two 8-value
    // chunks of an even/odd thread pair; same arithmetic as nvfp4_quantize_kernel.
    const int groups = hidden >> 4;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
      const int c = threadIdx.x + i * blockDim.x;  // chunk index; block g = c / 2
      float bmax = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) bmax = fmaxf(bmax, fabsf(v[i][j]));
      bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 1));
      if (c < chunks_per_row) {
        const float raw = __fdiv_rn(__fmul_rn(bmax, nv.divisor), 6.0f);
        const uint32_t sc = f32x2_to_e4m3x2(raw, 0.0f) & 0xffu;
        const float sd = e4m3_to_f32(sc);
        uint32_t packed = 0u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t byte;
          if (sd == 0.0f) {
            byte = (signbit(v[i][2 * j]) ? 0x08u : 0u) | (signbit(v[i][2 * j + 1]) ? 0x80u : 0u);
          } else {
            byte = f32x2_to_e2m1x2(__fdiv_rn(__fmul_rn(v[i][2 * j], nv.divisor), sd),
                                   __fdiv_rn(__fmul_rn(v[i][2 * j + 1], nv.divisor), sd)) & 0xffu;
          }
          packed |= byte << (8 * j);
        }
        *reinterpret_cast<uint32_t*>(nv.codes + static_cast<size_t>(row) * (hidden >> 1) + c * 4) = packed;
        if ((c & 1) == 0) {
          const int g = c >> 1;
          const size_t off = (static_cast<size_t>(row >> 7) * (groups >> 2) + (g >> 2)) * 512 +
                             static_cast<size_t>(row & 31) * 16 + ((row & 127) >> 5) * 4 + (g & 3);
          nv.scales[off] = static_cast<uint8_t>(sc);
        }
      }
    }
  }

  if (DO_QUANT) {
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
    }
    amax = block_reduce<true>(amax, scratch);
    if (!(amax <= 3.0e38f) && threadIdx.x == 0) atomicOr(status, STATUS_NONFINITE_INPUT);
    const float scale = (amax == 0.0f) ? 1.0f : __fdiv_rn(amax, 448.0f);
    if (threadIdx.x == 0) scales[row] = scale;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < chunks_per_row) {
        uint32_t q[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          q[j] = f32x2_to_e4m3x2(__fdiv_rn(v[i][2 * j], scale), __fdiv_rn(v[i][2 * j + 1], scale));
        }
        uint2 packed;
        packed.x = q[0] | (q[1] << 16);
        packed.y = q[2] | (q[3] << 16);
        *reinterpret_cast<uint2*>(codes + row_off + c * 8) = packed;
      }
    }
  }
}

template <bool HAS_BRANCH, bool DO_NORM, bool DO_QUANT>
cudaError_t launch_chunks(cudaStream_t stream, int rows, int hidden, int threads, int chunks,
                          const uint16_t* x, const uint16_t* branch, const uint16_t* weight,
                          uint16_t* residual_out, uint16_t* normalized_out, uint8_t* codes,
                          float* scales, float eps, uint32_t* status, const Nvfp4Out& nv) {
#define TK100_LAUNCH(C)                                                                       \
  launch_kernel(resnorm_quant_kernel<HAS_BRANCH, DO_NORM, DO_QUANT, C>, dim3(rows), dim3(threads), \
                0, stream, x, branch, weight, residual_out, normalized_out, codes, scales, hidden, \
                eps, status, nv)
  switch (chunks) {
    case 1: return TK100_LAUNCH(1);
    case 2: return TK100_LAUNCH(2);
    case 3: return TK100_LAUNCH(3);
    default: return TK100_LAUNCH(4);
  }
#undef TK100_LAUNCH
}

}  // namespace

namespace {
bool g_pdl = true;
uint32_t g_debug = 0;
unsigned long long* g_stamps = nullptr;
}  // namespace

void read_process_switches() {
  const char* v = std::getenv("TK100_PDL");
  g_pdl = !(v && v[0] == '0');
#ifdef TK100_EXPERIMENT
  const char* d = std::getenv("TK100_DEBUG");
  g_debug = d ? static_cast<uint32_t>(std::atoi(d)) : 0u;
  const char* sp = std::getenv("TK100_STAMPS_PTR");
  g_stamps = sp ? reinterpret_cast<unsigned long long*>(std::strtoull(sp, nullptr, 0)) : nullptr;
#endif
}

bool pdl_enabled() { return g_pdl; }

uint32_t debug_flags() { return g_debug; }

unsigned long long* debug_stamps() { return g_stamps; }

bool norm_geometry(int hidden, int* threads, int* chunks) {
  if (hidden <= 0 || (hidden & 7) != 0) return false;
  const int row_chunks = hidden >> 3;
  // One chunk per thread while the row fits a 1024-thread CTA, warp-multiple CTAs.
  int c = (row_chunks + 1023) / 1024;
  if (c > kMaxChunks) return false;
  // Prefer CTAs of at most 640 threads (three co-resident per SM) when that costs
  // no extra chunk, e.g. 5120 -> 640 x 1, 17408 -> 544 x 4.
  int t = (row_chunks + c - 1) / c;
  if (t > 704 && c < kMaxChunks) {
    c = (row_chunks + 639) / 640;
    if (c > kMaxChunks) c = kMaxChunks;
    t = (row_chunks + c - 1) / c;
  }
  t = (t + 31) & ~31;
  if (t > 1024) return false;
  *threads = t;
  *chunks = c;
  return true;
}

cudaError_t launch_resnorm_quant(cudaStream_t stream, int rows, int hidden, const uint16_t* x,
                                 const uint16_t* branch, const uint16_t* weight,
                                 uint16_t* residual_out, uint16_t* normalized_out, uint8_t* codes,
                                 float* scales, float eps, uint32_t* status, uint8_t* nvfp4_codes,
                                 uint8_t* nvfp4_scales, float nvfp4_divisor) {
  const Nvfp4Out nv{nvfp4_codes, nvfp4_scales, nvfp4_divisor};
  int threads = 0, chunks = 0;
  if (!norm_geometry(hidden, &threads, &chunks)) return cudaErrorInvalidValue;
  // A row per CTA: with one 16-byte chunk per thread (640 threads for 5120 columns) three CTAs
  // share an SM, so 256 or 512 rows run as one and a bit, or two, waves of CTAs that each sit
  // through two block reductions.  More chunks per thread = smaller CTAs = more rows in flight per
  // SM: take the fewest chunks that put all rows into one wave, the most when none does.
  {
    static int sms = 0;
    if (sms == 0) {
      int device = 0;
      if (cudaGetDevice(&device) != cudaSuccess ||
          cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
        sms = 148;
      }
    }
    const int row_chunks = hidden >> 3;
    while (chunks * 2 <= kMaxChunks && rows > sms * (2048 / threads)) {
      const int c = chunks * 2;
      const int t = ((row_chunks + c - 1) / c + 31) & ~31;
      if (t < 128) break;
      chunks = c;
      threads = t;
    }
  }
  const bool has_branch = branch != nullptr;
  const bool do_norm = normalized_out != nullptr;
  const bool do_quant = codes != nullptr;
#define TK100_CASE(B, N, Q)                                                                      \
  if (has_branch == B && do_norm == N && do_quant == Q)                                          \
  return launch_chunks<B, N, Q>(stream, rows, hidden, threads, chunks, x, branch, weight,        \
                                residual_out, normalized_out, codes, scales, eps, status, nv)
  TK100_CASE(true, true, true);
  TK100_CASE(true, true, false);
  TK100_CASE(false, true, true);
  TK100_CASE(false, true, false);
  TK100_CASE(false, false, true);
#undef TK100_CASE
  return cudaErrorInvalidValue;
}

}  // namespace tk100
