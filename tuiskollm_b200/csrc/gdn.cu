// Gated-delta-net decode step either side of the FP8 GDN projections: the control mat-vecs and
// the width-4 causal convolution ("prepare"), and the FP32 state recurrence with its gated
// RMSNorm.  Replaces tuisko-kernels-sm120/src/gdn/prepare.rs:41-102 (bodies
// src/device/gdn_prepare.rs:34-142) and src/gdn/recurrence.rs:41-88 (body
// src/device/gdn_recurrence.rs:42-186).
//
// Both steps are HBM- and latency-bound byte movers (0.98 MB of control weights, 6.29 MB of
// state per token), so the work here is in how the bytes move:
//   * prepare is ONE launch: CTAs [0, 96) each own one control row for all tokens of the batch
//     (the weight row is read once, 16 bytes per load), the remaining CTAs run the convolution
//     on 8 channels per thread (history, weights, input and output as 16-byte accesses);
//   * the recurrence gives every (token, value head) a cluster of 4 CTAs, 32 state rows each:
//     four times the CTAs in flight of a head-per-CTA grid at batch 1, every state byte loaded
//     as part of an independent 16-byte request issued before any arithmetic, q/k normalised by
//     each warp for itself (no block barrier in front of the state math), and the one value that
//     couples the rows -- the mean square of the 128 recurrent outputs -- exchanged through
//     distributed shared memory with a single cluster barrier.
#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tk100 {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float ex2_approx(float v) {
  float r;
  asm("ex2.approx.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float lg2_approx(float v) {
  float r;
  asm("lg2.approx.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float rsqrt_approx(float v) {
  float r;
  asm("rsqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
// The reference's forms (device/gdn_prepare.rs:14-31): exp through ex2.approx, an IEEE divide.
__device__ __forceinline__ float fast_exp(float v) { return ex2_approx(v * kLog2e); }
__device__ __forceinline__ float sigmoid_ref(float v) { return __fdiv_rn(1.0f, 1.0f + fast_exp(-v)); }
__device__ __forceinline__ float softplus_ref(float v) {
  return v > 20.0f ? v : lg2_approx(1.0f + fast_exp(v)) * kLn2;
}

__device__ __forceinline__ uint4 ldg16(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// Sum over 8 BF16 pairs-of-chunks: acc += x[j] * w[j] for the 8 values packed in two uint4.
__device__ __forceinline__ float dot8(const uint4& x, const uint4& w, float acc) {
  acc = fmaf(bf16x2_lo(x.x), bf16x2_lo(w.x), acc);
  acc = fmaf(bf16x2_hi(x.x), bf16x2_hi(w.x), acc);
  acc = fmaf(bf16x2_lo(x.y), bf16x2_lo(w.y), acc);
  acc = fmaf(bf16x2_hi(x.y), bf16x2_hi(w.y), acc);
  acc = fmaf(bf16x2_lo(x.z), bf16x2_lo(w.z), acc);
  acc = fmaf(bf16x2_hi(x.z), bf16x2_hi(w.z), acc);
  acc = fmaf(bf16x2_lo(x.w), bf16x2_lo(w.w), acc);
  acc = fmaf(bf16x2_hi(x.w), bf16x2_hi(w.w), acc);
  return acc;
}

constexpr int kPrepThreads = 320;
constexpr int kPrepWarps = kPrepThreads / 32;
constexpr int kMaxChunksPerThread = 4;  // hidden <= 320 * 4 * 8 = 10240

// --------------------------------------------------------------------------- prepare
// CTAs [0, 2 * control_rows): one fused control row each, all tokens.
// CTAs beyond: the convolution, 8 channels per thread.
__global__ void __launch_bounds__(kPrepThreads) gdn_prepare_kernel(GdnPrepareParams p) {
  __shared__ float partial[kPrepWarps][kGdnMaxBatch];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int control_ctas = 2 * p.control_rows;

  if (static_cast<int>(blockIdx.x) < control_ctas) {
    const int row = blockIdx.x;
    const int chunks = p.hidden / 8;
    // Weights do not depend on the predecessor: request them before waiting for it.
    uint4 w[kMaxChunksPerThread];
#pragma unroll
    for (int c = 0; c < kMaxChunksPerThread; ++c) {
      const int chunk = tid + c * kPrepThreads;
      w[c] = chunk < chunks ? ldg16(p.control_weights + static_cast<size_t>(row) * p.hidden + chunk * 8)
                            : make_uint4(0, 0, 0, 0);
    }
    pdl_wait();
    pdl_trigger();
    // Two chunk columns at a time: all tokens' loads of a column pair are requested before the
    // first FMA on them, so a batch of 8 costs one round trip to L2 per pair, not eight.
    float acc[kGdnMaxBatch];
#pragma unroll
    for (int t = 0; t < kGdnMaxBatch; ++t) acc[t] = 0.0f;
#pragma unroll
    for (int c0 = 0; c0 < kMaxChunksPerThread; c0 += 2) {
      uint4 x[kGdnMaxBatch][2];
#pragma unroll
      for (int t = 0; t < kGdnMaxBatch; ++t) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int chunk = tid + (c0 + c) * kPrepThreads;
          x[t][c] = (t < p.batch && chunk < chunks)
                        ? ldg16(p.input + static_cast<size_t>(t) * p.hidden + chunk * 8)
                        : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int t = 0; t < kGdnMaxBatch; ++t) {
        acc[t] = dot8(x[t][0], w[c0], acc[t]);
        acc[t] = dot8(x[t][1], w[c0 + 1], acc[t]);
      }
    }
#pragma unroll
    for (int t = 0; t < kGdnMaxBatch; ++t) {
      if (t < p.batch) {
        const float s = warp_sum(acc[t]);
        if (lane == 0) partial[warp][t] = s;
      }
    }
    __syncthreads();
    if (tid < p.batch) {
      float sum = partial[0][tid];
#pragma unroll
      for (int i = 1; i < kPrepWarps; ++i) sum += partial[i][tid];
      if (row < p.control_rows) {
        const float control = sum + bf16_bits_to_f32(p.dt_bias[row]);
        p.log_decay[tid * p.control_rows + row] =
            -fast_exp(bf16_bits_to_f32(p.a_log[row])) * softplus_ref(control);
      } else {
        p.beta[tid * p.control_rows + row - p.control_rows] = sigmoid_ref(sum);
      }
    }
    return;
  }

  // Convolution: 8 adjacent channels of one token per thread.
  const int groups = p.qkv_rows / 8;
  const int index = (static_cast<int>(blockIdx.x) - control_ctas) * kPrepThreads + tid;
  pdl_wait();
  pdl_trigger();
  if (index >= p.batch * groups) return;
  const int token = index / groups;
  const int channel = (index - token * groups) * 8;
  const size_t state_row = p.state_rows[token];
  uint16_t* hist = p.history + (state_row * p.qkv_rows + channel) * 3;  // 48 bytes, 16-aligned
  const uint4 cur4 = ldg16(p.projected + static_cast<size_t>(token) * p.input_rows + channel);
  const uint4 h4[3] = {*reinterpret_cast<const uint4*>(hist), *reinterpret_cast<const uint4*>(hist + 8),
                       *reinterpret_cast<const uint4*>(hist + 16)};
  uint4 w4[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) w4[i] = ldg16(p.convolution_weights + static_cast<size_t>(channel) * 4 + i * 8);

  const uint32_t hw[12] = {h4[0].x, h4[0].y, h4[0].z, h4[0].w, h4[1].x, h4[1].y,
                           h4[1].z, h4[1].w, h4[2].x, h4[2].y, h4[2].z, h4[2].w};
  const uint32_t ww[16] = {w4[0].x, w4[0].y, w4[0].z, w4[0].w, w4[1].x, w4[1].y, w4[1].z, w4[1].w,
                           w4[2].x, w4[2].y, w4[2].z, w4[2].w, w4[3].x, w4[3].y, w4[3].z, w4[3].w};
  const uint32_t cw[4] = {cur4.x, cur4.y, cur4.z, cur4.w};
  auto half_of = [](const uint32_t* words, int i) -> uint32_t {
    return (words[i >> 1] >> ((i & 1) * 16)) & 0xffffu;
  };
  uint32_t new_hist[24];
  uint32_t out_bits[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t h0 = half_of(hw, 3 * c), h1 = half_of(hw, 3 * c + 1), h2 = half_of(hw, 3 * c + 2);
    const uint32_t cur = half_of(cw, c);
    new_hist[3 * c] = h1;
    new_hist[3 * c + 1] = h2;
    new_hist[3 * c + 2] = cur;
    // Same association as the reference: w0*h0 + (w1*h1 + (w2*h2 + w3*cur)), each step one FMA.
    const float sum = fmaf(
        bf16_bits_to_f32(half_of(ww, 4 * c)), bf16_bits_to_f32(h0),
        fmaf(bf16_bits_to_f32(half_of(ww, 4 * c + 1)), bf16_bits_to_f32(h1),
             fmaf(bf16_bits_to_f32(half_of(ww, 4 * c + 2)), bf16_bits_to_f32(h2),
                  bf16_bits_to_f32(half_of(ww, 4 * c + 3)) * bf16_bits_to_f32(cur))));
    out_bits[c] = f32_to_bf16_bits(sum * sigmoid_ref(sum));
  }
  uint4 s[3];
  uint32_t* sw = reinterpret_cast<uint32_t*>(s);
#pragma unroll
  for (int i = 0; i < 12; ++i) sw[i] = new_hist[2 * i] | (new_hist[2 * i + 1] << 16);
  *reinterpret_cast<uint4*>(hist) = s[0];
  *reinterpret_cast<uint4*>(hist + 8) = s[1];
  *reinterpret_cast<uint4*>(hist + 16) = s[2];
  uint4 o;
  o.x = out_bits[0] | (out_bits[1] << 16);
  o.y = out_bits[2] | (out_bits[3] << 16);
  o.z = out_bits[4] | (out_bits[5] << 16);
  o.w = out_bits[6] | (out_bits[7] << 16);
  *reinterpret_cast<uint4*>(p.convolved + static_cast<size_t>(token) * p.qkv_rows + channel) = o;
}

// ------------------------------------------------------------------------ recurrence
constexpr int kHeadDim = 128;
constexpr int kKeyHeads = 16;
constexpr int kValueHeads = 48;
constexpr int kQkWidth = kKeyHeads * kHeadDim;
constexpr int kRecThreads = 256;
constexpr int kRecWarps = kRecThreads / 32;
constexpr float kRmsEpsilon = 1.0e-6f;
constexpr float kDeltaScale = 0.08838835f;  // 1 / sqrt(128)

__device__ __forceinline__ float dot4(const float4& a, const float4& b) {
  return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, a.w * b.w)));
}

// Four BF16 values at p (8-byte aligned) as floats.
__device__ __forceinline__ float4 load_bf16x4(const uint16_t* p) {
  const uint2 w = __ldg(reinterpret_cast<const uint2*>(p));
  return make_float4(bf16x2_lo(w.x), bf16x2_hi(w.x), bf16x2_lo(w.y), bf16x2_hi(w.y));
}

// SPLIT = CTAs (one cluster) per (token, value head): 4 up to batch 4 (at most 768 CTAs of 32 state
// rows), 2 beyond (at most 768 CTAs of 64 rows), so that every batch runs as one wave.
template <int SPLIT>
__global__ void __cluster_dims__(SPLIT, 1, 1) __launch_bounds__(kRecThreads)
    gdn_recurrence_kernel(GdnRecurrenceParams p) {
  constexpr int kRecSplit = SPLIT;
  constexpr int kRowsPerCta = kHeadDim / kRecSplit;
  constexpr int kRowsPerWarp = kRowsPerCta / kRecWarps;
  // Every CTA of the cluster holds all partial sums of squares (pushed by their owners) and
  // its own 32 recurrent outputs.
  __shared__ float squares[kRecSplit * kRecWarps];
  __shared__ float recurrent[kRowsPerCta];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t rank = cluster_cta_rank();
  const int unit = blockIdx.x / kRecSplit;
  const int token = unit / kValueHeads;
  const int value_head = unit - token * kValueHeads;
  const int key_head = value_head / (kValueHeads / kKeyHeads);
  const int row0 = static_cast<int>(rank) * kRowsPerCta + warp * kRowsPerWarp;

  // First half of the "every CTA of the cluster is running" barrier a remote shared-memory store
  // needs; the second half sits in front of the push, behind the state math.
  cluster_arrive();
  pdl_wait();
  pdl_trigger();

  const size_t state_row = p.state_rows[token];
  float* state = p.state + ((state_row * kValueHeads + value_head) * kHeadDim + row0) * kHeadDim;
  // All state bytes of this warp in flight before anything depends on them.
  float4 old_state[kRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i)
    old_state[i] = *reinterpret_cast<const float4*>(state + i * kHeadDim + lane * 4);

  const uint16_t* token_qkv = p.qkv + static_cast<size_t>(token) * p.qkv_rows;
  float4 q = load_bf16x4(token_qkv + key_head * kHeadDim + lane * 4);
  float4 k = load_bf16x4(token_qkv + kQkWidth + key_head * kHeadDim + lane * 4);
  const uint16_t* value_row = token_qkv + 2 * kQkWidth + value_head * kHeadDim + row0;
  float value[kRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) value[i] = bf16_bits_to_f32(__ldg(value_row + i));
  const int control = token * kValueHeads + value_head;
  const float decay = ex2_approx(__ldg(p.log_decay + control) * kLog2e);
  const float beta = __ldg(p.beta + control);

  // L2 normalisation of q and k over the head (device/gdn_recurrence.rs:79-105); each warp for itself.
  const float q_norm = rsqrt_approx(warp_sum(dot4(q, q)) + kRmsEpsilon);
  const float k_norm = rsqrt_approx(warp_sum(dot4(k, k)) + kRmsEpsilon);
  q.x *= q_norm; q.y *= q_norm; q.z *= q_norm; q.w *= q_norm;
  k.x *= k_norm; k.y *= k_norm; k.z *= k_norm; k.w *= k_norm;

  float state_key[kRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) state_key[i] = dot4(old_state[i], k);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) state_key[i] += __shfl_xor_sync(0xffffffffu, state_key[i], o);
  }
  float rec[kRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    const float update = beta * (value[i] - decay * state_key[i]);
    float4 s;
    s.x = fmaf(old_state[i].x, decay, k.x * update);
    s.y = fmaf(old_state[i].y, decay, k.y * update);
    s.z = fmaf(old_state[i].z, decay, k.z * update);
    s.w = fmaf(old_state[i].w, decay, k.w * update);
    // Four-CTA clusters (batches up to 4) keep the new rows and store them behind the push below;
    // with two-CTA clusters the registers that takes cost the sixth resident CTA per SM, and the
    // 768 CTAs of batch 8 would no longer run as one wave.
    if constexpr (kRecSplit == 4) old_state[i] = s;
    else *reinterpret_cast<float4*>(state + i * kHeadDim + lane * 4) = s;
    rec[i] = dot4(s, q);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) rec[i] += __shfl_xor_sync(0xffffffffu, rec[i], o);
  }
  float square = 0.0f;
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    rec[i] *= kDeltaScale;
    square = fmaf(rec[i], rec[i], square);
  }
  if (lane < kRowsPerWarp) {
    float mine = rec[0];
#pragma unroll
    for (int i = 1; i < kRowsPerWarp; ++i) mine = lane == i ? rec[i] : mine;
    recurrent[warp * kRowsPerWarp + lane] = mine;
  }
  // Lane r pushes this warp's sum of squares into CTA r of the cluster.  Four-CTA clusters store
  // the new state rows between the two halves of the barrier: its release half would otherwise
  // wait for those global stores before it lets the peers see the sums (batch 1: 4.9 -> 4.6 us).
  cluster_wait();
  if (lane < kRecSplit)
    st_dsmem_f32(mapa_u32(smem_u32(&squares[rank * kRecWarps + warp]), lane), square);
  cluster_arrive();
  if constexpr (kRecSplit == 4) {
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i)
      *reinterpret_cast<float4*>(state + i * kHeadDim + lane * 4) = old_state[i];
  }
  cluster_wait();

  if (tid < kRowsPerCta) {
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < kRecSplit * kRecWarps; ++i) total += squares[i];
    const float inverse_rms = rsqrt_approx(total / static_cast<float>(kHeadDim) + kRmsEpsilon);
    const int row = static_cast<int>(rank) * kRowsPerCta + tid;
    const float normalized = recurrent[tid] * inverse_rms * bf16_bits_to_f32(__ldg(p.norm_weight + row));
    const float gate = bf16_bits_to_f32(__ldg(
        p.projected + static_cast<size_t>(token) * p.input_rows + p.qkv_rows + value_head * kHeadDim + row));
    const float silu = __fdiv_rn(gate, 1.0f + ex2_approx(-gate * kLog2e));
    p.output[static_cast<size_t>(token) * (kValueHeads * kHeadDim) + value_head * kHeadDim + row] =
        static_cast<uint16_t>(f32_to_bf16_bits(normalized * silu));
  }
}

}  // namespace

bool gdn_geometry_ok(int hidden, int control_rows, int qkv_rows, int input_rows) {
  return hidden > 0 && hidden % 8 == 0 && hidden <= kPrepThreads * kMaxChunksPerThread * 8 &&
         control_rows == kValueHeads && qkv_rows == 2 * kQkWidth + kValueHeads * kHeadDim &&
         input_rows == qkv_rows + kValueHeads * kHeadDim;
}

cudaError_t launch_gdn_prepare(cudaStream_t stream, const GdnPrepareParams& p) {
  const int conv_threads = p.batch * (p.qkv_rows / 8);
  const int grid = 2 * p.control_rows + (conv_threads + kPrepThreads - 1) / kPrepThreads;
  return launch_kernel(gdn_prepare_kernel, dim3(grid), dim3(kPrepThreads), 0, stream, p);
}

cudaError_t launch_gdn_recurrence(cudaStream_t stream, const GdnRecurrenceParams& p) {
  // The cluster shape is compiled into the kernel (__cluster_dims__).
  if (p.batch <= 4)
    return launch_kernel(gdn_recurrence_kernel<4>, dim3(p.batch * kValueHeads * 4), dim3(kRecThreads),
                         0, stream, p);
  return launch_kernel(gdn_recurrence_kernel<2>, dim3(p.batch * kValueHeads * 2), dim3(kRecThreads), 0,
                       stream, p);
}

}  // namespace tk100
