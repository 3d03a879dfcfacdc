// Checkpoint planes -> run-time planes on the device, replacing the host loops of
// tuisko-model/src/materialize.rs: the fused QKV gather (:33-103, gather_source_planes :295-314)
// and the NVFP4 block-scale permutation into 128 x 4 tiles (swizzle_scale_planes :353-408,
// nvfp4_scale_offset :410-422).  Both are lossless byte movers: source planes are uploaded as the
// checkpoint stores them and rearranged in HBM, so the host never walks 11 MB of scale codes
// byte by byte.
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tk100 {
namespace {

constexpr int kGatherThreads = 256;

// Concatenation of up to kMaterializeMaxPlanes planes.  VEC: every plane is a whole number of
// 16-byte words at a 16-byte aligned address; otherwise bytes.
template <bool VEC>
__global__ void __launch_bounds__(kGatherThreads) gather_planes_kernel(GatherParams p) {
  using Word = typename std::conditional<VEC, uint4, uint8_t>::type;
  const size_t total = p.offset[p.planes] / sizeof(Word);
  const size_t stride = static_cast<size_t>(gridDim.x) * kGatherThreads;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kGatherThreads + threadIdx.x; i < total; i += stride) {
    const size_t byte = i * sizeof(Word);
    int plane = 0;
#pragma unroll
    for (int k = 1; k < kMaterializeMaxPlanes; ++k) plane += (k < p.planes && byte >= p.offset[k]) ? 1 : 0;
    const Word* source = reinterpret_cast<const Word*>(p.source[plane] + (byte - p.offset[plane]));
    reinterpret_cast<Word*>(p.output)[i] = *source;
  }
}

// One CTA permutes 128 rows x 64 groups (16 tiles of 512 bytes): rows are read as 64-byte runs
// (4 threads x 16 bytes per row), staged in shared memory, and every thread then writes one
// 16-byte piece of a tile -- the four quartile rows of one `row mod 32`, four groups each.
constexpr int kSwizzleThreads = 512;
constexpr int kSwizzleGroups = 64;

__global__ void __launch_bounds__(kSwizzleThreads) swizzle_scales_kernel(SwizzleParams p) {
  __shared__ __align__(16) uint8_t tile[128][kSwizzleGroups + 16];  // +16: rows land in different banks
  const int tid = threadIdx.x;
  const size_t row_tile = blockIdx.y;
  const size_t group0 = static_cast<size_t>(blockIdx.x) * kSwizzleGroups;
  const int groups_here = static_cast<int>(min(static_cast<size_t>(kSwizzleGroups), p.groups_per_row - group0));

  {
    const int r = tid >> 2, piece = tid & 3;  // 128 rows x 4 pieces of 16 groups
    const size_t row = row_tile * 128 + r;
    const size_t plane = row / p.rows_per_plane, source_row = row % p.rows_per_plane;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (piece * 16 < groups_here) {
      const uint8_t* src = p.source[plane] + source_row * p.groups_per_row + group0 + piece * 16;
      if (p.vector_loads && piece * 16 + 16 <= groups_here) {
        v = __ldg(reinterpret_cast<const uint4*>(src));
      } else {
        uint8_t* bytes = reinterpret_cast<uint8_t*>(&v);
        for (int j = 0; j < 16 && piece * 16 + j < groups_here; ++j) bytes[j] = src[j];
      }
      // validate_nvfp4_scales (tuisko-model/src/bindings.rs:1105-1120): no negative or NaN code.
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      bool bad = false;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const uint32_t code = (w[j] >> (8 * b)) & 0xffu;
          const bool live = piece * 16 + j * 4 + b < groups_here;
          bad |= live && ((code & 0x80u) != 0 || code == 0x7fu);
        }
      }
      if (bad) atomicOr(p.status, STATUS_BAD_ARGUMENT);
    }
    *reinterpret_cast<uint4*>(&tile[r][piece * 16]) = v;
  }
  __syncthreads();

  // 16 tiles x 32 pieces of 16 bytes.
  const int t = tid >> 5, row_mod32 = tid & 31;
  if (t * 4 < groups_here) {
    uint32_t w[4];
#pragma unroll
    for (int quartile = 0; quartile < 4; ++quartile)
      w[quartile] = *reinterpret_cast<const uint32_t*>(&tile[quartile * 32 + row_mod32][t * 4]);
    const size_t tiles_per_row = p.groups_per_row / 4;
    uint8_t* dst = p.output + (row_tile * tiles_per_row + group0 / 4 + t) * 512 + row_mod32 * 16;
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace

cudaError_t launch_gather_planes(cudaStream_t stream, const GatherParams& p, bool vector_words) {
  const size_t words = p.offset[p.planes] / (vector_words ? 16 : 1);
  if (words == 0) return cudaSuccess;
  const size_t want = (words + kGatherThreads - 1) / kGatherThreads;
  const unsigned grid = static_cast<unsigned>(want < 148 * 16 ? want : 148 * 16);
  return vector_words ? launch_kernel(gather_planes_kernel<true>, dim3(grid), dim3(kGatherThreads), 0, stream, p)
                      : launch_kernel(gather_planes_kernel<false>, dim3(grid), dim3(kGatherThreads), 0, stream, p);
}

cudaError_t launch_swizzle_scales(cudaStream_t stream, const SwizzleParams& p) {
  const size_t rows = p.rows_per_plane * p.planes;
  const dim3 grid(static_cast<unsigned>((p.groups_per_row + kSwizzleGroups - 1) / kSwizzleGroups),
                  static_cast<unsigned>(rows / 128));
  return launch_kernel(swizzle_scales_kernel, grid, dim3(kSwizzleThreads), 0, stream, p);
}

}  // namespace tk100
