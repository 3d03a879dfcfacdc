// tk100_fp8_projection_static: the FP8 projection for hosts that must not allocate.
//
// tk100_create() calls cudaMalloc for the split-K scratch, so a host that is not allowed
// to allocate device memory cannot even build a context.  Two kinds of caller are in that
// position: an engine that hands its whole device budget to one arena at start-up and
// treats any later allocation as a failed "no allocation after warm-up" gate, and code
// that runs inside somebody else's process (a plugin, a callback) where the CUDA allocator
// belongs to the embedding application.  For them this one entry point needs no context:
// the split-K partial tiles, the tile tickets and a fault word live in a fixed array that
// is part of the library image.
//
// What that costs: every GPU that loads the library carries kStaticScratchBytes (8 MiB +
// 16 KiB) of device memory until the process exits, and problems whose scratch need is
// larger are refused rather than served more slowly.
#include <cudaTypedefs.h>

#include <cstdio>
#include <mutex>

#include "../../include/tuisko_sm100.h"
#include "kernels.h"
#include "ptx.cuh"

namespace tk100 {
namespace {

constexpr size_t kStaticPartialBytes = 8u << 20;  // split-K partial tiles
constexpr size_t kStaticCounters = 2048;          // tile tickets (uint32)
constexpr size_t kStaticTailBytes = 16u << 10;    // tickets + fault word + padding
constexpr size_t kStaticScratchBytes = kStaticPartialBytes + kStaticTailBytes;
static_assert(kStaticCounters * sizeof(unsigned int) + 256 <= kStaticTailBytes, "tail too small");

// The scratch itself.  In host code this name is only a stand-in for the symbol; the
// device address is looked up once per device with cudaGetSymbolAddress (below).
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
struct DeviceState {
  bool ready = false;
  unsigned char* scratch = nullptr;  // device address of g_static_scratch on this device
  int sm_count = 0;
  void* encode_fn = nullptr;
};
DeviceState g_devices[kMaxDevices];
std::mutex g_mutex;
// Destination of the failure text for the call in progress on this thread.
thread_local char* g_message = nullptr;
thread_local size_t g_message_capacity = 0;

tk100_status fail(tk100_status code, const char* fmt, long long a = 0, long long b = 0) {
  if (g_message && g_message_capacity > 0) std::snprintf(g_message, g_message_capacity, fmt, a, b);
  return code;
}

// Once per device, with that device current: resolve the scratch address, the SM count,
// the tensor-map encoder and the kernels' shared-memory attributes.  No allocation.
tk100_status setup_current_device(DeviceState** out) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) {
    return fail(TK100_ERR_DRIVER, "[gpu.driver] cudaGetDevice failed (%lld)", e);
  }
  if (device < 0 || device >= kMaxDevices) {
    return fail(TK100_ERR_CONTEXT, "[gpu.context] device ordinal %lld is not supported", device);
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& st = g_devices[device];
  if (!st.ready) {
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (e != cudaSuccess || major != 10) {
      return fail(TK100_ERR_MODULE,
                  "[gpu.module] device %lld is not compute capability 10.x (sm_100a only)", device);
    }
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      return fail(TK100_ERR_DRIVER, "[gpu.driver] cudaGetSymbolAddress(static scratch) failed (%lld)",
                  e);
    }
    e = cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) {
      return fail(TK100_ERR_DRIVER, "[gpu.driver] reading the SM count failed (%lld)", e);
    }
    cudaDriverEntryPointQueryResult q;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &st.encode_fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !st.encode_fn) {
      return fail(TK100_ERR_MODULE, "[gpu.module] cuTensorMapEncodeTiled is not available");
    }
    if ((e = fp8_projection_prepare()) != cudaSuccess) {
      return fail(TK100_ERR_MODULE, "[gpu.module] preparing the FP8 projection routes failed (%lld)",
                  e);
    }
    read_process_switches();
    st.scratch = static_cast<unsigned char*>(ptr);
    st.ready = true;
  }
  *out = &st;
  return TK100_OK;
}

tk100_status encode_map(const DeviceState& st, const void* base, uint64_t rows, uint64_t row_bytes,
                        uint32_t box_rows, CUtensorMap* map) {
  auto encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(st.encode_fn);
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {128u, box_rows};
  const cuuint32_t elem[2] = {1u, 1u};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                      box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return fail(TK100_ERR_DRIVER, "[gpu.driver] cuTensorMapEncodeTiled failed with CUresult %lld", r);
  }
  return TK100_OK;
}

bool misaligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; }

}  // namespace

}  // namespace tk100

extern "C" TK100_API tk100_status tk100_fp8_projection_static(
    tk100_stream stream, int rows, int out_rows, int columns, const uint8_t* activation_codes,
    const float* activation_scales, const uint8_t* weight_codes, const uint16_t* weight_scales,
    uint16_t* output, char* message, size_t message_capacity) {
  using namespace tk100;
  g_message = message;
  g_message_capacity = message_capacity;
  if (message && message_capacity > 0) message[0] = '\0';
  if (rows < 1 || rows > TK100_STATIC_MAX_ROWS) {
    return fail(TK100_ERR_LAUNCH,
                "[gpu.launch] static FP8 projection: row count %lld is outside 1..=%lld", rows,
                static_cast<long long>(TK100_STATIC_MAX_ROWS));
  }
  if (out_rows < 16 || out_rows % 16 != 0) {
    return fail(TK100_ERR_LAUNCH,
                "[gpu.launch] static FP8 projection: %lld output rows (need a multiple of 16)",
                out_rows);
  }
  if (columns < 128 || columns % 128 != 0) {
    return fail(TK100_ERR_LAUNCH,
                "[gpu.launch] static FP8 projection: %lld columns (need a multiple of 128)", columns);
  }
  if (!activation_codes || !activation_scales || !weight_codes || !weight_scales || !output) {
    return fail(TK100_ERR_LAUNCH, "[gpu.launch] static FP8 projection: a plane is null");
  }
  if (misaligned(activation_codes, 128) || misaligned(weight_codes, 128) ||
      misaligned(activation_scales, 4) || misaligned(weight_scales, 2) || misaligned(output, 2)) {
    return fail(TK100_ERR_LAUNCH, "[gpu.launch] static FP8 projection: a plane is misaligned");
  }
  DeviceState* st = nullptr;
  tk100_status s = setup_current_device(&st);
  if (s != TK100_OK) return s;

  // Same tiling rule as the context route: 128-row tiles, token tile by row count, K split
  // so that the tiles fill the SMs.
  const int block_tok = rows <= 16 ? 16 : rows <= 32 ? 32 : rows <= 64 ? 64 : 128;
  const long long tiles_n = (out_rows + 127) / 128;
  const long long tiles = tiles_n * ((rows + block_tok - 1) / block_tok);
  const long long slots =
      static_cast<long long>(st->sm_count) * (block_tok <= 32 ? 3 : block_tok <= 128 ? 2 : 1);
  int splits = static_cast<int>(slots / tiles);
  if (splits > 8) splits = 8;
  if (splits > columns / 128) splits = columns / 128;
  if (splits < 1) splits = 1;
  if (splits > 1) {
    const unsigned long long need =
        static_cast<unsigned long long>(splits) * tiles * block_tok * 128ull * sizeof(float);
    if (need > kStaticPartialBytes) {
      return fail(TK100_ERR_ARENA,
                  "[gpu.arena] static FP8 projection: needs %lld bytes of split-K scratch, the "
                  "static scratch holds %lld",
                  static_cast<long long>(need), static_cast<long long>(kStaticPartialBytes));
    }
    if (tiles > static_cast<long long>(kStaticCounters)) {
      return fail(TK100_ERR_ARENA,
                  "[gpu.arena] static FP8 projection: %lld output tiles, the static scratch has "
                  "%lld tickets",
                  tiles, static_cast<long long>(kStaticCounters));
    }
  }

  CUtensorMap map_w, map_a;
  if ((s = encode_map(*st, weight_codes, static_cast<uint64_t>(out_rows),
                      static_cast<uint64_t>(columns), 128, &map_w)) != TK100_OK) {
    return s;
  }
  if ((s = encode_map(*st, activation_codes, static_cast<uint64_t>(rows),
                      static_cast<uint64_t>(columns), static_cast<uint32_t>(block_tok), &map_a)) !=
      TK100_OK) {
    return s;
  }

  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  unsigned char* tail = st->scratch + kStaticPartialBytes;
  // The scratch keeps whatever the previous call left: the tickets must start at zero
  // (partials are fully rewritten before they are read).  The fault word behind the tickets is
  // NOT cleared here: it collects the faults of all calls until
  // tk100_fp8_projection_static_status reads and clears it.
  cudaError_t e = cudaMemsetAsync(tail, 0, kStaticCounters * sizeof(unsigned int), cs);
  if (e != cudaSuccess) {
    return fail(TK100_ERR_DRIVER, "[gpu.driver] clearing the static scratch failed (%lld)", e);
  }
  Fp8ProjParams p{};
  p.rows = rows;
  p.out_rows = out_rows;
  p.k = columns;
  p.splits = splits;
  p.act_scales = activation_scales;
  p.w_scales = weight_scales;
  p.out = output;
  p.partials = reinterpret_cast<float*>(st->scratch);
  p.counters = reinterpret_cast<unsigned int*>(tail);
  p.status = reinterpret_cast<uint32_t*>(tail + kStaticCounters * sizeof(unsigned int));
  e = launch_fp8_projection(cs, block_tok, map_w, map_a, p);
  if (e != cudaSuccess) {
    return fail(TK100_ERR_DRIVER, "[gpu.driver] launching the static FP8 projection failed (%lld)",
                e);
  }
  return TK100_OK;
}

extern "C" TK100_API tk100_status tk100_fp8_projection_static_status(tk100_stream stream,
                                                                     uint32_t* word) {
  using namespace tk100;
  g_message = nullptr;
  g_message_capacity = 0;
  if (!word) return TK100_ERR_LAUNCH;
  DeviceState* st = nullptr;
  tk100_status s = setup_current_device(&st);
  if (s != TK100_OK) return s;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  unsigned char* fault = st->scratch + kStaticPartialBytes + kStaticCounters * sizeof(unsigned int);
  cudaError_t e = cudaMemcpyAsync(word, fault, sizeof(uint32_t), cudaMemcpyDeviceToHost, cs);
  if (e == cudaSuccess) e = cudaMemsetAsync(fault, 0, sizeof(uint32_t), cs);
  if (e == cudaSuccess) e = cudaStreamSynchronize(cs);
  return e == cudaSuccess ? TK100_OK : TK100_ERR_DRIVER;
}
