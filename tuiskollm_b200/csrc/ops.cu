// Operator layer and the extern "C" boundary.
#include "ops.hpp"

#include <cudaTypedefs.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "ptx.cuh"

namespace tk100 {

namespace {

thread_local std::string g_create_error;

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

int env_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  return (v && v[0]) ? std::atoi(v) : fallback;
}

}  // namespace

Tuning Tuning::from_environment() {
  Tuning t;
  t.splits = env_int("TK100_SPLITS", t.splits);
  t.block_tok = env_int("TK100_BLOCK_TOK", t.block_tok);
  t.slots_per_sm = env_int("TK100_SLOTS_PER_SM", t.slots_per_sm);
  t.deep_ring = env_int("TK100_DEEP_RING", t.deep_ring);
  t.l2_prefetch = env_int("TK100_L2_PREFETCH", t.l2_prefetch);
  t.nvfp4_l2_prefetch = env_int("TK100_NVFP4_L2_PREFETCH", t.nvfp4_l2_prefetch);
  t.cluster = env_int("TK100_CLUSTER", t.cluster);
  t.fp8_pair = env_int("TK100_FP8_PAIR", t.fp8_pair);
  t.fp8_pair_min_rows = env_int("TK100_FP8_PAIR_MIN_ROWS", t.fp8_pair_min_rows);
  t.nvfp4_pair = env_int("TK100_PAIR", t.nvfp4_pair);
  t.nvfp4_pair_min_rows = env_int("TK100_PAIR_MIN_ROWS", t.nvfp4_pair_min_rows);
  t.swiglu_pairs = env_int("TK100_SWIGLU_PAIRS", t.swiglu_pairs);
  t.fp8_persist = env_int("TK100_FP8_PERSIST", t.fp8_persist);
  t.fp8_stream_k = env_int("TK100_FP8_STREAMK", t.fp8_stream_k);
  t.nvfp4_wide = env_int("TK100_NVFP4_WIDE", t.nvfp4_wide);
  t.nvfp4_wide_min_rows = env_int("TK100_NVFP4_WIDE_MIN_ROWS", t.nvfp4_wide_min_rows);
  t.nvfp4_persist = env_int("TK100_PERSIST", t.nvfp4_persist);
  t.nvfp4_persist_min_rows = env_int("TK100_PERSIST_MIN_ROWS", t.nvfp4_persist_min_rows);
  t.fused_exchange = env_int("TK100_FUSED_TAIL", t.fused_exchange);
  t.argmax_spread = env_int("TK100_ARGMAX_SPREAD", t.argmax_spread);
  t.fused_quant = env_int("TK100_FUSED_QUANT", t.fused_quant);
  return t;
}

// --------------------------------------------------------------------- Context

Status Context::check(cudaError_t e, const char* operation) {
  if (e == cudaSuccess) return TK100_OK;
  return fail(TK100_ERR_DRIVER,
              std::string("[gpu.driver] ") + operation + ": " + cudaGetErrorString(e));
}

Status Context::create(const tk100_config& in, Context** out, std::string* error) {
  tk100_config cfg = in;
  if (cfg.abi_version != TK100_ABI_VERSION) {
    *error = "[gpu.module] tk100_config.abi_version does not match this library";
    return TK100_ERR_MODULE;
  }
  if (cfg.hidden == 0) cfg.hidden = 5120;
  if (cfg.intermediate == 0) cfg.intermediate = 17408;
  if (cfg.rms_norm_epsilon == 0.0f) cfg.rms_norm_epsilon = 1.0e-6f;
  if (cfg.max_rows == 0) cfg.max_rows = 2048;
  if (cfg.workspace_bytes == 0) cfg.workspace_bytes = 64ull << 20;
  // tuisko-kernels-sm120/src/fp8/projection.rs require_fp8_geometry: the reduction
  // length must tile; here one TMA stage is 128 bytes of K.
  int threads = 0, chunks = 0;
  if (cfg.hidden % 128 != 0 || !norm_geometry(static_cast<int>(cfg.hidden), &threads, &chunks)) {
    *error = "[gpu.launch] hidden size " + std::to_string(cfg.hidden) +
             " is not admitted (multiple of 128, at most 32768)";
    return TK100_ERR_LAUNCH;
  }

  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count <= 0) {
    *error = std::string("[gpu.driver] no CUDA device: ") + cudaGetErrorString(e);
    return TK100_ERR_DRIVER;
  }
  if (cfg.device < 0 || cfg.device >= count) {
    *error = "[gpu.context] device ordinal " + std::to_string(cfg.device) + " out of range";
    return TK100_ERR_CONTEXT;
  }
  if ((e = cudaSetDevice(cfg.device)) != cudaSuccess) {
    *error = std::string("[gpu.driver] cudaSetDevice: ") + cudaGetErrorString(e);
    return TK100_ERR_DRIVER;
  }
  cudaDeviceProp prop{};
  if ((e = cudaGetDeviceProperties(&prop, cfg.device)) != cudaSuccess) {
    *error = std::string("[gpu.driver] cudaGetDeviceProperties: ") + cudaGetErrorString(e);
    return TK100_ERR_DRIVER;
  }
  if (prop.major != 10) {
    *error = "[gpu.module] device has compute capability " + std::to_string(prop.major) + "." +
             std::to_string(prop.minor) + ", expected 10.x (sm_100a kernels only)";
    return TK100_ERR_MODULE;
  }

  Context* ctx = new (std::nothrow) Context();
  if (!ctx) {
    *error = "[gpu.driver] out of host memory";
    return TK100_ERR_DRIVER;
  }
  ctx->config_ = cfg;
  ctx->sm_count_ = prop.multiProcessorCount;
  read_process_switches();
  ctx->tuning_ = Tuning::from_environment();

  cudaDriverEntryPointQueryResult q;
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ctx->encode_fn_, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !ctx->encode_fn_) {
    *error = "[gpu.module] cuTensorMapEncodeTiled is not available from this driver";
    delete ctx;
    return TK100_ERR_MODULE;
  }
  if ((e = fp8_projection_prepare()) != cudaSuccess) {
    *error = std::string("[gpu.module] preparing the FP8 projection routes: ") +
             cudaGetErrorString(e);
    delete ctx;
    return TK100_ERR_MODULE;
  }
  if ((e = fp8_swiglu_prepare()) != cudaSuccess) {
    *error = std::string("[gpu.module] preparing the FP8 SwiGLU routes: ") + cudaGetErrorString(e);
    delete ctx;
    return TK100_ERR_MODULE;
  }
  if ((e = fp8_pair_persist_prepare()) != cudaSuccess) {
    *error = std::string("[gpu.module] preparing the persistent FP8 pair kernel: ") + cudaGetErrorString(e);
    delete ctx;
    return TK100_ERR_MODULE;
  }
  if ((e = fp8_pair_prepare()) != cudaSuccess) {
    *error = std::string("[gpu.module] preparing the FP8 pair route: ") + cudaGetErrorString(e);
    delete ctx;
    return TK100_ERR_MODULE;
  }
  if ((e = nvfp4_pair_prepare()) != cudaSuccess) {
    *error = std::string("[gpu.module] preparing the NVFP4 pair routes: ") + cudaGetErrorString(e);
    delete ctx;
    return TK100_ERR_MODULE;
  }
  if ((e = nvfp4_persist_prepare(&ctx->persist_pairs_)) != cudaSuccess) {
    *error = std::string("[gpu.module] preparing the persistent NVFP4 routes: ") + cudaGetErrorString(e);
    delete ctx;
    return TK100_ERR_MODULE;
  }
  if ((e = nvfp4_prepare()) != cudaSuccess) {
    *error = std::string("[gpu.module] preparing the NVFP4 projection routes: ") +
             cudaGetErrorString(e);
    delete ctx;
    return TK100_ERR_MODULE;
  }

  ctx->partial_bytes_ = cfg.workspace_bytes;
  ctx->counter_count_ = 1 << 16;
  bool ok = cudaMalloc(&ctx->partials_, ctx->partial_bytes_) == cudaSuccess &&
            cudaMalloc(&ctx->counters_, ctx->counter_count_ * sizeof(unsigned int)) ==
                cudaSuccess &&
            cudaMalloc(&ctx->status_, sizeof(uint32_t)) == cudaSuccess &&
            cudaMalloc(&ctx->exchange_step_, 2 * sizeof(unsigned int)) == cudaSuccess &&
            cudaMemset(ctx->exchange_step_, 0, 2 * sizeof(unsigned int)) == cudaSuccess &&
            cudaMalloc(&ctx->argmax_spread_, kArgmaxSpreadBytes) == cudaSuccess &&
            cudaMemset(ctx->argmax_spread_, 0, kArgmaxSpreadBytes) == cudaSuccess &&
            cudaMalloc(&ctx->peer_sum_state_, 4 * sizeof(unsigned int)) == cudaSuccess &&
            cudaMemset(ctx->peer_sum_state_, 0, 4 * sizeof(unsigned int)) == cudaSuccess &&
            cudaMemset(ctx->counters_, 0, ctx->counter_count_ * sizeof(unsigned int)) ==
                cudaSuccess &&
            cudaMemset(ctx->status_, 0, sizeof(uint32_t)) == cudaSuccess &&
            cudaDeviceSynchronize() == cudaSuccess;
  if (!ok) {
    *error = std::string("[gpu.arena] allocating the context scratch: ") +
             cudaGetErrorString(cudaGetLastError());
    delete ctx;
    return TK100_ERR_ARENA;
  }
  *out = ctx;
  return TK100_OK;
}

Context::~Context() {
  if (partials_) cudaFree(partials_);
  if (counters_) cudaFree(counters_);
  if (status_) cudaFree(status_);
  if (exchange_step_) cudaFree(exchange_step_);
  if (argmax_spread_) cudaFree(argmax_spread_);
  if (peer_sum_state_) cudaFree(peer_sum_state_);
}

const char* Context::last_kernel() {
  char text[160];
  std::snprintf(text, sizeof text, "%s<%d,%d> splits=%d%s", route_.family, route_.a, route_.b,
                route_.splits, route_.cluster == 2 ? " cluster-leader" : route_.cluster ? " cluster" : "");
  route_text_ = text;
  return route_text_.c_str();
}

Status Context::encode_map(const MapKey& key, CUtensorMap* out) {
  auto encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(encode_fn_);
  const cuuint64_t dims[2] = {key.row_bytes, key.rows};
  const cuuint64_t strides[1] = {key.row_bytes};
  const cuuint32_t box[2] = {128u, key.box_rows};
  const cuuint32_t elem[2] = {1u, 1u};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(key.base), dims,
                      strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return fail(TK100_ERR_DRIVER, "[gpu.driver] cuTensorMapEncodeTiled failed with CUresult " +
                                      std::to_string(static_cast<int>(r)));
  }
  return TK100_OK;
}

Status Context::tensor_map(const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                           CUtensorMap* out) {
  const MapKey key{base, rows, row_bytes, box_rows, 0u};
  if (box_rows == 128u && !pinned_maps_.empty()) {
    auto pinned = pinned_maps_.find(key);
    if (pinned != pinned_maps_.end()) {
      *out = pinned->second;
      return TK100_OK;
    }
  }
  auto it = maps_.find(key);
  if (it != maps_.end()) {
    *out = it->second;
    return TK100_OK;
  }
  CUtensorMap map;
  Status s = encode_map(key, &map);
  if (s != TK100_OK) return s;
  if (maps_.size() > 4096) maps_.clear();
  maps_.emplace(key, map);
  *out = map;
  return TK100_OK;
}

Status Context::register_plane(const void* base, uint64_t rows, uint64_t row_bytes) {
  if (base == nullptr || !aligned(base, 128) || rows == 0 || row_bytes == 0 || row_bytes % 16 != 0) {
    return fail(TK100_ERR_LAUNCH,
                "[gpu.launch] register plane: a 128-byte aligned plane of rows x row_bytes "
                "(row_bytes a multiple of 16) is required");
  }
  const MapKey key{base, rows, row_bytes, 128u, 0u};
  CUtensorMap map;
  Status s = encode_map(key, &map);
  if (s != TK100_OK) return s;
  pinned_maps_[key] = map;
  return TK100_OK;
}

Status Context::scale_map(const void* base, uint64_t chunks, CUtensorMap* out) {
  const MapKey key{base, chunks, 512u, 4u, 1u};
  auto it = maps_.find(key);
  if (it != maps_.end()) {
    *out = it->second;
    return TK100_OK;
  }
  auto encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(encode_fn_);
  CUtensorMap map;
  const cuuint64_t dims[2] = {128, chunks};
  const cuuint64_t strides[1] = {512};
  const cuuint32_t box[2] = {128u, 4u};
  const cuuint32_t elem[2] = {1u, 1u};
  CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims,
                      strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return fail(TK100_ERR_DRIVER, "[gpu.driver] cuTensorMapEncodeTiled (scale plane) failed with "
                                  "CUresult " + std::to_string(static_cast<int>(r)));
  }
  if (maps_.size() > 4096) maps_.clear();
  maps_.emplace(key, map);
  *out = map;
  return TK100_OK;
}

// -------------------------------------------------------------- ResidualNormOp

namespace {

Status check_rows(Context& ctx, const char* what, int rows) {
  const int max_rows = static_cast<int>(ctx.config().max_rows);
  if (rows < 1 || rows > max_rows) {
    return ctx.fail(TK100_ERR_LAUNCH, std::string("[gpu.launch] ") + what + " row count " +
                                          std::to_string(rows) +
                                          " is outside the admitted routes 1..=" +
                                          std::to_string(max_rows));
  }
  return TK100_OK;
}

Status check_plane(Context& ctx, const char* what, const char* plane, const void* p,
                   size_t alignment) {
  if (p == nullptr) {
    return ctx.fail(TK100_ERR_LAUNCH,
                    std::string("[gpu.launch] ") + what + ": " + plane + " plane is null");
  }
  if (!aligned(p, alignment)) {
    return ctx.fail(TK100_ERR_LAUNCH, std::string("[gpu.launch] ") + what + ": " + plane +
                                          " plane is not " + std::to_string(alignment) +
                                          "-byte aligned");
  }
  return TK100_OK;
}

#define TK100_TRY(expr)                  \
  do {                                   \
    Status _s = (expr);                  \
    if (_s != TK100_OK) return _s;       \
  } while (0)

}  // namespace

// --------------------------------------------------------------- MaterializeOp

Status MaterializeOp::gather(cudaStream_t stream, int planes, const void* const* sources,
                             const uint64_t* bytes, void* output) {
  const char* what = "materialize gather";
  if (planes < 1 || planes > kMaterializeMaxPlanes || sources == nullptr || bytes == nullptr)
    return ctx_.fail(TK100_ERR_LAUNCH, std::string("[gpu.launch] ") + what + ": 1..=" +
                                           std::to_string(kMaterializeMaxPlanes) +
                                           " source planes are admitted");
  TK100_TRY(check_plane(ctx_, what, "output", output, 1));
  GatherParams p{};
  p.planes = planes;
  p.output = static_cast<uint8_t*>(output);
  bool vector_words = aligned(output, 16);
  size_t total = 0;
  for (int i = 0; i < planes; ++i) {
    if (bytes[i] != 0) TK100_TRY(check_plane(ctx_, what, "source", sources[i], 1));
    p.source[i] = static_cast<const uint8_t*>(sources[i]);
    p.offset[i] = total;
    if (total + bytes[i] < total)
      return ctx_.fail(TK100_ERR_LAUNCH, std::string("[gpu.launch] ") + what + ": length overflows");
    total += bytes[i];
    vector_words = vector_words && bytes[i] % 16 == 0 && aligned(sources[i], 16);
  }
  p.offset[planes] = total;
  if (total == 0) return TK100_OK;
  ctx_.count_launch();
  return ctx_.check(launch_gather_planes(stream, p, vector_words), "launching the plane gather");
}

Status MaterializeOp::swizzle_scales(cudaStream_t stream, int planes,
                                     const uint8_t* const* sources, uint64_t rows_per_plane,
                                     uint64_t groups_per_row, uint8_t* output) {
  const char* what = "NVFP4 scale layout";
  auto refuse = [&](const std::string& message) {
    return ctx_.fail(TK100_ERR_LAUNCH, "[checkpoint.source_binding] NVFP4 " + message);
  };
  if (planes < 1 || planes > 2 || sources == nullptr) return refuse("scale planes: 1 or 2 are admitted");
  const uint64_t rows = rows_per_plane * static_cast<uint64_t>(planes);
  // tuisko-model/src/materialize.rs:366-376
  if (rows == 0 || rows % 128 != 0)
    return refuse("scale rows " + std::to_string(rows) + " are not tiled by 128");
  if (groups_per_row == 0 || groups_per_row % 4 != 0)
    return refuse("scale groups " + std::to_string(groups_per_row) + " are not tiled by 4");
  TK100_TRY(check_plane(ctx_, what, "output", output, 16));
  SwizzleParams p{};
  p.planes = planes;
  p.rows_per_plane = rows_per_plane;
  p.groups_per_row = groups_per_row;
  p.vector_loads = groups_per_row % 16 == 0;
  for (int i = 0; i < planes; ++i) {
    TK100_TRY(check_plane(ctx_, what, "source", sources[i], 1));
    p.source[i] = sources[i];
    p.vector_loads = p.vector_loads && aligned(sources[i], 16);
  }
  p.output = output;
  p.status = ctx_.status_word();
  ctx_.count_launch();
  return ctx_.check(launch_swizzle_scales(stream, p), "launching the NVFP4 scale layout");
}

// ------------------------------------------------------------------- SamplerOp

Status SamplerOp::launch(cudaStream_t stream, int rows, int vocab, const uint16_t* logits,
                         const tk100_sampling_options* options, uint64_t* rng_state,
                         uint64_t* scratch, tk100_sample_decision* decisions, uint32_t* top_out) {
  const char* what = "sampler";
  auto refuse = [&](const std::string& message) {
    return ctx_.fail(TK100_ERR_LAUNCH, "[engine.sampling] " + message);
  };
  if (rows < 1 || rows > kSamplerMaxRows)
    return refuse("batch " + std::to_string(rows) + " is outside the admitted range 1..=" +
                  std::to_string(kSamplerMaxRows));
  if (vocab < kSamplerMaxTopK || vocab % 8 != 0)
    return refuse("sampling requires a BF16 logit row of a multiple of 8 values, at least " +
                  std::to_string(kSamplerMaxTopK) + ", got " + std::to_string(vocab));
  if (options == nullptr) return refuse("options are null");
  TK100_TRY(check_plane(ctx_, what, "logit", logits, 16));
  TK100_TRY(check_plane(ctx_, what, "generator state", rng_state, 8));
  TK100_TRY(check_plane(ctx_, what, "scratch", scratch, 8));
  TK100_TRY(check_plane(ctx_, what, "decision", decisions, 8));
  SamplerParams p{};
  p.rows = rows;
  p.vocab = vocab;
  p.logits = logits;
  for (int r = 0; r < rows; ++r) {
    const tk100_sampling_options& o = options[r];
    // tuisko-engine/src/sampling.rs:110-128 and :130-148
    if (!std::isfinite(o.temperature) || o.temperature < 0.0f)
      return refuse("temperature must be finite and non-negative");
    if (!std::isfinite(o.top_p) || o.top_p < 0.0f || o.top_p > 1.0f)
      return refuse("top_p must be finite and in 0..=1");
    if (o.top_k < 1 || o.top_k > static_cast<uint32_t>(vocab))
      return refuse("top_k must be in 1..=" + std::to_string(vocab));
    if (o.top_k > static_cast<uint32_t>(kSamplerMaxTopK))
      return refuse("top_k " + std::to_string(o.top_k) + " exceeds the device sampler's " +
                    std::to_string(kSamplerMaxTopK) + " candidates");
    if (o.stop_ids[0] == o.stop_ids[1])
      return refuse("generation stop-token identifiers must be distinct");
    for (uint32_t token : o.stop_ids)
      if (token >= static_cast<uint32_t>(vocab))
        return refuse("generation stop token " + std::to_string(token) + " is outside vocabulary 0.." +
                      std::to_string(vocab));
    p.temperature[r] = o.temperature;
    p.top_p[r] = o.top_p;
    p.top_k[r] = static_cast<int>(o.top_k);
    p.stop_ids[2 * r] = o.stop_ids[0];
    p.stop_ids[2 * r + 1] = o.stop_ids[1];
  }
  p.rng_state = rng_state;
  p.scratch = scratch;
  p.decisions = reinterpret_cast<uint32_t*>(decisions);
  p.top_out = top_out;
  p.status = ctx_.status_word();
  ctx_.count_launch();
  return ctx_.check(launch_sampler(stream, p), "launching the sampler");
}

// ------------------------------------------------------- GdnPrepareOp / GdnRecurrenceOp

namespace {
// Qwen3.8-27B gated-delta-net geometry (tuisko-model/src/lib.rs, Arch constants).
constexpr int kGdnControlRows = 48;
constexpr int kGdnQkvRows = 10240;
constexpr int kGdnInputRows = 16384;

Status check_gdn_batch(Context& ctx, const char* what, int batch) {
  if (batch < 1 || batch > kGdnMaxBatch) {
    return ctx.fail(TK100_ERR_LAUNCH, std::string("[gpu.launch] ") + what + " batch " +
                                          std::to_string(batch) +
                                          " is outside the admitted range 1..=" +
                                          std::to_string(kGdnMaxBatch));
  }
  if (!gdn_geometry_ok(static_cast<int>(ctx.config().hidden), kGdnControlRows, kGdnQkvRows,
                       kGdnInputRows)) {
    return ctx.fail(TK100_ERR_LAUNCH,
                    std::string("[gpu.launch] architecture geometry is incompatible with the ") +
                        what + " schedule");
  }
  return TK100_OK;
}
}  // namespace

Status GdnPrepareOp::launch(cudaStream_t stream, int batch, const uint16_t* input,
                            const uint16_t* control_weights, const uint16_t* a_log,
                            const uint16_t* dt_bias, const uint16_t* projected,
                            const uint16_t* convolution_weights, const uint32_t* state_rows,
                            uint16_t* history, float* log_decay, float* beta,
                            uint16_t* convolved) {
  const char* what = "GDN prepare";
  TK100_TRY(check_gdn_batch(ctx_, what, batch));
  TK100_TRY(check_plane(ctx_, what, "input", input, 16));
  TK100_TRY(check_plane(ctx_, what, "control weight", control_weights, 16));
  TK100_TRY(check_plane(ctx_, what, "a_log", a_log, 2));
  TK100_TRY(check_plane(ctx_, what, "dt_bias", dt_bias, 2));
  TK100_TRY(check_plane(ctx_, what, "projected", projected, 16));
  TK100_TRY(check_plane(ctx_, what, "convolution weight", convolution_weights, 16));
  TK100_TRY(check_plane(ctx_, what, "state row", state_rows, 4));
  TK100_TRY(check_plane(ctx_, what, "history", history, 16));
  TK100_TRY(check_plane(ctx_, what, "log_decay", log_decay, 4));
  TK100_TRY(check_plane(ctx_, what, "beta", beta, 4));
  TK100_TRY(check_plane(ctx_, what, "convolved", convolved, 16));
  GdnPrepareParams p{};
  p.batch = batch;
  p.hidden = static_cast<int>(ctx_.config().hidden);
  p.control_rows = kGdnControlRows;
  p.qkv_rows = kGdnQkvRows;
  p.input_rows = kGdnInputRows;
  p.input = input;
  p.control_weights = control_weights;
  p.a_log = a_log;
  p.dt_bias = dt_bias;
  p.projected = projected;
  p.convolution_weights = convolution_weights;
  p.state_rows = state_rows;
  p.history = history;
  p.log_decay = log_decay;
  p.beta = beta;
  p.convolved = convolved;
  ctx_.count_launch();
  return ctx_.check(launch_gdn_prepare(stream, p), "launching GDN prepare");
}

Status GdnRecurrenceOp::launch(cudaStream_t stream, int batch, const uint16_t* qkv,
                               const uint16_t* projected, const float* log_decay,
                               const float* beta, const uint16_t* norm_weight,
                               const uint32_t* state_rows, float* state, uint16_t* output) {
  const char* what = "GDN recurrence";
  TK100_TRY(check_gdn_batch(ctx_, what, batch));
  TK100_TRY(check_plane(ctx_, what, "qkv", qkv, 16));
  TK100_TRY(check_plane(ctx_, what, "projected", projected, 16));
  TK100_TRY(check_plane(ctx_, what, "log_decay", log_decay, 4));
  TK100_TRY(check_plane(ctx_, what, "beta", beta, 4));
  TK100_TRY(check_plane(ctx_, what, "norm weight", norm_weight, 2));
  TK100_TRY(check_plane(ctx_, what, "state row", state_rows, 4));
  TK100_TRY(check_plane(ctx_, what, "state", state, 16));
  TK100_TRY(check_plane(ctx_, what, "output", output, 16));
  GdnRecurrenceParams p{};
  p.batch = batch;
  p.qkv_rows = kGdnQkvRows;
  p.input_rows = kGdnInputRows;
  p.qkv = qkv;
  p.projected = projected;
  p.log_decay = log_decay;
  p.beta = beta;
  p.norm_weight = norm_weight;
  p.state_rows = state_rows;
  p.state = state;
  p.output = output;
  ctx_.count_launch();
  return ctx_.check(launch_gdn_recurrence(stream, p), "launching GDN recurrence");
}

Status ResidualNormOp::launch_plain(cudaStream_t stream, int batch, const uint16_t* input,
                                    const uint16_t* weight, uint16_t* output) {
  TK100_TRY(check_rows(ctx_, "residual norm", batch));
  TK100_TRY(check_plane(ctx_, "residual norm", "input", input, 16));
  TK100_TRY(check_plane(ctx_, "residual norm", "weight", weight, 16));
  TK100_TRY(check_plane(ctx_, "residual norm", "output", output, 16));
  ctx_.count_launch();
  return ctx_.check(
      launch_resnorm_quant(stream, batch, static_cast<int>(ctx_.config().hidden), input, nullptr,
                           weight, nullptr, output, nullptr, nullptr,
                           ctx_.config().rms_norm_epsilon, ctx_.status_word()),
      "launching RMSNorm");
}

Status ResidualNormOp::launch_residual(cudaStream_t stream, int batch,
                                       const uint16_t* residual_input, const uint16_t* branch,
                                       const uint16_t* weight, uint16_t* residual_output,
                                       uint16_t* normalized_output) {
  TK100_TRY(check_plane(ctx_, "residual norm", "branch", branch, 16));
  return launch_quantize(stream, batch, residual_input, branch, weight, residual_output,
                         normalized_output, nullptr, nullptr);
}

Status ResidualNormOp::launch_quantize(cudaStream_t stream, int batch,
                                       const uint16_t* residual_input, const uint16_t* branch,
                                       const uint16_t* weight, uint16_t* residual_output,
                                       uint16_t* normalized_output, uint8_t* activation_codes,
                                       float* activation_scales, float nvfp4_divisor,
                                       uint8_t* nvfp4_codes, uint8_t* nvfp4_scales) {
  TK100_TRY(check_rows(ctx_, "residual norm", batch));
  if (nvfp4_codes || nvfp4_scales) {
    if (ctx_.config().hidden % 64 != 0) {
      return ctx_.fail(TK100_ERR_LAUNCH,
                       "[gpu.launch] residual norm: NVFP4 output needs hidden % 64 == 0");
    }
    if (!std::isfinite(nvfp4_divisor) || nvfp4_divisor <= 0.0f) {
      return ctx_.fail(TK100_ERR_LAUNCH,
                       "[gpu.launch] NVFP4 input scale divisor must be finite and positive");
    }
    TK100_TRY(check_plane(ctx_, "residual norm", "NVFP4 activation codes", nvfp4_codes, 128));
    TK100_TRY(check_plane(ctx_, "residual norm", "NVFP4 activation scales", nvfp4_scales, 128));
  }
  TK100_TRY(check_plane(ctx_, "residual norm", "residual input", residual_input, 16));
  TK100_TRY(check_plane(ctx_, "residual norm", "weight", weight, 16));
  TK100_TRY(check_plane(ctx_, "residual norm", "normalized output", normalized_output, 16));
  if (branch) {
    TK100_TRY(check_plane(ctx_, "residual norm", "branch", branch, 16));
    TK100_TRY(check_plane(ctx_, "residual norm", "residual output", residual_output, 16));
  }
  if (activation_codes || activation_scales) {
    TK100_TRY(check_plane(ctx_, "residual norm", "activation codes", activation_codes, 128));
    TK100_TRY(check_plane(ctx_, "residual norm", "activation scales", activation_scales, 4));
  }
  ctx_.count_launch();
  return ctx_.check(
      launch_resnorm_quant(stream, batch, static_cast<int>(ctx_.config().hidden), residual_input,
                           branch, weight, branch ? residual_output : nullptr, normalized_output,
                           activation_codes, activation_scales, ctx_.config().rms_norm_epsilon,
                           ctx_.status_word(), nvfp4_codes, nvfp4_scales, nvfp4_divisor),
      "launching residual RMSNorm");
}

// ------------------------------------------------------------- Fp8ProjectionOp

Status Fp8ProjectionOp::quantize(cudaStream_t stream, int rows, int columns,
                                 const uint16_t* input, uint8_t* activation_codes,
                                 float* activation_scales) {
  TK100_TRY(check_rows(ctx_, name_, rows));
  int threads = 0, chunks = 0;
  if (!norm_geometry(columns, &threads, &chunks)) {
    return ctx_.fail(TK100_ERR_LAUNCH, std::string("[gpu.launch] ") + name_ + ": " +
                                           std::to_string(columns) +
                                           " columns are not admitted (multiple of 8, <= 32768)");
  }
  TK100_TRY(check_plane(ctx_, name_, "input", input, 16));
  TK100_TRY(check_plane(ctx_, name_, "activation codes", activation_codes, 16));
  TK100_TRY(check_plane(ctx_, name_, "activation scales", activation_scales, 4));
  ctx_.count_launch();
  return ctx_.check(launch_resnorm_quant(stream, rows, columns, input, nullptr, nullptr, nullptr,
                                         nullptr, activation_codes, activation_scales, 0.0f,
                                         ctx_.status_word()),
                    "launching the E4M3 activation quantiser");
}

Status Fp8ProjectionOp::launch(cudaStream_t stream, int rows, int out_rows, int columns,
                               const uint16_t* input, uint8_t* activation_codes,
                               float* activation_scales, const uint8_t* weight_codes,
                               const uint16_t* weight_scales, uint16_t* output, float* logits_f32,
                               unsigned long long* argmax_scratch, tk100_argmax_pair* pairs,
                               int vocab_offset, const ArgmaxTail* tail) {
  TK100_TRY(check_rows(ctx_, name_, rows));
  if (out_rows < 16 || out_rows % 16 != 0) {
    return ctx_.fail(TK100_ERR_LAUNCH, std::string("[gpu.launch] ") + name_ + ": " +
                                           std::to_string(out_rows) +
                                           " output rows are not admitted (multiple of 16)");
  }
  if (columns < 128 || columns % 128 != 0) {
    return ctx_.fail(TK100_ERR_LAUNCH, std::string("[gpu.launch] ") + name_ + ": " +
                                           std::to_string(columns) +
                                           " columns are not admitted (multiple of 128)");
  }
  TK100_TRY(check_plane(ctx_, name_, "activation codes", activation_codes, 128));
  TK100_TRY(check_plane(ctx_, name_, "activation scales", activation_scales, 4));
  TK100_TRY(check_plane(ctx_, name_, "weight codes", weight_codes, 128));
  TK100_TRY(check_plane(ctx_, name_, "weight scales", weight_scales, 2));
  if (output == nullptr && logits_f32 == nullptr && argmax_scratch == nullptr) {
    return ctx_.fail(TK100_ERR_LAUNCH,
                     std::string("[gpu.launch] ") + name_ + ": every output plane is null");
  }
  if (output) TK100_TRY(check_plane(ctx_, name_, "output", output, 2));
  if (pairs && argmax_scratch == nullptr) {
    return ctx_.fail(TK100_ERR_LAUNCH,
                     std::string("[gpu.launch] ") + name_ + ": argmax scratch plane is null");
  }
  if (argmax_scratch) TK100_TRY(check_plane(ctx_, name_, "argmax scratch", argmax_scratch, 8));
  ExchangePeers peers{};
  const int world = tail ? tail->world : 1;
  if (tail) {
    if (world < 1 || world > kMaxExchangeRanks || tail->rank < 0 || tail->rank >= world || !pairs ||
        rows > 4096 || (world > 1 && !tail->peer_buffers)) {
      return ctx_.fail(TK100_ERR_LAUNCH, std::string("[gpu.launch] ") + name_ +
                                             ": bad exchange argument (1 <= world <= 8, 0 <= rank < "
                                             "world, non-null pair and peer planes)");
    }
    for (int i = 0; i < world && world > 1; ++i) {
      if (tail->peer_buffers[i] == 0 || (tail->peer_buffers[i] & 7) != 0) {
        return ctx_.fail(TK100_ERR_LAUNCH, std::string("[gpu.launch] ") + name_ +
                                               ": peer buffer is null or misaligned");
      }
      peers.base[i] = reinterpret_cast<unsigned char*>(static_cast<uintptr_t>(tail->peer_buffers[i]));
    }
  }

  // Opt-in (TK100_FUSED_QUANT=1: launches of one wave, 2: every size): decode launches of at most
  // kFusedQuantRows rows quantise inside the projection kernel (every CTA derives the per-token
  // scale from the BF16 rows and makes its own code tiles; the codes and scales still reach the
  // caller's planes, bit for bit what the quantiser kernel writes).  Measured slower than the
  // quantiser launch in front, whose latency programmatic launch hides under the projection's
  // weight prefetch: LM-head shard of 31 040 rows 30.8 -> 32.4 us per step, 248 320 rows
  // 185.6 -> 188.2 us (the chain row load -> amax -> scale -> code tile delays the first UMMA of
  // every CTA).
  const long long fq_tiles = (out_rows + 127) / 128;
  const bool fuse_quant = input != nullptr && rows <= kFusedQuantRows && ctx_.tuning().fused_quant != 0 &&
                          (ctx_.forced_block_tok() == 0 || ctx_.forced_block_tok() == 16) &&
                          (fq_tiles <= 3LL * ctx_.sm_count() || ctx_.tuning().fused_quant == 2);
  if (input && fuse_quant) TK100_TRY(check_plane(ctx_, name_, "input", input, 16));
  if (input && !fuse_quant) {
    TK100_TRY(quantize(stream, rows, columns, input, activation_codes, activation_scales));
  }

  // Prefill shapes with a plain BF16 output: CTA pairs (256-row x 256-token pair tiles) halve
  // the operand bytes per MAC, which is what bounds the one-CTA kernel there.
  {
    const Tuning& tune = ctx_.tuning();
    const int min_rows = tune.fp8_pair_min_rows;
    // a launch of fewer than 32 pair CTAs (a small tensor-parallel shard of the plane) leaves
    // most SMs idle: the one-CTA kernel splits K instead (TK100_FP8_PAIR=2 takes the pair route
    // anyway).  Shards of 32-48 pair CTAs were measured faster on pairs than split.
    const long long pair_ctas = 2LL * ((rows + 255) / 256) * (out_rows / 256);
    // A long reduction on few pair tiles (the dense-FP8 down projection at 256 tokens: 40 CTAs
    // walking K = 17408) leaves most SMs idle as well; the one-CTA kernel splits K over clusters
    // there (measured 44.6 against 57.0 us).
    const bool long_k_few_tiles = pair_ctas < ctx_.sm_count() / 2 && columns >= 16384;
    // Stream-K on resident pairs (TK100_FP8_STREAMK=1, an experiment switch: measured slower than
    // the routes below at every benchmarked shape): every pair streams the same share of the
    // launch's tiles x K steps.
    const long long pair_tile_count = pair_ctas / 2;
    const int k_steps = columns / 128;
    bool stream_k = false;
    int stream_pairs = 0;
    if (tune.fp8_stream_k != 0 && ctx_.persist_pairs() > 0) {
      const long long steps = pair_tile_count * k_steps;
      stream_pairs = static_cast<int>(steps < ctx_.persist_pairs() ? steps : ctx_.persist_pairs());
      const bool fits = stream_pairs > 0 &&
                        fp8_pair_stream_k_scratch_bytes(stream_pairs) <= ctx_.partial_bytes() &&
                        static_cast<size_t>(2 * pair_tile_count) <= ctx_.counter_count();
      stream_k = fits;
    }
    if (tune.fp8_pair != 0 && rows >= min_rows && out_rows % 256 == 0 &&
        ((pair_ctas >= 32 && !long_k_few_tiles) || tune.fp8_pair == 2 || stream_k) && output &&
        !logits_f32 && !argmax_scratch && ctx_.forced_block_tok() == 0 && ctx_.forced_splits() == 0) {
      CUtensorMap map_w, map_a;
      TK100_TRY(ctx_.tensor_map(weight_codes, static_cast<uint64_t>(out_rows),
                                static_cast<uint64_t>(columns), 128, &map_w));
      TK100_TRY(ctx_.tensor_map(activation_codes, static_cast<uint64_t>(rows),
                                static_cast<uint64_t>(columns), 128, &map_a));
      Fp8ProjParams q{};
      q.rows = rows;
      q.out_rows = out_rows;
      q.k = columns;
      q.splits = 1;
      // at most one CTA per SM: the longer ring
      q.deep_ring = 2LL * ((rows + 255) / 256) * (out_rows / 256) <= ctx_.sm_count() ? 1 : 0;
      if (tune.deep_ring >= 0) q.deep_ring = tune.deep_ring != 0;
      q.act_scales = activation_scales;
      q.w_scales = weight_scales;
      q.out = output;
      q.status = ctx_.status_word();
      q.debug = debug_flags();
      q.stamps = debug_stamps();
      ctx_.count_launch();
      if (stream_k) {
        q.partials = ctx_.partials();
        q.counters = ctx_.counters();
        ctx_.note_route("fp8_pair_stream_k_kernel", 6, stream_pairs, 1, 1);
        return ctx_.check(launch_fp8_pair_persist(stream, stream_pairs, map_w, map_a, q, true),
                          "launching the stream-K FP8 pair projection");
      }
      // More pair tiles than pairs that fit the device at once: the resident pairs walk the tiles
      // with two accumulators in rotation (TK100_FP8_PERSIST).
      const long long pair_tiles = pair_ctas / 2;
      if (tune.fp8_persist != 0 && ctx_.persist_pairs() > 0 &&
          (pair_tiles > ctx_.persist_pairs() || tune.fp8_persist == 2)) {
        const int pairs = static_cast<int>(pair_tiles < ctx_.persist_pairs() ? pair_tiles : ctx_.persist_pairs());
        ctx_.note_route("fp8_pair_persist_kernel", 6, pairs, 1, 1);
        return ctx_.check(launch_fp8_pair_persist(stream, pairs, map_w, map_a, q, false),
                          "launching the persistent FP8 pair projection");
      }
      ctx_.note_route("fp8_pair_kernel", q.deep_ring ? 6 : 3, 0, 1, 1);
      return ctx_.check(launch_fp8_pair(stream, map_w, map_a, q), "launching the FP8 pair projection");
    }
  }

  // token tile: the smallest that holds all rows, 128-token tiles beyond that (two CTAs of
  // 128 tokens share an SM; a 256-token tile would leave one CTA per SM and no overlap)
  int block_tok = rows <= 16 ? 16 : rows <= 32 ? 32 : rows <= 64 ? 64 : 128;
  if (ctx_.forced_block_tok() == 16 || ctx_.forced_block_tok() == 32 ||
      ctx_.forced_block_tok() == 64 || ctx_.forced_block_tok() == 128 ||
      ctx_.forced_block_tok() == 256) {
    block_tok = ctx_.forced_block_tok();
  }
  const int tiles_n = (out_rows + 127) / 128;
  const int tiles_m = (rows + block_tok - 1) / block_tok;
  const long long tiles = static_cast<long long>(tiles_n) * tiles_m;
  const int kb_total = columns / 128;
  // Fill the SMs (two CTAs fit per SM up to 64-token tiles) by splitting K when the
  // plane has few 128-row tiles.
  // CTAs per SM by shared memory and registers: three up to 32-token tiles, two up to 128
  long long slots =
      static_cast<long long>(ctx_.sm_count()) * (block_tok <= 32 ? 3 : block_tok <= 128 ? 2 : 1);
  if (ctx_.tuning().slots_per_sm > 0) {
    slots = static_cast<long long>(ctx_.sm_count()) * ctx_.tuning().slots_per_sm;
  }
  int splits = static_cast<int>(slots / tiles);
  if (ctx_.forced_splits() > 0) splits = ctx_.forced_splits();
  if (splits > 8) splits = 8;
  if (splits > kb_total) splits = kb_total;
  if (splits < 1) splits = 1;
  while (splits > 1 &&
         (static_cast<size_t>(splits) * tiles * block_tok * 128 * sizeof(float) >
              ctx_.partial_bytes() ||
          static_cast<size_t>(tiles) > ctx_.counter_count())) {
    --splits;
  }

  CUtensorMap map_w, map_a;
  TK100_TRY(ctx_.tensor_map(weight_codes, static_cast<uint64_t>(out_rows),
                            static_cast<uint64_t>(columns), 128, &map_w));
  TK100_TRY(ctx_.tensor_map(activation_codes, static_cast<uint64_t>(rows),
                            static_cast<uint64_t>(columns), static_cast<uint32_t>(block_tok),
                            &map_a));

  Fp8ProjParams p{};
  p.rows = rows;
  p.out_rows = out_rows;
  p.k = columns;
  p.splits = splits;
  p.cluster = ctx_.tuning().cluster != 0 ? 1 : 0;
  if (p.cluster && splits > 1 && ctx_.tuning().cluster == 2) {
    // TK100_CLUSTER=2: split-K on a leader CTA when the peers' partial tiles fit its ring
    // ((splits - 1) tiles of [tokens][128 rows] fp32).  Measured against the symmetric reduction:
    // no gain at one token (QKV 10.0 -> 10.3 us: the "ring is free" handshake costs the hop that
    // the second cluster barrier used to), a loss at 32 (GDN-in 16.3 -> 21.5 us: one CTA finishes
    // every token), so it stays an experiment switch.
    const size_t ring = static_cast<size_t>(fp8_projection_stages(block_tok)) * (128 * 128 + block_tok * 128);
    const size_t land = static_cast<size_t>(splits - 1) * (rows < block_tok ? rows : block_tok) * 128 * sizeof(float);
    if (land <= ring) p.cluster = 2;
  }
  {
    const bool dr = ctx_.tuning().deep_ring >= 0;
    // unsplit launches with at most two CTAs per SM (an LM-head shard on 8 GPUs): measured
    // 26 us instead of 32 us for a 31 040-row shard; split launches are faster with three
    p.deep_ring = dr ? ctx_.tuning().deep_ring : (splits == 1 && tiles <= 2LL * ctx_.sm_count());
    // between three and four CTAs per SM worth of tiles: the 3-stage ring, four CTAs per SM, one
    // wave (a 4-way LM-head shard: 485 tiles on 148 SMs)
    if (!dr && splits == 1 && block_tok == 16 && tiles > 3LL * ctx_.sm_count() &&
        tiles <= 4LL * ctx_.sm_count()) {
      p.deep_ring = 2;
    }
  }
  {
    // Queueing the CTA's weight slice at L2 before the ring starts looked good only while the
    // rotating weight copies of the measurement still hit L2; on cold weights it costs
    // (N = 12288, M = 1: 12.7 -> 14.0 us), so it stays an experiment switch.
    p.l2_prefetch = ctx_.tuning().l2_prefetch;
  }
  p.act_scales = activation_scales;
  p.w_scales = weight_scales;
  p.out = output;
  p.logits_f32 = logits_f32;
  p.argmax_keys = argmax_scratch;  // pairs == null: the keys stay packed for tk100_argmax_exchange
  p.vocab_offset = vocab_offset;
  p.partials = ctx_.partials();
  p.counters = ctx_.counters();
  p.status = ctx_.status_word();
  p.debug = debug_flags();
  p.stamps = debug_stamps();
  if (fuse_quant) {
    p.x_bf16 = input;
    p.codes_out = activation_codes;
    p.scales_out = activation_scales;
  }
  // The last CTA of the launch unpacks the maxima (or exchanges them with the peers and merges):
  // no finalize / exchange launch behind the projection.
  const bool fuse_tail = pairs != nullptr && ctx_.tuning().fused_exchange != 0;
  if (fuse_tail) {
    p.tail_ticket = ctx_.tail_ticket();
    p.pairs_out = reinterpret_cast<ArgmaxPair*>(pairs);
    p.world = world;
    p.rank = tail ? tail->rank : 0;
    p.step_counter = ctx_.exchange_step();
    p.peers = peers;
    if (rows <= kArgmaxSpreadRows && ctx_.tuning().argmax_spread != 0) {
      p.spread_keys = ctx_.argmax_spread_keys();
      p.spread_tickets = ctx_.argmax_spread_tickets();
    }
  }
  ctx_.count_launch();
  {
    // the ring variant launch_fp8_projection picks for this tile size
    const int ring = (block_tok <= 32 && p.deep_ring == 1) ? 1 : (block_tok <= 16 && p.deep_ring == 2) ? 2 : 0;
    ctx_.note_route("fp8_projection_kernel", block_tok, ring, splits, splits > 1 ? p.cluster : 0);
  }
  TK100_TRY(ctx_.check(launch_fp8_projection(stream, block_tok, map_w, map_a, p),
                       "launching the FP8 projection"));
  if (pairs && !fuse_tail) {
    ctx_.count_launch();
    if (world > 1) {
      TK100_TRY(ctx_.check(launch_argmax_exchange(stream, rows, world, tail->rank, argmax_scratch, peers,
                                                  ctx_.exchange_step(),
                                                  reinterpret_cast<ArgmaxPair*>(pairs), ctx_.status_word()),
                           "launching the argmax exchange"));
    } else {
      TK100_TRY(ctx_.check(launch_argmax_finalize(stream, rows, argmax_scratch,
                                                  reinterpret_cast<ArgmaxPair*>(pairs)),
                           "launching the argmax finalizer"));
    }
  }
  return TK100_OK;
}

// ----------------------------------------------------------------- Fp8SwiGluOp

Status Fp8SwiGluOp::launch(cudaStream_t stream, int rows, const uint16_t* input,
                           uint8_t* activation_codes, float* activation_scales,
                           const uint8_t* weight_codes, const uint16_t* weight_scales,
                           uint16_t* output) {
  const char* name = "FP8 SwiGLU";
  TK100_TRY(check_rows(ctx_, name, rows));
  const int hidden = static_cast<int>(ctx_.config().hidden);
  const int inter = static_cast<int>(ctx_.config().intermediate);
  if (inter < 128 || inter % 128 != 0) {
    return ctx_.fail(TK100_ERR_LAUNCH, std::string("[gpu.launch] ") + name + ": intermediate size " +
                                           std::to_string(inter) + " is not admitted (multiple of 128)");
  }
  TK100_TRY(check_plane(ctx_, name, "activation codes", activation_codes, 128));
  TK100_TRY(check_plane(ctx_, name, "activation scales", activation_scales, 4));
  TK100_TRY(check_plane(ctx_, name, "weight codes", weight_codes, 128));
  TK100_TRY(check_plane(ctx_, name, "weight scales", weight_scales, 2));
  TK100_TRY(check_plane(ctx_, name, "output", output, 2));
  if (input) {
    TK100_TRY(Fp8ProjectionOp(ctx_, name).quantize(stream, rows, hidden, input, activation_codes,
                                                   activation_scales));
  }
  const int block_tok = rows <= 32 ? 32 : 128;
  CUtensorMap map_w, map_a;
  TK100_TRY(ctx_.tensor_map(weight_codes, static_cast<uint64_t>(2) * inter, static_cast<uint64_t>(hidden),
                            128, &map_w));
  TK100_TRY(ctx_.tensor_map(activation_codes, static_cast<uint64_t>(rows), static_cast<uint64_t>(hidden),
                            static_cast<uint32_t>(block_tok), &map_a));
  Fp8SwigluParams p{};
  p.rows = rows;
  p.intermediate = inter;
  p.k = hidden;
  p.act_scales = activation_scales;
  p.w_scales = weight_scales;
  p.out = output;
  p.status = ctx_.status_word();
  ctx_.count_launch();
  ctx_.note_route("fp8_swiglu_kernel", block_tok, block_tok == 128 && rows > 128 ? 1 : 0, 1, 0);
  return ctx_.check(launch_fp8_swiglu(stream, block_tok, map_w, map_a, p), "launching the FP8 SwiGLU");
}

// ------------------------------------------------------------------ Nvfp4MlpOp

Status Nvfp4MlpOp::quantize(cudaStream_t stream, int rows, int columns, const uint16_t* input,
                            float input_global_divisor, uint8_t* activation_codes,
                            uint8_t* activation_scales) {
  TK100_TRY(check_rows(ctx_, "NVFP4 activation quantiser", rows));
  if (columns < 64 || columns % 64 != 0) {
    return ctx_.fail(TK100_ERR_LAUNCH, "[gpu.launch] NVFP4 activation quantiser: " +
                                           std::to_string(columns) +
                                           " columns are not admitted (multiple of 64)");
  }
  if (!std::isfinite(input_global_divisor) || input_global_divisor <= 0.0f) {
    return ctx_.fail(TK100_ERR_LAUNCH,
                     "[gpu.launch] NVFP4 input scale divisor must be finite and positive");
  }
  TK100_TRY(check_plane(ctx_, "NVFP4 activation quantiser", "input", input, 32));
  TK100_TRY(check_plane(ctx_, "NVFP4 activation quantiser", "activation codes", activation_codes,
                        128));
  TK100_TRY(check_plane(ctx_, "NVFP4 activation quantiser", "activation scales",
                        activation_scales, 128));
  ctx_.count_launch();
  return ctx_.check(launch_nvfp4_quantize(stream, rows, columns, input, input_global_divisor,
                                          activation_codes, activation_scales),
                    "launching the NVFP4 activation quantiser");
}

Status Nvfp4MlpOp::launch(cudaStream_t stream, bool gate_up, int rows, int out_rows, int columns,
                          const uint16_t* input, uint8_t* activation_codes,
                          uint8_t* activation_scales, float input_global_divisor,
                          const uint8_t* weight_codes, const uint8_t* weight_scales,
                          float weight_scale_divisor, uint16_t* output, float* output_f32,
                          const Nvfp4NextQuant* next) {
  const char* name = gate_up ? "NVFP4 SwiGLU" : "NVFP4 down";
  TK100_TRY(check_rows(ctx_, name, rows));
  // tuisko-kernels-sm89/src/nvfp4/swiglu.rs:535-539
  if (!std::isfinite(weight_scale_divisor) || weight_scale_divisor <= 0.0f) {
    return ctx_.fail(TK100_ERR_LAUNCH,
                     "[gpu.launch] NVFP4 weight scale divisor must be finite and positive");
  }
  if (!std::isfinite(input_global_divisor) || input_global_divisor <= 0.0f) {
    return ctx_.fail(TK100_ERR_LAUNCH,
                     "[gpu.launch] NVFP4 input scale divisor must be finite and positive");
  }
  // the scale tiles cover 128 rows x 4 groups (tuisko-model/src/materialize.rs:366-376)
  if (out_rows < 128 || out_rows % 128 != 0) {
    return ctx_.fail(TK100_ERR_LAUNCH, std::string("[gpu.launch] ") + name + ": " +
                                           std::to_string(out_rows) +
                                           " output rows are not admitted (multiple of 128)");
  }
  // whole groups of four 16-column scale blocks (tuisko-model/src/materialize.rs:366-376)
  if (columns < 64 || columns % 64 != 0) {
    return ctx_.fail(TK100_ERR_LAUNCH, std::string("[gpu.launch] ") + name + ": " +
                                           std::to_string(columns) +
                                           " columns are not admitted (multiple of 64)");
  }
  TK100_TRY(check_plane(ctx_, name, "activation codes", activation_codes, 128));
  TK100_TRY(check_plane(ctx_, name, "activation scales", activation_scales, 128));
  TK100_TRY(check_plane(ctx_, name, "weight codes", weight_codes, 128));
  TK100_TRY(check_plane(ctx_, name, "weight scales", weight_scales, 128));
  if (output_f32) {
    if (gate_up) {
      return ctx_.fail(TK100_ERR_LAUNCH, "[gpu.launch] NVFP4 SwiGLU has no fp32 output");
    }
    TK100_TRY(check_plane(ctx_, name, "fp32 output", output_f32, 16));
  } else {
    TK100_TRY(check_plane(ctx_, name, "output", output, 2));
  }
  if (next) {
    if (!gate_up) {
      return ctx_.fail(TK100_ERR_LAUNCH, "[gpu.launch] only NVFP4 SwiGLU quantises its output");
    }
    if (!std::isfinite(next->divisor) || next->divisor <= 0.0f) {
      return ctx_.fail(TK100_ERR_LAUNCH,
                       "[gpu.launch] NVFP4 input scale divisor must be finite and positive");
    }
    TK100_TRY(check_plane(ctx_, name, "output codes", next->codes, 16));
    TK100_TRY(check_plane(ctx_, name, "output scales", next->scales, 16));
  }
  if (input) {
    TK100_TRY(quantize(stream, rows, columns, input, input_global_divisor, activation_codes,
                       activation_scales));
  }
  // Launches that do not quantise in their epilogue run the quantiser on the BF16 output.
  auto quantise_after = [&]() -> Status {
    if (!next) return TK100_OK;
    return quantize(stream, rows, out_rows, output, next->divisor, next->codes, next->scales);
  };

  // Prefill shapes: CTA pairs (256-row x 256-token pair tiles) halve the operand bytes per MAC.
  {
    const int pe = ctx_.tuning().nvfp4_pair;
    const int min_rows = ctx_.tuning().nvfp4_pair_min_rows;
    // Off unless TK100_PAIR=1 (down) or 2 (gate_up too): with two CTAs per SM the 128 x 128
    // tiles of the plain kernel overlap one CTA's epilogue with the other's loop and lose less
    // to the last wave (down at M = 2048: 149 us, CTA pairs 191 us).
    const bool allowed = pe == 1 || pe == 2;
    const bool this_op = gate_up ? pe == 2 : (out_rows % 256 == 0);
    if (allowed && this_op && rows >= min_rows) {
      const uint64_t w_rows = static_cast<uint64_t>(out_rows) * (gate_up ? 2 : 1);
      const uint64_t chunks_per_tile = static_cast<uint64_t>(columns / 64);
      CUtensorMap map_w, map_a, map_wsf, map_asf;
      TK100_TRY(ctx_.tensor_map(weight_codes, w_rows, static_cast<uint64_t>(columns / 2), 128, &map_w));
      TK100_TRY(ctx_.tensor_map(activation_codes, static_cast<uint64_t>(rows),
                                static_cast<uint64_t>(columns / 2), 128, &map_a));
      TK100_TRY(ctx_.scale_map(weight_scales, (w_rows / 128) * chunks_per_tile, &map_wsf));
      TK100_TRY(ctx_.scale_map(activation_scales,
                               static_cast<uint64_t>((rows + 127) / 128) * chunks_per_tile, &map_asf));
      Nvfp4Params q{};
      q.rows = rows;
      q.out_rows = out_rows;
      q.k = columns;
      q.splits = 1;
      q.up_row_offset = gate_up ? out_rows : 0;
      q.out_scale = 1.0f / (weight_scale_divisor * input_global_divisor);
      q.out = output;
      q.out_f32 = output_f32;
      q.status = ctx_.status_word();
      q.debug = debug_flags();
      q.stamps = debug_stamps();
      ctx_.count_launch();
      ctx_.note_route("nvfp4_pair_kernel", gate_up ? 1 : 0, 0, 1, 1);
      TK100_TRY(ctx_.check(launch_nvfp4_pair(stream, gate_up, map_w, map_a, map_wsf, map_asf, q),
                           "launching the NVFP4 pair projection"));
      return quantise_after();
    }
  }
  // Prefill shapes: persistent CTA pairs on 256-row x 256-token pair tiles (halves the operand
  // bytes per MAC through the SM's L2 port and the scale copies per MAC; the epilogue of one tile
  // runs under the next tile's MMAs).
  if (ctx_.tuning().nvfp4_persist != 0 && rows >= ctx_.tuning().nvfp4_persist_min_rows &&
      ctx_.persist_pairs() > 0 && (gate_up || out_rows % 256 == 0)) {
    const uint64_t w_rows = static_cast<uint64_t>(out_rows) * (gate_up ? 2 : 1);
    const uint64_t chunks_per_tile = static_cast<uint64_t>(columns / 64);
    CUtensorMap map_w, map_a, map_wsf, map_asf;
    TK100_TRY(ctx_.tensor_map(weight_codes, w_rows, static_cast<uint64_t>(columns / 2), 128, &map_w));
    TK100_TRY(ctx_.tensor_map(activation_codes, static_cast<uint64_t>(rows),
                              static_cast<uint64_t>(columns / 2), 128, &map_a));
    TK100_TRY(ctx_.scale_map(weight_scales, (w_rows / 128) * chunks_per_tile, &map_wsf));
    TK100_TRY(ctx_.scale_map(activation_scales,
                             static_cast<uint64_t>((rows + 127) / 128) * chunks_per_tile, &map_asf));
    Nvfp4Params q{};
    q.rows = rows;
    q.out_rows = out_rows;
    q.k = columns;
    q.splits = 1;
    q.up_row_offset = gate_up ? out_rows : 0;
    q.out_scale = 1.0f / (weight_scale_divisor * input_global_divisor);
    q.out = output;
    q.out_f32 = output_f32;
    q.status = ctx_.status_word();
    q.debug = debug_flags();
    q.stamps = debug_stamps();
    const long long tiles = static_cast<long long>((rows + 255) / 256) * (gate_up ? out_rows / 128 : out_rows / 256);
    const int pairs = static_cast<int>(tiles < ctx_.persist_pairs() ? tiles : ctx_.persist_pairs());
    ctx_.count_launch();
    ctx_.note_route("nvfp4_persist_kernel", gate_up ? 1 : 0, pairs, 1, 1);
    TK100_TRY(ctx_.check(launch_nvfp4_persist(stream, gate_up, pairs, map_w, map_a, map_wsf, map_asf, q),
                         "launching the persistent NVFP4 projection"));
    return quantise_after();
  }
  // 256-token tiles (one CTA per SM, a third fewer operand bytes and issue slots per MAC) for
  // prefill shapes: the plain projection unsplit, and the gate/up pairs.
  const bool pairs_wanted = gate_up && ctx_.tuning().swiglu_pairs != 0;
  const bool wide = rows >= ctx_.tuning().nvfp4_wide_min_rows &&
                    ((!gate_up && ctx_.tuning().nvfp4_wide >= 1) ||
                     (pairs_wanted && ctx_.tuning().nvfp4_wide >= 2));
  const int block_tok = rows <= 32 ? 32 : wide ? 256 : 128;
  const int tiles_n = out_rows / 128;
  const int tiles_m = (rows + block_tok - 1) / block_tok;
  const long long tiles = static_cast<long long>(tiles_n) * tiles_m;
  const int kb_total = (columns + 255) / 256;
  int splits = 1;
  if (!gate_up && !wide) {
    // two CTAs share an SM at <= 32 tokens
    // Clusters cannot straddle GPCs, so a launch that fills every slot spills into a second
    // wave: aim at ~80 % of the slots (measured on 5120 x 17408, M = 8: 6 splits 13.0 us, 7 splits
    // 20.6 us, 8 splits 19.3 us).
    const long long slots = static_cast<long long>(ctx_.sm_count()) * 2;
    splits = static_cast<int>(slots * 82 / 100 / tiles);
    if (ctx_.forced_splits() > 0) splits = ctx_.forced_splits();
    if (splits > 8) splits = 8;
    if (splits > kb_total) splits = kb_total;
    if (splits < 1) splits = 1;
    // Only the reduction through global scratch (TK100_CLUSTER=0) needs room for the partial
    // tiles and a ticket per tile; clusters reduce in shared memory.
    while (ctx_.tuning().cluster == 0 && splits > 1 &&
           (static_cast<size_t>(splits) * tiles * block_tok * 128 * sizeof(float) >
                ctx_.partial_bytes() ||
            static_cast<size_t>(tiles) > ctx_.counter_count())) {
      --splits;
    }
  }
  const uint64_t weight_rows = static_cast<uint64_t>(out_rows) * (gate_up ? 2 : 1);
  CUtensorMap map_w, map_a;
  TK100_TRY(ctx_.tensor_map(weight_codes, weight_rows, static_cast<uint64_t>(columns / 2), 128,
                            &map_w));
  TK100_TRY(ctx_.tensor_map(activation_codes, static_cast<uint64_t>(rows),
                            static_cast<uint64_t>(columns / 2), static_cast<uint32_t>(block_tok),
                            &map_a));
  Nvfp4Params p{};
  p.rows = rows;
  p.out_rows = out_rows;
  p.k = columns;
  p.splits = splits;
  p.cluster = ctx_.tuning().cluster != 0 ? 1 : 0;
  p.up_row_offset = gate_up ? out_rows : 0;
  // Queueing the slice at L2 first does not pay (measured at M = 1: gate/up 20.7 -> 22.0 us,
  // down 13.4 -> 14.9 us), so only TK100_NVFP4_L2_PREFETCH=n turns it on.
  p.l2_prefetch = ctx_.tuning().nvfp4_l2_prefetch;
  p.w_scales = weight_scales;
  p.a_scales = activation_scales;
  // the reference passes 1/divisor to its kernel (nvfp4/swiglu.rs:541); both divisors here
  p.out_scale = 1.0f / (weight_scale_divisor * input_global_divisor);
  p.out = output;
  p.out_f32 = output_f32;
  p.partials = ctx_.partials();
  p.counters = ctx_.counters();
  p.status = ctx_.status_word();
  p.debug = debug_flags();
  p.stamps = debug_stamps();
  // gate/up runs as clusters of two plain tiles (gate CTA, up CTA; two CTAs per SM) that swap
  // half of their accumulators over distributed shared memory, each finishing half of the
  // tokens.  Measured against the fused kernel (one CTA holds both tiles, one CTA per SM):
  // M = 1 24.4 -> 20.7 us, M = 256 51.6 -> 45.2 us, M = 2048 368 -> 318 us.  TK100_SWIGLU_PAIRS=0
  // selects the fused kernel.
  bool as_pairs = false;
  if (gate_up) as_pairs = ctx_.tuning().swiglu_pairs != 0;
  if (as_pairs) {
    p.pair_swiglu = 1;
    p.splits = 1;
  }
  if (p.cluster && ctx_.tuning().cluster != 1) {
    // Pushed exchange (one-way stores and barrier arrivals, no second cluster barrier) for the
    // gate/up pairs at 128-token tiles (M = 2048: 320.6 -> 313.0 us; at decode sizes it measured
    // the same or slightly slower, 21.9 -> 22.0 us).  TK100_CLUSTER=2 pushes everywhere it fits,
    // split K included (down, M = 1: 14.05 -> 14.6 us, so off by default).
    const size_t land = static_cast<size_t>(p.splits - 1) * (rows < block_tok ? rows : block_tok) * 128 * sizeof(float);
    const bool everywhere = ctx_.tuning().cluster == 2;
    if ((as_pairs && (block_tok >= 128 || everywhere)) ||
        (everywhere && p.splits > 1 && land <= nvfp4_ring_bytes(block_tok))) {
      p.cluster = 2;
    }
  }
  // Decode shapes quantise in the epilogue of the CTA that finishes the tokens (saves a launch:
  // M = 1 23.2 -> 22.1 us); from 128-token tiles on that epilogue work is not hidden and the
  // quantiser kernel after the projection is faster (M = 2048: 351 against 419 us).
  const bool in_epilogue = next && as_pairs && block_tok == 32;
  if (in_epilogue) {
    p.q_codes = next->codes;
    p.q_scales = next->scales;
    p.q_divisor = next->divisor;
  }
  ctx_.count_launch();
  ctx_.note_route("nvfp4_gemm_kernel", block_tok, gate_up && !as_pairs ? 1 : 0, p.splits,
                  (as_pairs || p.splits > 1) ? p.cluster : 0);
  TK100_TRY(ctx_.check(launch_nvfp4_gemm(stream, block_tok, gate_up && !as_pairs, map_w, map_a, p),
                       "launching the NVFP4 projection"));
  return in_epilogue ? TK100_OK : quantise_after();
}

}  // namespace tk100

// ------------------------------------------------------------------- C boundary

using tk100::Context;

struct tk100_ctx {
  Context* impl;
};

extern "C" {

tk100_status tk100_create(const tk100_config* config, tk100_ctx** out) {
  if (!config || !out) {
    tk100::g_create_error = "[gpu.launch] tk100_create: null argument";
    return TK100_ERR_LAUNCH;
  }
  Context* impl = nullptr;
  std::string error;
  tk100_status s = Context::create(*config, &impl, &error);
  if (s != TK100_OK) {
    tk100::g_create_error = error;
    return s;
  }
  *out = new tk100_ctx{impl};
  return TK100_OK;
}

void tk100_destroy(tk100_ctx* ctx) {
  if (!ctx) return;
  delete ctx->impl;
  delete ctx;
}

const char* tk100_last_error(const tk100_ctx* ctx) {
  return ctx ? ctx->impl->last_error().c_str() : tk100::g_create_error.c_str();
}

tk100_status tk100_device_status(tk100_ctx* ctx, tk100_stream stream, uint32_t* word) {
  if (!ctx || !word) return TK100_ERR_LAUNCH;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(word, ctx->impl->status_word(), sizeof(uint32_t),
                                  cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaMemsetAsync(ctx->impl->status_word(), 0, sizeof(uint32_t), s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e == cudaSuccess && (*word & tk100::STATUS_WAIT_TIMEOUT)) {
    // CTAs that gave up may have left split-K tickets, the LM head's tail ticket or its spread
    // maxima behind: re-arm them (the exchange's step number keeps counting).
    e = cudaMemsetAsync(ctx->impl->counters(), 0,
                        ctx->impl->counter_count() * sizeof(unsigned int), s);
    if (e == cudaSuccess) e = cudaMemsetAsync(ctx->impl->tail_ticket(), 0, sizeof(unsigned int), s);
    if (e == cudaSuccess) {
      e = cudaMemsetAsync(ctx->impl->argmax_spread_keys(), 0, tk100::kArgmaxSpreadBytes, s);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  }
  return ctx->impl->check(e, "reading the device status word");
}

uint64_t tk100_launch_count(const tk100_ctx* ctx) { return ctx ? ctx->impl->launches() : 0; }

const char* tk100_last_kernel(tk100_ctx* ctx) { return ctx ? ctx->impl->last_kernel() : ""; }

tk100_status tk100_rms_norm(tk100_ctx* ctx, tk100_stream stream, int rows, const uint16_t* input,
                            const uint16_t* weight, uint16_t* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::ResidualNormOp(*ctx->impl)
      .launch_plain(static_cast<cudaStream_t>(stream), rows, input, weight, output);
}

tk100_status tk100_residual_rms_norm(tk100_ctx* ctx, tk100_stream stream, int rows,
                                     const uint16_t* residual_input, const uint16_t* branch,
                                     const uint16_t* weight, uint16_t* residual_output,
                                     uint16_t* normalized_output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::ResidualNormOp(*ctx->impl)
      .launch_residual(static_cast<cudaStream_t>(stream), rows, residual_input, branch, weight,
                       residual_output, normalized_output);
}

tk100_status tk100_residual_rms_norm_quantize(tk100_ctx* ctx, tk100_stream stream, int rows,
                                              const uint16_t* residual_input,
                                              const uint16_t* branch, const uint16_t* weight,
                                              uint16_t* residual_output,
                                              uint16_t* normalized_output,
                                              uint8_t* activation_codes,
                                              float* activation_scales) {
  if (!ctx) return TK100_ERR_CONTEXT;
  if (!activation_codes || !activation_scales) {
    return ctx->impl->fail(TK100_ERR_LAUNCH,
                           "[gpu.launch] residual norm: activation code/scale plane is null");
  }
  return tk100::ResidualNormOp(*ctx->impl)
      .launch_quantize(static_cast<cudaStream_t>(stream), rows, residual_input, branch, weight,
                       residual_output, normalized_output, activation_codes, activation_scales);
}

tk100_status tk100_residual_rms_norm_quantize_nvfp4(
    tk100_ctx* ctx, tk100_stream stream, int rows, const uint16_t* residual_input,
    const uint16_t* branch, const uint16_t* weight, uint16_t* residual_output,
    uint16_t* normalized_output, uint8_t* activation_codes, float* activation_scales,
    float input_global_divisor, uint8_t* nvfp4_codes, uint8_t* nvfp4_scales) {
  if (!ctx) return TK100_ERR_CONTEXT;
  if (!nvfp4_codes || !nvfp4_scales) {
    return ctx->impl->fail(TK100_ERR_LAUNCH,
                           "[gpu.launch] residual norm: NVFP4 code/scale plane is null");
  }
  return tk100::ResidualNormOp(*ctx->impl)
      .launch_quantize(static_cast<cudaStream_t>(stream), rows, residual_input, branch, weight,
                       residual_output, normalized_output, activation_codes, activation_scales,
                       input_global_divisor, nvfp4_codes, nvfp4_scales);
}

tk100_status tk100_quantize_activation_e4m3(tk100_ctx* ctx, tk100_stream stream, int rows,
                                            int columns, const uint16_t* input,
                                            uint8_t* activation_codes, float* activation_scales) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::Fp8ProjectionOp(*ctx->impl, "FP8 activation quantiser")
      .quantize(static_cast<cudaStream_t>(stream), rows, columns, input, activation_codes,
                activation_scales);
}

tk100_status tk100_fp8_qkv(tk100_ctx* ctx, tk100_stream stream, int rows, int out_rows,
                           const uint16_t* input, uint8_t* activation_codes,
                           float* activation_scales, const uint8_t* weight_codes,
                           const uint16_t* weight_scales, uint16_t* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::FullAttentionQkvOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), rows, out_rows,
              static_cast<int>(ctx->impl->config().hidden), input, activation_codes,
              activation_scales, weight_codes, weight_scales, output);
}

tk100_status tk100_fp8_gdn_input(tk100_ctx* ctx, tk100_stream stream, int rows, int out_rows,
                                 const uint16_t* input, uint8_t* activation_codes,
                                 float* activation_scales, const uint8_t* weight_codes,
                                 const uint16_t* weight_scales, uint16_t* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::GdnInputProjectionOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), rows, out_rows,
              static_cast<int>(ctx->impl->config().hidden), input, activation_codes,
              activation_scales, weight_codes, weight_scales, output);
}

tk100_status tk100_fp8_projection(tk100_ctx* ctx, tk100_stream stream, int rows, int out_rows,
                                  int columns, const uint16_t* input, uint8_t* activation_codes,
                                  float* activation_scales, const uint8_t* weight_codes,
                                  const uint16_t* weight_scales, uint16_t* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::Fp8ProjectionOp(*ctx->impl, "FP8 projection")
      .launch(static_cast<cudaStream_t>(stream), rows, out_rows, columns, input,
              activation_codes, activation_scales, weight_codes, weight_scales, output);
}

tk100_status tk100_fp8_swiglu(tk100_ctx* ctx, tk100_stream stream, int rows, const uint16_t* input,
                              uint8_t* activation_codes, float* activation_scales,
                              const uint8_t* weight_codes, const uint16_t* weight_scales,
                              uint16_t* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::Fp8SwiGluOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), rows, input, activation_codes, activation_scales,
              weight_codes, weight_scales, output);
}

tk100_status tk100_fp8_down(tk100_ctx* ctx, tk100_stream stream, int rows, const uint16_t* input,
                            uint8_t* activation_codes, float* activation_scales,
                            const uint8_t* weight_codes, const uint16_t* weight_scales,
                            uint16_t* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  const tk100_config& c = ctx->impl->config();
  return tk100::Fp8DownOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), rows, static_cast<int>(c.hidden),
              static_cast<int>(c.intermediate), input, activation_codes, activation_scales,
              weight_codes, weight_scales, output);
}

tk100_status tk100_fp8_gdn_output(tk100_ctx* ctx, tk100_stream stream, int rows, int columns,
                                  const uint16_t* input, uint8_t* activation_codes,
                                  float* activation_scales, const uint8_t* weight_codes,
                                  const uint16_t* weight_scales, uint16_t* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::GdnOutputProjectionOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), rows, static_cast<int>(ctx->impl->config().hidden),
              columns, input, activation_codes, activation_scales, weight_codes, weight_scales, output);
}

tk100_status tk100_register_plane(tk100_ctx* ctx, const void* weight_codes, uint64_t rows,
                                  uint64_t row_bytes) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return ctx->impl->register_plane(weight_codes, rows, row_bytes);
}

void tk100_tensor_map_counts(const tk100_ctx* ctx, uint64_t* registered, uint64_t* transient) {
  if (registered) *registered = ctx ? ctx->impl->pinned_map_count() : 0;
  if (transient) *transient = ctx ? ctx->impl->transient_map_count() : 0;
}

tk100_status tk100_materialize_gather(tk100_ctx* ctx, tk100_stream stream, int planes,
                                      const void* const* sources, const uint64_t* bytes,
                                      void* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::MaterializeOp(*ctx->impl)
      .gather(static_cast<cudaStream_t>(stream), planes, sources, bytes, output);
}

tk100_status tk100_materialize_nvfp4_scales(tk100_ctx* ctx, tk100_stream stream, int planes,
                                            const uint8_t* const* sources,
                                            uint64_t rows_per_plane, uint64_t groups_per_row,
                                            uint8_t* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::MaterializeOp(*ctx->impl)
      .swizzle_scales(static_cast<cudaStream_t>(stream), planes, sources, rows_per_plane,
                      groups_per_row, output);
}

tk100_status tk100_sample(tk100_ctx* ctx, tk100_stream stream, int rows, int vocab,
                          const uint16_t* logits, const tk100_sampling_options* options,
                          uint64_t* rng_state, uint64_t* scratch, tk100_sample_decision* decisions,
                          uint32_t* top_out) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::SamplerOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), rows, vocab, logits, options, rng_state, scratch,
              decisions, top_out);
}

uint64_t tk100_sampler_initial_state(uint64_t seed) {
  // tuisko-engine/src/sampling.rs:247-250
  const uint64_t scramble = 0x9e3779b97f4a7c15ull;
  const uint64_t state = seed ^ scramble;
  return state == 0 ? scramble : state;
}

size_t tk100_sampler_scratch_bytes(int rows, int vocab) {
  return tk100::sampler_scratch_bytes(rows, vocab);
}

tk100_status tk100_gdn_prepare(tk100_ctx* ctx, tk100_stream stream, int batch,
                               const uint16_t* input, const uint16_t* control_weights,
                               const uint16_t* a_log, const uint16_t* dt_bias,
                               const uint16_t* projected, const uint16_t* convolution_weights,
                               const uint32_t* state_rows, uint16_t* history, float* log_decay,
                               float* beta, uint16_t* convolved) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::GdnPrepareOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), batch, input, control_weights, a_log, dt_bias,
              projected, convolution_weights, state_rows, history, log_decay, beta, convolved);
}

tk100_status tk100_gdn_recurrence(tk100_ctx* ctx, tk100_stream stream, int batch,
                                  const uint16_t* qkv, const uint16_t* projected,
                                  const float* log_decay, const float* beta,
                                  const uint16_t* norm_weight, const uint32_t* state_rows,
                                  float* state, uint16_t* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::GdnRecurrenceOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), batch, qkv, projected, log_decay, beta,
              norm_weight, state_rows, state, output);
}

tk100_status tk100_fp8_lm_head(tk100_ctx* ctx, tk100_stream stream, int rows, int vocab_rows,
                               int vocab_offset, const uint16_t* input, uint8_t* activation_codes,
                               float* activation_scales, const uint8_t* weight_codes,
                               const uint16_t* weight_scales, uint16_t* output, float* logits_f32,
                               uint64_t* argmax_scratch, tk100_argmax_pair* pairs) {
  if (!ctx) return TK100_ERR_CONTEXT;
  if (vocab_offset < 0) {
    return ctx->impl->fail(TK100_ERR_LAUNCH, "[gpu.launch] FP8 LM head: negative vocab offset");
  }
  return tk100::LmHeadOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), rows, vocab_rows,
              static_cast<int>(ctx->impl->config().hidden), input, activation_codes,
              activation_scales, weight_codes, weight_scales, output, logits_f32,
              reinterpret_cast<unsigned long long*>(argmax_scratch), pairs, vocab_offset);
}

tk100_status tk100_fp8_lm_head_sharded(tk100_ctx* ctx, tk100_stream stream, int rows, int vocab_rows,
                                       int vocab_offset, const uint16_t* input,
                                       uint8_t* activation_codes, float* activation_scales,
                                       const uint8_t* weight_codes, const uint16_t* weight_scales,
                                       uint16_t* output, float* logits_f32, uint64_t* argmax_scratch,
                                       int world, int rank, const uint64_t* peer_buffers,
                                       tk100_argmax_pair* merged_pairs) {
  if (!ctx) return TK100_ERR_CONTEXT;
  if (vocab_offset < 0) {
    return ctx->impl->fail(TK100_ERR_LAUNCH, "[gpu.launch] FP8 LM head: negative vocab offset");
  }
  tk100::ArgmaxTail tail;
  tail.world = world;
  tail.rank = rank;
  tail.peer_buffers = peer_buffers;
  return tk100::LmHeadOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), rows, vocab_rows,
              static_cast<int>(ctx->impl->config().hidden), input, activation_codes,
              activation_scales, weight_codes, weight_scales, output, logits_f32,
              reinterpret_cast<unsigned long long*>(argmax_scratch), merged_pairs, vocab_offset, &tail);
}

tk100_status tk100_argmax_merge(tk100_ctx* ctx, tk100_stream stream, int rows, int shards,
                                const tk100_argmax_pair* gathered, tk100_argmax_pair* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  if (rows < 1 || shards < 1 || !gathered || !output) {
    return ctx->impl->fail(TK100_ERR_LAUNCH, "[gpu.launch] argmax merge: bad argument");
  }
  ctx->impl->count_launch();
  return ctx->impl->check(
      tk100::launch_argmax_merge(static_cast<cudaStream_t>(stream), rows, shards,
                                 reinterpret_cast<const tk100::ArgmaxPair*>(gathered),
                                 reinterpret_cast<tk100::ArgmaxPair*>(output)),
      "launching the argmax merge");
}

tk100_status tk100_argmax_exchange(tk100_ctx* ctx, tk100_stream stream, int rows, int world,
                                   int rank, uint64_t* argmax_scratch,
                                   const uint64_t* peer_buffers, tk100_argmax_pair* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  if (rows < 1 || rows > 4096 || world < 1 || world > tk100::kMaxExchangeRanks || rank < 0 ||
      rank >= world || !argmax_scratch || !peer_buffers || !output) {
    return ctx->impl->fail(TK100_ERR_LAUNCH,
                           "[gpu.launch] argmax exchange: bad argument (1 <= world <= 8, "
                           "0 <= rank < world, non-null planes)");
  }
  tk100::ExchangePeers peers{};
  for (int i = 0; i < world; ++i) {
    if (peer_buffers[i] == 0 || (peer_buffers[i] & 7) != 0) {
      return ctx->impl->fail(TK100_ERR_LAUNCH,
                             "[gpu.launch] argmax exchange: peer buffer is null or misaligned");
    }
    peers.base[i] = reinterpret_cast<unsigned char*>(static_cast<uintptr_t>(peer_buffers[i]));
  }
  ctx->impl->count_launch();
  return ctx->impl->check(
      tk100::launch_argmax_exchange(static_cast<cudaStream_t>(stream), rows, world, rank,
                                    reinterpret_cast<unsigned long long*>(argmax_scratch), peers,
                                    ctx->impl->exchange_step(),
                                    reinterpret_cast<tk100::ArgmaxPair*>(output),
                                    ctx->impl->status_word()),
      "launching the argmax exchange");
}

namespace {
struct PeerSumLayout {
  long long chunk;       // two-shot chunk for `capacity` values
  long long one_shot;    // one-shot slot size in values
  size_t one_shot_offset, result_offset, flag_offset, bytes;
};
// Layout of a peer-sum exchange buffer sized for `capacity` values on `world` ranks.
PeerSumLayout peer_sum_layout(long long capacity, int world) {
  auto up = [](size_t v, size_t a) { return (v + a - 1) / a * a; };
  PeerSumLayout l{};
  l.chunk = static_cast<long long>(up(static_cast<size_t>((capacity + world - 1) / world), 8));
  l.one_shot = capacity < tk100::kPeerSumOneShotElems ? capacity : tk100::kPeerSumOneShotElems;
  l.one_shot = static_cast<long long>(up(static_cast<size_t>(l.one_shot), 8));
  // two-shot slots first, one-shot slots behind them: disjoint, so a rank that has moved on to a
  // step of the other form cannot touch what a slower rank still reads
  const size_t slots_two = up(static_cast<size_t>(world) * l.chunk * sizeof(float), 256);
  const size_t slots_one = 2 * static_cast<size_t>(world) * l.one_shot * sizeof(float);
  l.one_shot_offset = slots_two;
  l.result_offset = up(slots_two + slots_one, 256);
  l.flag_offset = l.result_offset + up(2 * static_cast<size_t>(world) * l.chunk * sizeof(uint16_t), 256);
  l.bytes = l.flag_offset + 256;
  return l;
}
}  // namespace

size_t tk100_peer_sum_bytes(size_t capacity_values, int world) {
  if (world < 1 || world > tk100::kMaxExchangeRanks || capacity_values == 0) return 0;
  return peer_sum_layout(static_cast<long long>(capacity_values), world).bytes;
}

tk100_status tk100_peer_sum_bf16(tk100_ctx* ctx, tk100_stream stream, size_t values,
                                 size_t capacity_values, int world, int rank, const float* partial,
                                 const uint64_t* peer_buffers, uint16_t* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  if (values == 0 || values % 8 != 0 || values > capacity_values || world < 1 ||
      world > tk100::kMaxExchangeRanks || rank < 0 || rank >= world || !partial || !peer_buffers ||
      !output || (reinterpret_cast<uintptr_t>(partial) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(output) & 7) != 0) {
    return ctx->impl->fail(TK100_ERR_LAUNCH,
                           "[gpu.launch] peer sum: bad argument (values a multiple of 8 within the "
                           "capacity, 1 <= world <= 8, 0 <= rank < world, aligned non-null planes)");
  }
  tk100::ExchangePeers peers{};
  for (int i = 0; i < world; ++i) {
    if (peer_buffers[i] == 0 || (peer_buffers[i] & 255) != 0) {
      return ctx->impl->fail(TK100_ERR_LAUNCH,
                             "[gpu.launch] peer sum: peer buffer is null or not 256-byte aligned");
    }
    peers.base[i] = reinterpret_cast<unsigned char*>(static_cast<uintptr_t>(peer_buffers[i]));
  }
  const PeerSumLayout l = peer_sum_layout(static_cast<long long>(capacity_values), world);
  tk100::PeerSumParams q{};
  q.elems = static_cast<long long>(values);
  q.world = world;
  q.rank = rank;
  q.one_shot = q.elems <= tk100::kPeerSumOneShotElems ? 1 : 0;
  // the chunk follows this call's size (a smaller sum still spreads over all ranks); it never
  // exceeds the chunk the buffer was sized for
  q.chunk = ((q.elems + world - 1) / world + 7) / 8 * 8;
  q.partial = partial;
  q.output = output;
  q.chunk_capacity = l.chunk;
  q.one_shot_stride4 = l.one_shot / 4;
  q.one_shot_offset = l.one_shot_offset;
  q.result_offset = l.result_offset;
  q.flag_offset = l.flag_offset;
  q.step_counter = ctx->impl->peer_sum_state();
  q.tickets = ctx->impl->peer_sum_state() + 1;
  q.status = ctx->impl->status_word();
  // all CTAs of the launch must be resident together (they wait for peers, never for each other)
  const long long vec = q.elems / 4;
  long long ctas = (vec + 256 * 4 - 1) / (256 * 4);
  if (ctas > ctx->impl->sm_count()) ctas = ctx->impl->sm_count();
  if (ctas < 1) ctas = 1;
  ctx->impl->count_launch();
  return ctx->impl->check(
      tk100::launch_peer_sum(static_cast<cudaStream_t>(stream), static_cast<int>(ctas), q, peers),
      "launching the peer sum");
}

tk100_status tk100_nvfp4_quantize_activation(tk100_ctx* ctx, tk100_stream stream, int rows,
                                             int columns, const uint16_t* input,
                                             float input_global_divisor,
                                             uint8_t* activation_codes,
                                             uint8_t* activation_scales) {
  if (!ctx) return TK100_ERR_CONTEXT;
  return tk100::Nvfp4MlpOp(*ctx->impl)
      .quantize(static_cast<cudaStream_t>(stream), rows, columns, input, input_global_divisor,
                activation_codes, activation_scales);
}

tk100_status tk100_nvfp4_gate_up_swiglu(tk100_ctx* ctx, tk100_stream stream, int rows,
                                        const uint16_t* input, uint8_t* activation_codes,
                                        uint8_t* activation_scales, float input_global_divisor,
                                        const uint8_t* weight_codes, const uint8_t* weight_scales,
                                        float weight_scale_divisor, uint16_t* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  const tk100_config& c = ctx->impl->config();
  return tk100::Nvfp4MlpOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), true, rows, static_cast<int>(c.intermediate),
              static_cast<int>(c.hidden), input, activation_codes, activation_scales,
              input_global_divisor, weight_codes, weight_scales, weight_scale_divisor, output);
}

tk100_status tk100_nvfp4_gate_up_swiglu_quantize(
    tk100_ctx* ctx, tk100_stream stream, int rows, const uint16_t* input, uint8_t* activation_codes,
    uint8_t* activation_scales, float input_global_divisor, const uint8_t* weight_codes,
    const uint8_t* weight_scales, float weight_scale_divisor, uint16_t* output,
    float output_global_divisor, uint8_t* output_codes, uint8_t* output_scales) {
  if (!ctx) return TK100_ERR_CONTEXT;
  const tk100_config& c = ctx->impl->config();
  const tk100::Nvfp4NextQuant next{output_global_divisor, output_codes, output_scales};
  return tk100::Nvfp4MlpOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), true, rows, static_cast<int>(c.intermediate),
              static_cast<int>(c.hidden), input, activation_codes, activation_scales,
              input_global_divisor, weight_codes, weight_scales, weight_scale_divisor, output,
              nullptr, &next);
}

tk100_status tk100_nvfp4_down(tk100_ctx* ctx, tk100_stream stream, int rows,
                              const uint16_t* input, uint8_t* activation_codes,
                              uint8_t* activation_scales, float input_global_divisor,
                              const uint8_t* weight_codes, const uint8_t* weight_scales,
                              float weight_scale_divisor, uint16_t* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  const tk100_config& c = ctx->impl->config();
  return tk100::Nvfp4MlpOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), false, rows, static_cast<int>(c.hidden),
              static_cast<int>(c.intermediate), input, activation_codes, activation_scales,
              input_global_divisor, weight_codes, weight_scales, weight_scale_divisor, output);
}

tk100_status tk100_nvfp4_down_partial(tk100_ctx* ctx, tk100_stream stream, int rows,
                                      const uint16_t* input, uint8_t* activation_codes,
                                      uint8_t* activation_scales, float input_global_divisor,
                                      const uint8_t* weight_codes, const uint8_t* weight_scales,
                                      float weight_scale_divisor, float* partial_output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  const tk100_config& c = ctx->impl->config();
  if (!partial_output) {
    return ctx->impl->fail(TK100_ERR_LAUNCH, "[gpu.launch] NVFP4 down: fp32 output plane is null");
  }
  return tk100::Nvfp4MlpOp(*ctx->impl)
      .launch(static_cast<cudaStream_t>(stream), false, rows, static_cast<int>(c.hidden),
              static_cast<int>(c.intermediate), input, activation_codes, activation_scales,
              input_global_divisor, weight_codes, weight_scales, weight_scale_divisor, nullptr,
              partial_output);
}

tk100_status tk100_f32_to_bf16(tk100_ctx* ctx, tk100_stream stream, size_t count,
                               const float* input, uint16_t* output) {
  if (!ctx) return TK100_ERR_CONTEXT;
  if (count == 0 || count % 4 != 0 || !input || !output ||
      (reinterpret_cast<uintptr_t>(input) & 15) || (reinterpret_cast<uintptr_t>(output) & 7)) {
    return ctx->impl->fail(TK100_ERR_LAUNCH,
                           "[gpu.launch] fp32 -> BF16: count must be a positive multiple of 4 and "
                           "the planes 16-byte aligned");
  }
  ctx->impl->count_launch();
  return ctx->impl->check(tk100::launch_f32_to_bf16(static_cast<cudaStream_t>(stream),
                                                    static_cast<long long>(count), input, output),
                          "launching fp32 -> BF16");
}

}  // extern "C"
