// Host-side operator layer: C++ counterparts of the reference's prepared operators
// (ResidualNormOp, FullAttentionQkvOp, GdnInputProjectionOp, LmHeadOp, Nvfp4SwiGluOp,
// Nvfp4DownOp) with the same method names, argument order and error behaviour.  The
// extern "C" functions of include/tuisko_sm100.h are one-line calls into these.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/tuisko_sm100.h"
#include "kernels.h"

namespace tk100 {

// Result of a launch: the reference's GpuResult<()> flattened to a status code; the
// message is kept on the context.
using Status = tk100_status;

// Route selectors for A/B measurements, read from TK100_* environment variables ONCE, when the
// context is created; no launch function reads the environment.  -1 / 0 = the library's choice.
struct Tuning {
  int splits = 0;             // TK100_SPLITS: forced K split
  int block_tok = 0;          // TK100_BLOCK_TOK: forced token tile
  int slots_per_sm = 0;       // TK100_SLOTS_PER_SM: CTA slots per SM assumed by the split choice
  int deep_ring = -1;         // TK100_DEEP_RING: ring variant of the FP8 projection
  int l2_prefetch = 0;        // TK100_L2_PREFETCH: FP8 weight k-blocks queued at L2 first
  int nvfp4_l2_prefetch = 0;  // TK100_NVFP4_L2_PREFETCH
  int cluster = 3;            // TK100_CLUSTER=0: split-K through global scratch instead of DSMEM,
                              // 1: symmetric two-barrier cluster exchange everywhere, 2: partial
                              // tiles pushed into the finishing CTA wherever they fit, 3 (default):
                              // pushed for the gate/up pairs at 128-token tiles only
  int fp8_pair = 1;           // TK100_FP8_PAIR: 0 off, 1 from 32 pair CTAs, 2 always
  int fp8_pair_min_rows = 256;
  int nvfp4_pair = 0;         // TK100_PAIR: 1 down, 2 gate_up too (cta_group::2 variant)
  int nvfp4_pair_min_rows = 1024;
  int nvfp4_persist = 0;      // TK100_PERSIST=1: persistent CTA-pair route for NVFP4 prefill shapes
  int nvfp4_persist_min_rows = 512;  // TK100_PERSIST_MIN_ROWS
  int fp8_stream_k = 0;       // TK100_FP8_STREAMK=1: stream-K on resident pairs wherever pairs can run (measured slower)
  int fp8_persist = 0;        // TK100_FP8_PERSIST=1: persistent CTA pairs with two accumulators for FP8
                              // prefill shapes of more pair tiles than resident pairs
  int nvfp4_wide = 0;         // TK100_NVFP4_WIDE: 256-token tiles (one CTA per SM) for NVFP4 prefill
                              // shapes: 1 down, 2 the gate/up pairs too
  int nvfp4_wide_min_rows = 512;  // TK100_NVFP4_WIDE_MIN_ROWS
  int swiglu_pairs = 1;       // TK100_SWIGLU_PAIRS=0: one CTA holds the gate and the up tile
  int fused_exchange = 1;     // TK100_FUSED_TAIL=0: argmax finalize / exchange as launches of their own
  int argmax_spread = 1;      // TK100_ARGMAX_SPREAD=0: every CTA's maxima go straight to the caller's keys
  int fused_quant = 0;        // TK100_FUSED_QUANT=1: launches of one wave and at most 4 rows quantise
                              // inside the projection kernel, 2: at every size (measured slower
                              // than the quantiser launch in front, so off by default)
  static Tuning from_environment();
};

class Context {
 public:
  static Status create(const tk100_config& config, Context** out, std::string* error);
  ~Context();

  Status fail(Status code, const std::string& message) {
    last_error_ = message;
    return code;
  }
  Status check(cudaError_t e, const char* operation);
  const std::string& last_error() const { return last_error_; }

  // Row-major u8 plane [rows, row_bytes] read through TMA in boxes of
  // 128 bytes x box_rows with the 128-byte swizzle.  Encoded once per distinct plane.
  Status tensor_map(const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                    CUtensorMap* out);

  // NVFP4 scale plane as rows of one 512-byte chunk (128 x u32), boxes of 4 chunks, unswizzled.
  Status scale_map(const void* base, uint64_t chunks, CUtensorMap* out);

  const tk100_config& config() const { return config_; }
  int sm_count() const { return sm_count_; }
  int persist_pairs() const { return persist_pairs_; }
  float* partials() const { return partials_; }
  size_t partial_bytes() const { return partial_bytes_; }
  unsigned int* counters() const { return counters_; }
  size_t counter_count() const { return counter_count_; }
  uint32_t* status_word() const { return status_; }
  unsigned int* exchange_step() const { return exchange_step_; }
  unsigned int* tail_ticket() const { return exchange_step_ + 1; }
  unsigned long long* argmax_spread_keys() const {
    return reinterpret_cast<unsigned long long*>(argmax_spread_);
  }
  unsigned int* argmax_spread_tickets() const {
    return reinterpret_cast<unsigned int*>(argmax_spread_ +
                                           static_cast<size_t>(kArgmaxGroups) * kArgmaxSpreadRows * 128);
  }
  unsigned int* peer_sum_state() const { return peer_sum_state_; }
  const Tuning& tuning() const { return tuning_; }
  int forced_splits() const { return tuning_.splits; }
  int forced_block_tok() const { return tuning_.block_tok; }
  void count_launch(int n = 1) { launches_ += static_cast<uint64_t>(n); }
  uint64_t launches() const { return launches_; }
  // Which kernel instantiation the last projection launch took (for reports and route tests):
  // a pointer and four integers per launch, formatted only when somebody asks.
  void note_route(const char* family, int a, int b, int splits, int cluster) {
    route_ = {family, a, b, splits, cluster};
  }
  const char* last_kernel();

 private:
  Context() = default;
  tk100_config config_{};
  int sm_count_ = 0;
  int persist_pairs_ = 0;  // CTA pairs of the persistent NVFP4 kernel that fit the device at once
  float* partials_ = nullptr;
  size_t partial_bytes_ = 0;
  unsigned int* counters_ = nullptr;
  size_t counter_count_ = 0;
  uint32_t* status_ = nullptr;
  unsigned int* exchange_step_ = nullptr;  // [0] device step counter of the peer argmax exchange,
                                           // [1] ticket of the LM head's fused tail
  uint8_t* argmax_spread_ = nullptr;  // LM head: per-group maxima and tickets (kArgmaxSpreadBytes)
  unsigned int* peer_sum_state_ = nullptr;  // peer sum: [0] step counter, [1..3] phase tickets
  Tuning tuning_;
  uint64_t launches_ = 0;
  struct RouteNote {
    const char* family = "";
    int a = 0, b = 0, splits = 0, cluster = 0;
  } route_;
  std::string route_text_;
  std::string last_error_;
  void* encode_fn_ = nullptr;
  // Encoded tensor maps by (base, rows, row bytes, box rows | kind): weight planes are encoded
  // on their first launch (or by tk100_register_plane) and found again by a hash look-up.
  struct MapKey {
    const void* base;
    uint64_t rows, row_bytes;
    uint32_t box_rows, kind;
    bool operator==(const MapKey& o) const {
      return base == o.base && rows == o.rows && row_bytes == o.row_bytes && box_rows == o.box_rows &&
             kind == o.kind;
    }
  };
  struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
      uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
      h ^= (k.rows + 0x7F4A7C15u) * 0xC2B2AE3D27D4EB4Full;
      h ^= (k.row_bytes << 17) ^ (static_cast<uint64_t>(k.box_rows) << 3) ^ k.kind;
      return static_cast<size_t>(h ^ (h >> 29));
    }
  };
  std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps_;
  // Maps of declared weight planes: encoded once by tk100_register_plane, never evicted.
  std::unordered_map<MapKey, CUtensorMap, MapKeyHash> pinned_maps_;
  Status encode_map(const MapKey& key, CUtensorMap* out);

 public:
  // Encodes the 128-row-box map of a weight-code plane ahead of its first launch.
  Status register_plane(const void* base, uint64_t rows, uint64_t row_bytes);
  size_t pinned_map_count() const { return pinned_maps_.size(); }
  size_t transient_map_count() const { return maps_.size(); }
};

// tuisko-kernels-sm120/src/residual_norm.rs:382-508
class ResidualNormOp {
 public:
  explicit ResidualNormOp(Context& ctx) : ctx_(ctx) {}
  Status launch_plain(cudaStream_t stream, int batch, const uint16_t* input,
                      const uint16_t* weight, uint16_t* output);
  Status launch_residual(cudaStream_t stream, int batch, const uint16_t* residual_input,
                         const uint16_t* branch, const uint16_t* weight,
                         uint16_t* residual_output, uint16_t* normalized_output);
  // Fused producer: norm (+ residual when branch != null) + per-token E4M3 quantisation.
  Status launch_quantize(cudaStream_t stream, int batch, const uint16_t* residual_input,
                         const uint16_t* branch, const uint16_t* weight,
                         uint16_t* residual_output, uint16_t* normalized_output,
                         uint8_t* activation_codes, float* activation_scales,
                         float nvfp4_divisor = 0.0f, uint8_t* nvfp4_codes = nullptr,
                         uint8_t* nvfp4_scales = nullptr);

 private:
  Context& ctx_;
};

// tuisko-model/src/materialize.rs: checkpoint planes -> run-time planes, on the device.
class MaterializeOp {
 public:
  explicit MaterializeOp(Context& ctx) : ctx_(ctx) {}
  // gather_source_planes (:295-314): `planes` device planes concatenated into `output`.
  Status gather(cudaStream_t stream, int planes, const void* const* sources,
                const uint64_t* bytes, void* output);
  // swizzle_scale_planes (:353-408) with validate_nvfp4_scales of every code.
  Status swizzle_scales(cudaStream_t stream, int planes, const uint8_t* const* sources,
                        uint64_t rows_per_plane, uint64_t groups_per_row, uint8_t* output);

 private:
  Context& ctx_;
};

// tuisko-engine/src/sampling.rs:56-95 (Sampler::new / Sampler::sample) for a decode batch of
// requests, on the device: option validation as the reference's, selection in one launch.
class SamplerOp {
 public:
  explicit SamplerOp(Context& ctx) : ctx_(ctx) {}
  Status launch(cudaStream_t stream, int rows, int vocab, const uint16_t* logits,
                const tk100_sampling_options* options, uint64_t* rng_state, uint64_t* scratch,
                tk100_sample_decision* decisions, uint32_t* top_out);

 private:
  Context& ctx_;
};

// tuisko-kernels-sm120/src/gdn/prepare.rs:176-290 (GdnPrepareOp::launch): control mat-vecs
// and the width-4 causal convolution of a decode batch of 1..=8 tokens, one launch.
class GdnPrepareOp {
 public:
  explicit GdnPrepareOp(Context& ctx) : ctx_(ctx) {}
  Status launch(cudaStream_t stream, int batch, const uint16_t* input,
                const uint16_t* control_weights, const uint16_t* a_log, const uint16_t* dt_bias,
                const uint16_t* projected, const uint16_t* convolution_weights,
                const uint32_t* state_rows, uint16_t* history, float* log_decay, float* beta,
                uint16_t* convolved);

 private:
  Context& ctx_;
};

// tuisko-kernels-sm120/src/gdn/recurrence.rs:171-236 (GdnRecurrenceOp::launch).
class GdnRecurrenceOp {
 public:
  explicit GdnRecurrenceOp(Context& ctx) : ctx_(ctx) {}
  Status launch(cudaStream_t stream, int batch, const uint16_t* qkv, const uint16_t* projected,
                const float* log_decay, const float* beta, const uint16_t* norm_weight,
                const uint32_t* state_rows, float* state, uint16_t* output);

 private:
  Context& ctx_;
};

// tuisko-kernels-sm120/src/fp8/projection.rs:510-794: one class serves the three planes;
// `name` only labels error messages ("FP8 QKV", "FP8 GDN input", "FP8 LM head", ...).
// How the LM head's per-shard maxima leave the projection: merged with the peers' over NVLink
// (world > 1) inside the same launch, or just unpacked (world == 1).
struct ArgmaxTail {
  int world = 1;
  int rank = 0;
  const uint64_t* peer_buffers = nullptr;  // `world` device addresses (tk100_argmax_exchange)
};

class Fp8ProjectionOp {
 public:
  Fp8ProjectionOp(Context& ctx, const char* name) : ctx_(ctx), name_(name) {}
  Status quantize(cudaStream_t stream, int rows, int columns, const uint16_t* input,
                  uint8_t* activation_codes, float* activation_scales);
  Status launch(cudaStream_t stream, int rows, int out_rows, int columns, const uint16_t* input,
                uint8_t* activation_codes, float* activation_scales, const uint8_t* weight_codes,
                const uint16_t* weight_scales, uint16_t* output, float* logits_f32 = nullptr,
                unsigned long long* argmax_scratch = nullptr, tk100_argmax_pair* pairs = nullptr,
                int vocab_offset = 0, const ArgmaxTail* tail = nullptr);

 private:
  Context& ctx_;
  const char* name_;
};

// tuisko-kernels-sm120/src/fp8/swiglu.rs:366-376: dense-FP8 gate/up projection + SwiGLU.
class Fp8SwiGluOp {
 public:
  explicit Fp8SwiGluOp(Context& ctx) : ctx_(ctx) {}
  Status launch(cudaStream_t stream, int rows, const uint16_t* input, uint8_t* activation_codes,
                float* activation_scales, const uint8_t* weight_codes, const uint16_t* weight_scales,
                uint16_t* output);

 private:
  Context& ctx_;
};

struct FullAttentionQkvOp : Fp8ProjectionOp {
  explicit FullAttentionQkvOp(Context& c) : Fp8ProjectionOp(c, "FP8 QKV") {}
};
struct GdnInputProjectionOp : Fp8ProjectionOp {
  explicit GdnInputProjectionOp(Context& c) : Fp8ProjectionOp(c, "FP8 GDN input") {}
};
struct LmHeadOp : Fp8ProjectionOp {
  explicit LmHeadOp(Context& c) : Fp8ProjectionOp(c, "FP8 LM head") {}
};
// tuisko-kernels-sm120/src/fp8/down.rs:197-207 (K = intermediate) and fp8/gdn_output.rs:178
// (K = the GDN value width): the same projection at other reduction lengths.
struct Fp8DownOp : Fp8ProjectionOp {
  explicit Fp8DownOp(Context& c) : Fp8ProjectionOp(c, "FP8 down") {}
};
struct GdnOutputProjectionOp : Fp8ProjectionOp {
  explicit GdnOutputProjectionOp(Context& c) : Fp8ProjectionOp(c, "FP8 GDN output") {}
};

// tuisko-kernels-sm89/src/nvfp4/swiglu.rs:470-571 and nvfp4/down.rs:455-556, with the
// activation side quantised to NVFP4 as well (caller-owned code / scale planes, like the FP8
// operators' activation planes) so that both operands feed the block-scaled tensor cores.
// Where gate_up + SwiGLU also leaves the NVFP4 form of its output for the down projection.
struct Nvfp4NextQuant {
  float divisor;    // input_global_divisor of the consumer
  uint8_t* codes;   // [rows, out_rows / 2]
  uint8_t* scales;  // swizzled [ceil(rows / 128) * 128, out_rows / 16]
};

class Nvfp4MlpOp {
 public:
  explicit Nvfp4MlpOp(Context& ctx) : ctx_(ctx) {}
  Status quantize(cudaStream_t stream, int rows, int columns, const uint16_t* input,
                  float input_global_divisor, uint8_t* activation_codes,
                  uint8_t* activation_scales);
  // gate_up = true: weights [2 * out_rows, columns / 2], output bf16(silu(gate) * up);
  // gate_up = false: weights [out_rows, columns / 2], plain projection.
  Status launch(cudaStream_t stream, bool gate_up, int rows, int out_rows, int columns,
                const uint16_t* input, uint8_t* activation_codes, uint8_t* activation_scales,
                float input_global_divisor, const uint8_t* weight_codes,
                const uint8_t* weight_scales, float weight_scale_divisor, uint16_t* output,
                float* output_f32 = nullptr, const Nvfp4NextQuant* next = nullptr);

 private:
  Context& ctx_;
};

}  // namespace tk100
