/*
 * tuisko-kernels-sm100: C ABI of the B200 (sm_100a) quantized projection operators.
 *
 * Each entry point stands in for one prepared-operator method of the reference's
 * sm_120 / sm_89 kernel crates (file:line cited per function, paths relative to the
 * blaind/tuiskollm tree) and keeps its pointer planes, layouts and scale conventions:
 *
 *   - BF16 planes are uint16_t bit patterns, row-major, token-major outputs [rows, N];
 *   - FP8 weights are E4M3FN codes [N, K] row-major (K contiguous) with ONE BF16 scale
 *     per output row; activations are quantised per token to E4M3FN with one fp32
 *     scale = amax/448 (1 when amax == 0);
 *   - NVFP4 weights are E2M1 codes [N, K/2] (low nibble = even column), E4M3 block
 *     scales per 16 columns stored in 128-row x 4-group tiles
 *     (tuisko-model/src/materialize.rs:410-422) and one fp32 global divisor;
 *   - the RMSNorm weight is stored zero-centred and applied as (1 + w).
 *
 * Conventions shared by every launch function:
 *   - the caller owns every buffer; launches allocate nothing, synchronise nothing and
 *     are stream-ordered on `stream` (a CUstream / cudaStream_t), so they can be
 *     recorded into a CUDA graph;
 *   - rows beyond `rows` of any output plane are never written;
 *   - pointers must be 16-byte aligned (the reference's arenas align to 256 bytes);
 *     FP8/NVFP4 code planes read through TMA must be 128-byte aligned;
 *   - the return value is a tk100_status; tk100_last_error() describes the failure.
 *     Nothing aborts or throws across this boundary.
 *
 * The library has no CPU fallback: without a CUDA device tk100_create fails.
 */
#ifndef TUISKO_SM100_H_
#define TUISKO_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TK100_ABI_VERSION 1

#if defined(__GNUC__)
#define TK100_API __attribute__((visibility("default")))
#else
#define TK100_API
#endif

/* Mirrors tuisko-gpu/src/error.rs:8-43 (GpuErrorCode) one to one. */
typedef enum tk100_status {
  TK100_OK = 0,
  TK100_ERR_DRIVER = 1,  /* gpu.driver  */
  TK100_ERR_ARENA = 2,   /* gpu.arena   */
  TK100_ERR_GRAPH = 3,   /* gpu.graph   */
  TK100_ERR_CONTEXT = 4, /* gpu.context */
  TK100_ERR_LAUNCH = 5,  /* gpu.launch  */
  TK100_ERR_MODULE = 6   /* gpu.module  */
} tk100_status;

/* Bits of the device status word returned by tk100_device_status(). */
#define TK100_DEVICE_WAIT_TIMEOUT 1u    /* a bounded in-kernel wait gave up */
#define TK100_DEVICE_NONFINITE_LOGIT 2u /* LM head produced NaN/Inf (sampling.rs:233-242) */
#define TK100_DEVICE_NONFINITE_INPUT 4u /* quantiser met NaN/Inf */
#define TK100_DEVICE_BAD_ARGUMENT 8u

typedef struct tk100_ctx tk100_ctx;
typedef void* tk100_stream; /* CUstream / cudaStream_t */

/* Model geometry, the run-time counterpart of the reference's `Arch` constants
 * (tuisko-model/src/lib.rs:29-137).  Zero fields take the Qwen3.8-27B values. */
typedef struct tk100_config {
  uint32_t abi_version;     /* TK100_ABI_VERSION */
  int32_t device;           /* CUDA device ordinal; must be current-able by the caller */
  uint32_t hidden;          /* 5120 */
  uint32_t intermediate;    /* 17408 */
  float rms_norm_epsilon;   /* 1e-6 */
  uint32_t max_rows;        /* largest `rows` any launch will pass (default 2048) */
  uint64_t workspace_bytes; /* split-K scratch allocated once by tk100_create (default 64 MiB) */
} tk100_config;

/* (max, index) of one token row, index in global vocabulary numbering; -1 = no row. */
typedef struct tk100_argmax_pair {
  float value;
  int32_t index;
} tk100_argmax_pair;

/* Replaces `*Op::new(&Arc<CudaContext>)` (tuisko-kernels-sm120/src/residual_norm.rs:396-416,
 * src/fp8/projection.rs:525-545, :629, :720; tuisko-kernels-sm89/src/nvfp4/swiglu.rs:495):
 * validates the geometry, prepares every kernel route and allocates the only memory the
 * library ever owns (split-K scratch, tile tickets, the status word).  No launches. */
TK100_API tk100_status tk100_create(const tk100_config* config, tk100_ctx** out);
TK100_API void tk100_destroy(tk100_ctx* ctx);
/* Message of the last failure on this context (or of tk100_create when ctx is NULL). */
TK100_API const char* tk100_last_error(const tk100_ctx* ctx);
/* Reads and clears the device status word; synchronises `stream`.  When the word reports a wait
 * that ran out, the tickets and keys a kernel that gave up may have left behind (split-K tile
 * tickets, the LM head's tail ticket and per-group maxima) are zeroed as well, so the context can
 * be used again; the results of the launches before the call are invalid. */
TK100_API tk100_status tk100_device_status(tk100_ctx* ctx, tk100_stream stream, uint32_t* word);
/* Number of kernels this context has launched (for launch accounting). */
TK100_API uint64_t tk100_launch_count(const tk100_ctx* ctx);
/* Name of the kernel instantiation the last projection launch on this context took, e.g.
 * "fp8_projection_kernel<16,1> splits=1" (token tile, ring variant) -- for reports and route
 * tests; valid until the next call.  No counterpart in the reference. */
TK100_API const char* tk100_last_kernel(tk100_ctx* ctx);

/* Declares a weight-code plane (`rows` x `row_bytes` bytes, 128-byte aligned: an FP8 plane has
 * row_bytes = K, a packed NVFP4 plane K / 2) so that its TMA tensor map is encoded now, at load
 * time, instead of on the plane's first launch; registered maps are never evicted.  Replaces the
 * per-operator `prepare` step of the reference (`*Op::new`, e.g.
 * tuisko-kernels-sm120/src/fp8/projection.rs:525-545).  Optional: an undeclared plane is encoded
 * on first use and cached.  Not stream-ordered, host work only. */
TK100_API tk100_status tk100_register_plane(tk100_ctx* ctx, const void* weight_codes, uint64_t rows,
                                            uint64_t row_bytes);
/* Number of registered and of lazily cached tensor maps (for tests and reports). */
TK100_API void tk100_tensor_map_counts(const tk100_ctx* ctx, uint64_t* registered,
                                       uint64_t* transient);

/* ResidualNormOp::launch_plain (tuisko-kernels-sm120/src/residual_norm.rs:425-456). */
TK100_API tk100_status tk100_rms_norm(tk100_ctx* ctx, tk100_stream stream, int rows, const uint16_t* input,
                            const uint16_t* weight, uint16_t* output);

/* ResidualNormOp::launch_residual (tuisko-kernels-sm120/src/residual_norm.rs:467-507).
 * residual_input and branch may alias each other; residual_output may be residual_input. */
TK100_API tk100_status tk100_residual_rms_norm(tk100_ctx* ctx, tk100_stream stream, int rows,
                                     const uint16_t* residual_input, const uint16_t* branch,
                                     const uint16_t* weight, uint16_t* residual_output,
                                     uint16_t* normalized_output);

/* The fused producer: launch_residual / launch_plain (branch == NULL, residual_output
 * ignored) plus the per-token E4M3 quantiser that the reference launches separately
 * (tuisko-kernels-sm120/src/fp8/projection.rs:71-88, device/fp8_projection.rs:54-126),
 * in ONE kernel.  activation_codes [rows, hidden] u8, activation_scales [rows] f32. */
TK100_API tk100_status tk100_residual_rms_norm_quantize(tk100_ctx* ctx, tk100_stream stream, int rows,
                                              const uint16_t* residual_input,
                                              const uint16_t* branch, const uint16_t* weight,
                                              uint16_t* residual_output,
                                              uint16_t* normalized_output,
                                              uint8_t* activation_codes,
                                              float* activation_scales);

/* The fused producer with both quantised forms of the normalised row: E4M3 codes + scale for
 * the FP8 projections (optional: activation_codes / activation_scales may both be NULL) and
 * NVFP4 codes + block scales for the W4A4 MLP (definition at tk100_nvfp4_quantize_activation;
 * no reference counterpart), all in the one kernel that reads x (+ branch) once.  The NVFP4
 * planes then go to tk100_nvfp4_gate_up_swiglu with input == NULL.  hidden % 64 == 0. */
TK100_API tk100_status tk100_residual_rms_norm_quantize_nvfp4(
    tk100_ctx* ctx, tk100_stream stream, int rows, const uint16_t* residual_input,
    const uint16_t* branch, const uint16_t* weight, uint16_t* residual_output,
    uint16_t* normalized_output, uint8_t* activation_codes, float* activation_scales,
    float input_global_divisor, uint8_t* nvfp4_codes, uint8_t* nvfp4_scales);

/* quantize_activation_e4m3 alone (tuisko-kernels-sm120/src/fp8/projection.rs:71-88),
 * for rows of `columns` BF16 values (columns % 8 == 0). */
TK100_API tk100_status tk100_quantize_activation_e4m3(tk100_ctx* ctx, tk100_stream stream, int rows,
                                            int columns, const uint16_t* input,
                                            uint8_t* activation_codes, float* activation_scales);

/* FullAttentionQkvOp::launch / GdnInputProjectionOp::launch
 * (tuisko-kernels-sm120/src/fp8/projection.rs:557-611, :660-702), same argument order.
 * `out_rows` is the weight row count N (the reference fixes it per Arch; here it is a
 * run-time value, N % 16 == 0) and the reduction length is config.hidden.
 * input != NULL: quantise `input` into activation_codes/scales, then project (the
 * reference's two launches).  input == NULL: activation_codes/scales already hold the
 * fused producer's output and only the projection runs.
 * Admitted rows: 1 <= rows <= config.max_rows; anything else is TK100_ERR_LAUNCH. */
TK100_API tk100_status tk100_fp8_qkv(tk100_ctx* ctx, tk100_stream stream, int rows, int out_rows,
                           const uint16_t* input, uint8_t* activation_codes,
                           float* activation_scales, const uint8_t* weight_codes,
                           const uint16_t* weight_scales, uint16_t* output);
TK100_API tk100_status tk100_fp8_gdn_input(tk100_ctx* ctx, tk100_stream stream, int rows, int out_rows,
                                 const uint16_t* input, uint8_t* activation_codes,
                                 float* activation_scales, const uint8_t* weight_codes,
                                 const uint16_t* weight_scales, uint16_t* output);
/* Same operator for any reduction length `columns` (% 128 == 0): the GDN-output and
 * dense-FP8 down planes (tuisko-kernels-sm120/src/fp8/gdn_output.rs:38-76, fp8/down.rs:197-207). */
TK100_API tk100_status tk100_fp8_projection(tk100_ctx* ctx, tk100_stream stream, int rows, int out_rows,
                                  int columns, const uint16_t* input, uint8_t* activation_codes,
                                  float* activation_scales, const uint8_t* weight_codes,
                                  const uint16_t* weight_scales, uint16_t* output);

/* Dense-FP8 MLP (tuisko-engine/src/dense_fp8_mlp.rs:404-452 calls the two in this order).
 * Fp8SwiGluOp::launch (tuisko-kernels-sm120/src/fp8/swiglu.rs:366-376), same argument order:
 * weight_codes [2 * intermediate, hidden] E4M3 with the gate rows first, weight_scales
 * [2 * intermediate] BF16; output [rows, intermediate] = bf16(silu(gate) * up), SiLU as
 * v / (1 + 2^(-v log2 e)) (device/fp8_swiglu.rs:13-15).  input == NULL: the activation planes
 * already hold the fused producer's codes and scales. */
TK100_API tk100_status tk100_fp8_swiglu(tk100_ctx* ctx, tk100_stream stream, int rows,
                                        const uint16_t* input, uint8_t* activation_codes,
                                        float* activation_scales, const uint8_t* weight_codes,
                                        const uint16_t* weight_scales, uint16_t* output);
/* Fp8DownOp::launch (tuisko-kernels-sm120/src/fp8/down.rs:197-207): input / activation planes
 * are [rows, intermediate] (the per-token E4M3 quantisation runs over the whole 17 408-wide
 * row), weight_codes [hidden, intermediate], output [rows, hidden]. */
TK100_API tk100_status tk100_fp8_down(tk100_ctx* ctx, tk100_stream stream, int rows,
                                      const uint16_t* input, uint8_t* activation_codes,
                                      float* activation_scales, const uint8_t* weight_codes,
                                      const uint16_t* weight_scales, uint16_t* output);
/* GdnOutputProjectionOp::launch (tuisko-kernels-sm120/src/fp8/gdn_output.rs:178): reduction
 * length `columns` = the GDN value width (6144 for the reference's model, % 128 == 0), weight_codes
 * [hidden, columns], output [rows, hidden]. */
TK100_API tk100_status tk100_fp8_gdn_output(tk100_ctx* ctx, tk100_stream stream, int rows, int columns,
                                            const uint16_t* input, uint8_t* activation_codes,
                                            float* activation_scales, const uint8_t* weight_codes,
                                            const uint16_t* weight_scales, uint16_t* output);

/* gather_source_planes (tuisko-model/src/materialize.rs:295-314), the body of
 * FullAttentionQkvBindings::materialize (:33-103) and MtpBindings::materialize_qkv (:119-152):
 * concatenates `planes` (1..=3) device planes of `bytes[i]` bytes each into `output`, in order,
 * without changing a byte.  `sources` and `bytes` are HOST arrays; the planes are device memory
 * (the checkpoint's query/gate, key and value tensors as uploaded). */
TK100_API tk100_status tk100_materialize_gather(tk100_ctx* ctx, tk100_stream stream, int planes,
                                                const void* const* sources, const uint64_t* bytes,
                                                void* output);

/* swizzle_scale_planes (tuisko-model/src/materialize.rs:353-408): permutes 1 (down) or 2 (gate
 * rows, then up rows) row-major E4M3 block-scale planes `[rows_per_plane, groups_per_row]` into
 * the 128-row x 4-group tile order of nvfp4_scale_offset (:410-422) that the NVFP4 kernels
 * consume.  Geometry is refused with the reference's messages (rows tiled by 128, groups by 4);
 * a negative or NaN scale code (validate_nvfp4_scales, bindings.rs:1105-1120) sets device status
 * bit 3.  `sources` is a HOST array of device pointers. */
TK100_API tk100_status tk100_materialize_nvfp4_scales(tk100_ctx* ctx, tk100_stream stream,
                                                      int planes, const uint8_t* const* sources,
                                                      uint64_t rows_per_plane,
                                                      uint64_t groups_per_row, uint8_t* output);

/* Per-request sampling controls (tuisko-engine/src/sampling.rs:11-22 SamplingOptions, plus the
 * request's two stop-token identifiers, :57-60). */
typedef struct tk100_sampling_options {
  float temperature;    /* 0 selects greedy decoding */
  float top_p;          /* cumulative probability kept after top-k, 0..=1 */
  uint32_t top_k;       /* 1..=32 on the device (the generation contract's default is 20) */
  uint32_t stop_ids[2]; /* distinct, below `vocab` */
} tk100_sampling_options;

/* tuisko-engine/src/sampling.rs:47-53 SampleDecision. */
typedef struct tk100_sample_decision {
  uint32_t token_id;
  uint32_t stopped; /* 1 when token_id is one of the request's stop identifiers */
} tk100_sample_decision;

/* Sampler::sample (tuisko-engine/src/sampling.rs:76-95) for `rows` (1..=8) requests at once, on
 * the device: `logits` is BF16 [rows, vocab] in device memory (the LM head's output plane), so the
 * row never travels to the host.  `options` is a HOST array of `rows` entries, validated with the
 * reference's rules and messages (:110-148) before anything is launched; a top_k above 32 is
 * refused (the host sampler remains for it).  `rng_state` [rows] holds each request's xorshift64
 * state in device memory -- start it from tk100_sampler_initial_state(seed); it advances once per
 * sampled (non-greedy) token, like the reference's.  `scratch` is
 * tk100_sampler_scratch_bytes(rows, vocab) bytes of device memory, zero before the first call.
 * `top_out`, when not NULL, receives the top_k survivors of each row as [rows, 32, 2] words
 * (f32 value bits, token index) in the reference's order.  A non-finite logit sets
 * TK100 status bit 1 (see tk100_device_status) where the reference returns an error. */
TK100_API tk100_status tk100_sample(tk100_ctx* ctx, tk100_stream stream, int rows, int vocab,
                                    const uint16_t* logits, const tk100_sampling_options* options,
                                    uint64_t* rng_state, uint64_t* scratch,
                                    tk100_sample_decision* decisions, uint32_t* top_out);
/* XorShift64::new (tuisko-engine/src/sampling.rs:247-250); host arithmetic only. */
TK100_API uint64_t tk100_sampler_initial_state(uint64_t seed);
TK100_API size_t tk100_sampler_scratch_bytes(int rows, int vocab);

/* GdnPrepareOp::launch (tuisko-kernels-sm120/src/gdn/prepare.rs:226-290): for a decode batch of
 * 1..=8 tokens, (a) the fused control mat-vecs -- rows [0,48) of `control_weights` give
 * log_decay = -exp(a_log) * softplus(x.w + dt_bias), rows [48,96) give beta = sigmoid(x.w) --
 * and (b) the width-4 causal convolution + SiLU over the first 10240 channels of `projected`
 * ([batch,16384] BF16), which also shifts each token's 3-tap history
 * (`history[state_rows[token], channel, 0..3]`, BF16) in place.  One launch where the reference
 * has two.  Outputs: log_decay, beta FP32 [batch,48]; convolved BF16 [batch,10240].  State rows of
 * one batch must be distinct.  Same argument order as the reference. */
TK100_API tk100_status tk100_gdn_prepare(tk100_ctx* ctx, tk100_stream stream, int batch,
                                         const uint16_t* input, const uint16_t* control_weights,
                                         const uint16_t* a_log, const uint16_t* dt_bias,
                                         const uint16_t* projected,
                                         const uint16_t* convolution_weights,
                                         const uint32_t* state_rows, uint16_t* history,
                                         float* log_decay, float* beta, uint16_t* convolved);

/* GdnRecurrenceOp::launch (tuisko-kernels-sm120/src/gdn/recurrence.rs:184-236): gated delta
 * rule on the FP32 state `[state rows, 48, 128, 128]` (updated in place at
 * `state_rows[token]`), then RMSNorm over each head's 128 outputs times `norm_weight`, times
 * SiLU of the gate (`projected[token, 10240 + ...]`), BF16 `[batch, 6144]`.  qkv is the
 * convolved plane `[batch,10240]`: 16 query heads, 16 key heads, 48 value heads of 128. */
TK100_API tk100_status tk100_gdn_recurrence(tk100_ctx* ctx, tk100_stream stream, int batch,
                                            const uint16_t* qkv, const uint16_t* projected,
                                            const float* log_decay, const float* beta,
                                            const uint16_t* norm_weight,
                                            const uint32_t* state_rows, float* state,
                                            uint16_t* output);

/* LmHeadOp::launch (tuisko-kernels-sm120/src/fp8/projection.rs:751-793) with the greedy
 * selection of tuisko-engine/src/sampling.rs:162-173 folded into the same kernel.
 * vocab_rows / vocab_offset describe this rank's contiguous shard of the vocabulary
 * (248320 / 0 on one GPU).  output (BF16 logits [rows, vocab_rows]) is the reference's
 * plane; logits_f32 and pairs are optional (NULL to skip; with pairs == NULL and
 * argmax_scratch != NULL the packed maxima are left in argmax_scratch).  argmax_scratch is a
 * caller-owned array of `rows` 64-bit words that must be zero before the first launch;
 * every launch leaves it zero again (with pairs != NULL and up to 32 rows the CTAs collect their
 * maxima in keys owned by the context, one cache line per token and group of CTAs, and the
 * caller's array is not written at all).  Launches on one context that write pairs must be
 * ordered on one stream: they share those keys and the ticket that elects the finishing CTA.
 * pairs[i].index is a global vocabulary index. */
TK100_API tk100_status tk100_fp8_lm_head(tk100_ctx* ctx, tk100_stream stream, int rows, int vocab_rows,
                               int vocab_offset, const uint16_t* input, uint8_t* activation_codes,
                               float* activation_scales, const uint8_t* weight_codes,
                               const uint16_t* weight_scales, uint16_t* output, float* logits_f32,
                               uint64_t* argmax_scratch, tk100_argmax_pair* pairs);

/* LmHeadOp::launch for one rank of a vocabulary-sharded LM head, with the exchange and the merge
 * in the SAME launch (no reference counterpart: the reference is single-GPU and selects on the
 * host): the last CTA of the projection to finish stores this shard's (max, index) pairs into
 * every peer's exchange buffer over NVLink (step-tagged 8-byte words, plain peer stores), waits
 * -- bounded, ~2 s, then TK100_DEVICE_WAIT_TIMEOUT -- for the peers' pairs and writes the merged
 * pairs [rows], identical on every rank.  world == 1 degenerates to tk100_fp8_lm_head with
 * pairs.  Arguments as tk100_fp8_lm_head and tk100_argmax_exchange (peer_buffers may be NULL
 * when world == 1); every rank makes the same sequence of calls. */
TK100_API tk100_status tk100_fp8_lm_head_sharded(
    tk100_ctx* ctx, tk100_stream stream, int rows, int vocab_rows, int vocab_offset,
    const uint16_t* input, uint8_t* activation_codes, float* activation_scales,
    const uint8_t* weight_codes, const uint16_t* weight_scales, uint16_t* output, float* logits_f32,
    uint64_t* argmax_scratch, int world, int rank, const uint64_t* peer_buffers,
    tk100_argmax_pair* merged_pairs);

/* Reduces the gathered per-shard pairs [shards, rows] to [rows] with the same rule as
 * greedy_index (first maximum in total order; lowest global index on ties). */
TK100_API tk100_status tk100_argmax_merge(tk100_ctx* ctx, tk100_stream stream, int rows, int shards,
                                const tk100_argmax_pair* gathered, tk100_argmax_pair* output);

/* Vocabulary-sharded greedy selection fused with its exchange (no reference counterpart: the
 * reference is single-GPU and selects on the host).  Call tk100_fp8_lm_head with
 * pairs == NULL so that the packed per-shard maxima stay in argmax_scratch, then this: one
 * small kernel per rank unpacks them, stores the (max, index) pairs straight into every
 * peer's exchange buffer over NVLink as 8-byte words tagged with the step number (no fence, no
 * separate flag), waits (bounded, ~2 s, then TK100_DEVICE_WAIT_TIMEOUT) for all peers' words of
 * the step and merges with the first-maximum rule into `output` [rows] -- identical on every
 * rank.  No collective library call is involved.
 * peer_buffers: host array of `world` device addresses, entry i = rank i's exchange buffer as
 * mapped in THIS process (peer access enabled; e.g. torch symmetric memory), each
 * TK100_EXCHANGE_BYTES(rows, world) bytes, zero-filled once before the first call.  Every
 * rank must make the same sequence of calls (the kernels meet by step number). */
#define TK100_EXCHANGE_BYTES(rows, world) (2u * (world) * (rows) * 16u)
TK100_API tk100_status tk100_argmax_exchange(tk100_ctx* ctx, tk100_stream stream, int rows, int world,
                                   int rank, uint64_t* argmax_scratch,
                                   const uint64_t* peer_buffers, tk100_argmax_pair* output);

/* NVFP4 activation quantiser for the W4A4 tensor-core route.  The reference's NVFP4
 * operators multiply BF16 activations (A16) and have no such step; the definition is this
 * library's own, symmetric to the weight convention: per 16 columns
 *   scale = e4m3_rne_sat((amax * divisor) / 6),  code = e2m1_rne_sat((x * divisor) / scale),
 * represented value = e2m1 * scale / divisor.  activation_codes [rows, columns/2] (low
 * nibble = even column); activation_scales in the same 128-row x 4-group tiles as weight
 * scales with row = token, sized ceil(rows/128)*128 * columns/16 bytes.  columns % 64 == 0. */
TK100_API tk100_status tk100_nvfp4_quantize_activation(tk100_ctx* ctx, tk100_stream stream, int rows,
                                             int columns, const uint16_t* input,
                                             float input_global_divisor,
                                             uint8_t* activation_codes,
                                             uint8_t* activation_scales);

/* Nvfp4SwiGluOp::launch (tuisko-kernels-sm89/src/nvfp4/swiglu.rs:525-571): weight_codes is the
 * fused [2 * intermediate, hidden/2] plane (gate rows, then up rows), weight_scales its
 * swizzled [2 * intermediate, hidden/16] E4M3 plane, weight_scale_divisor finite and > 0;
 * output [rows, intermediate] = bf16(silu(gate) * up).  Added to the reference signature:
 * the activation code / scale planes (caller-owned, as for the FP8 operators) and the
 * checkpoint's input_global_scale divisor (tuisko-model/src/bindings.rs:880-883), because
 * the contraction runs W4A4 on tcgen05.mma kind::mxf4nvf4.block_scale.
 * input != NULL: quantise it first; input == NULL: the planes already hold codes/scales. */
TK100_API tk100_status tk100_nvfp4_gate_up_swiglu(tk100_ctx* ctx, tk100_stream stream, int rows,
                                        const uint16_t* input, uint8_t* activation_codes,
                                        uint8_t* activation_scales, float input_global_divisor,
                                        const uint8_t* weight_codes, const uint8_t* weight_scales,
                                        float weight_scale_divisor, uint16_t* output);

/* Tensor-parallel layer: sum of every rank's fp32 partial output (tk100_nvfp4_down_partial),
 * rounded to BF16 once, by one kernel per rank over NVLink peer memory instead of a collective
 * library call plus tk100_f32_to_bf16.  peer_buffers[i] is the device address, valid on this
 * rank, of rank i's exchange buffer (entry `rank` is this rank's own): tk100_peer_sum_bytes
 * (capacity_values, world) bytes each, 256-byte aligned, zeroed once, the same capacity on every
 * rank and in every call.  values % 8 == 0, values <= capacity_values.  Up to 16 384 values every
 * rank receives the whole partials (one NVLink latency); beyond that rank d adds chunk d of all
 * partials and sends the BF16 chunk to everyone.  The partials are added in rank order on every
 * rank, so all ranks end with identical bits.  All ranks must call it the same number of
 * times; a peer that does not arrive within 2 s sets TK100_DEVICE_WAIT_TIMEOUT.  Ranks are
 * processes on different GPUs (the kernel waits for its peers).  No counterpart in the
 * reference (single GPU). */
TK100_API size_t tk100_peer_sum_bytes(size_t capacity_values, int world);
TK100_API tk100_status tk100_peer_sum_bf16(tk100_ctx* ctx, tk100_stream stream, size_t values,
                                           size_t capacity_values, int world, int rank,
                                           const float* partial, const uint64_t* peer_buffers,
                                           uint16_t* output);

/* tk100_nvfp4_gate_up_swiglu that also leaves the NVFP4 form of its output (codes
 * [rows, intermediate/2], swizzled block scales, definition at tk100_nvfp4_quantize_activation
 * with output_global_divisor) for tk100_nvfp4_down(input == NULL).  Up to 32 rows the
 * quantisation runs in the projection's epilogue instead of a launch of its own; beyond that
 * the call launches the quantiser after the projection.  Both planes are always written.  No
 * counterpart in the reference (its down kernel reads BF16). */
TK100_API tk100_status tk100_nvfp4_gate_up_swiglu_quantize(
    tk100_ctx* ctx, tk100_stream stream, int rows, const uint16_t* input, uint8_t* activation_codes,
    uint8_t* activation_scales, float input_global_divisor, const uint8_t* weight_codes,
    const uint8_t* weight_scales, float weight_scale_divisor, uint16_t* output,
    float output_global_divisor, uint8_t* output_codes, uint8_t* output_scales);

/* Nvfp4DownOp::launch (tuisko-kernels-sm89/src/nvfp4/down.rs:510-556): weight_codes
 * [hidden, intermediate/2], weight_scales swizzled [hidden, intermediate/16];
 * input / activation planes are [rows, intermediate]; output [rows, hidden]. */
TK100_API tk100_status tk100_nvfp4_down(tk100_ctx* ctx, tk100_stream stream, int rows,
                              const uint16_t* input, uint8_t* activation_codes,
                              uint8_t* activation_scales, float input_global_divisor,
                              const uint8_t* weight_codes, const uint8_t* weight_scales,
                              float weight_scale_divisor, uint16_t* output);

/* Tensor-parallel form of tk100_nvfp4_down (no reference counterpart: the reference is
 * single-GPU).  A rank that owns a slice of the reduction (config.intermediate = its slice,
 * a multiple of 64 columns; weight and activation planes hold only that slice) writes its
 * unrounded fp32 partial sums [rows, hidden]; the ranks' partials are summed with one NCCL
 * all-reduce and rounded once with tk100_f32_to_bf16. */
TK100_API tk100_status tk100_nvfp4_down_partial(tk100_ctx* ctx, tk100_stream stream, int rows,
                                      const uint16_t* input, uint8_t* activation_codes,
                                      uint8_t* activation_scales, float input_global_divisor,
                                      const uint8_t* weight_codes, const uint8_t* weight_scales,
                                      float weight_scale_divisor, float* partial_output);
/* fp32 -> BF16, round to nearest even; count % 4 == 0. */
TK100_API tk100_status tk100_f32_to_bf16(tk100_ctx* ctx, tk100_stream stream, size_t count,
                               const float* input, uint16_t* output);

/* No counterpart in the reference.  The FP8 projection (activation codes and scales already
 * produced, as with input == NULL above) for hosts that must not allocate device memory and
 * therefore cannot use tk100_create, which allocates the split-K scratch: an engine that
 * gives its whole device budget to one arena at start-up and fails its "no allocation after
 * warm-up" gate on any later cudaMalloc, or code that runs as a guest inside a process whose
 * CUDA allocator it does not own.  It takes no context; its scratch (split-K partial tiles,
 * tile tickets, a fault word) is a fixed array inside the library image.
 *
 * Limits and rules:
 *   - every GPU that loads this library holds TK100_STATIC_SCRATCH_BYTES of device memory
 *     for that array until the process exits, whether or not this function is ever called;
 *   - rows <= TK100_STATIC_MAX_ROWS; a problem whose split-K scratch would exceed the array
 *     is refused with TK100_ERR_ARENA (nothing is launched), it is not run more slowly;
 *   - the first call on each device looks up the array's device address, the SM count and
 *     the kernel attributes (the device must be current); make that first call before any
 *     stream capture begins;
 *   - all calls on a device share the one array: each call clears the tickets on `stream`
 *     before its kernel, and two calls whose kernels could overlap on the GPU (different
 *     streams, no dependency) race on it -- serialise them;
 *   - a bounded in-kernel wait that runs out leaves TK100_DEVICE_WAIT_TIMEOUT in the array's
 *     fault word and the output of that call (and of later calls, whose CTAs leave at once
 *     while the bit is set) is invalid; tk100_fp8_projection_static_status reads and clears it;
 *   - it calls no cudaMalloc / cudaFree and no allocating library routine.
 * `message` (may be NULL) receives the failure text, at most message_capacity bytes. */
#define TK100_STATIC_MAX_ROWS 256
#define TK100_STATIC_SCRATCH_BYTES ((8u << 20) + (16u << 10))
TK100_API tk100_status tk100_fp8_projection_static(
    tk100_stream stream, int rows, int out_rows, int columns, const uint8_t* activation_codes,
    const float* activation_scales, const uint8_t* weight_codes, const uint16_t* weight_scales,
    uint16_t* output, char* message, size_t message_capacity);
/* No counterpart in the reference.  Reads and clears the fault word of the static scratch on the
 * current device (the counterpart of tk100_device_status for the context-free entry point; same
 * TK100_DEVICE_* bits); synchronises `stream`, allocates nothing.  Call it on the stream the
 * static launches used, after them. */
TK100_API tk100_status tk100_fp8_projection_static_status(tk100_stream stream, uint32_t* word);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* TUISKO_SM100_H_ */
