// Internal launch interface between the operator layer (ops.cu) and the kernels.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

namespace tk100 {

// Process-wide switches, read from the environment by read_process_switches() when a context
// is created (or the context-free entry point sets a device up) and never by a launch:
// TK100_PDL=0 turns programmatic stream serialisation off (with it a kernel's set-up and weight
// prefetch overlap the tail of its predecessor).
void read_process_switches();
bool pdl_enabled();

// Performance-experiment switches (1 = skip the epilogue, 2 = skip the UMMA issue, 4 = skip the
// activation loads; results are wrong when any is set).  They exist only in a library built
// with -DTK100_EXPERIMENT, which reads them from TK100_DEBUG; the default build compiles every
// test of them to `false`.
enum : uint32_t { DBG_NO_EPILOGUE = 1, DBG_NO_MMA = 2, DBG_NO_ACT = 4 };
#ifdef TK100_EXPERIMENT
#define TK100_DBG(p, bits) (((p).debug & (bits)) != 0)
#else
#define TK100_DBG(p, bits) false
#endif
uint32_t debug_flags();
// Experiment builds only: a kernel writes %globaltimer at a few points of CTA `c` into
// stamps[c * 8 + k] (k: 0 entry, 1 set-up done, 2 producer past the dependency wait, 3 first stage
// full, 4 last UMMA issued, 5 accumulator complete, 6 epilogue done, 7 exit) when the plane is set
// (its device address comes from TK100_STAMPS_PTR, read with the other switches).
#ifdef TK100_EXPERIMENT
#define TK100_STAMP(p, k)                                                                          \
  do {                                                                                             \
    if ((p).stamps) {                                                                              \
      const size_t _c = blockIdx.x + static_cast<size_t>(gridDim.x) * (blockIdx.y + static_cast<size_t>(gridDim.y) * blockIdx.z); \
      unsigned long long _t;                                                                       \
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(_t));                                       \
      (p).stamps[_c * 8 + (k)] = _t;                                                               \
    }                                                                                              \
  } while (0)
#else
#define TK100_STAMP(p, k) do { } while (0)
#endif
unsigned long long* debug_stamps();

// A cluster shape other than (1, 1, 1) launches thread-block clusters of that shape.
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t stream, dim3 cluster, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned int n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster.x * cluster.y * cluster.z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster.x;
    attr[n].val.clusterDim.y = cluster.y;
    attr[n].val.clusterDim.z = cluster.z;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, Args&&... args) {
  return launch_kernel_cluster(kernel, grid, block, smem, stream, dim3(1, 1, 1),
                               std::forward<Args>(args)...);
}

// ---------------------------------------------------------------- norm_quant.cu
// threads/chunks for a row of `hidden` BF16 values; false when the row is not admitted.
bool norm_geometry(int hidden, int* threads, int* chunks);

// One launch covering any of: residual add (branch != null), RMSNorm
// (normalized_out != null) and E4M3 quantisation (codes != null).
cudaError_t launch_resnorm_quant(cudaStream_t stream, int rows, int hidden, const uint16_t* x,
                                 const uint16_t* branch, const uint16_t* weight,
                                 uint16_t* residual_out, uint16_t* normalized_out, uint8_t* codes,
                                 float* scales, float eps, uint32_t* status,
                                 uint8_t* nvfp4_codes = nullptr, uint8_t* nvfp4_scales = nullptr,
                                 float nvfp4_divisor = 0.0f);

// ----------------------------------------------------------------------- gdn.cu
// Decode batches the gated-delta-net steps admit (tuisko-kernels-sm120/src/gdn/prepare.rs:13-24).
constexpr int kGdnMaxBatch = 8;
struct GdnPrepareParams {
  int batch;
  int hidden;        // 5120
  int control_rows;  // 48 decay rows followed by 48 beta rows in `control_weights`
  int qkv_rows;      // 10240 convolved channels
  int input_rows;    // 16384 = row stride of `projected`
  const uint16_t* input;                // [batch, hidden] BF16
  const uint16_t* control_weights;      // [2 * control_rows, hidden] BF16
  const uint16_t* a_log;                // [control_rows] BF16
  const uint16_t* dt_bias;              // [control_rows] BF16
  const uint16_t* projected;            // [batch, input_rows] BF16
  const uint16_t* convolution_weights;  // [qkv_rows, 4] BF16
  const uint32_t* state_rows;           // [batch]
  uint16_t* history;                    // [state rows, qkv_rows, 3] BF16, updated in place
  float* log_decay;                     // [batch, control_rows]
  float* beta;                          // [batch, control_rows]
  uint16_t* convolved;                  // [batch, qkv_rows] BF16
};
struct GdnRecurrenceParams {
  int batch;
  int qkv_rows;
  int input_rows;
  const uint16_t* qkv;          // [batch, qkv_rows] BF16: q (16 x 128), k (16 x 128), v (48 x 128)
  const uint16_t* projected;    // [batch, input_rows] BF16; the gate follows the qkv rows
  const float* log_decay;       // [batch, 48]
  const float* beta;            // [batch, 48]
  const uint16_t* norm_weight;  // [128] BF16
  const uint32_t* state_rows;   // [batch]
  float* state;                 // [state rows, 48, 128, 128] FP32, updated in place
  uint16_t* output;             // [batch, 48 * 128] BF16
};
// True for the one geometry the kernels are written for (16 key heads, 48 value heads of 128).
bool gdn_geometry_ok(int hidden, int control_rows, int qkv_rows, int input_rows);
cudaError_t launch_gdn_prepare(cudaStream_t stream, const GdnPrepareParams& p);
cudaError_t launch_gdn_recurrence(cudaStream_t stream, const GdnRecurrenceParams& p);

// --------------------------------------------------------------- materialize.cu
constexpr int kMaterializeMaxPlanes = 3;
struct GatherParams {
  int planes;                                    // 1..=3
  const uint8_t* source[kMaterializeMaxPlanes];  // device planes, concatenated in this order
  size_t offset[kMaterializeMaxPlanes + 1];      // byte offset of each plane in `output`; [planes] = total
  uint8_t* output;
};
struct SwizzleParams {
  int planes;                // 1 (down) or 2 (gate rows then up rows)
  const uint8_t* source[2];  // [rows_per_plane, groups_per_row] E4M3 codes, row-major
  size_t rows_per_plane;
  size_t groups_per_row;     // multiple of 4
  int vector_loads;          // sources 16-byte aligned and groups_per_row a multiple of 16
  uint8_t* output;           // [planes * rows_per_plane * groups_per_row] in 128 x 4 tiles
  uint32_t* status;
};
cudaError_t launch_gather_planes(cudaStream_t stream, const GatherParams& p, bool vector_words);
cudaError_t launch_swizzle_scales(cudaStream_t stream, const SwizzleParams& p);

// ------------------------------------------------------------------- sampler.cu
constexpr int kSamplerMaxRows = 8;
constexpr int kSamplerMaxTopK = 32;
struct SamplerParams {
  int rows;   // 1..=8 requests of a decode batch
  int vocab;  // values per row, a multiple of 8
  const uint16_t* logits;  // [rows, vocab] BF16
  float temperature[kSamplerMaxRows];
  float top_p[kSamplerMaxRows];
  int top_k[kSamplerMaxRows];  // 1..=32
  uint32_t stop_ids[2 * kSamplerMaxRows];
  uint64_t* rng_state;  // [rows] xorshift64 states, advanced in place
  uint64_t* scratch;    // sampler_scratch_bytes(rows, vocab), zero before the first launch
  uint32_t* decisions;  // [rows, 2]: token id, stopped flag
  uint32_t* top_out;    // optional [rows, 32, 2]: value bits (f32) and index of the survivors
  uint32_t* status;
};
int sampler_slices(int vocab);
size_t sampler_scratch_bytes(int rows, int vocab);
cudaError_t launch_sampler(cudaStream_t stream, const SamplerParams& p);

// ------------------------------------------------------------------ fp8_proj.cu
// ------------------------------------------------------------------- fp8_mlp.cu
struct Fp8SwigluParams {
  int rows;          // active tokens M
  int intermediate;  // outputs per token I; the weight plane holds gate rows [0, I) then up rows [I, 2I)
  int k;             // reduction length, multiple of 128
  const float* act_scales;   // [rows]
  const uint16_t* w_scales;  // [2 * I] BF16
  uint16_t* out;             // [rows, I] BF16
  uint32_t* status;
};
cudaError_t fp8_swiglu_prepare();
// block_tok 32 or 128.
cudaError_t launch_fp8_swiglu(cudaStream_t stream, int block_tok, const CUtensorMap& tmap_w,
                              const CUtensorMap& tmap_a, const Fp8SwigluParams& p);

struct ArgmaxPair {
  float value;
  int32_t index;
};
// Peer exchange buffers of the vocabulary-sharded argmax (device addresses, one per rank;
// entry `rank` is this rank's own buffer).
constexpr int kMaxExchangeRanks = 8;
struct ExchangePeers {
  unsigned char* base[kMaxExchangeRanks];
};
// Largest row count whose activation quantiser the projection kernel runs itself.
constexpr int kFusedQuantRows = 4;

constexpr int kArgmaxGroups = 8;
constexpr int kArgmaxSpreadRows = 32;
constexpr size_t kArgmaxSpreadBytes =
    static_cast<size_t>(kArgmaxGroups) * (kArgmaxSpreadRows + 1) * 128;  // keys, then the tickets

struct Fp8ProjParams {
  int rows;       // active tokens M
  int out_rows;   // weight rows N (this shard)
  int k;          // reduction length, multiple of 128
  int splits;     // K splits (grid.z)
  int deep_ring;  // 1: longer ring, two CTAs per SM (launches with few CTAs); 2: 3-stage ring, four
                  // CTAs per SM (16-token tiles, tile counts between 3 and 4 per SM)
  int l2_prefetch;  // > 0: before waiting for the predecessor, ask L2 for up to this many weight
                    // k-blocks beyond the ring (short weight streams that fit L2)
  int cluster;    // 1: the splits of a tile form a thread-block cluster and reduce over
                  // distributed shared memory (every CTA finishes a share of the tokens, two
                  // cluster barriers); 2: the peers store their partial tiles into the leader's
                  // shared memory and leave, the leader finishes every token;
                  // 0: fp32 partial tiles in `partials` + tickets
  const float* act_scales;      // [rows]
  const uint16_t* w_scales;     // [out_rows] BF16
  uint16_t* out;                // [rows, out_rows] BF16, may be null for the LM head
  float* logits_f32;            // [rows, out_rows] or null
  unsigned long long* argmax_keys;  // [rows] packed (key, ~index) or null
  int vocab_offset;             // global index of this shard's row 0
  float* partials;              // split-K scratch
  unsigned int* counters;       // one per output tile, zero between launches
  uint32_t* status;
  uint32_t debug;               // experiment switches (debug_flags()); 0 in normal use
  unsigned long long* stamps;   // experiment builds: timestamp plane (TK100_STAMP), else null
  // Fused activation quantiser (16-token tiles, rows <= kFusedQuantRows): when x_bf16 is set the
  // CTA computes the per-token scales from the BF16 rows itself and writes each stage's code tile
  // into shared memory (tmap_a is not read); the CTAs of output tile 0 also publish the codes
  // and scales to codes_out / scales_out, the planes the unfused quantiser would have written.
  const uint16_t* x_bf16;       // [rows, k] or null
  uint8_t* codes_out;           // [rows, k]
  float* scales_out;            // [rows]
  // Fused tail of the LM head: the last CTA of the launch to finish (ticket) unpacks the packed
  // maxima into pairs_out (world == 1) or exchanges them with the peers and merges (world > 1),
  // and clears argmax_keys.  Null ticket = no fused tail.
  unsigned int* tail_ticket;
  ArgmaxPair* pairs_out;        // [rows]
  // Spread maxima (fused tail, rows <= kArgmaxSpreadRows): the CTAs of one wave finish together,
  // and their atomics on one token's key -- and on the keys of the other tokens in the same
  // 128-byte line -- queue behind one another at one L2 slice while the CTAs hold their SM slots.
  // With spread_keys set, CTA tile_n works on group tile_n % kArgmaxGroups: key (group, token)
  // sits in a line of its own ([group][kArgmaxSpreadRows] lines of 16 words, word 0 used), and
  // tickets are drawn per group (spread_tickets, one line each) with only the last CTA of a group
  // drawing from tail_ticket.  The CTA that draws the last one folds the groups, clears them and
  // leaves argmax_keys untouched (world == 1) or holding the folded keys for the exchange.
  unsigned long long* spread_keys;  // library-owned, zero between launches; null = direct keys
  unsigned int* spread_tickets;     // [kArgmaxGroups] lines of 32 words, word 0 used
  int world, rank;
  unsigned int* step_counter;   // device step number of the exchange
  ExchangePeers peers;
};

// block_tok is the token tile (16, 32, 64, 128 or 256).
cudaError_t launch_fp8_projection(cudaStream_t stream, int block_tok, const CUtensorMap& tmap_w,
                                  const CUtensorMap& tmap_a, const Fp8ProjParams& p);
size_t fp8_projection_smem_bytes(int block_tok);
int fp8_projection_stages(int block_tok);
cudaError_t fp8_projection_prepare();  // sets the dynamic shared-memory attributes once
// fp8_pair.cu: prefill route on CTA pairs (256-row x 256-token pair tiles, BF16 output only,
// unsplit K; out_rows must be a multiple of 256).
// Persistent form (fp8_pair_persist.cu): `pairs` resident CTA pairs walk the pair tiles.
cudaError_t fp8_pair_persist_prepare();
// stream_k: the pairs share the launch's tiles x K steps evenly; pieces of a tile meet in
// p.partials (fp8_pair_stream_k_scratch_bytes) under tickets in p.counters (two per pair tile).
cudaError_t launch_fp8_pair_persist(cudaStream_t stream, int pairs, const CUtensorMap& tmap_w,
                                    const CUtensorMap& tmap_a, const Fp8ProjParams& p, bool stream_k);
size_t fp8_pair_stream_k_scratch_bytes(int pairs);
cudaError_t fp8_pair_prepare();
cudaError_t launch_fp8_pair(cudaStream_t stream, const CUtensorMap& tmap_w, const CUtensorMap& tmap_a,
                            const Fp8ProjParams& p);

// keys -> pairs, and clears the keys for the next launch.
cudaError_t launch_argmax_finalize(cudaStream_t stream, int rows, unsigned long long* keys,
                                   ArgmaxPair* pairs);
cudaError_t launch_argmax_exchange(cudaStream_t stream, int rows, int world, int rank,
                                   unsigned long long* keys, const ExchangePeers& peers,
                                   unsigned int* step_counter, ArgmaxPair* out, uint32_t* status);
// peer_reduce.cu: sum of the ranks' fp32 partials over peer memory, rounded to BF16 once.
constexpr long long kPeerSumOneShotElems = 16384;  // up to here every rank receives whole partials
struct PeerSumParams {
  long long elems;        // values per rank, multiple of 8
  long long chunk;        // two-shot: values of one rank's chunk (multiple of 8); world * chunk >= elems
  long long chunk_capacity;  // the chunk of a call at the buffer's full capacity: slot / result stride
  long long one_shot_stride4;  // one-shot slot stride in float4 (fixed by the capacity)
  size_t one_shot_offset;  // byte offset of the one-shot slots inside every rank's buffer
  int world, rank;
  int one_shot;
  const float* partial;   // this rank's [elems] fp32
  uint16_t* output;       // this rank's [elems] BF16 sum
  size_t result_offset;   // byte offsets inside every rank's exchange buffer
  size_t flag_offset;
  unsigned int* tickets;  // 3 zeroed counters of this rank
  unsigned int* step_counter;
  uint32_t* status;
};
cudaError_t launch_peer_sum(cudaStream_t stream, int ctas, const PeerSumParams& q,
                            const ExchangePeers& peers);
// [shards, rows] pairs -> [rows] pairs with the first-maximum rule.
cudaError_t launch_argmax_merge(cudaStream_t stream, int rows, int shards,
                                const ArgmaxPair* gathered, ArgmaxPair* out);

// -------------------------------------------------------------------- nvfp4.cu
struct Nvfp4Params {
  int rows;            // active tokens M
  int out_rows;        // outputs per token (weight rows of one tile family), multiple of 128
  int k;               // reduction length in elements, multiple of 256
  int splits;          // K splits (1 with gate/up fusion)
  int cluster;         // 1: the splits of a tile (or a gate/up pair) reduce over distributed shared
                       // memory with two cluster barriers; 2: partial tiles are pushed into the
                       // CTA that finishes them (split K: the leader; pairs: the partner)
  int pair_swiglu;     // 1: plain tiles in clusters of two (gate tile, up tile): the up CTA hands
                       // its accumulator to the gate CTA, which writes bf16(silu(gate) * up)
  int up_row_offset;   // gate/up fusion: first weight row of the up half (= out_rows)
  int l2_prefetch;     // > 0: queue up to this many weight k-blocks of the CTA's slice at L2 first
  const uint8_t* w_scales;  // swizzled E4M3 weight scales
  const uint8_t* a_scales;  // swizzled E4M3 activation scales
  float out_scale;     // 1 / (weight divisor * activation divisor)
  uint16_t* out;       // [rows, out_rows] BF16
  float* out_f32;      // when set (plain projection only): unrounded fp32 output instead
  // gate/up on cluster pairs at <= 32 tokens: also quantise the rounded outputs to NVFP4 for
  // the next projection (codes [rows, out_rows / 2], swizzled block scales, row = token)
  uint8_t* q_codes;
  uint8_t* q_scales;
  float q_divisor;
  float* partials;
  unsigned int* counters;
  uint32_t* status;
  uint32_t debug;      // experiment switches (debug_flags()); 0 in normal use
  unsigned long long* stamps;  // experiment builds: timestamp plane (TK100_STAMP), else null
};

cudaError_t nvfp4_prepare();
// Bytes of the shared-memory ring of the plain projection kernel at this token tile (what a
// pushed reduction may land in).
size_t nvfp4_ring_bytes(int block_tok);
// block_tok 32 or 128.  gate_up: weight plane holds gate rows then up rows; output is
// bf16(silu(gate) * up).
cudaError_t launch_nvfp4_gemm(cudaStream_t stream, int block_tok, bool gate_up,
                              const CUtensorMap& tmap_w, const CUtensorMap& tmap_a,
                              const Nvfp4Params& p);
// nvfp4_pair.cu: prefill route on CTA pairs (256-row x 256-token pair tiles).
cudaError_t nvfp4_pair_prepare();
cudaError_t launch_nvfp4_pair(cudaStream_t stream, bool gate_up, const CUtensorMap& tmap_w,
                              const CUtensorMap& tmap_a, const CUtensorMap& tmap_wsf,
                              const CUtensorMap& tmap_asf, const Nvfp4Params& p);
// nvfp4_persist.cu: prefill route on persistent CTA pairs (256-row x 256-token pair tiles, one
// pair per two SMs walking its share of the tiles).  `max_pairs`: pairs resident at once.
cudaError_t nvfp4_persist_prepare(int* max_pairs);
cudaError_t launch_nvfp4_persist(cudaStream_t stream, bool gate_up, int pairs, const CUtensorMap& tmap_w,
                                 const CUtensorMap& tmap_a, const CUtensorMap& tmap_wsf,
                                 const CUtensorMap& tmap_asf, const Nvfp4Params& p);
cudaError_t launch_f32_to_bf16(cudaStream_t stream, long long n, const float* in, uint16_t* out);
cudaError_t launch_nvfp4_quantize(cudaStream_t stream, int rows, int k, const uint16_t* x,
                                  float divisor, uint8_t* codes, uint8_t* scales);

}  // namespace tk100
