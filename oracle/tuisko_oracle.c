/*
 * CPU oracle for the quantized projection path: a plain-C restatement of the
 * reference's host-side qualification formulas.  TEST INFRASTRUCTURE ONLY: it
 * is the checker for the CUDA kernels and the timed CPU baseline; nothing the
 * library ships links, loads or calls it.
 *
 * Every function names the reference file:line whose arithmetic it follows
 * (paths are relative to the blaind/tuiskollm tree).
 *
 * Parity status: pinned.  tests/test_oracle_kat.py checks this file against
 * every known-answer value the reference's own unit tests hold for the path
 * (codec pins, swizzle offsets, structured fixtures with closed-form sums).
 * One part is NOT pinned: NVFP4 *activation* quantisation (tko_nvfp4_quantize*)
 * has no implementation or test in the reference; it is this build's own
 * definition, written by symmetry with the pinned weight convention, and is
 * labelled "parity unpinned" wherever it is used.
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define TKO_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- codecs */

/* qual/src/fp8_projection_oracle.rs:106-108 */
TKO_API float tko_bf16_to_f32(uint16_t bits) {
  uint32_t w = (uint32_t)bits << 16;
  float f;
  memcpy(&f, &w, 4);
  return f;
}

/* qual/src/fp8_projection_oracle.rs:99-104 (round to nearest even, no NaN case) */
TKO_API uint16_t tko_f32_to_bf16(float value) {
  uint32_t bits;
  memcpy(&bits, &value, 4);
  uint32_t rounded = bits + (0x7fffu + ((bits >> 16) & 1u));
  return (uint16_t)(rounded >> 16);
}

/* qual/src/fp8_projection_oracle.rs:81-97; returns 0 on success, -1 for a NaN code */
TKO_API int tko_e4m3_decode(uint8_t code, float* out) {
  float sign = (code & 0x80) ? -1.0f : 1.0f;
  int exponent = (code >> 3) & 0x0f;
  int fraction = code & 0x07;
  float magnitude;
  if (exponent == 0 && fraction == 0) {
    magnitude = 0.0f;
  } else if (exponent == 0) {
    magnitude = (float)fraction * ldexpf(1.0f, -9);
  } else if (exponent == 15 && fraction == 7) {
    return -1;
  } else {
    magnitude = (1.0f + (float)fraction / 8.0f) * ldexpf(1.0f, exponent - 7);
  }
  *out = sign * magnitude;
  return 0;
}

static float e4m3_lut[256];
static double e4m3_lut64[256];
static int lut_ready = 0;

static void build_luts(void) {
  if (lut_ready) return;
  for (int c = 0; c < 256; ++c) {
    float v = 0.0f;
    if (tko_e4m3_decode((uint8_t)c, &v) != 0) v = NAN;
    e4m3_lut[c] = v;
    e4m3_lut64[c] = (double)v;
  }
  lut_ready = 1;
}

TKO_API void tko_init(void) { build_luts(); }

/* qual/src/fp8_projection_oracle.rs:52-79: exhaustive nearest-code search, the
 * reference encoder.  Returns the code, or -1 when the input is not finite. */
TKO_API int tko_e4m3_encode_search(float value) {
  build_luts();
  if (!isfinite(value)) return -1;
  if (value == 0.0f) return signbit(value) ? 0x80 : 0x00;
  if (value > 448.0f) value = 448.0f;
  if (value < -448.0f) value = -448.0f;
  int best = 0;
  float best_distance = INFINITY;
  for (int code = 0; code < 256; ++code) {
    if (code == 0x7f || code == 0xff) continue;
    float represented = e4m3_lut[code];
    if (represented == 0.0f && (signbit(represented) != 0) != (signbit(value) != 0)) continue;
    float distance = fabsf(value - represented);
    if (distance < best_distance || (distance == best_distance && (code & 1) == 0)) {
      best = code;
      best_distance = distance;
    }
  }
  return best;
}

/* Arithmetic round-to-nearest-even E4M3FN encoder with saturation to +-448.
 * Same contract as tko_e4m3_encode_search; the test suite proves the two equal
 * on every BF16 input over a sweep of scales before this one is trusted. */
TKO_API int tko_e4m3_encode(float value) {
  if (!isfinite(value)) return -1;
  int sign = signbit(value) ? 0x80 : 0x00;
  float a = fabsf(value);
  if (a == 0.0f) return sign;
  if (a >= 448.0f) return sign | 0x7e;
  int e;
  (void)frexpf(a, &e); /* a = m * 2^e, m in [0.5, 1) -> binade exponent e-1 */
  int exp2 = e - 1;
  if (exp2 < -6) exp2 = -6; /* subnormal and lowest normal binade share a step of 2^-9 */
  float step = ldexpf(1.0f, exp2 - 3);
  float q = a / step; /* exact: division by a power of two */
  float r = rintf(q); /* default rounding mode: nearest even */
  int n = (int)r;     /* value = n * step */
  int code;
  if (exp2 == -6 && n < 8) {
    code = n; /* subnormal (or zero) */
  } else {
    int ebits = exp2 + 7;
    if (n == 16) { /* rounded up into the next binade */
      ebits += 1;
      n = 8;
    }
    code = (ebits << 3) | (n - 8);
  }
  if (code > 0x7e) code = 0x7e;
  return sign | code;
}

/* Counts BF16 inputs (all 65536 bit patterns, finite ones only) for which the two
 * encoders disagree on value/scale; first_bad receives one offending pattern. */
TKO_API long tko_e4m3_encoder_disagreements(float scale, uint32_t* first_bad) {
  long bad = 0;
  for (uint32_t bits = 0; bits < 65536u; ++bits) {
    float v = tko_bf16_to_f32((uint16_t)bits);
    if (!isfinite(v)) continue;
    float q = v / scale;
    if (!isfinite(q)) continue;
    if (tko_e4m3_encode(q) != tko_e4m3_encode_search(q)) {
      if (bad == 0 && first_bad) *first_bad = bits;
      ++bad;
    }
  }
  return bad;
}

/* qual/src/nvfp4_swiglu.rs:373-378 */
TKO_API float tko_e2m1_decode(uint8_t code) {
  static const float mags[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  float m = mags[code & 7];
  return (code & 8) ? -m : m;
}

/* Round-to-nearest-even E2M1 encoder with saturation to +-6 (this build's own
 * definition; the reference never encodes E2M1).  Ties go to the code whose low
 * bit is zero, which is what IEEE nearest-even on the 1-bit mantissa gives. */
TKO_API int tko_e2m1_encode(float value) {
  static const float mags[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  int sign = signbit(value) ? 8 : 0;
  float a = fabsf(value);
  if (!(a == a)) return -1;
  int best = 7;
  for (int c = 0; c < 7; ++c) {
    float mid = 0.5f * (mags[c] + mags[c + 1]); /* exact */
    if (a < mid || (a == mid && (c & 1) == 0)) {
      best = c;
      break;
    }
  }
  return sign | best;
}

/* tuisko-model/src/materialize.rs:410-422 (same formula at
 * tuisko-kernels-sm89/src/nvfp4/swiglu.rs:47-61 and qual/src/nvfp4_swiglu.rs:359-371) */
TKO_API size_t tko_nvfp4_scale_offset(size_t row, size_t group, size_t groups_per_row) {
  size_t tile = row / 128;
  size_t row_in_tile = row & 127;
  size_t scale_tile = group / 4;
  size_t scale_lane = group & 3;
  size_t row_mod32 = row_in_tile & 31;
  size_t row_quartile = row_in_tile >> 5;
  return (tile * (groups_per_row / 4) + scale_tile) * 512 + row_mod32 * 16 + row_quartile * 4 +
         scale_lane;
}

/* ------------------------------------------------- residual add + RMSNorm */

/* qual/src/residual_norm.rs:228-232: residual = bf16(f32(x) + f32(branch)) */
TKO_API void tko_residual_add(const uint16_t* x, const uint16_t* branch, size_t n, uint16_t* out) {
  for (size_t i = 0; i < n; ++i)
    out[i] = tko_f32_to_bf16(tko_bf16_to_f32(x[i]) + tko_bf16_to_f32(branch[i]));
}

/* qual/src/residual_norm.rs:328-348: f64 RMSNorm with a zero-centred weight */
TKO_API void tko_rms_norm(const uint16_t* input, const uint16_t* weight, size_t hidden, float eps,
                          uint16_t* out) {
  double squared_sum = 0.0;
  for (size_t i = 0; i < hidden; ++i) {
    double v = (double)tko_bf16_to_f32(input[i]);
    squared_sum += v * v;
  }
  double mean = squared_sum / (double)hidden;
  double inverse_rms = 1.0 / sqrt(mean + (double)eps);
  for (size_t i = 0; i < hidden; ++i) {
    double v = (double)tko_bf16_to_f32(input[i]);
    double w = (double)tko_bf16_to_f32(weight[i]);
    out[i] = tko_f32_to_bf16((float)(v * inverse_rms * (1.0 + w)));
  }
}

/* rows x hidden driver for the two functions above (branch may be NULL) */
TKO_API void tko_residual_rms_norm_rows(const uint16_t* x, const uint16_t* branch,
                                        const uint16_t* weight, size_t rows, size_t hidden,
                                        float eps, uint16_t* residual_out,
                                        uint16_t* normalized_out) {
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows; ++r) {
    const uint16_t* src = x + (size_t)r * hidden;
    if (branch) {
      tko_residual_add(src, branch + (size_t)r * hidden, hidden, residual_out + (size_t)r * hidden);
      src = residual_out + (size_t)r * hidden;
    }
    tko_rms_norm(src, weight, hidden, eps, normalized_out + (size_t)r * hidden);
  }
}

/* ------------------------------------------- per-token E4M3 quantisation */

/* qual/src/fp8_projection_oracle.rs:23-50.  search != 0 selects the reference's
 * exhaustive encoder, 0 the arithmetic one.  Returns 0, or -1 on non-finite input. */
TKO_API int tko_quantize_e4m3(const uint16_t* input, size_t hidden, int search, uint8_t* codes,
                              float* scale_out, double* represented_sum) {
  build_luts();
  float maximum = 0.0f;
  for (size_t i = 0; i < hidden; ++i) {
    float a = fabsf(tko_bf16_to_f32(input[i]));
    if (a > maximum) maximum = a; /* f32::max folding from 0.0 */
  }
  float scale = (maximum == 0.0f) ? 1.0f : maximum / 448.0f;
  double sum = 0.0;
  for (size_t i = 0; i < hidden; ++i) {
    float q = tko_bf16_to_f32(input[i]) / scale;
    int code = search ? tko_e4m3_encode_search(q) : tko_e4m3_encode(q);
    if (code < 0) return -1;
    codes[i] = (uint8_t)code;
    sum += e4m3_lut64[code];
  }
  *scale_out = scale;
  if (represented_sum) *represented_sum = sum;
  return 0;
}

TKO_API int tko_quantize_e4m3_rows(const uint16_t* input, size_t rows, size_t hidden, int search,
                                   uint8_t* codes, float* scales) {
  int status = 0;
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows; ++r) {
    if (tko_quantize_e4m3(input + (size_t)r * hidden, hidden, search, codes + (size_t)r * hidden,
                          scales + r, NULL) != 0) {
#pragma omp atomic write
      status = -1;
    }
  }
  return status;
}

/* ------------------------------------------------------- FP8 projection */

/* qual/src/dense_fp8_gdn_layer.rs:417-433 (fp8_dot) and :400-415 (whole plane);
 * same formula at qual/src/dense_fp8_mlp.rs:295-312, qual/src/text_endpoint.rs:233-261:
 *   out[m, n] = (sum_k dec(a[m,k]) * dec(w[n,k]))_f64 * f64(a_scale[m]) * f64(bf16(w_scale[n]))
 * out is f64 [rows, out_rows] (token-major).  Returns -1 when a NaN code is met. */
TKO_API int tko_fp8_projection(const uint8_t* act_codes, const float* act_scales,
                               const uint8_t* w_codes, const uint16_t* w_scales, size_t rows,
                               size_t out_rows, size_t k, double* out) {
  build_luts();
  int status = 0;
#pragma omp parallel for schedule(static)
  for (long n = 0; n < (long)out_rows; ++n) {
    const uint8_t* w = w_codes + (size_t)n * k;
    double ws = (double)tko_bf16_to_f32(w_scales[n]);
    for (size_t m = 0; m < rows; ++m) {
      const uint8_t* a = act_codes + m * k;
      double sum = 0.0;
      int bad = 0;
      for (size_t i = 0; i < k; ++i) {
        bad |= (a[i] & 0x7f) == 0x7f;
        bad |= (w[i] & 0x7f) == 0x7f;
        sum += e4m3_lut64[a[i]] * e4m3_lut64[w[i]];
      }
      if (bad) {
#pragma omp atomic write
        status = -1;
      }
      out[m * out_rows + (size_t)n] = sum * (double)act_scales[m] * ws;
    }
  }
  return status;
}

/* Same, for a list of selected weight rows (row_index[j] picks w row); used to
 * check a sample of a plane that is too large to evaluate whole on the CPU. */
TKO_API int tko_fp8_projection_rows(const uint8_t* act_codes, const float* act_scales,
                                    const uint8_t* w_codes_sel, const uint16_t* w_scales_sel,
                                    size_t rows, size_t n_sel, size_t k, double* out) {
  return tko_fp8_projection(act_codes, act_scales, w_codes_sel, w_scales_sel, rows, n_sel, k, out);
}

/* ------------------------------------------------------- greedy argmax */

/* tuisko-engine/src/sampling.rs:162-173 and :233-242.  First maximum under the
 * IEEE total order wins (+0 > -0); any non-finite logit is an error (-1 - index). */
TKO_API long tko_greedy_index(const uint16_t* logits, size_t n) {
  long best = -1;
  int32_t best_key = 0;
  for (size_t i = 0; i < n; ++i) {
    uint32_t bits = (uint32_t)logits[i] << 16;
    if ((bits & 0x7f800000u) == 0x7f800000u) return -1 - (long)i;
    /* total_cmp key: flip the magnitude bits of negatives, compare as signed */
    int32_t key = (int32_t)bits;
    key ^= (int32_t)(((uint32_t)(key >> 31)) >> 1);
    if (best < 0 || key > best_key) {
      best = (long)i;
      best_key = key;
    }
  }
  return best;
}

/* tuisko-engine/src/sampling.rs:212-231 (top_k_select): `k` best (index, value) pairs, value
 * descending under the IEEE total order, ties by ascending index -- a candidate displaces a
 * retained one only when strictly greater.  Returns the count kept, or -1 - index of the first
 * non-finite logit. */
static int32_t tko_total_key(float v) {
  int32_t key;
  memcpy(&key, &v, 4);
  key ^= (int32_t)(((uint32_t)(key >> 31)) >> 1);
  return key;
}

TKO_API long tko_top_k_select(const uint16_t* logits, size_t n, size_t k, uint32_t* top_index,
                              float* top_value) {
  size_t kept = 0;
  for (size_t token = 0; token < n; ++token) {
    uint32_t bits = (uint32_t)logits[token] << 16;
    if ((bits & 0x7f800000u) == 0x7f800000u) return -1 - (long)token;
    float value;
    memcpy(&value, &bits, 4);
    int32_t key = tko_total_key(value);
    if (kept == k && !(key > tko_total_key(top_value[kept - 1]))) continue;
    /* partition point: first position whose retained value is below `value` */
    size_t at = 0;
    while (at < kept && tko_total_key(top_value[at]) >= key) ++at;
    size_t last = kept < k ? kept : k - 1;
    for (size_t i = last; i > at; --i) {
      top_value[i] = top_value[i - 1];
      top_index[i] = top_index[i - 1];
    }
    top_value[at] = value;
    top_index[at] = (uint32_t)token;
    if (kept < k) ++kept;
  }
  return (long)kept;
}

/* tuisko-engine/src/sampling.rs:244-260 (XorShift64). */
TKO_API uint64_t tko_xorshift_new(uint64_t seed) {
  const uint64_t scramble = 0x9e3779b97f4a7c15ull;
  uint64_t state = seed ^ scramble;
  return state == 0 ? scramble : state;
}

TKO_API double tko_xorshift_unit(uint64_t* state) {
  uint64_t value = *state;
  value ^= value << 13;
  value ^= value >> 7;
  value ^= value << 17;
  *state = value;
  return (double)(value >> 11) * (1.0 / 9007199254740992.0);
}

/* tuisko-engine/src/sampling.rs:76-95 and :175-210 (Sampler::sample): one token from a BF16
 * logit row; the generator state advances only on the sampled route.  Returns the token, or
 * -1 - index of a non-finite logit, or -(n + 2) when the distribution has no finite mass. */
TKO_API long tko_sample(const uint16_t* logits, size_t n, float temperature, float top_p,
                        size_t top_k, uint64_t* rng_state) {
  if (temperature == 0.0f || top_k == 1) return tko_greedy_index(logits, n);
  uint32_t* index = (uint32_t*)malloc(top_k * sizeof(uint32_t));
  float* value = (float*)malloc(top_k * sizeof(float));
  double* weight = (double*)malloc(top_k * sizeof(double));
  long result;
  long kept = tko_top_k_select(logits, n, top_k, index, value);
  if (kept < 0) {
    result = kept;
  } else {
    float maximum = value[0];
    double total = 0.0;
    for (long i = 0; i < kept; ++i) {
      weight[i] = (double)expf((value[i] - maximum) / temperature);
      total += weight[i];
    }
    float floor_p = top_p > FLT_MIN ? top_p : FLT_MIN;
    double cutoff = (double)floor_p * total;
    double retained_total = 0.0;
    long retained = 0;
    for (long i = 0; i < kept; ++i) {
      retained_total += weight[i];
      ++retained;
      if (retained_total >= cutoff) break;
    }
    if (retained == 0 || !isfinite(retained_total) || retained_total <= 0.0) {
      result = -((long)n + 2);
    } else {
      double threshold = tko_xorshift_unit(rng_state) * retained_total;
      double cumulative = 0.0;
      result = (long)index[retained - 1];
      for (long i = 0; i < retained; ++i) {
        cumulative += weight[i];
        if (cumulative >= threshold) {
          result = (long)index[i];
          break;
        }
      }
    }
  }
  free(index);
  free(value);
  free(weight);
  return result;
}

/* ------------------------------------------------------------- NVFP4 */

/* Weight value: e2m1 * e4m3(block scale) / global divisor
 * (tuisko-kernels-sm89/src/nvfp4/swiglu.rs:211-212; qual/src/nvfp4_swiglu.rs:317-357).
 * A16 dot: bf16 activations x decoded weights, f64 accumulation, one output per
 * (token, weight row).  w_codes is [rows_w, k/2] (low nibble = even column),
 * w_scales the swizzled E4M3 plane.  out is f64 [tokens, rows_w]. */
TKO_API int tko_nvfp4_a16_dot(const uint16_t* x, size_t tokens, size_t k, const uint8_t* w_codes,
                              const uint8_t* w_scales, float weight_scale_divisor, size_t rows_w,
                              double* out) {
  build_luts();
  size_t groups = k / 16;
  int status = 0;
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows_w; ++r) {
    for (size_t t = 0; t < tokens; ++t) {
      double acc = 0.0;
      for (size_t g = 0; g < groups; ++g) {
        uint8_t sc = w_scales[tko_nvfp4_scale_offset((size_t)r, g, groups)];
        if ((sc & 0x7f) == 0x7f) {
#pragma omp atomic write
          status = -1;
        }
        double gsum = 0.0;
        for (size_t c = 0; c < 16; ++c) {
          uint8_t packed = w_codes[(size_t)r * (k / 2) + g * 8 + c / 2];
          uint8_t code = (c & 1) ? (packed >> 4) : (packed & 15);
          gsum += (double)tko_bf16_to_f32(x[t * k + g * 16 + c]) * (double)tko_e2m1_decode(code);
        }
        acc += gsum * e4m3_lut64[sc];
      }
      out[t * rows_w + (size_t)r] = acc / (double)weight_scale_divisor;
    }
  }
  return status;
}

/* qual/src/nvfp4_swiglu.rs:306-315: silu(gate) * up in f64 with exact exp */
TKO_API double tko_silu_mul(double gate, double up) { return gate / (1.0 + exp(-gate)) * up; }

/* NVFP4 activation quantisation -- PARITY UNPINNED (no reference counterpart).
 * Definition, per token row and 16-wide block, all in f32 with IEEE operations:
 *   amax   = max |x|
 *   s_code = e4m3_rne_sat((amax * divisor) / 6)      (non-negative E4M3FN)
 *   s      = decode(s_code)
 *   code_j = (s == 0) ? signed zero : e2m1_rne_sat((x_j * divisor) / s)
 * Represented value = e2m1 * s / divisor, the same form as the weights.
 * codes: [rows, k/2], low nibble = even column.  scales: swizzled 128x4 tiles
 * addressed by tko_nvfp4_scale_offset(row = token, group), plane sized for
 * ceil(rows/128)*128 rows; entries of rows >= `rows` are not written. */
TKO_API void tko_nvfp4_quantize_rows(const uint16_t* x, size_t rows, size_t k, float divisor,
                                     uint8_t* codes, uint8_t* scales) {
  build_luts();
  size_t groups = k / 16;
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows; ++r) {
    for (size_t g = 0; g < groups; ++g) {
      const uint16_t* blk = x + (size_t)r * k + g * 16;
      float amax = 0.0f;
      for (int j = 0; j < 16; ++j) {
        float a = fabsf(tko_bf16_to_f32(blk[j]));
        if (a > amax) amax = a;
      }
      float raw = (amax * divisor) / 6.0f;
      int sc = tko_e4m3_encode(raw);
      if (sc < 0) sc = 0x7e;
      scales[tko_nvfp4_scale_offset((size_t)r, g, groups)] = (uint8_t)sc;
      float s = e4m3_lut[sc];
      for (int j = 0; j < 16; j += 2) {
        int lo, hi;
        float v0 = tko_bf16_to_f32(blk[j]), v1 = tko_bf16_to_f32(blk[j + 1]);
        if (s == 0.0f) {
          lo = signbit(v0) ? 8 : 0;
          hi = signbit(v1) ? 8 : 0;
        } else {
          lo = tko_e2m1_encode((v0 * divisor) / s);
          hi = tko_e2m1_encode((v1 * divisor) / s);
        }
        codes[(size_t)r * (k / 2) + g * 8 + j / 2] = (uint8_t)((hi << 4) | lo);
      }
    }
  }
}

/* W4A4 dot over represented values (own definition, see above):
 *   out[t, r] = (sum_g (sum_j e2m1(a)*e2m1(w)) * s_a[t,g] * s_w[r,g]) / (div_a * div_w)
 * f64 accumulation; out is f64 [tokens, rows_w]. */
TKO_API int tko_nvfp4_w4a4_dot(const uint8_t* a_codes, const uint8_t* a_scales, float a_divisor,
                               size_t tokens, size_t k, const uint8_t* w_codes,
                               const uint8_t* w_scales, float w_divisor, size_t rows_w,
                               double* out) {
  build_luts();
  size_t groups = k / 16;
  int status = 0;
  static const int8_t twice[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows_w; ++r) {
    for (size_t t = 0; t < tokens; ++t) {
      double acc = 0.0;
      for (size_t g = 0; g < groups; ++g) {
        uint8_t sw = w_scales[tko_nvfp4_scale_offset((size_t)r, g, groups)];
        uint8_t sa = a_scales[tko_nvfp4_scale_offset(t, g, groups)];
        if ((sw & 0x7f) == 0x7f || (sa & 0x7f) == 0x7f) {
#pragma omp atomic write
          status = -1;
        }
        int isum = 0; /* products of doubled magnitudes: exact small integers */
        const uint8_t* wp = w_codes + (size_t)r * (k / 2) + g * 8;
        const uint8_t* ap = a_codes + t * (k / 2) + g * 8;
        for (int b = 0; b < 8; ++b) {
          isum += twice[wp[b] & 15] * twice[ap[b] & 15];
          isum += twice[wp[b] >> 4] * twice[ap[b] >> 4];
        }
        acc += 0.25 * (double)isum * e4m3_lut64[sw] * e4m3_lut64[sa];
      }
      out[t * rows_w + (size_t)r] = acc / ((double)a_divisor * (double)w_divisor);
    }
  }
  return status;
}

TKO_API int tko_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Sets the OpenMP team size for the loops above (a launcher such as torch.distributed.run
 * exports OMP_NUM_THREADS=1 to its ranks; the CPU baseline wants all online cores). */
TKO_API void tko_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
