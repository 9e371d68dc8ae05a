/*
 * q3x_oracle.c -- see q3x_oracle.h.  TEST INFRASTRUCTURE ONLY: the checker for the CUDA
 * path, never a fallback for it.
 *
 * Build: gcc -std=c11 -O2 -ffp-contract=off -fPIC -shared q3x_oracle.c -lm
 * (-ffp-contract=off keeps a*b-c*d and the sum-of-squares loops un-fused, which is what an
 * ISO build of the reference computes.)
 */
#include "q3x_oracle.h"

#include <float.h>
#include <math.h>
#include <string.h>

#define BF16_ROWS_OVERFLOW(a, b) ((b) != 0 && (a) > SIZE_MAX / (b))

/* ---------------------------------------------------------------- bf16 codec */

/* src/runtime/reference/decode_ops.cpp:15-20 */
float q3x_oracle_decode_bf16(uint16_t bits) {
  uint32_t wide = (uint32_t)bits << 16;
  float f;
  memcpy(&f, &wide, sizeof f);
  return f;
}

/* src/runtime/reference/decode_ops.cpp:22-33: RNE; a NaN keeps sign and top payload and
 * gets the quiet bit so a small payload can never round into infinity. */
uint16_t q3x_oracle_encode_bf16(float value) {
  uint32_t u;
  memcpy(&u, &value, sizeof u);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

#define DEC q3x_oracle_decode_bf16
#define ENC q3x_oracle_encode_bf16

static int eps_ok(float eps) { return isfinite(eps) && eps > 0.0f; }

int q3x_oracle_fp32_to_bf16(const float* in, size_t count, uint16_t* out) {
  if (count == 0) return Q3X_ORACLE_OK;
  if (!in || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t i = 0; i < count; ++i) out[i] = ENC(in[i]);
  return Q3X_ORACLE_OK;
}

/* ---------------------------------------------------------------- embedding */

int q3x_oracle_embedding_gather(const uint16_t* table, size_t vocab, size_t hidden,
                                const uint32_t* token_ids, size_t token_count, uint16_t* out) {
  if (BF16_ROWS_OVERFLOW(vocab, hidden) || BF16_ROWS_OVERFLOW(token_count, hidden))
    return Q3X_ORACLE_SIZE_OVERFLOW;
  if (token_count == 0 || hidden == 0) return Q3X_ORACLE_OK;
  if (!table || !token_ids || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  int status = Q3X_ORACLE_OK;
  for (size_t t = 0; t < token_count; ++t) {
    size_t id = token_ids[t];
    if (id >= vocab) {
      status = Q3X_ORACLE_TOKEN_OUT_OF_RANGE;
      continue;
    }
    memcpy(out + t * hidden, table + id * hidden, hidden * sizeof(uint16_t));
  }
  return status;
}

/* ---------------------------------------------------------------- RMS norms */

/* One row of src/runtime/reference/decode_ops.cpp:69-82 / :109-129.  The sum of squares is
 * a sequential FP32 sum; the product order is x * inv * gamma, then (optionally) the SiLU
 * of the gate multiplies in FP32 before the single rounding. */
static void norm_row(const uint16_t* x, const uint16_t* w, const uint16_t* gate, size_t n,
                     float eps, int centered, uint16_t* y) {
  float ss = 0.0f;
  for (size_t i = 0; i < n; ++i) {
    float v = DEC(x[i]);
    ss += v * v;
  }
  float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (size_t i = 0; i < n; ++i) {
    float gamma = DEC(w[i]) + (centered ? 1.0f : 0.0f);
    float v = DEC(x[i]) * inv * gamma;
    if (gate) {
      float g = DEC(gate[i]);
      v *= g / (1.0f + expf(-g));
    }
    y[i] = ENC(v);
  }
}

int q3x_oracle_rms_norm(const uint16_t* in, const uint16_t* weight, size_t width, float eps,
                        int centered, uint16_t* out) {
  if (!eps_ok(eps)) return Q3X_ORACLE_INVALID_ARGUMENT;
  if (width == 0) return Q3X_ORACLE_OK;
  if (!in || !weight || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  norm_row(in, weight, NULL, width, eps, centered, out);
  return Q3X_ORACLE_OK;
}

int q3x_oracle_headwise_rms_norm(const uint16_t* in, const uint16_t* weight,
                                 const uint16_t* gate, size_t heads, size_t dim, float eps,
                                 int centered, uint16_t* out) {
  if (!eps_ok(eps)) return Q3X_ORACLE_INVALID_ARGUMENT;
  if (BF16_ROWS_OVERFLOW(heads, dim)) return Q3X_ORACLE_SIZE_OVERFLOW;
  if (heads == 0 || dim == 0) return Q3X_ORACLE_OK;
  if (!in || !weight || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t h = 0; h < heads; ++h)
    norm_row(in + h * dim, weight, gate ? gate + h * dim : NULL, dim, eps, centered,
             out + h * dim);
  return Q3X_ORACLE_OK;
}

/* ---------------------------------------------------------------- pointwise */

int q3x_oracle_residual_add(const uint16_t* left, const uint16_t* right, size_t count,
                            uint16_t* out) {
  if (count == 0) return Q3X_ORACLE_OK;
  if (!left || !right || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t i = 0; i < count; ++i) out[i] = ENC(DEC(left[i]) + DEC(right[i]));
  return Q3X_ORACLE_OK;
}

int q3x_oracle_residual_add_rms_norm(const uint16_t* left, const uint16_t* right,
                                     const uint16_t* weight, size_t tokens, size_t hidden,
                                     float eps, uint16_t* residual, uint16_t* normalized) {
  if (!eps_ok(eps)) return Q3X_ORACLE_INVALID_ARGUMENT;
  if (BF16_ROWS_OVERFLOW(tokens, hidden)) return Q3X_ORACLE_SIZE_OVERFLOW;
  if (tokens == 0 || hidden == 0) return Q3X_ORACLE_OK;
  if (!left || !right || !weight || !residual) return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t t = 0; t < tokens; ++t) {
    const size_t o = t * hidden;
    /* the norm may overwrite `right` exactly, so finish the row's add first */
    for (size_t i = 0; i < hidden; ++i) residual[o + i] = ENC(DEC(left[o + i]) + DEC(right[o + i]));
    if (normalized) norm_row(residual + o, weight, NULL, hidden, eps, 1, normalized + o);
  }
  return Q3X_ORACLE_OK;
}

int q3x_oracle_silu_mul(const uint16_t* gate, const uint16_t* up, size_t count, uint16_t* out) {
  if (count == 0) return Q3X_ORACLE_OK;
  if (!gate || !up || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t i = 0; i < count; ++i) {
    float g = DEC(gate[i]);
    float s = g / (1.0f + expf(-g));
    out[i] = ENC(s * DEC(up[i]));
  }
  return Q3X_ORACLE_OK;
}

int q3x_oracle_silu_mul_merged(const uint16_t* merged, size_t tokens, size_t intermediate,
                               uint16_t* out) {
  if (BF16_ROWS_OVERFLOW(tokens, intermediate) || BF16_ROWS_OVERFLOW(tokens * intermediate, 2))
    return Q3X_ORACLE_SIZE_OVERFLOW;
  if (tokens == 0 || intermediate == 0) return Q3X_ORACLE_OK;
  if (!merged || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t t = 0; t < tokens; ++t) {
    const uint16_t* row = merged + t * 2 * intermediate;
    int st = q3x_oracle_silu_mul(row, row + intermediate, intermediate, out + t * intermediate);
    if (st) return st;
  }
  return Q3X_ORACLE_OK;
}

int q3x_oracle_sigmoid_gate(const uint16_t* value, const uint16_t* gate, size_t count,
                            uint16_t* out) {
  if (count == 0) return Q3X_ORACLE_OK;
  if (!value || !gate || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t i = 0; i < count; ++i) {
    float g = DEC(gate[i]);
    /* branch-stable form, decode_ops.cpp:334-337 */
    float s = g >= 0.0f ? 1.0f / (1.0f + expf(-g)) : expf(g) / (1.0f + expf(g));
    out[i] = ENC(DEC(value[i]) * s);
  }
  return Q3X_ORACLE_OK;
}

int q3x_oracle_l2_normalize_heads(const uint16_t* in, size_t heads, size_t dim, float eps,
                                  float scale, uint16_t* out) {
  if (!eps_ok(eps)) return Q3X_ORACLE_INVALID_ARGUMENT;
  if (BF16_ROWS_OVERFLOW(heads, dim)) return Q3X_ORACLE_SIZE_OVERFLOW;
  if (heads == 0 || dim == 0) return Q3X_ORACLE_OK;
  if (!in || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t h = 0; h < heads; ++h) {
    const uint16_t* x = in + h * dim;
    float ss = 0.0f;
    for (size_t i = 0; i < dim; ++i) {
      float v = DEC(x[i]);
      ss += v * v;
    }
    /* no mean: this is an L2 norm, not an RMS norm (decode_ops.cpp:369) */
    float inv = 1.0f / sqrtf(ss + eps);
    if (scale != 1.0f) inv = inv * scale;
    for (size_t i = 0; i < dim; ++i) out[h * dim + i] = ENC(DEC(x[i]) * inv);
  }
  return Q3X_ORACLE_OK;
}

/* ---------------------------------------------------------------- RoPE */

int q3x_oracle_partial_neox_rope_256_64(const uint16_t* in, const float* cosines,
                                        const float* sines, size_t heads, uint16_t* out) {
  enum { D = 256, ROT = 64, HALF = 32 };
  if (BF16_ROWS_OVERFLOW(heads, (size_t)D)) return Q3X_ORACLE_SIZE_OVERFLOW;
  if (heads == 0) return Q3X_ORACLE_OK;
  if (!in || !cosines || !sines || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t h = 0; h < heads; ++h) {
    const uint16_t* x = in + h * D;
    uint16_t* y = out + h * D;
    for (int d = 0; d < HALF; ++d) {
      float a = DEC(x[d]);
      float b = DEC(x[d + HALF]);
      /* plain mul/sub and mul/add, no FMA (decode_ops.cpp:399-403) */
      uint16_t lo = ENC(a * cosines[d] - b * sines[d]);
      uint16_t hi = ENC(b * cosines[d] + a * sines[d]);
      y[d] = lo;
      y[d + HALF] = hi;
    }
    if (y != x) memmove(y + ROT, x + ROT, (D - ROT) * sizeof(uint16_t));
  }
  return Q3X_ORACLE_OK;
}

static float bf16_round_trip(float v) { return DEC(ENC(v)); }

void q3x_oracle_rope_tables(size_t first_position, size_t positions, float* cosines,
                            float* sines) {
  const float theta = 10000000.0f;
  for (size_t p = 0; p < positions; ++p) {
    for (size_t pair = 0; pair < 32; ++pair) {
      float exponent = 2.0f * (float)pair / 64.0f;
      float inv_freq = 1.0f / powf(theta, exponent);
      float angle = (float)(first_position + p) * inv_freq;
      /* cos/sin of a finite angle is never NaN, so the NaN branch of ENC is moot and this
       * equals the reference's bf16_round_trip (request_state.cpp:326-334). */
      cosines[p * 32 + pair] = bf16_round_trip(cosf(angle));
      sines[p * 32 + pair] = bf16_round_trip(sinf(angle));
    }
  }
}

/* ---------------------------------------------------------------- layout */

static int ranges_overlap(const void* a, size_t abytes, const void* b, size_t bbytes) {
  uintptr_t x = (uintptr_t)a, y = (uintptr_t)b;
  return x < y + bbytes && y < x + abytes;
}

int q3x_oracle_split_interleaved_q_gate(const uint16_t* in, size_t heads, size_t dim,
                                        uint16_t* q_out, uint16_t* gate_out) {
  if (BF16_ROWS_OVERFLOW(heads, dim) || BF16_ROWS_OVERFLOW(heads * dim, 2 * sizeof(uint16_t)))
    return Q3X_ORACLE_SIZE_OVERFLOW;
  if (heads == 0 || dim == 0) return Q3X_ORACLE_OK;
  if (!in || !q_out || !gate_out) return Q3X_ORACLE_INVALID_ARGUMENT;
  size_t obytes = heads * dim * sizeof(uint16_t);
  if (ranges_overlap(in, 2 * obytes, q_out, obytes) || ranges_overlap(in, 2 * obytes, gate_out, obytes) ||
      ranges_overlap(q_out, obytes, gate_out, obytes))
    return Q3X_ORACLE_INVALID_ALIAS;
  for (size_t h = 0; h < heads; ++h) {
    memcpy(q_out + h * dim, in + (2 * h) * dim, dim * sizeof(uint16_t));
    memcpy(gate_out + h * dim, in + (2 * h + 1) * dim, dim * sizeof(uint16_t));
  }
  return Q3X_ORACLE_OK;
}

int q3x_oracle_full_attention_preprocess(const uint16_t* interleaved_q_gate, uint16_t* key,
                                         const uint16_t* q_weight, const uint16_t* k_weight,
                                         float eps, uint16_t* q_out, uint16_t* gate_out,
                                         const float* cosines, const float* sines,
                                         size_t first_position, size_t tokens) {
  enum { QH = 24, KH = 4, D = 256 };
  if (!eps_ok(eps)) return Q3X_ORACLE_INVALID_ARGUMENT;
  if (tokens == 0) return Q3X_ORACLE_OK;
  if (!interleaved_q_gate || !key || !q_weight || !k_weight || !q_out || !gate_out || !cosines ||
      !sines)
    return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t t = 0; t < tokens; ++t) {
    uint16_t* q = q_out + t * QH * D;
    uint16_t* k = key + t * KH * D;
    const float* c = cosines + (first_position + t) * 32;
    const float* s = sines + (first_position + t) * 32;
    int st = q3x_oracle_split_interleaved_q_gate(interleaved_q_gate + t * QH * 2 * D, QH, D, q,
                                                 gate_out + t * QH * D);
    if (st) return st;
    /* normalised values are rounded to bf16 BEFORE the rotation reads them */
    st = q3x_oracle_headwise_rms_norm(q, q_weight, NULL, QH, D, eps, 1, q);
    if (st) return st;
    st = q3x_oracle_headwise_rms_norm(k, k_weight, NULL, KH, D, eps, 1, k);
    if (st) return st;
    st = q3x_oracle_partial_neox_rope_256_64(q, c, s, QH, q);
    if (st) return st;
    st = q3x_oracle_partial_neox_rope_256_64(k, c, s, KH, k);
    if (st) return st;
  }
  return Q3X_ORACLE_OK;
}

/* ---------------------------------------------------------------- causal conv1d */

int q3x_oracle_causal_conv1d_silu(const uint16_t* raw, size_t tokens, size_t channels,
                                  const uint16_t* weight, uint16_t* history, uint16_t* out) {
  if (BF16_ROWS_OVERFLOW(tokens, channels)) return Q3X_ORACLE_SIZE_OVERFLOW;
  if (tokens == 0 || channels == 0) return Q3X_ORACLE_OK;
  if (!raw || !weight || !history || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  if (raw == weight || raw == history || weight == history || weight == out || history == out)
    return Q3X_ORACLE_INVALID_ALIAS;
  for (size_t t = 0; t < tokens; ++t) {
    const uint16_t* x = raw + t * channels;
    uint16_t* y = out + t * channels;
    for (size_t c = 0; c < channels; ++c) {
      uint16_t* h = history + c * 3;
      const uint16_t* w = weight + c * 4;
      uint16_t cur = x[c];
      /* fused multiply-adds, oldest tap first (gdn_decode.cpp:163-175) */
      float acc = 0.0f;
      acc = fmaf(DEC(h[0]), DEC(w[0]), acc);
      acc = fmaf(DEC(h[1]), DEC(w[1]), acc);
      acc = fmaf(DEC(h[2]), DEC(w[2]), acc);
      acc = fmaf(DEC(cur), DEC(w[3]), acc);
      y[c] = ENC(acc / (1.0f + expf(-acc)));
      h[0] = h[1];
      h[1] = h[2];
      h[2] = cur; /* the RAW input, not the convolved value */
    }
  }
  return Q3X_ORACLE_OK;
}

/* ---------------------------------------------------------------- NVFP4 */

/* src/quantization/nvfp4.cpp:9-12 */
float q3x_oracle_decode_e2m1(uint8_t nibble) {
  static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  float m = mag[nibble & 7u];
  return (nibble & 8u) ? -m : m;
}

/* src/quantization/nvfp4.cpp:27-50: bias 7, subnormals mantissa * 2^-9, 0x7f/0xff NaN */
float q3x_oracle_decode_e4m3fn(uint8_t bits) {
  unsigned e = (bits >> 3) & 0xfu, m = bits & 7u;
  float v;
  if (e == 0xfu && m == 7u)
    v = NAN;
  else if (e == 0)
    v = ldexpf((float)m, -9);
  else
    v = ldexpf(1.0f + (float)m / 8.0f, (int)e - 7);
  return copysignf(v, (bits & 0x80u) ? -1.0f : 1.0f);
}

/* Nearest finite E4M3 magnitude code with ties to the even code, after clamping to 448:
 * the same result as the reference's exhaustive nearest search
 * (gemv_reference.cpp:42-57), obtained arithmetically.  The E4M3 grid spacing inside the
 * binade of v is 2^(e-3) (2^-9 below 2^-6), so v / spacing rounded to nearest-even is exact. */
uint8_t q3x_oracle_encode_e4m3fn(float value) {
  if (isnan(value)) return 0x7f;
  uint8_t sign = signbit(value) ? 0x80u : 0;
  float a = fabsf(value);
  if (a > 448.0f) a = 448.0f;
  int e = -126;
  if (a != 0.0f) (void)frexpf(a, &e); /* a = f * 2^e, f in [0.5,1) -> a in [2^(e-1), 2^e) */
  int binade = e - 1;
  if (binade < -6) binade = -6; /* zero and the subnormal range share the 2^-9 grid */
  float spacing = ldexpf(1.0f, binade - 3);
  float steps = nearbyintf(a / spacing); /* default rounding mode: nearest-even; exact divide */
  /* steps in [0,8] for the subnormal range, [8,16] above; 16 carries into the next binade */
  int n = (int)steps;
  unsigned code;
  if (binade == -6 && n < 8)
    code = (unsigned)n;
  else {
    if (n == 16) {
      n = 8;
      binade += 1;
    }
    code = ((unsigned)(binade + 7) << 3) | (unsigned)(n - 8);
  }
  if (code > 0x7eu) code = 0x7eu;
  return (uint8_t)(sign | code);
}

/* Ladder over the midpoints of {0,.5,1,1.5,2,3,4,6}; a value exactly on a midpoint goes to
 * the neighbour whose code is even (0.25->0, 0.75->1.0, 1.25->1.0, 1.75->2.0, 2.5->2.0,
 * 3.5->4.0, 5.0->4.0).  Infinity saturates to 6 with its sign; NaN gives +6 (0x7). */
uint8_t q3x_oracle_encode_e2m1(float value) {
  if (isnan(value)) return 0x7;
  uint8_t sign = signbit(value) ? 0x8u : 0;
  float a = fabsf(value);
  uint8_t m;
  if (a <= 0.25f) m = 0;
  else if (a < 0.75f) m = 1;
  else if (a <= 1.25f) m = 2;
  else if (a < 1.75f) m = 3;
  else if (a <= 2.5f) m = 4;
  else if (a < 3.5f) m = 5;
  else if (a <= 5.0f) m = 6;
  else m = 7;
  return (uint8_t)(sign | m);
}

int q3x_oracle_nvfp4_dequantize(const uint8_t* codes, const uint8_t* scales, float global_scale,
                                size_t rows, size_t cols, float* out) {
  if (cols % 16 != 0) return Q3X_ORACLE_INVALID_COLUMN_COUNT;
  if (!isfinite(global_scale) || global_scale < 0.0f) return Q3X_ORACLE_INVALID_ARGUMENT;
  if (BF16_ROWS_OVERFLOW(rows, cols)) return Q3X_ORACLE_SIZE_OVERFLOW;
  if (rows == 0 || cols == 0) return Q3X_ORACLE_OK;
  if (!codes || !scales || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) {
      uint8_t byte = codes[r * (cols / 2) + c / 2];
      uint8_t nib = (c & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0xf);
      /* product order of nvfp4.cpp:57-58 */
      out[r * cols + c] = q3x_oracle_decode_e2m1(nib) *
                          q3x_oracle_decode_e4m3fn(scales[r * (cols / 16) + c / 16]) * global_scale;
    }
  return Q3X_ORACLE_OK;
}

/* magnitude bits of a finite bf16, else 0: bf16 magnitudes order like their bit patterns */
static uint16_t finite_mag(uint16_t bits) {
  uint16_t m = bits & 0x7fffu;
  return m < 0x7f80u ? m : 0;
}

static size_t group_count(size_t rows, size_t rows_per_scale) {
  if (rows_per_scale == 0) return rows ? 1 : 0;
  return (rows + rows_per_scale - 1) / rows_per_scale;
}

int q3x_oracle_group_amax(const uint16_t* in, size_t rows, size_t cols, size_t rows_per_scale,
                          float* amax_out) {
  if (BF16_ROWS_OVERFLOW(rows, cols)) return Q3X_ORACLE_SIZE_OVERFLOW;
  if (rows == 0 || cols == 0) return Q3X_ORACLE_OK;
  if (!in || !amax_out) return Q3X_ORACLE_INVALID_ARGUMENT;
  size_t per = rows_per_scale ? rows_per_scale : rows;
  size_t groups = group_count(rows, rows_per_scale);
  for (size_t g = 0; g < groups; ++g) {
    size_t r0 = g * per, r1 = r0 + per < rows ? r0 + per : rows;
    uint16_t top = 0;
    for (size_t i = r0 * cols; i < r1 * cols; ++i) {
      uint16_t m = finite_mag(in[i]);
      if (m > top) top = m;
    }
    amax_out[g] = DEC(top);
  }
  return Q3X_ORACLE_OK;
}

static float global_scale_from_amax(float amax) { return amax == 0.0f ? 1.0f : amax / 2688.0f; }

int q3x_oracle_nvfp4_quantize_with_scales(const uint16_t* in, size_t rows, size_t cols,
                                          size_t rows_per_scale, const float* global_scales,
                                          uint8_t* codes, uint8_t* scales) {
  if (cols % 16 != 0) return Q3X_ORACLE_INVALID_COLUMN_COUNT;
  if (BF16_ROWS_OVERFLOW(rows, cols)) return Q3X_ORACLE_SIZE_OVERFLOW;
  if (rows == 0 || cols == 0) return Q3X_ORACLE_OK;
  if (!in || !global_scales || !codes || !scales) return Q3X_ORACLE_INVALID_ARGUMENT;
  size_t per = rows_per_scale ? rows_per_scale : rows;
  for (size_t r = 0; r < rows; ++r) {
    const float global = global_scales[r / per];
    const float k = 1.0f / (global * 6.0f);
    for (size_t b = 0; b < cols / 16; ++b) {
      const uint16_t* x = in + r * cols + b * 16;
      uint16_t top = 0;
      for (int i = 0; i < 16; ++i) {
        uint16_t m = finite_mag(x[i]);
        if (m > top) top = m;
      }
      uint8_t s = top == 0 ? 0 : q3x_oracle_encode_e4m3fn(DEC(top) * k);
      scales[r * (cols / 16) + b] = s;
      float d = q3x_oracle_decode_e4m3fn(s) * global;
      float inv = 0.0f;
      if (d != 0.0f) {
        inv = 1.0f / d;
        if (!(inv <= FLT_MAX)) inv = FLT_MAX;
      }
      for (int i = 0; i < 16; i += 2) {
        uint8_t lo = q3x_oracle_encode_e2m1(DEC(x[i]) * inv);
        uint8_t hi = q3x_oracle_encode_e2m1(DEC(x[i + 1]) * inv);
        codes[r * (cols / 2) + b * 8 + i / 2] = (uint8_t)(lo | (hi << 4));
      }
    }
  }
  return Q3X_ORACLE_OK;
}

int q3x_oracle_nvfp4_quantize(const uint16_t* in, size_t rows, size_t cols, size_t rows_per_scale,
                              uint8_t* codes, uint8_t* scales, float* global_scales) {
  if (cols % 16 != 0) return Q3X_ORACLE_INVALID_COLUMN_COUNT;
  if (BF16_ROWS_OVERFLOW(rows, cols)) return Q3X_ORACLE_SIZE_OVERFLOW;
  if (rows == 0 || cols == 0) return Q3X_ORACLE_OK;
  if (!in || !codes || !scales || !global_scales) return Q3X_ORACLE_INVALID_ARGUMENT;
  int st = q3x_oracle_group_amax(in, rows, cols, rows_per_scale, global_scales);
  if (st) return st;
  size_t groups = group_count(rows, rows_per_scale);
  for (size_t g = 0; g < groups; ++g) global_scales[g] = global_scale_from_amax(global_scales[g]);
  return q3x_oracle_nvfp4_quantize_with_scales(in, rows, cols, rows_per_scale, global_scales,
                                               codes, scales);
}
