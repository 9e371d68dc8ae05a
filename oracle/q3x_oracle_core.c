/*
 * q3x_oracle_core.c -- CPU restatement of the reference host ops that sit BETWEEN the fused
 * elementwise / normalisation operators: the gated-delta-net recurrence step, softmax, GQA
 * attention (+ the sigmoid output gate), greedy argmax and the batch-one GEMVs.
 *
 * TEST INFRASTRUCTURE ONLY, like q3x_oracle.c: the checker for the CUDA path, never part of it.
 * Built into the same libq3x_oracle.so with -ffp-contract=off; every sum is the reference's own
 * left-to-right FP32 sum (std::fma where the reference calls std::fma), so results are bit-identical
 * to the reference's sources compiled with an ISO-conforming compiler, which the tests check against
 * oracle/_ref.
 */
#include <math.h>
#include <string.h>

#include "q3x_oracle.h"

#define DEC q3x_oracle_decode_bf16
#define ENC q3x_oracle_encode_bf16

enum { QK_HEADS = 16, V_HEADS = 48, HEAD = 128, Q_OFF = 0, K_OFF = 2048, V_OFF = 4096, CHANNELS = 10240 };

/* src/runtime/reference/gdn_decode.cpp:62-73 */
static float stable_softplus(float v) { return v > 20.0f ? v : log1pf(expf(v)); }
static float stable_sigmoid(float v) {
  if (v >= 0.0f) return 1.0f / (1.0f + expf(-v));
  const float e = expf(v);
  return e / (1.0f + e);
}

/* One recurrence step: gated_delta_net_update_reference_cpu,
 * src/runtime/reference/gdn_decode.cpp:186-293.  state [48,128(v),128(k)] bf16, in place allowed. */
static void gdn_step(const uint16_t* conv_qkv, const uint16_t* a, const uint16_t* b, const uint16_t* A_log,
                     const uint16_t* dt_bias, const uint16_t* state_in, uint16_t* state_out, float l2_eps,
                     uint16_t* out) {
  const float inv_sqrt_dim = 1.0f / sqrtf((float)HEAD);
  float qn[HEAD], kn[HEAD];
  for (size_t h = 0; h < V_HEADS; ++h) {
    const size_t qk = h / 3;
    const uint16_t* q = conv_qkv + Q_OFF + qk * HEAD;
    const uint16_t* k = conv_qkv + K_OFF + qk * HEAD;
    float qs = 0.0f, ks = 0.0f;
    for (size_t d = 0; d < HEAD; ++d) {
      const float qv = DEC(q[d]), kv = DEC(k[d]);
      qs = fmaf(qv, qv, qs);
      ks = fmaf(kv, kv, ks);
    }
    const float q_scale = 1.0f / sqrtf(qs + l2_eps) * inv_sqrt_dim;
    const float k_scale = 1.0f / sqrtf(ks + l2_eps);
    for (size_t d = 0; d < HEAD; ++d) {
      qn[d] = DEC(q[d]) * q_scale;
      kn[d] = DEC(k[d]) * k_scale;
    }
    const float gate_in = DEC(a[h]) + DEC(dt_bias[h]);
    const float g = -expf(DEC(A_log[h])) * stable_softplus(gate_in);
    const float alpha = expf(g);
    const float beta = stable_sigmoid(DEC(b[h]));
    for (size_t v = 0; v < HEAD; ++v) {
      const size_t row = (h * HEAD + v) * HEAD;
      float pred = 0.0f;
      for (size_t d = 0; d < HEAD; ++d) pred = fmaf(alpha * DEC(state_in[row + d]), kn[d], pred);
      const float delta = (DEC(conv_qkv[V_OFF + h * HEAD + v]) - pred) * beta;
      float result = 0.0f;
      for (size_t d = 0; d < HEAD; ++d) {
        const float updated = fmaf(delta, kn[d], alpha * DEC(state_in[row + d]));
        state_out[row + d] = ENC(updated);
        result = fmaf(updated, qn[d], result);
      }
      out[h * HEAD + v] = ENC(result);
    }
  }
}

/* Token-sequential form (the tile launchers, include/q3x/runtime/gdn_decode.h:95-110): every step
 * reads the bf16 state the previous step persisted; its output uses that step's FP32 state. */
int q3x_oracle_gated_delta_net_update(const uint16_t* conv_qkv, size_t tokens, const uint16_t* a,
                                      const uint16_t* b, const uint16_t* A_log, const uint16_t* dt_bias,
                                      const uint16_t* state_in, uint16_t* state_out, float l2_eps,
                                      uint16_t* out) {
  if (!(isfinite(l2_eps) && l2_eps > 0.0f)) return Q3X_ORACLE_INVALID_ARGUMENT;
  if (tokens == 0) return Q3X_ORACLE_OK;
  if (!conv_qkv || !a || !b || !A_log || !dt_bias || !state_in || !state_out || !out)
    return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t t = 0; t < tokens; ++t)
    gdn_step(conv_qkv + t * CHANNELS, a + t * V_HEADS, b + t * V_HEADS, A_log, dt_bias,
             t == 0 ? state_in : state_out, state_out, l2_eps, out + t * V_HEADS * HEAD);
  return Q3X_ORACLE_OK;
}

/* softmax_reference_cpu, src/runtime/reference/decode_ops.cpp:413-443 */
int q3x_oracle_softmax(const float* in, size_t rows, size_t cols, float* out) {
  if (rows == 0 || cols == 0) return Q3X_ORACLE_OK;
  if (!in || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t r = 0; r < rows; ++r) {
    const float* x = in + r * cols;
    float* y = out + r * cols;
    float m = -INFINITY;
    for (size_t c = 0; c < cols; ++c) m = x[c] > m ? x[c] : m; /* std::max(maximum, x): keeps maximum on NaN */
    float den = 0.0f;
    for (size_t c = 0; c < cols; ++c) den += expf(x[c] - m);
    for (size_t c = 0; c < cols; ++c) y[c] = expf(x[c] - m) / den;
  }
  return Q3X_ORACLE_OK;
}

/* gqa_attention_reference_cpu, src/runtime/reference/decode_ops.cpp:445-508: one query token against
 * `length` cached positions; caches [position, kv_heads, dim]; scratch [q_heads, length] receives the
 * probabilities. */
int q3x_oracle_gqa_attention(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, size_t q_heads,
                             size_t kv_heads, size_t length, size_t dim, float scale, float* scratch,
                             uint16_t* out) {
  if (!q || !k_cache || !v_cache || !scratch || !out || kv_heads == 0 || q_heads % kv_heads != 0 || length == 0 ||
      dim == 0 || !isfinite(scale))
    return Q3X_ORACLE_INVALID_ARGUMENT;
  const size_t per_kv = q_heads / kv_heads;
  for (size_t h = 0; h < q_heads; ++h) {
    const size_t kv = h / per_kv;
    for (size_t p = 0; p < length; ++p) {
      const uint16_t* k = k_cache + (p * kv_heads + kv) * dim;
      float s = 0.0f;
      for (size_t d = 0; d < dim; ++d) s += DEC(q[h * dim + d]) * DEC(k[d]);
      scratch[h * length + p] = s * scale;
    }
  }
  q3x_oracle_softmax(scratch, q_heads, length, scratch);
  for (size_t h = 0; h < q_heads; ++h) {
    const size_t kv = h / per_kv;
    for (size_t d = 0; d < dim; ++d) {
      float v = 0.0f;
      for (size_t p = 0; p < length; ++p) v += scratch[h * length + p] * DEC(v_cache[(p * kv_heads + kv) * dim + d]);
      out[h * dim + d] = ENC(v);
    }
  }
  return Q3X_ORACLE_OK;
}

/* Attention followed by the sigmoid output gate with the bf16 boundary between them kept
 * (launch_gqa_attention_sigmoid_gate_24_4_256_cuda, include/q3x/runtime/decode_ops.h:384-395). */
int q3x_oracle_gqa_attention_sigmoid_gate(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache,
                                          size_t q_heads, size_t kv_heads, size_t length, size_t dim, float scale,
                                          float* scratch, const uint16_t* gate, uint16_t* out) {
  const int st = q3x_oracle_gqa_attention(q, k_cache, v_cache, q_heads, kv_heads, length, dim, scale, scratch, out);
  if (st != Q3X_ORACLE_OK) return st;
  return q3x_oracle_sigmoid_gate(out, gate, q_heads * dim, out);
}

/* Greedy argmax over bf16 logits, the rule of bf16_greedy_argmax_kernel
 * (src/kernels/reference/decode_ops.cu:246-345): non-finite inputs are skipped and flagged; among the
 * finite ones the largest FP32 value wins and equal maxima (signed zeros included) keep the smallest
 * index; no finite input at all gives index 0xffffffff and value bits 0. */
int q3x_oracle_bf16_greedy_argmax(const uint16_t* in, size_t count, uint32_t* index, uint16_t* value_bits,
                                  uint16_t* has_nonfinite) {
  if (count && !in) return Q3X_ORACLE_INVALID_ARGUMENT;
  uint32_t best = 0xffffffffu;
  uint16_t bits = 0, bad = 0;
  float top = -INFINITY;
  for (size_t i = 0; i < count; ++i) {
    if ((in[i] & 0x7f80u) == 0x7f80u) {
      bad = 1;
      continue;
    }
    const float v = DEC(in[i]);
    if (best == 0xffffffffu || v > top) {
      best = (uint32_t)i;
      bits = in[i];
      top = v;
    }
  }
  *index = best;
  *value_bits = bits;
  *has_nonfinite = bad;
  return Q3X_ORACLE_OK;
}

/* Batch-one GEMVs, src/kernels/reference/gemv_reference.cpp: bf16 weights (:84-110) and the canonical
 * NVFP4 layout (:179-225: packed [rows, cols/2] even k in the low nibble, E4M3 block scales
 * [rows, cols/16], value = E2M1 * E4M3 * weight_scale_2), FP32 left-to-right accumulation. */
int q3x_oracle_bf16_gemv(const uint16_t* w, const uint16_t* x, size_t rows, size_t cols, float* out) {
  if (rows == 0 || cols == 0) return Q3X_ORACLE_OK;
  if (!w || !x || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t r = 0; r < rows; ++r) {
    float s = 0.0f;
    for (size_t c = 0; c < cols; ++c) s += DEC(w[r * cols + c]) * DEC(x[c]);
    out[r] = s;
  }
  return Q3X_ORACLE_OK;
}

int q3x_oracle_nvfp4_gemv(const uint8_t* packed, const uint8_t* block_scales, float weight_scale_2,
                          const uint16_t* x, size_t rows, size_t cols, float* out) {
  if (cols % 16 != 0) return Q3X_ORACLE_INVALID_COLUMN_COUNT;
  if (!(isfinite(weight_scale_2) && weight_scale_2 >= 0.0f)) return Q3X_ORACLE_INVALID_ARGUMENT;
  if (rows == 0 || cols == 0) return Q3X_ORACLE_OK;
  if (!packed || !block_scales || !x || !out) return Q3X_ORACLE_INVALID_ARGUMENT;
  for (size_t r = 0; r < rows; ++r) {
    float s = 0.0f;
    for (size_t c = 0; c < cols; ++c) {
      const uint8_t byte = packed[r * (cols / 2) + c / 2];
      const uint8_t nibble = (c & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0xf);
      /* dequantize_nvfp4_value, src/quantization/nvfp4.cpp:52-59: (e2m1 * e4m3) * scale_2 */
      const float wv = q3x_oracle_decode_e2m1(nibble) * q3x_oracle_decode_e4m3fn(block_scales[r * (cols / 16) + c / 16]) *
                       weight_scale_2;
      s += wv * DEC(x[c]);
    }
    out[r] = s;
  }
  return Q3X_ORACLE_OK;
}
