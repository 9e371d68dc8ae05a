// ref_shim.cpp -- C entry points over the reference project's own host reference ops, so the
// restatement in q3x_oracle.c can be compared with them bit for bit.
//
// TEST INFRASTRUCTURE ONLY.  This file is compiled together with the reference's unmodified
// sources (src/runtime/reference/{decode_ops,layout_ops,gdn_decode}.cpp,
// src/quantization/nvfp4.cpp, src/kernels/reference/gemv_reference.cpp), taken from where the
// reference checkout lies, into oracle/_ref/libq3x_ref.so (see oracle/Makefile).  Nothing of the
// reference is copied into this repository; when no reference checkout is present the library
// is simply not built and the tests that need it skip.
#include <cstddef>
#include <cstdint>

#include "q3x/kernels/reference_gemv.h"
#include "q3x/quantization/nvfp4.h"
#include "q3x/runtime/decode_ops.h"
#include "q3x/runtime/gdn_decode.h"
#include "q3x/runtime/layout_ops.h"

namespace rt = q3x::runtime;
namespace qz = q3x::quantization;

extern "C" {

int ref_embedding_gather(const std::uint16_t* table, std::size_t vocab, std::size_t hidden,
                         std::size_t token_id, std::uint16_t* out) {
  return static_cast<int>(rt::embedding_gather_reference_cpu(table, vocab, hidden, token_id, out));
}
int ref_centered_rms_norm(const std::uint16_t* in, const std::uint16_t* w, std::size_t n, float eps,
                          std::uint16_t* out) {
  return static_cast<int>(rt::centered_rms_norm_reference_cpu(in, w, n, eps, out));
}
int ref_plain_rms_norm(const std::uint16_t* in, const std::uint16_t* w, std::size_t n, float eps,
                       std::uint16_t* out) {
  return static_cast<int>(rt::plain_rms_norm_reference_cpu(in, w, n, eps, out));
}
int ref_headwise_centered_rms_norm(const std::uint16_t* in, const std::uint16_t* w, std::size_t heads,
                                   std::size_t dim, float eps, std::uint16_t* out) {
  return static_cast<int>(rt::headwise_centered_rms_norm_reference_cpu(in, w, heads, dim, eps, out));
}
int ref_headwise_plain_rms_norm(const std::uint16_t* in, const std::uint16_t* w, std::size_t heads,
                                std::size_t dim, float eps, std::uint16_t* out) {
  return static_cast<int>(rt::headwise_plain_rms_norm_reference_cpu(in, w, heads, dim, eps, out));
}
int ref_headwise_plain_rms_norm_silu_gate(const std::uint16_t* in, const std::uint16_t* w,
                                          const std::uint16_t* gate, std::size_t heads, std::size_t dim,
                                          float eps, std::uint16_t* out) {
  return static_cast<int>(
      rt::headwise_plain_rms_norm_silu_gate_reference_cpu(in, w, gate, heads, dim, eps, out));
}
int ref_residual_add(const std::uint16_t* l, const std::uint16_t* r, std::size_t n, std::uint16_t* out) {
  return static_cast<int>(rt::residual_add_reference_cpu(l, r, n, out));
}
int ref_fp32_to_bf16(const float* in, std::size_t n, std::uint16_t* out) {
  return static_cast<int>(rt::fp32_to_bf16_reference_cpu(in, n, out));
}
int ref_silu_mul(const std::uint16_t* g, const std::uint16_t* u, std::size_t n, std::uint16_t* out) {
  return static_cast<int>(rt::silu_mul_reference_cpu(g, u, n, out));
}
int ref_sigmoid_gate(const std::uint16_t* v, const std::uint16_t* g, std::size_t n, std::uint16_t* out) {
  return static_cast<int>(rt::sigmoid_gate_reference_cpu(v, g, n, out));
}
int ref_l2_normalize_heads(const std::uint16_t* in, std::size_t heads, std::size_t dim, float eps,
                           std::uint16_t* out) {
  return static_cast<int>(rt::l2_normalize_heads_reference_cpu(in, heads, dim, eps, out));
}
int ref_partial_neox_rope_256_64(const std::uint16_t* in, const float* c, const float* s,
                                 std::size_t heads, std::uint16_t* out) {
  return static_cast<int>(rt::partial_neox_rope_256_64_reference_cpu(in, c, s, heads, out));
}
int ref_split_interleaved_q_gate(const std::uint16_t* in, std::size_t heads, std::size_t dim,
                                 std::uint16_t* q, std::uint16_t* gate) {
  return static_cast<int>(rt::split_interleaved_q_gate_reference_cpu(in, heads, dim, q, gate));
}
int ref_causal_conv1d_silu_update(const std::uint16_t* raw, const std::uint16_t* w, std::uint16_t* history,
                                  std::uint16_t* out) {
  return static_cast<int>(rt::causal_conv1d_silu_update_reference_cpu(raw, w, history, out));
}
float ref_decode_e2m1(std::uint8_t nibble) { return qz::decode_e2m1(nibble); }
float ref_decode_e4m3fn(std::uint8_t bits) { return qz::decode_e4m3fn(bits); }
std::uint8_t ref_unpack_e2m1_nibble(std::uint8_t packed, int high) {
  return qz::unpack_e2m1_nibble(packed, high != 0);
}
int ref_dequantize_nvfp4(const std::uint8_t* codes, const std::uint8_t* scales, float global,
                         std::size_t rows, std::size_t cols, float* out) {
  return static_cast<int>(qz::dequantize_nvfp4_reference(codes, scales, global, rows, cols, out));
}
// The reference's E4M3 activation quantiser is file-local; its value is observable through the
// static W8A8 GEMV with one row, one column and a weight of 1.0 (code 0x38):
// output = decode(quantise(x / input_scale)) * weight_scale * input_scale.
int ref_e4m3_quantised_value(std::uint16_t activation_bf16, float input_scale, float* out) {
  const std::uint8_t one = 0x38U;
  return static_cast<int>(q3x::kernels::fp8_static_gemv_reference_cpu(&one, 1.0F, input_scale,
                                                                       &activation_bf16, 1U, 1U, out));
}


// ---- the GDN recurrence, GQA attention and softmax host ops ---------------------------------------
int ref_gated_delta_net_update(const std::uint16_t* conv_qkv, const std::uint16_t* a, const std::uint16_t* b,
                               const std::uint16_t* A_log, const std::uint16_t* dt_bias,
                               const std::uint16_t* state_in, std::uint16_t* state_out, float l2_eps,
                               std::uint16_t* out) {
  return static_cast<int>(
      rt::gated_delta_net_update_reference_cpu(conv_qkv, a, b, A_log, dt_bias, state_in, state_out, l2_eps, out));
}
int ref_softmax(const float* in, std::size_t rows, std::size_t cols, float* out) {
  return static_cast<int>(rt::softmax_reference_cpu(in, rows, cols, out));
}
int ref_gqa_attention(const std::uint16_t* q, const std::uint16_t* k_cache, const std::uint16_t* v_cache,
                      std::size_t q_heads, std::size_t kv_heads, std::size_t length, std::size_t dim, float scale,
                      float* scratch, std::size_t scratch_elements, std::uint16_t* out) {
  return static_cast<int>(rt::gqa_attention_reference_cpu(q, k_cache, v_cache, q_heads, kv_heads, length, dim, scale,
                                                          scratch, scratch_elements, out));
}

int ref_bf16_gemv(const std::uint16_t* w, const std::uint16_t* x, std::size_t rows, std::size_t cols, float* out) {
  return static_cast<int>(q3x::kernels::bf16_gemv_reference_cpu(w, x, rows, cols, out));
}
int ref_nvfp4_gemv(const std::uint8_t* packed, const std::uint8_t* scales, float scale_2, const std::uint16_t* x,
                   std::size_t rows, std::size_t cols, float* out) {
  return static_cast<int>(q3x::kernels::nvfp4_gemv_reference_cpu(packed, scales, scale_2, x, rows, cols, out));
}

// ---- per-token host ops applied to a run of token rows --------------------------------------------
// The reference's host ops for the embedding, the conv, the q|gate split and the rotation take ONE token;
// its runner loops over tokens around them.  These wrappers are that loop, in C++, so that a timing of
// the host path spends its time in the reference's functions and not in the caller's per-token loop.
int ref_embedding_gather_rows(const std::uint16_t* table, std::size_t vocab, std::size_t hidden,
                              const std::uint32_t* ids, std::size_t tokens, std::uint16_t* out) {
  for (std::size_t t = 0; t < tokens; ++t) {
    const int st = static_cast<int>(rt::embedding_gather_reference_cpu(table, vocab, hidden, ids[t], out + t * hidden));
    if (st != 0) return st;
  }
  return 0;
}
int ref_causal_conv1d_silu_update_rows(const std::uint16_t* raw, std::size_t tokens, const std::uint16_t* w,
                                       std::uint16_t* history, std::uint16_t* out) {
  for (std::size_t t = 0; t < tokens; ++t) {
    const int st = static_cast<int>(rt::causal_conv1d_silu_update_reference_cpu(
        raw + t * rt::kGdnQkvChannels, w, history, out + t * rt::kGdnQkvChannels));
    if (st != 0) return st;
  }
  return 0;
}
// split + centred q/k head norm + partial RoPE of `tokens` rows starting at `first_position`: the
// call sequence of the full-attention pre-processing, token by token.
int ref_full_attention_preprocess_rows(const std::uint16_t* q_gate, std::uint16_t* key, const std::uint16_t* q_w,
                                       const std::uint16_t* k_w, float eps, std::uint16_t* q_out,
                                       std::uint16_t* gate_out, const float* cosines, const float* sines,
                                       std::size_t first_position, std::size_t tokens) {
  constexpr std::size_t Q = 24U, KV = 4U, D = 256U;
  for (std::size_t t = 0; t < tokens; ++t) {
    std::uint16_t* q = q_out + t * Q * D;
    std::uint16_t* k = key + t * KV * D;
    int st = static_cast<int>(rt::split_interleaved_q_gate_reference_cpu(q_gate + t * 2U * Q * D, Q, D, q,
                                                                         gate_out + t * Q * D));
    if (st == 0) st = static_cast<int>(rt::headwise_centered_rms_norm_reference_cpu(q, q_w, Q, D, eps, q));
    if (st == 0) st = static_cast<int>(rt::headwise_centered_rms_norm_reference_cpu(k, k_w, KV, D, eps, k));
    const float* c = cosines + (first_position + t) * 32U;
    const float* s = sines + (first_position + t) * 32U;
    if (st == 0) st = static_cast<int>(rt::partial_neox_rope_256_64_reference_cpu(q, c, s, Q, q));
    if (st == 0) st = static_cast<int>(rt::partial_neox_rope_256_64_reference_cpu(k, c, s, KV, k));
    if (st != 0) return st;
  }
  return 0;
}

}  // extern "C"
