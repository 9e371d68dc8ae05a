// Definitions of the mirrored launchers: the reference's own argument limits, then a forward to the
// C ABI, which performs the pointer / overlap / overflow checks and enqueues the sm_100a kernels.
#include "q3x_b200_ops.hpp"

#include "q3x_b200.h"

namespace q3x::runtime {
namespace {

constexpr int kInvalidValue = 1;  // cudaErrorInvalidValue

bool default_gdn(const GdnDimensions& d) noexcept {
  return d.qk_head_count == kGdnQkHeadCount && d.value_head_count == kGdnValueHeadCount &&
         d.head_dimension == kGdnHeadDimension;
}

}  // namespace

int launch_embedding_gather_reference_cuda(const std::uint16_t* table, std::size_t vocab, std::size_t hidden,
                                           std::size_t token_id, std::uint16_t* output, void* stream) noexcept {
  return q3x_b200_embedding_gather_one(table, vocab, hidden, token_id, output, stream);
}

int launch_embedding_gather_prompt_reference_cuda(const std::uint16_t* table, std::size_t vocab, std::size_t hidden,
                                                  const std::uint32_t* token_ids, std::size_t token_count,
                                                  std::uint16_t* output, void* stream) noexcept {
  // the reference rejects an empty prompt and an empty row here (decode_ops.cu:2792-2823)
  if (token_count == 0U || hidden == 0U || vocab == 0U) return kInvalidValue;
  return q3x_b200_embedding_gather(table, vocab, hidden, token_ids, token_count, output, stream);
}

int launch_centered_rms_norm_reference_cuda(const std::uint16_t* input, const std::uint16_t* weight,
                                            std::size_t hidden, float eps, std::uint16_t* output,
                                            void* stream) noexcept {
  return q3x_b200_rms_norm(input, weight, hidden == 0U ? 0U : 1U, hidden, eps, 1, output, stream);
}

int launch_plain_rms_norm_reference_cuda(const std::uint16_t* input, const std::uint16_t* weight, std::size_t hidden,
                                         float eps, std::uint16_t* output, void* stream) noexcept {
  return q3x_b200_rms_norm(input, weight, hidden == 0U ? 0U : 1U, hidden, eps, 0, output, stream);
}

int launch_headwise_centered_rms_norm_reference_cuda(const std::uint16_t* input, const std::uint16_t* weight,
                                                     std::size_t heads, std::size_t dim, float eps,
                                                     std::uint16_t* output, void* stream) noexcept {
  return q3x_b200_rms_norm(input, weight, heads, dim, eps, 1, output, stream);
}

int launch_headwise_plain_rms_norm_reference_cuda(const std::uint16_t* input, const std::uint16_t* weight,
                                                  std::size_t heads, std::size_t dim, float eps,
                                                  std::uint16_t* output, void* stream) noexcept {
  return q3x_b200_rms_norm(input, weight, heads, dim, eps, 0, output, stream);
}

int launch_headwise_plain_rms_norm_silu_gate_reference_cuda(const std::uint16_t* input, const std::uint16_t* weight,
                                                            const std::uint16_t* gate, std::size_t heads,
                                                            std::size_t dim, float eps, std::uint16_t* output,
                                                            void* stream) noexcept {
  return q3x_b200_rms_norm_silu_gate(input, weight, gate, heads, dim, eps, output, stream);
}

int launch_residual_add_reference_cuda(const std::uint16_t* left, const std::uint16_t* right, std::size_t count,
                                       std::uint16_t* output, void* stream) noexcept {
  return q3x_b200_residual_add(left, right, count, output, stream);
}

int launch_residual_add_centered_rms_norm_5120_cuda(const std::uint16_t* left, const std::uint16_t* right,
                                                    const std::uint16_t* weight, float eps,
                                                    std::uint16_t* residual_output, std::uint16_t* normalized_output,
                                                    void* stream) noexcept {
  if (normalized_output == nullptr) return kInvalidValue;  // both boundaries are published (decode_ops.cu:2945-2968)
  return q3x_b200_residual_add_rms_norm(left, right, weight, 1U, kResidualNormHiddenSize, eps, residual_output,
                                        normalized_output, stream);
}

int launch_residual_add_headwise_centered_rms_norm_m32_5120_cuda(const std::uint16_t* left,
                                                                 const std::uint16_t* right,
                                                                 const std::uint16_t* weight, std::size_t tokens,
                                                                 std::size_t hidden, float eps,
                                                                 std::uint16_t* residual_output,
                                                                 std::uint16_t* normalized_output,
                                                                 void* stream) noexcept {
  if (tokens != 32U) return kInvalidValue;  // exact-M32 boundary (decode_ops.cu:1955-1968)
  return launch_residual_add_headwise_centered_rms_norm_prefill_5120_cuda(left, right, weight, tokens, hidden, eps,
                                                                          residual_output, normalized_output, stream);
}

int launch_residual_add_headwise_centered_rms_norm_prefill_5120_cuda(const std::uint16_t* left,
                                                                     const std::uint16_t* right,
                                                                     const std::uint16_t* weight, std::size_t tokens,
                                                                     std::size_t hidden, float eps,
                                                                     std::uint16_t* residual_output,
                                                                     std::uint16_t* normalized_output,
                                                                     void* stream) noexcept {
  if (tokens == 0U || tokens > kResidualNormPrefillMaximumTokens || hidden != kResidualNormHiddenSize ||
      normalized_output == nullptr)
    return kInvalidValue;
  return q3x_b200_residual_add_rms_norm(left, right, weight, tokens, hidden, eps, residual_output, normalized_output,
                                        stream);
}

int launch_fp32_to_bf16_reference_cuda(const float* input, std::size_t count, std::uint16_t* output,
                                       void* stream) noexcept {
  return q3x_b200_fp32_to_bf16(input, count, output, stream);
}

int launch_silu_mul_reference_cuda(const std::uint16_t* gate, const std::uint16_t* up, std::size_t count,
                                   std::uint16_t* output, void* stream) noexcept {
  return q3x_b200_silu_mul(gate, up, count, output, stream);
}

int launch_sigmoid_gate_reference_cuda(const std::uint16_t* value, const std::uint16_t* gate, std::size_t count,
                                       std::uint16_t* output, void* stream) noexcept {
  return q3x_b200_sigmoid_gate(value, gate, count, output, stream);
}

int launch_l2_normalize_heads_reference_cuda(const std::uint16_t* input, std::size_t heads, std::size_t dim, float eps,
                                             std::uint16_t* output, void* stream) noexcept {
  return q3x_b200_l2_normalize_heads(input, heads, dim, eps, 1.0F, output, stream);
}

int launch_partial_neox_rope_256_64_reference_cuda(const std::uint16_t* input, const float* cosines,
                                                   const float* sines, std::size_t heads, std::uint16_t* output,
                                                   void* stream) noexcept {
  return q3x_b200_partial_neox_rope_256_64(input, cosines, sines, heads, output, stream);
}

int launch_qk_partial_neox_rope_tile_24_4_256_64_cuda(std::uint16_t* query, std::uint16_t* key, const float* cosines,
                                                      const float* sines, std::size_t first_position,
                                                      std::size_t tokens, void* stream) noexcept {
  if (tokens == 0U || tokens > kQkRopeTileMaximumTokens) return kInvalidValue;  // decode_ops.cu:3138
  return q3x_b200_qk_partial_neox_rope(query, key, cosines, sines, first_position, tokens, stream);
}

int launch_full_attention_preprocess_24_4_256_64_reference_256_cuda(
    const std::uint16_t* q_gate, std::uint16_t* key, const std::uint16_t* q_weight, const std::uint16_t* k_weight,
    float eps, std::uint16_t* q_out, std::uint16_t* gate_out, const float* cosines, const float* sines,
    std::size_t first_position, std::size_t tokens, void* stream) noexcept {
  if (tokens == 0U || tokens > kFullAttentionPreprocessMaximumTokens) return kInvalidValue;  // decode_ops.cu:3182
  return q3x_b200_full_attention_preprocess(q_gate, key, q_weight, k_weight, eps, q_out, gate_out, cosines, sines,
                                            first_position, tokens, stream);
}

int launch_full_attention_preprocess_24_4_256_64_prompt_wide_p8000_cuda(
    const std::uint16_t* q_gate, std::uint16_t* key, const std::uint16_t* q_weight, const std::uint16_t* k_weight,
    float eps, std::uint16_t* q_out, std::uint16_t* gate_out, const float* cosines, const float* sines,
    std::size_t first_position, std::size_t tokens, void* stream) noexcept {
  // the reference compiles this panel entry only under an admission option and otherwise answers
  // cudaErrorNotSupported (decode_ops.cu:3298-3317); here the same kernel serves any size
  if (!can_launch_full_attention_preprocess_prompt_wide_p8000(first_position, tokens)) return kInvalidValue;
  return q3x_b200_full_attention_preprocess(q_gate, key, q_weight, k_weight, eps, q_out, gate_out, cosines, sines,
                                            first_position, tokens, stream);
}

int launch_full_attention_preprocess_24_4_256_64_cuda(const std::uint16_t* q_gate, std::uint16_t* key,
                                                      const std::uint16_t* q_weight, const std::uint16_t* k_weight,
                                                      float eps, std::uint16_t* q_out, std::uint16_t* gate_out,
                                                      const float* cosines, const float* sines,
                                                      std::size_t first_position, std::size_t tokens,
                                                      void* stream) noexcept {
  return launch_full_attention_preprocess_24_4_256_64_reference_256_cuda(q_gate, key, q_weight, k_weight, eps, q_out,
                                                                         gate_out, cosines, sines, first_position,
                                                                         tokens, stream);
}

int launch_split_interleaved_q_gate_reference_cuda(const std::uint16_t* input, std::size_t heads, std::size_t dim,
                                                   std::uint16_t* q_out, std::uint16_t* gate_out,
                                                   void* stream) noexcept {
  return q3x_b200_split_interleaved_q_gate(input, heads, dim, q_out, gate_out, stream);
}

int launch_causal_conv1d_silu_update_reference_cuda(const std::uint16_t* raw, const std::uint16_t* weight,
                                                    std::uint16_t* history, std::uint16_t* out,
                                                    GdnDimensions dimensions, void* stream) noexcept {
  if (!default_gdn(dimensions)) return kInvalidValue;  // gdn_decode.cu:1901-1907
  return q3x_b200_causal_conv1d_silu(raw, 1U, kGdnQkvChannels, weight, history, out, stream);
}

int launch_causal_conv1d_silu_update_tile_reference_cuda(const std::uint16_t* raw, std::size_t tokens,
                                                         const std::uint16_t* weight, std::uint16_t* history,
                                                         std::uint16_t* out, GdnDimensions dimensions,
                                                         void* stream) noexcept {
  if (!default_gdn(dimensions) || tokens == 0U || tokens > kGdnMaximumTileTokenCount) return kInvalidValue;
  return q3x_b200_causal_conv1d_silu(raw, tokens, kGdnQkvChannels, weight, history, out, stream);
}

namespace gdn_prefill_whole_span_conv_detail {

int launch_causal_conv1d_silu_update_whole_span_exact_cuda(const std::uint16_t* raw, std::size_t tokens,
                                                           const std::uint16_t* weight, std::uint16_t* history,
                                                           std::uint16_t* out, void* stream) noexcept {
  if (tokens == 0U || tokens > kMaximumTokenCount) return kInvalidValue;  // gdn_prefill_whole_span_conv_sm87.cu:537
  return q3x_b200_causal_conv1d_silu(raw, tokens, kGdnQkvChannels, weight, history, out, stream);
}

int launch_causal_conv1d_silu_update_token_parallel_exact_cuda(const std::uint16_t* raw, std::size_t tokens,
                                                               const std::uint16_t* weight, std::uint16_t* history,
                                                               std::uint16_t* out, void* stream) noexcept {
  // this form requires a disjoint output (gdn_prefill_whole_span_conv_sm87.cu:553-566)
  if (tokens == 0U || tokens > kMaximumTokenCount || raw == out) return kInvalidValue;
  return q3x_b200_causal_conv1d_silu(raw, tokens, kGdnQkvChannels, weight, history, out, stream);
}

}  // namespace gdn_prefill_whole_span_conv_detail
}  // namespace q3x::runtime
