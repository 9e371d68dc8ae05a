// Definitions of the mirrored launchers: the reference's own argument limits, then a forward to the
// C ABI, which performs the pointer / overlap / overflow checks and enqueues the sm_100a kernels.
#include "q3x_b200_ops.hpp"

#include <cmath>

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

// ---- decode attention, softmax, argmax ------------------------------------------------------------------

int launch_softmax_reference_cuda(const float* input, std::size_t rows, std::size_t columns, float* output,
                                  void* stream) noexcept {
  return q3x_b200_softmax(input, rows, columns, output, stream);
}

std::size_t gqa_attention_splitkv_sigmoid_gate_24_4_256_workspace_elements(std::size_t sequence_length) noexcept {
  if (sequence_length <= kFusedGqaMaximumSequenceLength || sequence_length > kDecodeGqaSplitKvMaximumSequenceLength)
    return 0U;  // outside the entry point's range there is nothing to size
  return q3x_b200_gqa_decode_workspace_floats(sequence_length);
}

int launch_gqa_attention_splitkv_sigmoid_gate_24_4_256_cuda(const std::uint16_t* query, const std::uint16_t* key_cache,
                                                            const std::uint16_t* value_cache,
                                                            std::size_t sequence_length, float attention_scale,
                                                            float* workspace, std::size_t workspace_elements,
                                                            const std::uint16_t* gate, std::uint16_t* output,
                                                            void* stream) noexcept {
  // the reference admits (64, 4096] here and requires the gate (decode_ops.h:405-410)
  if (sequence_length <= kFusedGqaMaximumSequenceLength || sequence_length > kDecodeGqaSplitKvMaximumSequenceLength ||
      gate == nullptr)
    return kInvalidValue;
  return q3x_b200_gqa_attention_decode_sigmoid_gate(query, key_cache, value_cache, sequence_length, attention_scale,
                                                    workspace, workspace_elements, gate, output, stream);
}

namespace {
// the tile forms admit 2..512 tokens, the panel form up to its own maximum (decode_ops.h:452-500); the gate is required
int bulk_causal(const std::uint16_t* q, const std::uint16_t* k, const std::uint16_t* v, const std::uint16_t* gate,
                std::size_t first_position, std::size_t token_count, std::size_t maximum_tokens, std::uint16_t* out,
                void* stream) noexcept {
  if (token_count < 2U || token_count > maximum_tokens || first_position > kBulkCausalGqaMaximumSequenceLength - token_count ||
      gate == nullptr)
    return kInvalidValue;
  return q3x_b200_gqa_attention_prefill_sigmoid_gate(q, k, v, gate, first_position, token_count, 0.0625F, out, stream);
}
}  // namespace

int launch_bulk_causal_gqa_sigmoid_gate_24_4_256_cuda(const std::uint16_t* query_tile, const std::uint16_t* key_cache,
                                                      const std::uint16_t* value_cache, const std::uint16_t* gate_tile,
                                                      std::size_t first_position, std::size_t token_count,
                                                      std::uint16_t* output_tile, void* stream) noexcept {
  return bulk_causal(query_tile, key_cache, value_cache, gate_tile, first_position, token_count, 512U, output_tile, stream);
}

int launch_bulk_causal_gqa_sigmoid_gate_24_4_256_fixed_cuda(const std::uint16_t* query_tile,
                                                            const std::uint16_t* key_cache,
                                                            const std::uint16_t* value_cache,
                                                            const std::uint16_t* gate_tile, std::size_t first_position,
                                                            std::size_t token_count, std::uint16_t* output_tile,
                                                            void* stream) noexcept {
  return bulk_causal(query_tile, key_cache, value_cache, gate_tile, first_position, token_count, 512U, output_tile, stream);
}

int launch_bulk_causal_gqa_sigmoid_gate_24_4_256_group_q64_panel_fixed_cuda(
    const std::uint16_t* query_panel, const std::uint16_t* key_cache, const std::uint16_t* value_cache,
    const std::uint16_t* gate_panel, std::size_t first_position, std::size_t token_count, std::uint16_t* output_panel,
    void* stream) noexcept {
  if (first_position >= (static_cast<std::size_t>(1) << 18)) return kInvalidValue;  // decode_ops.h:493-497
  return bulk_causal(query_panel, key_cache, value_cache, gate_panel, first_position, token_count,
                     kBulkCausalGqaGroupQ64PanelMaximumTokens, output_panel, stream);
}

int launch_bf16_greedy_argmax_cuda(const std::uint16_t* input, std::size_t element_count,
                                   Bf16GreedyArgmaxResult* result_workspace, void* stream) noexcept {
  return q3x_b200_bf16_greedy_argmax(input, element_count, result_workspace, stream);
}

// ---- gated-delta-net recurrence ----------------------------------------------------------------------------

bool supports_gated_delta_net_update_plain_rms_norm_silu_gate_fusion(std::size_t token_count, GdnDimensions dimensions,
                                                                     std::size_t norm_head_count,
                                                                     std::size_t norm_head_dimension) noexcept {
  return token_count == 1U && default_gdn(dimensions) && norm_head_count == kGdnValueHeadCount &&
         norm_head_dimension == kGdnHeadDimension;
}

int launch_gated_delta_net_update_reference_cuda(const std::uint16_t* conv_qkv, const std::uint16_t* a,
                                                 const std::uint16_t* b, const std::uint16_t* A_log,
                                                 const std::uint16_t* dt_bias, const std::uint16_t* state_input,
                                                 std::uint16_t* state_output, float l2_epsilon, std::uint16_t* output,
                                                 GdnDimensions dimensions, void* stream) noexcept {
  if (!default_gdn(dimensions)) return kInvalidValue;
  return q3x_b200_gated_delta_net_update(conv_qkv, 1U, a, b, A_log, dt_bias, state_input, state_output, l2_epsilon,
                                         output, stream);
}

int launch_gated_delta_net_update_tile_reference_cuda(const std::uint16_t* conv_qkv, std::size_t token_count,
                                                      const std::uint16_t* a, const std::uint16_t* b,
                                                      const std::uint16_t* A_log, const std::uint16_t* dt_bias,
                                                      const std::uint16_t* state_input, std::uint16_t* state_output,
                                                      float l2_epsilon, std::uint16_t* output, GdnDimensions dimensions,
                                                      void* stream) noexcept {
  if (!default_gdn(dimensions) || token_count == 0U || token_count > kGdnMaximumTileTokenCount) return kInvalidValue;
  return q3x_b200_gated_delta_net_update(conv_qkv, token_count, a, b, A_log, dt_bias, state_input, state_output,
                                         l2_epsilon, output, stream);
}

int launch_gated_delta_net_update_warp_parallel_cuda(const std::uint16_t* conv_qkv, const std::uint16_t* a,
                                                     const std::uint16_t* b, const std::uint16_t* A_log,
                                                     const std::uint16_t* dt_bias, const std::uint16_t* state_input,
                                                     std::uint16_t* state_output, float l2_epsilon,
                                                     std::uint16_t* output, GdnDimensions dimensions,
                                                     void* stream) noexcept {
  return launch_gated_delta_net_update_reference_cuda(conv_qkv, a, b, A_log, dt_bias, state_input, state_output,
                                                      l2_epsilon, output, dimensions, stream);
}

int launch_gated_delta_net_update_tile_warp_parallel_cuda(const std::uint16_t* conv_qkv, std::size_t token_count,
                                                          const std::uint16_t* a, const std::uint16_t* b,
                                                          const std::uint16_t* A_log, const std::uint16_t* dt_bias,
                                                          const std::uint16_t* state_input,
                                                          std::uint16_t* state_output, float l2_epsilon,
                                                          std::uint16_t* output, GdnDimensions dimensions,
                                                          void* stream) noexcept {
  return launch_gated_delta_net_update_tile_reference_cuda(conv_qkv, token_count, a, b, A_log, dt_bias, state_input,
                                                           state_output, l2_epsilon, output, dimensions, stream);
}

int gdn_decode_detail::launch_gated_delta_net_update_plain_rms_norm_silu_gate_exact_cuda(
    const std::uint16_t* conv_qkv, const std::uint16_t* a, const std::uint16_t* b, const std::uint16_t* A_log,
    const std::uint16_t* dt_bias, const std::uint16_t* state_input, std::uint16_t* state_output, float l2_epsilon,
    const std::uint16_t* norm_weight, const std::uint16_t* silu_gate, float norm_epsilon, std::uint16_t* output,
    void* stream) noexcept {
  return q3x_b200_gated_delta_net_update_rms_norm_silu_gate(conv_qkv, 1U, a, b, A_log, dt_bias, state_input,
                                                            state_output, l2_epsilon, norm_weight, silu_gate,
                                                            norm_epsilon, output, stream);
}

std::size_t gdn_prefill_chunk64_native_detail::workspace_bytes() noexcept {
  return q3x_b200_gated_delta_net_chunked_workspace_bytes(kMaximumTokenCount);
}

int gdn_prefill_chunk64_native_detail::launch(void* workspace, std::size_t workspace_capacity_bytes,
                                              const std::uint16_t* conv_qkv, std::size_t token_count,
                                              const std::uint16_t* a, const std::uint16_t* b, const std::uint16_t* A_log,
                                              const std::uint16_t* dt_bias, const std::uint16_t* state_input,
                                              std::uint16_t* state_output, float l2_epsilon,
                                              const std::uint16_t* norm_weight, const std::uint16_t* silu_gate,
                                              float norm_epsilon, std::uint16_t* output, void* stream) noexcept {
  // the reference's admission: 1 to 512 tokens, every pointer present, both epsilons finite and positive, the whole
  // workspace whatever the token count; all before the first enqueue
  if (token_count == 0U || token_count > kMaximumTokenCount || workspace == nullptr ||
      workspace_capacity_bytes < workspace_bytes() || norm_weight == nullptr || silu_gate == nullptr ||
      !std::isfinite(norm_epsilon) || norm_epsilon <= 0.0F)
    return kInvalidValue;
  if (const int status = q3x_b200_gated_delta_net_update_chunked(conv_qkv, token_count, a, b, A_log, dt_bias, state_input,
                                                                 state_output, l2_epsilon, output, workspace,
                                                                 workspace_capacity_bytes, stream);
      status != 0)
    return status;
  return q3x_b200_rms_norm_silu_gate(output, norm_weight, silu_gate, token_count * 48U, 128U, norm_epsilon, output, stream);
}

int gdn_prefill_chunk64_native_detail::launch_fixed_production(
    void* workspace, std::size_t workspace_capacity_bytes, const std::uint16_t* conv_qkv, std::size_t token_count,
    const std::uint16_t* a, const std::uint16_t* b, const std::uint16_t* A_log, const std::uint16_t* dt_bias,
    const std::uint16_t* state_input, std::uint16_t* state_output, float l2_epsilon, const std::uint16_t* norm_weight,
    const std::uint16_t* silu_gate, float norm_epsilon, std::uint16_t* output, void* stream) noexcept {
  // one tactic here, so the sealed entry is the same call
  return launch(workspace, workspace_capacity_bytes, conv_qkv, token_count, a, b, A_log, dt_bias, state_input,
                state_output, l2_epsilon, norm_weight, silu_gate, norm_epsilon, output, stream);
}

int launch_gated_delta_net_update_plain_rms_norm_silu_gate_cuda(
    const std::uint16_t* conv_qkv, const std::uint16_t* a, const std::uint16_t* b, const std::uint16_t* A_log,
    const std::uint16_t* dt_bias, const std::uint16_t* state_input, std::uint16_t* state_output, float l2_epsilon,
    const std::uint16_t* norm_weight, const std::uint16_t* silu_gate, std::size_t norm_head_count,
    std::size_t norm_head_dimension, float norm_epsilon, std::uint16_t* output, GdnDimensions dimensions,
    void* stream) noexcept {
  if (!default_gdn(dimensions) || norm_head_count == 0U || norm_head_dimension == 0U ||
      norm_head_count > kGdnValueHeadCount * kGdnHeadDimension ||
      norm_head_count * norm_head_dimension != kGdnValueHeadCount * kGdnHeadDimension)
    return kInvalidValue;
  if (supports_gated_delta_net_update_plain_rms_norm_silu_gate_fusion(1U, dimensions, norm_head_count,
                                                                      norm_head_dimension))
    return q3x_b200_gated_delta_net_update_rms_norm_silu_gate(conv_qkv, 1U, a, b, A_log, dt_bias, state_input,
                                                              state_output, l2_epsilon, norm_weight, silu_gate,
                                                              norm_epsilon, output, stream);
  // any other norm partition of the 6144 outputs: the recurrence, then the gated norm in place (gdn_decode.h:171-178)
  const int st = q3x_b200_gated_delta_net_update(conv_qkv, 1U, a, b, A_log, dt_bias, state_input, state_output,
                                                 l2_epsilon, output, stream);
  if (st != 0) return st;
  return q3x_b200_rms_norm_silu_gate(output, norm_weight, silu_gate, norm_head_count, norm_head_dimension, norm_epsilon,
                                     output, stream);
}

namespace gdn_prefill_whole_span_conv_detail {

int launch_causal_conv1d_silu_update_token_parallel_compact_qk_exact_cuda(
    const std::uint16_t* raw, std::size_t tokens, const std::uint16_t* weight, std::uint16_t* history,
    std::uint16_t* out, float l2_epsilon, std::uint16_t* compact_q, std::uint16_t* compact_k, void* stream) noexcept {
  if (tokens == 0U || tokens > kMaximumTokenCount || raw == out) return kInvalidValue;
  // q carries the extra 1 / sqrt(128) in this layout (gdn_prefill_whole_span_conv_sm87.cu:355-357)
  return q3x_b200_causal_conv1d_silu_compact_qk(raw, tokens, weight, history, out, l2_epsilon, 0.08838834764831845F,
                                                compact_q, compact_k, stream);
}

int launch_causal_conv1d_silu_update_prompt_wide_p40_compact_qk_exact_cuda(
    const std::uint16_t* raw, std::size_t tokens, const std::uint16_t* weight, std::uint16_t* history,
    std::uint16_t* out, float l2_epsilon, std::uint16_t* compact_q, std::uint16_t* compact_k, void* stream) noexcept {
  // admits exactly the prompt-wide length (gdn_prefill_whole_span_conv_sm87.cu:612-619); here it is one launch of
  // the same kernel as every other length
  if (tokens != kPromptWideP40TokenCount || raw == out) return kInvalidValue;
  return q3x_b200_causal_conv1d_silu_compact_qk(raw, tokens, weight, history, out, l2_epsilon, 0.08838834764831845F,
                                                compact_q, compact_k, stream);
}

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

namespace q3x::kernels {

int launch_bf16_gemv_reference_cuda(const std::uint16_t* weights, const std::uint16_t* activation, std::size_t rows,
                                    std::size_t columns, float* output, void* stream) noexcept {
  if (rows != 0U && columns != 0U && output == nullptr) return 1;
  return q3x_b200_bf16_gemv(weights, activation, rows, columns, output, nullptr, stream);
}
int launch_bf16_gemv_bf16_cuda(const std::uint16_t* weights, const std::uint16_t* activation, std::size_t rows,
                               std::size_t columns, std::uint16_t* output, void* stream) noexcept {
  if (rows != 0U && columns != 0U && output == nullptr) return 1;
  return q3x_b200_bf16_gemv(weights, activation, rows, columns, nullptr, output, stream);
}
int launch_fp8_gemv_reference_cuda(const std::uint8_t* weights, float weight_scale, const std::uint16_t* activation,
                                   std::size_t rows, std::size_t columns, float* output, void* stream) noexcept {
  if (rows != 0U && columns != 0U && output == nullptr) return 1;
  return q3x_b200_fp8_gemv(weights, weight_scale, activation, rows, columns, output, nullptr, stream);
}
int launch_nvfp4_gemv_reference_cuda(const std::uint8_t* packed_weights, const std::uint8_t* block_scales,
                                     float weight_scale_2, const std::uint16_t* activation, std::size_t rows,
                                     std::size_t columns, float* output, void* stream) noexcept {
  if (rows != 0U && columns != 0U && output == nullptr) return 1;
  return q3x_b200_nvfp4_gemv(packed_weights, block_scales, weight_scale_2, activation, rows, columns, output, nullptr,
                             stream);
}

}  // namespace q3x::kernels
