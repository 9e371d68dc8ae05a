// C++17 mirror of the reference project's operator API for the fused layer-op path.
//
// Every function below has the namespace, name, parameter list, default arguments and return
// convention of the declaration it stands in for in the reference headers
// (include/q3x/runtime/decode_ops.h, layout_ops.h, gdn_decode.h and
// src/kernels/reference/gdn_prefill_whole_span_conv_sm87.h), so a reference build that links
// libq3x_b200_host.so instead of compiling its own .cu files resolves the same symbols.  Each one
// validates what the reference validates (its argument limits are part of its contract), then
// forwards to the C ABI of libq3x_b200.so.  Nothing here allocates, copies or synchronises.
//
// Only CUDA launchers are mirrored.  The `*_reference_cpu` functions of the same headers are the
// reference's CPU path; this library has no CPU path.
#pragma once

#include <cstddef>
#include <cstdint>

namespace q3x::runtime {

// ---- constants and types the signatures need (decode_ops.h:8-59, gdn_decode.h:8-36) -------------
inline constexpr std::size_t kLinearAttentionHeadDimension = 128U;
inline constexpr std::size_t kFullAttentionHeadDimension = 256U;
inline constexpr std::size_t kQwenRotaryDimension = 64U;
inline constexpr std::size_t kQkRopeTileMaximumTokens = 16U;
inline constexpr std::size_t kFullAttentionPreprocessMaximumTokens = 512U;
inline constexpr std::size_t kFullAttentionPreprocessPromptWideP8000Tokens = 8'000U;
inline constexpr std::size_t kFullAttentionPreprocessPromptWideP8000PanelCount = 5U;
inline constexpr std::size_t kResidualNormPrefillMaximumTokens = 512U;  // decode_ops.cu:1913-1953
inline constexpr std::size_t kResidualNormHiddenSize = 5'120U;

inline constexpr std::size_t kFusedGqaMaximumSequenceLength = 64U;            // decode_ops.h:10
inline constexpr std::size_t kDecodeGqaSplitKvMaximumSequenceLength = 4'096U;  // decode_ops.h:11

// decode_ops.h:61-69
struct Bf16GreedyArgmaxResult {
  std::uint32_t index = 0U;
  std::uint16_t value_bits = 0U;
  std::uint16_t has_nonfinite = 0U;
};
static_assert(sizeof(Bf16GreedyArgmaxResult) == 8U);
inline constexpr std::size_t kBf16GreedyArgmaxWorkspaceResults = 33U;

inline constexpr std::size_t kGdnQkHeadCount = 16U;
inline constexpr std::size_t kGdnValueHeadCount = 48U;
inline constexpr std::size_t kGdnHeadDimension = 128U;
inline constexpr std::size_t kGdnConvHistoryWidth = 3U;
inline constexpr std::size_t kGdnConvKernelWidth = 4U;
inline constexpr std::size_t kGdnMaximumTileTokenCount = 16U;
inline constexpr std::size_t kGdnQkvChannels = (2U * kGdnQkHeadCount + kGdnValueHeadCount) * kGdnHeadDimension;

enum class DecodeOpStatus : std::uint8_t {
  kSuccess = 0, kInvalidArgument, kInvalidDimension, kSizeOverflow, kTokenOutOfRange, kInsufficientScratch,
};
enum class LayoutOpStatus : std::uint8_t { kSuccess = 0, kInvalidArgument, kSizeOverflow, kOverlappingStorage };
enum class GdnStatus : std::uint8_t { kSuccess = 0, kInvalidArgument, kInvalidDimension, kSizeOverflow, kInvalidAlias };

struct GdnDimensions {
  std::size_t qk_head_count = kGdnQkHeadCount;
  std::size_t value_head_count = kGdnValueHeadCount;
  std::size_t head_dimension = kGdnHeadDimension;
};

[[nodiscard]] constexpr bool can_launch_full_attention_preprocess_prompt_wide_p8000(
    const std::size_t first_position, const std::size_t token_count) noexcept {
  return token_count == kFullAttentionPreprocessPromptWideP8000Tokens &&
         first_position % kFullAttentionPreprocessPromptWideP8000Tokens == 0U &&
         first_position / kFullAttentionPreprocessPromptWideP8000Tokens <
             kFullAttentionPreprocessPromptWideP8000PanelCount;
}

// ---- decode_ops.h launchers (all return cudaError_t as int; cuda_stream is a cudaStream_t) -------
[[nodiscard]] int launch_embedding_gather_reference_cuda(const std::uint16_t* embedding_table,
                                                         std::size_t vocabulary_size, std::size_t hidden_size,
                                                         std::size_t token_id, std::uint16_t* output,
                                                         void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_embedding_gather_prompt_reference_cuda(const std::uint16_t* embedding_table,
                                                                std::size_t vocabulary_size, std::size_t hidden_size,
                                                                const std::uint32_t* token_ids,
                                                                std::size_t token_count, std::uint16_t* output,
                                                                void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_centered_rms_norm_reference_cuda(const std::uint16_t* input, const std::uint16_t* weight,
                                                          std::size_t hidden_size, float epsilon,
                                                          std::uint16_t* output, void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_plain_rms_norm_reference_cuda(const std::uint16_t* input, const std::uint16_t* weight,
                                                       std::size_t hidden_size, float epsilon, std::uint16_t* output,
                                                       void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_headwise_centered_rms_norm_reference_cuda(const std::uint16_t* input,
                                                                   const std::uint16_t* shared_weight,
                                                                   std::size_t head_count, std::size_t head_dimension,
                                                                   float epsilon, std::uint16_t* output,
                                                                   void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_headwise_plain_rms_norm_reference_cuda(const std::uint16_t* input,
                                                                const std::uint16_t* shared_weight,
                                                                std::size_t head_count, std::size_t head_dimension,
                                                                float epsilon, std::uint16_t* output,
                                                                void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_headwise_plain_rms_norm_silu_gate_reference_cuda(
    const std::uint16_t* input, const std::uint16_t* shared_weight, const std::uint16_t* gate, std::size_t head_count,
    std::size_t head_dimension, float epsilon, std::uint16_t* output, void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_residual_add_reference_cuda(const std::uint16_t* left, const std::uint16_t* right,
                                                     std::size_t element_count, std::uint16_t* output,
                                                     void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_residual_add_centered_rms_norm_5120_cuda(const std::uint16_t* left,
                                                                  const std::uint16_t* right,
                                                                  const std::uint16_t* weight, float epsilon,
                                                                  std::uint16_t* residual_output,
                                                                  std::uint16_t* normalized_output,
                                                                  void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_residual_add_headwise_centered_rms_norm_m32_5120_cuda(
    const std::uint16_t* left, const std::uint16_t* right, const std::uint16_t* weight, std::size_t token_count,
    std::size_t hidden_size, float epsilon, std::uint16_t* residual_output, std::uint16_t* normalized_output,
    void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_residual_add_headwise_centered_rms_norm_prefill_5120_cuda(
    const std::uint16_t* left, const std::uint16_t* right, const std::uint16_t* weight, std::size_t token_count,
    std::size_t hidden_size, float epsilon, std::uint16_t* residual_output, std::uint16_t* normalized_output,
    void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_fp32_to_bf16_reference_cuda(const float* input, std::size_t element_count,
                                                     std::uint16_t* output, void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_silu_mul_reference_cuda(const std::uint16_t* gate, const std::uint16_t* up,
                                                 std::size_t element_count, std::uint16_t* output,
                                                 void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_sigmoid_gate_reference_cuda(const std::uint16_t* value, const std::uint16_t* gate,
                                                     std::size_t element_count, std::uint16_t* output,
                                                     void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_l2_normalize_heads_reference_cuda(const std::uint16_t* input, std::size_t head_count,
                                                           std::size_t head_dimension, float epsilon,
                                                           std::uint16_t* output, void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_partial_neox_rope_256_64_reference_cuda(const std::uint16_t* input, const float* cosines,
                                                                 const float* sines, std::size_t head_count,
                                                                 std::uint16_t* output,
                                                                 void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_qk_partial_neox_rope_tile_24_4_256_64_cuda(std::uint16_t* query, std::uint16_t* key,
                                                                    const float* cosines, const float* sines,
                                                                    std::size_t first_position,
                                                                    std::size_t token_count,
                                                                    void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_full_attention_preprocess_24_4_256_64_reference_256_cuda(
    const std::uint16_t* interleaved_q_gate, std::uint16_t* key, const std::uint16_t* q_weight,
    const std::uint16_t* k_weight, float epsilon, std::uint16_t* query_output, std::uint16_t* gate_output,
    const float* cosines, const float* sines, std::size_t first_position, std::size_t token_count,
    void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_full_attention_preprocess_24_4_256_64_prompt_wide_p8000_cuda(
    const std::uint16_t* interleaved_q_gate, std::uint16_t* key, const std::uint16_t* q_weight,
    const std::uint16_t* k_weight, float epsilon, std::uint16_t* query_output, std::uint16_t* gate_output,
    const float* cosines, const float* sines, std::size_t first_position, std::size_t token_count,
    void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_full_attention_preprocess_24_4_256_64_cuda(
    const std::uint16_t* interleaved_q_gate, std::uint16_t* key, const std::uint16_t* q_weight,
    const std::uint16_t* k_weight, float epsilon, std::uint16_t* query_output, std::uint16_t* gate_output,
    const float* cosines, const float* sines, std::size_t first_position, std::size_t token_count,
    void* cuda_stream = nullptr) noexcept;

[[nodiscard]] int launch_softmax_reference_cuda(const float* input, std::size_t rows, std::size_t columns,
                                                float* output, void* cuda_stream = nullptr) noexcept;
// decode_ops.h:397-423: sequence_length in (64, 4096]
[[nodiscard]] std::size_t gqa_attention_splitkv_sigmoid_gate_24_4_256_workspace_elements(
    std::size_t sequence_length) noexcept;
[[nodiscard]] int launch_gqa_attention_splitkv_sigmoid_gate_24_4_256_cuda(
    const std::uint16_t* query, const std::uint16_t* key_cache, const std::uint16_t* value_cache,
    std::size_t sequence_length, float attention_scale, float* workspace, std::size_t workspace_elements,
    const std::uint16_t* gate, std::uint16_t* output, void* cuda_stream = nullptr) noexcept;
// decode_ops.h:17-21,419-505: bulk causal attention of a prefill tile / panel with the sigmoid output gate.
// token_count in [2, 512] for the tile forms; query / gate / output are tile-local [token_count, 24, 256], the caches
// are global [position, 4, 256], first_position is the append position of the tile's first token.
inline constexpr std::size_t kBulkCausalGqaMaximumSequenceLength = 262'144U;
inline constexpr std::size_t kBulkCausalGqaGroupQ64PanelMaximumTokens = 8'192U;
[[nodiscard]] int launch_bulk_causal_gqa_sigmoid_gate_24_4_256_cuda(
    const std::uint16_t* query_tile, const std::uint16_t* key_cache, const std::uint16_t* value_cache,
    const std::uint16_t* gate_tile, std::size_t first_position, std::size_t token_count, std::uint16_t* output_tile,
    void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_bulk_causal_gqa_sigmoid_gate_24_4_256_fixed_cuda(
    const std::uint16_t* query_tile, const std::uint16_t* key_cache, const std::uint16_t* value_cache,
    const std::uint16_t* gate_tile, std::size_t first_position, std::size_t token_count, std::uint16_t* output_tile,
    void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_bulk_causal_gqa_sigmoid_gate_24_4_256_group_q64_panel_fixed_cuda(
    const std::uint16_t* query_panel, const std::uint16_t* key_cache, const std::uint16_t* value_cache,
    const std::uint16_t* gate_panel, std::size_t first_position, std::size_t token_count, std::uint16_t* output_panel,
    void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_bf16_greedy_argmax_cuda(const std::uint16_t* input, std::size_t element_count,
                                                 Bf16GreedyArgmaxResult* result_workspace,
                                                 void* cuda_stream = nullptr) noexcept;

// ---- layout_ops.h -------------------------------------------------------------------------------
[[nodiscard]] int launch_split_interleaved_q_gate_reference_cuda(const std::uint16_t* input, std::size_t head_count,
                                                                 std::size_t head_dimension,
                                                                 std::uint16_t* query_output,
                                                                 std::uint16_t* gate_output,
                                                                 void* cuda_stream = nullptr) noexcept;

// ---- gdn_decode.h (conv launchers) ----------------------------------------------------------------
[[nodiscard]] int launch_causal_conv1d_silu_update_reference_cuda(const std::uint16_t* raw_qkv,
                                                                  const std::uint16_t* conv_weight,
                                                                  std::uint16_t* history_in_out,
                                                                  std::uint16_t* conv_qkv_output,
                                                                  GdnDimensions dimensions = {},
                                                                  void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_causal_conv1d_silu_update_tile_reference_cuda(
    const std::uint16_t* raw_qkv, std::size_t token_count, const std::uint16_t* conv_weight,
    std::uint16_t* history_in_out, std::uint16_t* conv_qkv_output, GdnDimensions dimensions = {},
    void* cuda_stream = nullptr) noexcept;

// ---- gdn_decode.h (recurrence launchers, :85-188) ----------------------------------------------------------
[[nodiscard]] bool supports_gated_delta_net_update_plain_rms_norm_silu_gate_fusion(
    std::size_t token_count, GdnDimensions dimensions, std::size_t norm_head_count,
    std::size_t norm_head_dimension) noexcept;
[[nodiscard]] int launch_gated_delta_net_update_reference_cuda(
    const std::uint16_t* conv_qkv, const std::uint16_t* a, const std::uint16_t* b, const std::uint16_t* A_log,
    const std::uint16_t* dt_bias, const std::uint16_t* state_input, std::uint16_t* state_output, float l2_epsilon,
    std::uint16_t* output, GdnDimensions dimensions = {}, void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_gated_delta_net_update_tile_reference_cuda(
    const std::uint16_t* conv_qkv, std::size_t token_count, const std::uint16_t* a, const std::uint16_t* b,
    const std::uint16_t* A_log, const std::uint16_t* dt_bias, const std::uint16_t* state_input,
    std::uint16_t* state_output, float l2_epsilon, std::uint16_t* output, GdnDimensions dimensions = {},
    void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_gated_delta_net_update_warp_parallel_cuda(
    const std::uint16_t* conv_qkv, const std::uint16_t* a, const std::uint16_t* b, const std::uint16_t* A_log,
    const std::uint16_t* dt_bias, const std::uint16_t* state_input, std::uint16_t* state_output, float l2_epsilon,
    std::uint16_t* output, GdnDimensions dimensions = {}, void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_gated_delta_net_update_tile_warp_parallel_cuda(
    const std::uint16_t* conv_qkv, std::size_t token_count, const std::uint16_t* a, const std::uint16_t* b,
    const std::uint16_t* A_log, const std::uint16_t* dt_bias, const std::uint16_t* state_input,
    std::uint16_t* state_output, float l2_epsilon, std::uint16_t* output, GdnDimensions dimensions = {},
    void* cuda_stream = nullptr) noexcept;
namespace gdn_decode_detail {
// gdn_decode.h:152-168: the exact-shape (one token, 48 heads of 128) form behind the composite below
[[nodiscard]] int launch_gated_delta_net_update_plain_rms_norm_silu_gate_exact_cuda(
    const std::uint16_t* conv_qkv, const std::uint16_t* a, const std::uint16_t* b, const std::uint16_t* A_log,
    const std::uint16_t* dt_bias, const std::uint16_t* state_input, std::uint16_t* state_output, float l2_epsilon,
    const std::uint16_t* norm_weight, const std::uint16_t* silu_gate, float norm_epsilon, std::uint16_t* output,
    void* cuda_stream = nullptr) noexcept;
}  // namespace gdn_decode_detail
[[nodiscard]] int launch_gated_delta_net_update_plain_rms_norm_silu_gate_cuda(
    const std::uint16_t* conv_qkv, const std::uint16_t* a, const std::uint16_t* b, const std::uint16_t* A_log,
    const std::uint16_t* dt_bias, const std::uint16_t* state_input, std::uint16_t* state_output, float l2_epsilon,
    const std::uint16_t* norm_weight, const std::uint16_t* silu_gate, std::size_t norm_head_count,
    std::size_t norm_head_dimension, float norm_epsilon, std::uint16_t* output, GdnDimensions dimensions = {},
    void* cuda_stream = nullptr) noexcept;

namespace gdn_prefill_chunk64_native_detail {
inline constexpr std::size_t kMaximumTokenCount = 512U;
// src/kernels/sm87/gdn_prefill_chunk64_native_sm87.h:96-122: the GDN recurrence of a prefill tile of 1 to 512 tokens
// in chunks of 64 (WY form), then the gated RMSNorm of its output in place.  One reusable caller-owned workspace of at
// least workspace_bytes() bytes, whatever the token count.
[[nodiscard]] std::size_t workspace_bytes() noexcept;
[[nodiscard]] int launch(void* workspace, std::size_t workspace_capacity_bytes, const std::uint16_t* conv_qkv,
                         std::size_t token_count, const std::uint16_t* a, const std::uint16_t* b,
                         const std::uint16_t* A_log, const std::uint16_t* dt_bias, const std::uint16_t* state_input,
                         std::uint16_t* state_output, float l2_epsilon, const std::uint16_t* norm_weight,
                         const std::uint16_t* silu_gate, float norm_epsilon, std::uint16_t* output,
                         void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_fixed_production(void* workspace, std::size_t workspace_capacity_bytes,
                                          const std::uint16_t* conv_qkv, std::size_t token_count, const std::uint16_t* a,
                                          const std::uint16_t* b, const std::uint16_t* A_log,
                                          const std::uint16_t* dt_bias, const std::uint16_t* state_input,
                                          std::uint16_t* state_output, float l2_epsilon,
                                          const std::uint16_t* norm_weight, const std::uint16_t* silu_gate,
                                          float norm_epsilon, std::uint16_t* output,
                                          void* cuda_stream = nullptr) noexcept;
}  // namespace gdn_prefill_chunk64_native_detail

namespace gdn_prefill_whole_span_conv_detail {
inline constexpr std::size_t kMaximumTokenCount = 512U;
// src/kernels/reference/gdn_prefill_whole_span_conv_sm87.h:59-67
[[nodiscard]] int launch_causal_conv1d_silu_update_token_parallel_compact_qk_exact_cuda(
    const std::uint16_t* raw_qkv, std::size_t token_count, const std::uint16_t* conv_weight,
    std::uint16_t* history_in_out, std::uint16_t* conv_qkv_output, float l2_epsilon, std::uint16_t* compact_q,
    std::uint16_t* compact_k, void* cuda_stream = nullptr) noexcept;
// :69-80: the same operator for the one prompt length (40000 tokens) of the reference's prompt-wide chunk graph
inline constexpr std::size_t kPromptWideP40TokenCount = 40'000U;
[[nodiscard]] int launch_causal_conv1d_silu_update_prompt_wide_p40_compact_qk_exact_cuda(
    const std::uint16_t* raw_qkv, std::size_t token_count, const std::uint16_t* conv_weight,
    std::uint16_t* history_in_out, std::uint16_t* conv_qkv_output, float l2_epsilon, std::uint16_t* compact_q,
    std::uint16_t* compact_k, void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_causal_conv1d_silu_update_whole_span_exact_cuda(
    const std::uint16_t* raw_qkv, std::size_t token_count, const std::uint16_t* conv_weight,
    std::uint16_t* history_in_out, std::uint16_t* conv_qkv_output, void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_causal_conv1d_silu_update_token_parallel_exact_cuda(
    const std::uint16_t* raw_qkv, std::size_t token_count, const std::uint16_t* conv_weight,
    std::uint16_t* history_in_out, std::uint16_t* conv_qkv_output, void* cuda_stream = nullptr) noexcept;
}  // namespace gdn_prefill_whole_span_conv_detail

}  // namespace q3x::runtime

// ---- include/q3x/kernels/reference_gemv.h:64-130: the batch-one projection launchers ------------------------
namespace q3x::kernels {
[[nodiscard]] int launch_bf16_gemv_reference_cuda(const std::uint16_t* weights, const std::uint16_t* activation,
                                                  std::size_t rows, std::size_t columns, float* output,
                                                  void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_bf16_gemv_bf16_cuda(const std::uint16_t* weights, const std::uint16_t* activation,
                                             std::size_t rows, std::size_t columns, std::uint16_t* output,
                                             void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_fp8_gemv_reference_cuda(const std::uint8_t* weights, float weight_scale,
                                                 const std::uint16_t* activation, std::size_t rows,
                                                 std::size_t columns, float* output,
                                                 void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_nvfp4_gemv_reference_cuda(const std::uint8_t* packed_weights,
                                                   const std::uint8_t* block_scales, float weight_scale_2,
                                                   const std::uint16_t* activation, std::size_t rows,
                                                   std::size_t columns, float* output,
                                                   void* cuda_stream = nullptr) noexcept;
}  // namespace q3x::kernels

#include "q3x_b200_dispatch.hpp"
#include "q3x_b200_prefill_bindings.hpp"
