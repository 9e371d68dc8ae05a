// Projection-backend dispatch: the reference's batch-one projection composites, served by this library.
//
// The reference selects its projection kernels with `enum class ProjectionBackend`
// (include/q3x/runtime/model_weights.h:373-376) and describes a projection's weights with
// `LinearWeight = std::variant<Bf16LinearWeight, Fp8LinearWeight, NvFp4LinearWeight>` (:226-363).  Its
// dispatcher (src/kernels/reference/projection_dispatch.cpp) defines, among others, the composites that
// CONTAIN operators of the fused layer-op path:
//   launch_projection_to_bf16_cuda                                         (model_weights.h:794-798)
//   launch_mlp_gate_up_silu_to_bf16_cuda                                   (:928-934)
//   launch_post_attention_residual_norm_mlp_gate_up_silu_to_bf16_cuda      (:945-956)
//   launch_decode_runner_post_attention_residual_norm_mlp_gate_up_silu_dead_up_to_bf16_cuda (:965-976)
//   launch_mlp_down_residual_norm_to_bf16_cuda                             (:989-999)
// q3x_b200_dispatch.cpp defines exactly these symbols: the batch-one projections run this library's GEMV
// kernels (bf16, FP8 with a per-tensor scale, NVFP4 weight-only -- the reference path's semantics, :646-690),
// the elementwise halves its fused operators.  Every valid backend value is served by the same sm_100a
// kernels (there is one implementation here, so the value only has to be valid); kB200LayerOps is a third
// value a caller may use to say so explicitly.
//
// Two ways to compile:
//   * inside the reference tree, with -DQ3X_B200_USE_REFERENCE_HEADERS and the reference's include
//     directory: the types and declarations are the reference's own (model_weights.h), so its callers link
//     against these definitions unchanged;
//   * stand-alone (this repository's build and tests): the mirror types below, which keep the names,
//     namespaces and the leading fields of the reference's structs -- enough for identical mangled
//     signatures.  The reference's structs carry further trailing fields (pre-swizzled sidecars), so objects
//     must not be passed between code compiled in different modes.
#pragma once

#include <cstddef>
#include <cstdint>

#if defined(Q3X_B200_USE_REFERENCE_HEADERS)
#include "q3x/runtime/model_weights.h"
#else
#include <variant>
#endif

namespace q3x::runtime {

#if !defined(Q3X_B200_USE_REFERENCE_HEADERS)

struct Bf16LinearWeight {  // model_weights.h:283-287
  const std::uint16_t* weight = nullptr;
  std::size_t output_size = 0U;
  std::size_t input_size = 0U;
};
struct Fp8LinearWeight {  // model_weights.h:289-296 (leading fields)
  const std::uint8_t* weight = nullptr;
  const float* weight_scale_device = nullptr;
  const float* input_scale_device = nullptr;
  float weight_scale = 0.0F;
  float input_scale = 0.0F;
  std::size_t output_size = 0U;
  std::size_t input_size = 0U;
};
struct NvFp4LinearWeight {  // model_weights.h:321-329 (leading fields)
  const std::uint8_t* packed_weight = nullptr;
  const std::uint8_t* block_scale = nullptr;
  const float* weight_scale_2_device = nullptr;
  const float* input_scale_device = nullptr;
  float weight_scale_2 = 0.0F;
  float input_scale = 0.0F;
  std::size_t output_size = 0U;
  std::size_t input_size = 0U;
};
using LinearWeight = std::variant<Bf16LinearWeight, Fp8LinearWeight, NvFp4LinearWeight>;  // :362-363
enum class LinearWeightKind : std::uint8_t { kBf16, kFp8, kNvFp4 };                        // :365-369

// Same underlying type and the same first two values as the reference's enum (:373-376).
enum class ProjectionBackend : std::uint8_t {
  kReference = 0,
  kSm87WeightOnly,
  kB200LayerOps,
};

[[nodiscard]] constexpr bool is_valid_projection_backend(const ProjectionBackend backend) noexcept {
  return static_cast<std::uint8_t>(backend) <= static_cast<std::uint8_t>(ProjectionBackend::kB200LayerOps);
}

// model_weights.h:393-398
[[nodiscard]] LinearWeightKind linear_weight_kind(const LinearWeight& weight) noexcept;
[[nodiscard]] std::size_t linear_output_size(const LinearWeight& weight) noexcept;
[[nodiscard]] std::size_t linear_input_size(const LinearWeight& weight) noexcept;
// model_weights.h:400-466: shape / type / payload eligibility of the fused routes (host only)
[[nodiscard]] bool supports_bf16_projection_pair(ProjectionBackend backend, const LinearWeight& first_weight,
                                                 const LinearWeight& second_weight) noexcept;
[[nodiscard]] bool supports_fp8_projection_pair(ProjectionBackend backend, const LinearWeight& first_weight,
                                                const LinearWeight& second_weight) noexcept;
[[nodiscard]] bool supports_fp8_qkv_z_projection_pair(ProjectionBackend backend, const LinearWeight& qkv_weight,
                                                      const LinearWeight& z_weight) noexcept;
[[nodiscard]] bool supports_linear_attention_qkv_z_ab_projection_fusion(ProjectionBackend backend,
                                                                        const LinearWeight& qkv_weight,
                                                                        const LinearWeight& z_weight,
                                                                        const LinearWeight& a_weight,
                                                                        const LinearWeight& b_weight) noexcept;
[[nodiscard]] bool supports_fp8_q_kv_projection_fusion(ProjectionBackend backend, const LinearWeight& q_weight,
                                                       const LinearWeight& key_weight,
                                                       const LinearWeight& value_weight) noexcept;
[[nodiscard]] bool supports_nvfp4_gate_up_silu_fusion(ProjectionBackend backend, const LinearWeight& gate_weight,
                                                      const LinearWeight& up_weight) noexcept;
[[nodiscard]] bool supports_nvfp4_down_residual_norm_fusion(ProjectionBackend backend,
                                                            const LinearWeight& down_weight) noexcept;
// model_weights.h:770-787: FP32 output, and the two-step form that also leaves the FP32 result in the scratch
[[nodiscard]] int launch_projection_reference_cuda(const LinearWeight& weight, const std::uint16_t* input, float* output,
                                                   void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_projection_to_bf16_reference_cuda(const LinearWeight& weight, const std::uint16_t* input,
                                                           float* fp32_scratch, std::size_t scratch_elements,
                                                           std::uint16_t* output, void* cuda_stream = nullptr) noexcept;
// model_weights.h:885-918: two, three and four projections over one shared activation
[[nodiscard]] int launch_projection_pair_tile_to_bf16_cuda(ProjectionBackend backend, const LinearWeight& first_weight,
                                                           const LinearWeight& second_weight, const std::uint16_t* input,
                                                           std::size_t token_count, float* fp32_scratch,
                                                           std::size_t scratch_elements, std::uint16_t* first_output,
                                                           std::uint16_t* second_output,
                                                           void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_linear_attention_qkv_z_ab_to_bf16_cuda(
    ProjectionBackend backend, const LinearWeight& qkv_weight, const LinearWeight& z_weight, const LinearWeight& a_weight,
    const LinearWeight& b_weight, const std::uint16_t* input, std::uint16_t* qkv_output, std::uint16_t* z_output,
    std::uint16_t* a_output, std::uint16_t* b_output, void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_full_attention_q_kv_to_bf16_cuda(ProjectionBackend backend, const LinearWeight& q_weight,
                                                          const LinearWeight& key_weight,
                                                          const LinearWeight& value_weight, const std::uint16_t* input,
                                                          float* fp32_scratch, std::size_t scratch_elements,
                                                          std::uint16_t* q_output, std::uint16_t* key_output,
                                                          std::uint16_t* value_output,
                                                          void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_projection_to_bf16_cuda(ProjectionBackend backend, const LinearWeight& weight,
                                                 const std::uint16_t* input, float* fp32_scratch,
                                                 std::size_t scratch_elements, std::uint16_t* output,
                                                 void* cuda_stream = nullptr) noexcept;
// model_weights.h:387,800-826: the sequence-tile form, token_count in [1, 64]
inline constexpr std::size_t kMaximumProjectionTileTokenCount = 64U;
[[nodiscard]] int launch_projection_tile_to_bf16_cuda(ProjectionBackend backend, const LinearWeight& weight,
                                                      const std::uint16_t* input, std::size_t token_count,
                                                      float* fp32_scratch, std::size_t scratch_elements,
                                                      std::uint16_t* output, void* cuda_stream = nullptr) noexcept;
// model_weights.h:828-847: one FP8 projection over a whole prefill chunk (256 or 512 tokens, the five attention /
// GDN projection shapes); anything else is cudaErrorNotSupported so that the caller keeps its tiled schedule
[[nodiscard]] int launch_exact_fp8_whole_chunk_projection_to_bf16_cuda(ProjectionBackend backend,
                                                                       const LinearWeight& weight,
                                                                       const std::uint16_t* input,
                                                                       std::size_t token_count, std::uint16_t* output,
                                                                       void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_mlp_gate_up_silu_to_bf16_cuda(ProjectionBackend backend, const LinearWeight& gate_weight,
                                                       const LinearWeight& up_weight, const std::uint16_t* input,
                                                       float* fp32_scratch, std::size_t scratch_elements,
                                                       std::uint16_t* gate_output, std::uint16_t* up_output,
                                                       void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_post_attention_residual_norm_mlp_gate_up_silu_to_bf16_cuda(
    ProjectionBackend backend, const LinearWeight& gate_weight, const LinearWeight& up_weight,
    const std::uint16_t* residual_left, std::uint16_t* residual_right_and_normalized,
    const std::uint16_t* norm_weight, float epsilon, float* fp32_scratch, std::size_t scratch_elements,
    std::uint16_t* residual_output, std::uint16_t* gate_output, std::uint16_t* up_output,
    void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_decode_runner_post_attention_residual_norm_mlp_gate_up_silu_dead_up_to_bf16_cuda(
    ProjectionBackend backend, const LinearWeight& gate_weight, const LinearWeight& up_weight,
    const std::uint16_t* residual_left, std::uint16_t* residual_right_and_normalized,
    const std::uint16_t* norm_weight, float epsilon, float* fp32_scratch, std::size_t scratch_elements,
    std::uint16_t* residual_output, std::uint16_t* gate_output, std::uint16_t* up_workspace,
    void* cuda_stream = nullptr) noexcept;
[[nodiscard]] int launch_mlp_down_residual_norm_to_bf16_cuda(
    ProjectionBackend backend, const LinearWeight& down_weight, const std::uint16_t* activation,
    const std::uint16_t* residual_left, const std::uint16_t* norm_weight, float epsilon, float* fp32_scratch,
    std::size_t scratch_elements, std::uint16_t* raw_down_output, std::uint16_t* residual_output,
    std::uint16_t* normalized_output, void* cuda_stream = nullptr) noexcept;

#endif  // !Q3X_B200_USE_REFERENCE_HEADERS

// The third backend value, spelled so that it exists in both compile modes.
inline constexpr ProjectionBackend kProjectionBackendB200LayerOps = static_cast<ProjectionBackend>(2);

// True for the values this library serves: the reference's two and the explicit third.
[[nodiscard]] constexpr bool projection_backend_served_by_b200(const ProjectionBackend backend) noexcept {
  return static_cast<std::uint8_t>(backend) <= 2U;
}

// ---- the elementwise halves on their own, for callers that run their own projections ---------------
// (no counterpart in the reference: there the halves only exist inside the composites above)

// gate_output <- bf16(silu(gate_output) * up_output) over token_count x intermediate_size elements.
[[nodiscard]] int launch_mlp_gate_up_silu_epilogue_cuda(ProjectionBackend backend, std::uint16_t* gate_output,
                                                        const std::uint16_t* up_output, std::size_t token_count,
                                                        std::size_t intermediate_size,
                                                        void* cuda_stream = nullptr) noexcept;
// residual add + centred RMSNorm; residual_right_and_normalized is read as the right operand and receives
// the normalised rows, residual_output the rounded residual (hidden_size must be 5120).
[[nodiscard]] int launch_post_attention_residual_norm_prologue_cuda(ProjectionBackend backend,
                                                                    const std::uint16_t* residual_left,
                                                                    std::uint16_t* residual_right_and_normalized,
                                                                    const std::uint16_t* norm_weight, float epsilon,
                                                                    std::size_t token_count, std::size_t hidden_size,
                                                                    std::uint16_t* residual_output,
                                                                    void* cuda_stream = nullptr) noexcept;
// raw_down_output + residual_left -> residual_output, then the next layer's input norm into
// normalized_output.  The three outputs are distinct buffers.
[[nodiscard]] int launch_mlp_down_residual_norm_epilogue_cuda(ProjectionBackend backend,
                                                              const std::uint16_t* raw_down_output,
                                                              const std::uint16_t* residual_left,
                                                              const std::uint16_t* norm_weight, float epsilon,
                                                              std::size_t token_count, std::size_t hidden_size,
                                                              std::uint16_t* residual_output,
                                                              std::uint16_t* normalized_output,
                                                              void* cuda_stream = nullptr) noexcept;

}  // namespace q3x::runtime
