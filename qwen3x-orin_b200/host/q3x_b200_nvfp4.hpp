// C++17 front end of the NVFP4 activation operators of libq3x_b200.so.
//
// The reference project has no activation quantiser (its NVFP4 code decodes checkpoint weights,
// include/q3x/quantization/nvfp4.h), so these functions have no declaration to mirror; they follow
// the conventions of the reference's launchers all the same (decode_ops.h:172-176): `int` is a
// cudaError_t, pointers are device pointers, the caller owns every buffer including the scratch,
// nothing is allocated, copied or synchronised, `cuda_stream` is a cudaStream_t.
#pragma once

#include <cstddef>
#include <cstdint>

namespace q3x::quantization {

inline constexpr std::size_t kNvFp4ActivationBlock = 16U;       // elements per E4M3 block scale (nvfp4.h:8)
inline constexpr std::size_t kNvFp4PrefillScaleScope = 512U;    // rows per global scale: one prefill chunk

// include/q3x/quantization/nvfp4.h:41-46, same enumerators and values
enum class NvFp4Status : std::uint8_t {
  kSuccess = 0,
  kInvalidArgument,
  kInvalidColumnCount,
  kSizeOverflow,
};
[[nodiscard]] const char* nvfp4_status_string(NvFp4Status status) noexcept;
// Host-side shape check of a [rows, cols] activation tensor, in the reference's status vocabulary: cols must be
// a multiple of 16 (kInvalidColumnCount), rows * cols * 2 must fit size_t (kSizeOverflow).
[[nodiscard]] NvFp4Status validate_nvfp4_activation_shape(std::size_t rows, std::size_t cols) noexcept;

// Caller-owned buffers of one call on a [rows, cols] tensor.
struct NvFp4ActivationBuffers {
  std::uint32_t* scratch = nullptr;       // nvfp4_activation_scratch_words(rows, rows_per_scale) words
  float* global_scales = nullptr;         // nvfp4_activation_scale_groups(rows, rows_per_scale) floats
  std::uint8_t* codes = nullptr;          // rows * cols / 2 bytes, even column in the low nibble
  std::uint8_t* block_scales = nullptr;   // rows * cols / 16 E4M3 bytes, row-major, un-swizzled
};

// Block scales re-laid out in the 128 x 4 tiles block-scaled tensor-core MMA reads (see q3x_b200.h).
[[nodiscard]] std::size_t nvfp4_swizzled_block_scale_bytes(std::size_t rows, std::size_t cols) noexcept;
[[nodiscard]] int launch_nvfp4_swizzle_block_scales_cuda(const std::uint8_t* row_major, std::size_t rows,
                                                         std::size_t cols, std::uint8_t* swizzled,
                                                         void* cuda_stream = nullptr) noexcept;

// The projection that consumes those operands: out [tokens, out_features] bf16 = activations x weights^T, both
// NVFP4 (codes, swizzled block scales, FP32 second-level scales: one per activation scale group, one for the
// weights), on the block-scaled tensor cores.  It stands where the reference's prefill arm of
// launch_projection_to_bf16_cuda (model_weights.h:794-841) multiplies bf16 activations with NVFP4 weights.
struct NvFp4ProjectionWeight {
  const std::uint8_t* codes = nullptr;                  // [out_features, in_features / 2]
  const std::uint8_t* block_scales_swizzled = nullptr;  // nvfp4_swizzled_block_scale_bytes(out_features, in_features)
  float scale_2 = 1.0F;                                 // NvFp4LinearWeight::weight_scale_2
  std::size_t out_features = 0U;
  std::size_t in_features = 0U;
};
[[nodiscard]] std::size_t nvfp4_projection_workspace_bytes(std::size_t token_count, std::size_t out_features,
                                                           std::size_t in_features, std::size_t rows_per_scale) noexcept;
[[nodiscard]] int launch_nvfp4_projection_to_bf16_cuda(const NvFp4ProjectionWeight& weight,
                                                       const std::uint8_t* activation_codes,
                                                       const std::uint8_t* activation_block_scales_swizzled,
                                                       const float* activation_global_scales,
                                                       std::size_t rows_per_scale, std::size_t token_count,
                                                       std::uint16_t* output, void* workspace,
                                                       std::size_t workspace_bytes, void* cuda_stream = nullptr) noexcept;

[[nodiscard]] std::size_t nvfp4_activation_scale_groups(std::size_t rows, std::size_t rows_per_scale) noexcept;
[[nodiscard]] std::size_t nvfp4_activation_scratch_words(std::size_t rows, std::size_t rows_per_scale) noexcept;

// Any bf16 tensor: group amax -> global scales -> codes and block scales.
[[nodiscard]] int launch_nvfp4_quantize_activations_cuda(const std::uint16_t* input, std::size_t rows, std::size_t cols,
                                                         std::size_t rows_per_scale, NvFp4ActivationBuffers buffers,
                                                         void* cuda_stream = nullptr) noexcept;

// launch_residual_add_centered_rms_norm_*_5120_cuda (decode_ops.h:238-272) with the NVFP4 operand of the
// next projection produced in the same kernel; normalized_output is required.
[[nodiscard]] int launch_residual_add_centered_rms_norm_nvfp4_cuda(
    const std::uint16_t* left, const std::uint16_t* right, const std::uint16_t* weight, std::size_t token_count,
    std::size_t hidden_size, float epsilon, std::size_t rows_per_scale, std::uint16_t* residual_output,
    std::uint16_t* normalized_output, NvFp4ActivationBuffers buffers, void* cuda_stream = nullptr) noexcept;

// launch_headwise_plain_rms_norm_silu_gate_reference_cuda (decode_ops.h:218-222) over tokens of
// `heads_per_token` heads, plus NVFP4 of each token's row.
[[nodiscard]] int launch_headwise_plain_rms_norm_silu_gate_nvfp4_cuda(
    const std::uint16_t* input, const std::uint16_t* weight, const std::uint16_t* gate, std::size_t token_count,
    std::size_t heads_per_token, std::size_t head_dimension, float epsilon, std::size_t rows_per_scale,
    std::uint16_t* output, NvFp4ActivationBuffers buffers, void* cuda_stream = nullptr) noexcept;

// launch_silu_mul_reference_cuda (decode_ops.h:290-293) plus NVFP4 of its output (the down projection's operand).
[[nodiscard]] int launch_silu_mul_nvfp4_cuda(const std::uint16_t* gate, const std::uint16_t* up,
                                             std::size_t token_count, std::size_t intermediate_size,
                                             std::size_t rows_per_scale, std::uint16_t* output,
                                             NvFp4ActivationBuffers buffers, void* cuda_stream = nullptr) noexcept;

// launch_sigmoid_gate_reference_cuda (decode_ops.h:295-298) plus NVFP4 of its output (the attention output
// projection's operand).
[[nodiscard]] int launch_sigmoid_gate_nvfp4_cuda(const std::uint16_t* value, const std::uint16_t* gate,
                                                 std::size_t token_count, std::size_t width,
                                                 std::size_t rows_per_scale, std::uint16_t* output,
                                                 NvFp4ActivationBuffers buffers, void* cuda_stream = nullptr) noexcept;

}  // namespace q3x::quantization
