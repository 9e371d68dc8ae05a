// Thin forwards from the C++ front end of the NVFP4 activation operators to the C ABI.
#include "q3x_b200_nvfp4.hpp"

#include "q3x_b200.h"

namespace q3x::quantization {

const char* nvfp4_status_string(const NvFp4Status status) noexcept {
  switch (status) {
    case NvFp4Status::kSuccess: return "success";
    case NvFp4Status::kInvalidArgument: return "invalid argument";
    case NvFp4Status::kInvalidColumnCount: return "column count is not a multiple of the NVFP4 group size";
    case NvFp4Status::kSizeOverflow: return "NVFP4 tensor element count overflows size_t";
  }
  return "unknown NVFP4 status";
}

NvFp4Status validate_nvfp4_activation_shape(const std::size_t rows, const std::size_t cols) noexcept {
  if (cols % kNvFp4ActivationBlock != 0U) return NvFp4Status::kInvalidColumnCount;
  if (cols != 0U && rows > static_cast<std::size_t>(-1) / cols / 2U) return NvFp4Status::kSizeOverflow;
  return NvFp4Status::kSuccess;
}

std::size_t nvfp4_swizzled_block_scale_bytes(std::size_t rows, std::size_t cols) noexcept {
  return q3x_b200_nvfp4_swizzled_scale_bytes(rows, cols);
}

int launch_nvfp4_swizzle_block_scales_cuda(const std::uint8_t* row_major, std::size_t rows, std::size_t cols,
                                           std::uint8_t* swizzled, void* cuda_stream) noexcept {
  return q3x_b200_nvfp4_swizzle_block_scales(row_major, rows, cols, swizzled, cuda_stream);
}

std::size_t nvfp4_projection_workspace_bytes(std::size_t token_count, std::size_t out_features, std::size_t in_features,
                                             std::size_t rows_per_scale) noexcept {
  return q3x_b200_nvfp4_gemm_workspace_bytes(token_count, out_features, in_features, rows_per_scale);
}

int launch_nvfp4_projection_to_bf16_cuda(const NvFp4ProjectionWeight& weight, const std::uint8_t* activation_codes,
                                         const std::uint8_t* activation_block_scales_swizzled,
                                         const float* activation_global_scales, std::size_t rows_per_scale,
                                         std::size_t token_count, std::uint16_t* output, void* workspace,
                                         std::size_t workspace_bytes, void* cuda_stream) noexcept {
  return q3x_b200_nvfp4_gemm_bf16(activation_codes, activation_block_scales_swizzled, activation_global_scales,
                                  rows_per_scale, weight.codes, weight.block_scales_swizzled, weight.scale_2, token_count,
                                  weight.out_features, weight.in_features, output, workspace, workspace_bytes, cuda_stream);
}

std::size_t nvfp4_activation_scale_groups(std::size_t rows, std::size_t rows_per_scale) noexcept {
  return q3x_b200_nvfp4_group_count(rows, rows_per_scale);
}

std::size_t nvfp4_activation_scratch_words(std::size_t rows, std::size_t rows_per_scale) noexcept {
  return q3x_b200_nvfp4_scratch_words(rows, rows_per_scale);
}

int launch_nvfp4_quantize_activations_cuda(const std::uint16_t* input, std::size_t rows, std::size_t cols,
                                           std::size_t rows_per_scale, NvFp4ActivationBuffers b,
                                           void* cuda_stream) noexcept {
  return q3x_b200_nvfp4_quantize_dynamic(input, rows, cols, rows_per_scale, b.scratch, b.global_scales, b.codes,
                                         b.block_scales, cuda_stream);
}

int launch_residual_add_centered_rms_norm_nvfp4_cuda(const std::uint16_t* left, const std::uint16_t* right,
                                                     const std::uint16_t* weight, std::size_t token_count,
                                                     std::size_t hidden_size, float epsilon,
                                                     std::size_t rows_per_scale, std::uint16_t* residual_output,
                                                     std::uint16_t* normalized_output, NvFp4ActivationBuffers b,
                                                     void* cuda_stream) noexcept {
  return q3x_b200_residual_add_rms_norm_nvfp4(left, right, weight, token_count, hidden_size, epsilon, rows_per_scale,
                                              residual_output, normalized_output, b.scratch, b.global_scales, b.codes,
                                              b.block_scales, cuda_stream);
}

int launch_headwise_plain_rms_norm_silu_gate_nvfp4_cuda(const std::uint16_t* input, const std::uint16_t* weight,
                                                        const std::uint16_t* gate, std::size_t token_count,
                                                        std::size_t heads_per_token, std::size_t head_dimension,
                                                        float epsilon, std::size_t rows_per_scale,
                                                        std::uint16_t* output, NvFp4ActivationBuffers b,
                                                        void* cuda_stream) noexcept {
  return q3x_b200_rms_norm_silu_gate_nvfp4(input, weight, gate, token_count, heads_per_token, head_dimension, epsilon,
                                           rows_per_scale, output, b.scratch, b.global_scales, b.codes,
                                           b.block_scales, cuda_stream);
}

int launch_silu_mul_nvfp4_cuda(const std::uint16_t* gate, const std::uint16_t* up, std::size_t token_count,
                               std::size_t intermediate_size, std::size_t rows_per_scale, std::uint16_t* output,
                               NvFp4ActivationBuffers b, void* cuda_stream) noexcept {
  return q3x_b200_silu_mul_nvfp4(gate, up, token_count, intermediate_size, rows_per_scale, output, b.scratch,
                                 b.global_scales, b.codes, b.block_scales, cuda_stream);
}

int launch_sigmoid_gate_nvfp4_cuda(const std::uint16_t* value, const std::uint16_t* gate, std::size_t token_count,
                                   std::size_t width, std::size_t rows_per_scale, std::uint16_t* output,
                                   NvFp4ActivationBuffers b, void* cuda_stream) noexcept {
  return q3x_b200_sigmoid_gate_nvfp4(value, gate, token_count, width, rows_per_scale, output, b.scratch,
                                     b.global_scales, b.codes, b.block_scales, cuda_stream);
}

}  // namespace q3x::quantization
