#include "q3x_b200_dispatch.hpp"

#include "q3x_b200.h"

namespace q3x::runtime {
namespace {
constexpr int kInvalidValue = 1;    // cudaErrorInvalidValue
constexpr int kNotSupported = 801;  // cudaErrorNotSupported
constexpr std::size_t kHidden = 5120U;

// Invalid backend -> invalid value; a valid backend this library does not serve -> not supported.
int route(const ProjectionBackend backend) noexcept {
  if (!is_valid_projection_backend(backend)) return kInvalidValue;
  return projection_backend_uses_b200_layer_ops(backend) ? 0 : kNotSupported;
}
}  // namespace

int launch_mlp_gate_up_silu_epilogue_cuda(const ProjectionBackend backend, std::uint16_t* gate_output,
                                          const std::uint16_t* up_output, const std::size_t token_count,
                                          const std::size_t intermediate_size, void* cuda_stream) noexcept {
  if (const int r = route(backend); r != 0) return r;
  if (intermediate_size != 0U && token_count > static_cast<std::size_t>(-1) / intermediate_size) return kInvalidValue;
  return q3x_b200_silu_mul(gate_output, up_output, token_count * intermediate_size, gate_output, cuda_stream);
}

int launch_post_attention_residual_norm_prologue_cuda(const ProjectionBackend backend,
                                                      const std::uint16_t* residual_left,
                                                      std::uint16_t* residual_right_and_normalized,
                                                      const std::uint16_t* norm_weight, const float epsilon,
                                                      const std::size_t token_count, const std::size_t hidden_size,
                                                      std::uint16_t* residual_output, void* cuda_stream) noexcept {
  if (const int r = route(backend); r != 0) return r;
  if (hidden_size != kHidden || token_count == 0U) return kInvalidValue;  // projection_dispatch.cpp:483-534
  return q3x_b200_residual_add_rms_norm(residual_left, residual_right_and_normalized, norm_weight, token_count,
                                        hidden_size, epsilon, residual_output, residual_right_and_normalized,
                                        cuda_stream);
}

int launch_mlp_down_residual_norm_epilogue_cuda(const ProjectionBackend backend, const std::uint16_t* raw_down_output,
                                                const std::uint16_t* residual_left, const std::uint16_t* norm_weight,
                                                const float epsilon, const std::size_t token_count,
                                                const std::size_t hidden_size, std::uint16_t* residual_output,
                                                std::uint16_t* normalized_output, void* cuda_stream) noexcept {
  if (const int r = route(backend); r != 0) return r;
  // three distinct boundaries (model_weights.h:977-983): raw down stays observable
  if (hidden_size != kHidden || token_count == 0U || normalized_output == nullptr ||
      normalized_output == raw_down_output)
    return kInvalidValue;
  return q3x_b200_residual_add_rms_norm(residual_left, raw_down_output, norm_weight, token_count, hidden_size, epsilon,
                                        residual_output, normalized_output, cuda_stream);
}

}  // namespace q3x::runtime
