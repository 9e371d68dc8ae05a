// Projection-backend dispatch, as far as the fused layer ops are concerned.
//
// The reference selects its projection kernels with `enum class ProjectionBackend`
// (include/q3x/runtime/model_weights.h:373-376) and exposes three composites that CONTAIN
// operators of this path: launch_mlp_gate_up_silu_to_bf16_cuda,
// launch_post_attention_residual_norm_mlp_gate_up_silu_to_bf16_cuda (and its decode-runner twin) and
// launch_mlp_down_residual_norm_to_bf16_cuda (model_weights.h:928-992).  Their GEMV arms are dense
// contractions and stay with the reference; what it does around them when no fused kernel applies
// (src/kernels/reference/projection_dispatch.cpp:1411,1558,1661) is call the elementwise launchers.
// The functions here are those elementwise halves, taking the projection outputs as inputs, so the
// reference's dispatcher can route them to this library by backend value.
#pragma once

#include <cstddef>
#include <cstdint>

namespace q3x::runtime {

// Same underlying type and the same first two values as the reference's enum; the third value
// selects this library for the elementwise halves.
enum class ProjectionBackend : std::uint8_t {
  kReference = 0,
  kSm87WeightOnly,
  kB200LayerOps,
};

[[nodiscard]] constexpr bool is_valid_projection_backend(const ProjectionBackend backend) noexcept {
  return static_cast<std::uint8_t>(backend) <= static_cast<std::uint8_t>(ProjectionBackend::kB200LayerOps);
}
// True when this library serves the elementwise half for `backend`; every other valid backend gets
// cudaErrorNotSupported from the functions below so that the caller falls back
// (model_weights.h:835-841 describes that convention).
[[nodiscard]] constexpr bool projection_backend_uses_b200_layer_ops(const ProjectionBackend backend) noexcept {
  return backend == ProjectionBackend::kB200LayerOps;
}

// gate_output <- bf16(silu(gate_output) * up_output) over token_count x intermediate_size elements:
// the tail of launch_mlp_gate_up_silu_to_bf16_cuda once both projections have been written.
[[nodiscard]] int launch_mlp_gate_up_silu_epilogue_cuda(ProjectionBackend backend, std::uint16_t* gate_output,
                                                        const std::uint16_t* up_output, std::size_t token_count,
                                                        std::size_t intermediate_size,
                                                        void* cuda_stream = nullptr) noexcept;

// The head of launch_post_attention_residual_norm_mlp_gate_up_silu_to_bf16_cuda: residual add +
// centred RMSNorm; residual_right_and_normalized is read as the right operand and receives the
// normalised rows, residual_output the rounded residual (hidden_size must be 5120).
[[nodiscard]] int launch_post_attention_residual_norm_prologue_cuda(ProjectionBackend backend,
                                                                    const std::uint16_t* residual_left,
                                                                    std::uint16_t* residual_right_and_normalized,
                                                                    const std::uint16_t* norm_weight, float epsilon,
                                                                    std::size_t token_count, std::size_t hidden_size,
                                                                    std::uint16_t* residual_output,
                                                                    void* cuda_stream = nullptr) noexcept;

// The tail of launch_mlp_down_residual_norm_to_bf16_cuda: raw_down_output (already written by the
// down projection) + residual_left -> residual_output, then the next layer's input norm into
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
