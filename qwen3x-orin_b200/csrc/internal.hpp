// Declarations shared between the translation units of libq3x_b200.so (not part of the ABI).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace q3x {

enum class NormMode : int {
  kCentered = 0,       // y = x * inv_rms * (1 + w)
  kPlain = 1,          // y = x * inv_rms * w
  kPlainSiluGate = 2,  // y = x * inv_rms * w * silu(z)
  kL2 = 3,             // y = x * scale / sqrt(sum x^2 + eps)
};

// Enqueues the row-norm kernel that fits the shape; arguments are already validated.
//   a / b        input (or left / right when residual_out != nullptr)
//   out          normalised rows (nullptr allowed only together with residual_out)
//   coherent     an output aliases an input exactly: use coherent loads
//   amax_bits    when non-null, atomically raised to the bf16 magnitude bits of the largest
//                finite output of each group of rows_per_amax_group rows (vector paths only)
void launch_norm_rows(NormMode mode, const uint16_t* a, const uint16_t* b, const uint16_t* weight,
                      const uint16_t* gate, size_t rows, size_t width, float eps, float l2_scale,
                      uint16_t* residual_out, uint16_t* out, bool coherent, uint32_t* amax_bits,
                      size_t rows_per_amax_group, cudaStream_t stream);

bool norm_rows_vector_path(const void* a, const void* b, const void* weight, const void* gate, size_t width,
                           const void* residual_out, const void* out, NormMode mode);

int check_residual_norm(const uint16_t* left, const uint16_t* right, const uint16_t* weight, size_t tokens,
                        size_t hidden, float eps, const uint16_t* residual_out, const uint16_t* normalized_out,
                        bool* done);

}  // namespace q3x

namespace q3x {

// Scratch words (uint32) of the NVFP4 entry points for `groups` scale groups:
// either [0,rows) per-row amax words (single-pass kernels) or [0,G) group amax words (multi-kernel
// path); the last word is the error flag.
size_t fused_scratch_words(size_t rows, size_t groups);

// Single-pass kernels (fused_nvfp4.cu).  Return false, with nothing enqueued, when the fused path does
// not apply; the caller then takes the multi-kernel path, which produces the same bytes.
bool launch_residual_norm_nvfp4_fused(const uint16_t* left, const uint16_t* right, const uint16_t* weight,
                                      size_t tokens, size_t hidden, float eps, size_t rows_per_scale,
                                      uint16_t* residual_out, uint16_t* normalized_out, uint32_t* scratch,
                                      float* global_scales_out, uint8_t* codes, uint8_t* scales, cudaStream_t s);
bool launch_silu_mul_nvfp4_fused(const uint16_t* gate, const uint16_t* up, size_t tokens, size_t intermediate,
                                 size_t rows_per_scale, uint16_t* out, uint32_t* scratch, float* global_scales_out,
                                 uint8_t* codes, uint8_t* scales, cudaStream_t s);
bool launch_sigmoid_gate_nvfp4_fused(const uint16_t* value, const uint16_t* gate, size_t tokens, size_t width,
                                     size_t rows_per_scale, uint16_t* out, uint32_t* scratch,
                                     float* global_scales_out, uint8_t* codes, uint8_t* scales, cudaStream_t s);
bool launch_gated_norm_nvfp4_fused(const uint16_t* in, const uint16_t* weight, const uint16_t* gate, size_t tokens,
                                   size_t heads_per_row, size_t dim, float eps, size_t rows_per_scale, uint16_t* out,
                                   uint32_t* scratch, float* global_scales_out, uint8_t* codes, uint8_t* scales,
                                   cudaStream_t s);

}  // namespace q3x
