// Arithmetic shared by the row-norm kernels: the sum of squares of one 128-bit vector, the inverse
// RMS exactly as the host reference spells it, and the scaling of eight elements in each mode.
#pragma once

#include "device_utils.cuh"
#include "internal.hpp"

namespace q3x {

__device__ __forceinline__ float sum_squares8(const uint4& v) {
  float f[8];
  unpack8(v, f);
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s = fmaf(f[i], f[i], s);
  return s;
}

// 1 / sqrt(sum / n + eps)  (src/runtime/reference/decode_ops.cpp:74-76)
__device__ __forceinline__ float inverse_rms(float sum, float n, float eps) {
  return 1.0f / sqrtf(__fadd_rn(__fdiv_rn(sum, n), eps));
}

template <NormMode MODE>
__device__ __forceinline__ uint4 scale8(const uint4& x, const uint4& w, const uint4& z, float inv) {
  float xf[8], wf[8], zf[8], y[8];
  unpack8(x, xf);
  if (MODE != NormMode::kL2) unpack8(w, wf);
  if (MODE == NormMode::kPlainSiluGate) unpack8(z, zf);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (MODE == NormMode::kL2) {
      y[i] = xf[i] * inv;
    } else {
      const float gamma = MODE == NormMode::kCentered ? wf[i] + 1.0f : wf[i];
      y[i] = xf[i] * inv * gamma;  // (x * inv) * gamma, the reference's product order
      if (MODE == NormMode::kPlainSiluGate) y[i] *= silu(zf[i]);
    }
  }
  return pack8(y);
}

}  // namespace q3x
