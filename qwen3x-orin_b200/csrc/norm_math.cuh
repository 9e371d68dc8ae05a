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

// 1 / sqrt(t) from MUFU.RSQ plus one Newton step: relative error about 2^-23, the accuracy class of
// the IEEE divide / sqrt / divide chain it stands in for, at a fifth of the instructions (every
// lane of a row evaluates it).
__device__ __forceinline__ float refined_rsqrt(float t) {
  float r;
  asm("rsqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(t));
  const float half_t = 0.5f * t;
  const float refined = r * fmaf(-half_t * r, r, 1.5f);
  // an overflowed sum (t = inf) gives r = 0 like the IEEE chain; the Newton step would turn it into NaN
  return t < 3.0e38f ? refined : r;
}

// inverse RMS: 1 / sqrt(sum / n + eps)  (src/runtime/reference/decode_ops.cpp:74-76); inv_n = 1 / n.
// eps > 0 keeps the argument positive and normal; an infinite or NaN sum propagates as 0 / NaN.
__device__ __forceinline__ float inverse_rms(float sum, float inv_n, float eps) {
  return refined_rsqrt(fmaf(sum, inv_n, eps));
}
// inverse L2 norm: 1 / sqrt(sum + eps)  (decode_ops.cpp:369)
__device__ __forceinline__ float inverse_l2(float sum, float eps) { return refined_rsqrt(sum + eps); }

// Scales eight elements; *top (when given) is raised to the largest finite magnitude of the result
// after rounding (see amax8_float).
template <NormMode MODE, bool kTrackAmax = false>
__device__ __forceinline__ uint4 scale8(const uint4& x, const uint4& w, const uint4& z, float inv,
                                        float* top = nullptr) {
  float xf[8], wf[8], zf[8], y[8];
  unpack8(x, xf);
  if (MODE != NormMode::kL2) unpack8(w, wf);
  if (MODE == NormMode::kPlainSiluGate) unpack8(z, zf);
  // two elements per instruction (fma2 / mul2 / add2 round each half like the scalar operation)
  const float2 inv2 = make_float2(inv, inv);
#pragma unroll
  for (int i = 0; i < 8; i += 2) {
    float2 v = mul2(make_float2(xf[i], xf[i + 1]), inv2);
    if (MODE != NormMode::kL2) {
      float2 gamma = make_float2(wf[i], wf[i + 1]);
      if (MODE == NormMode::kCentered) gamma = add2(gamma, make_float2(1.0f, 1.0f));
      v = mul2(v, gamma);  // (x * inv) * gamma, the reference's product order
      if (MODE == NormMode::kPlainSiluGate) v = mul2(v, silu2(make_float2(zf[i], zf[i + 1])));
    }
    y[i] = v.x;
    y[i + 1] = v.y;
  }
  const uint4 packed = pack8(y);
  if (kTrackAmax) *top = fmaxf(*top, amax8_float(y, packed));
  return packed;
}

}  // namespace q3x
