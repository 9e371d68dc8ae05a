// Device arithmetic of the NVFP4 activation quantiser (see nvfp4.cu for the specification):
// the two hardware narrow conversions, the exact E4M3 decode and the per-block reciprocal.
#pragma once

#include <cfloat>

#include "device_utils.cuh"

namespace q3x {

// round-to-nearest-even onto E4M3 with saturation at 448
__device__ __forceinline__ uint32_t encode_e4m3(float v) {
  uint16_t pair;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(0.0f), "f"(v));
  return pair & 0xffu;
}

// Non-negative E4M3 code -> float (exact).
__device__ __forceinline__ float decode_e4m3_positive(uint32_t code) {
  const uint32_t e = (code >> 3) & 0xfu, m = code & 7u;
  if (e == 0) return static_cast<float>(m) * 0.001953125f;     // m * 2^-9
  if (code == 0x7fu) return __uint_as_float(0x7fffffffu);        // NaN (never produced by encode)
  return __uint_as_float(((e + 120u) << 23) | (m << 20));        // (1 + m/8) * 2^(e-7)
}

// Eight floats -> eight E2M1 codes in one word, element i in nibble i (RNE, saturation at 6).
__device__ __forceinline__ uint32_t encode_e2m1x8(const float (&r)[8]) {
  uint32_t out;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "}"
      : "=r"(out)
      : "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]));
  return out;
}

// global scale of a group from its amax bits: A == 0 ? 1 : A / 2688
__device__ __forceinline__ float global_scale_from_amax_bits(uint32_t amax_bits) {
  const float amax = __uint_as_float(amax_bits << 16);
  return amax == 0.0f ? 1.0f : __fdiv_rn(amax, 2688.0f);
}
// k = 1 / (global * 6): multiplies a block amax into the E4M3 scale domain
__device__ __forceinline__ float block_scale_factor(float global) {
  return __fdiv_rn(1.0f, __fmul_rn(global, 6.0f));
}
// E4M3 code of one block scale from the block's amax (magnitude of its largest finite element)
__device__ __forceinline__ uint32_t block_scale_code(float amax, float k) {
  return amax == 0.0f ? 0u : encode_e4m3(__fmul_rn(amax, k));
}
__device__ __forceinline__ uint32_t block_scale_code(uint32_t amax_bits, float k) {
  return block_scale_code(__uint_as_float(amax_bits << 16), k);
}
// inv = d == 0 ? 0 : min(1 / d, FLT_MAX) with d = decode(scale) * global
__device__ __forceinline__ float block_inverse(uint32_t scale_code, float global) {
  const float d = __fmul_rn(decode_e4m3_positive(scale_code), global);
  return d == 0.0f ? 0.0f : fminf(__frcp_rn(d), FLT_MAX);
}
// the eight codes of one vector under a block's reciprocal
__device__ __forceinline__ uint32_t quantize8(const float (&x)[8], float inv) {
  float f[8];
  const float2 inv2 = make_float2(inv, inv);
#pragma unroll
  for (int i = 0; i < 8; i += 2) {  // two products per instruction, each rounded like __fmul_rn
    const float2 p = mul2(make_float2(x[i], x[i + 1]), inv2);
    f[i] = p.x;
    f[i + 1] = p.y;
  }
  return encode_e2m1x8(f);
}
__device__ __forceinline__ uint32_t quantize8(const uint4& x, float inv) {
  float f[8];
  unpack8(x, f);
  return quantize8(f, inv);
}

}  // namespace q3x
