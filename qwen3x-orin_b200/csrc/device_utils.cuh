// Device helpers shared by every kernel of the library: the bfloat16 codec, 128-bit global
// accesses with cache hints, warp / block reductions and the SiLU / sigmoid forms.
//
// Numerical contract (the reference's host ops, src/runtime/reference/decode_ops.cpp:15-33):
// bf16 -> FP32 is exact; FP32 -> bf16 rounds to nearest-even; no fast-math anywhere.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace q3x {

constexpr int kWarp = 32;
constexpr unsigned kFullMask = 0xffffffffu;

// ---------------------------------------------------------------------------- bf16 codec

__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }
__device__ __forceinline__ float bf16_to_float(uint16_t bits) {
  return __uint_as_float(static_cast<uint32_t>(bits) << 16);
}

// Exact integer rule of the reference: RNE, a NaN keeps sign and upper payload and gets the quiet
// bit.  Needed where an FP32 NaN arrives from memory with an arbitrary payload.
__device__ __forceinline__ uint16_t float_to_bf16_exact(float value) {
  uint32_t u = __float_as_uint(value);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

// Two FP32 results of arithmetic -> packed bf16 (first in the low half).  The hardware
// conversion is RNE with overflow to infinity, identical to the integer rule for every
// non-NaN value; a NaN produced by GPU arithmetic is always the canonical 0x7fffffff, which
// both rules map to 0x7fff (sign aside), so the single instruction is exact here.
__device__ __forceinline__ uint32_t pack_bf16x2(float first, float second) {
  uint32_t out;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(out) : "f"(second), "f"(first));
  return out;
}
__device__ __forceinline__ uint16_t float_to_bf16(float value) {
  return static_cast<uint16_t>(pack_bf16x2(value, 0.0f) & 0xffffu);
}

// Eight bf16 (one 128-bit vector) <-> eight floats.
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x);
  f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z);
  f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]);
  v.y = pack_bf16x2(f[2], f[3]);
  v.z = pack_bf16x2(f[4], f[5]);
  v.w = pack_bf16x2(f[6], f[7]);
  return v;
}

// ---------------------------------------------------------------------------- memory

// Streaming 128-bit load: read-only path, no L1 allocation (every byte is used once).
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Plain coherent 128-bit load (for buffers the same launch may also write, e.g. in-place ops).
__device__ __forceinline__ uint4 ld_vec(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st_vec(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }
// Streaming store: the line is not expected to be re-read by this kernel.
__device__ __forceinline__ void st_stream(void* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// Small read-mostly operands (weights, tables): keep them cached.
__device__ __forceinline__ uint4 ld_weight(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// Coherent load served by L2 (data another CTA of the same launch has written): bypasses L1.
__device__ __forceinline__ uint4 ld_l2(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_u32(void* p, uint32_t v) { *reinterpret_cast<uint32_t*>(p) = v; }

// ---------------------------------------------------------------------------- kernel overlap
// Programmatic dependent launch, for the batch-one operators whose cost is mostly the gap between two
// kernels.  A kernel launched with the stream-serialisation attribute (host::launch_kernel) may start
// while the kernel before it in the stream is still running; wait_for_prior_kernels() then blocks until
// that kernel has completed and its writes are visible, and it must come before the kernel's first
// access to global memory.  release_next_kernel() lets the NEXT kernel of the stream start early (it will
// sit in its own wait).  Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void wait_for_prior_kernels() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void release_next_kernel() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------- reductions

template <int LANES>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
  return v;
}
template <int LANES>
__device__ __forceinline__ uint32_t group_max_u32(uint32_t v) {
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(kFullMask, v, o));
  return v;
}

// Sum over a CTA of WARPS warps; every thread receives the total.  `scratch` holds WARPS floats.
template <int WARPS>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = group_sum<32>(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) total += scratch[w];  // same order in every thread
  return total;
}

// ---------------------------------------------------------------------------- activations

// exp(-|g|) in (0, 1] from one MUFU.EX2.  ex2.approx has a relative error of 2^-22; the rounded
// argument adds |g| * 2^-24, so the total stays below 2e-6 for |g| <= 20 and below 1e-5 wherever the
// result is not yet a bf16 subnormal.
// It is evaluated as the square of exp(-|g|/2): the single-instruction (flushing) form of ex2 then
// only flushes beyond |g| = 174, where the result is below every bf16 subnormal anyway, while the
// product keeps FP32 subnormals -- the tail of silu for g in (-92, -87) needs them.
__device__ __forceinline__ float exp_neg_abs(float g) {
  float h;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(h) : "f"(-fabsf(g) * 0.7213475204444817f));
  return h * h;
}
// 1 / b for b in [1, 2]: one MUFU.RCP (relative error 2^-23; no subnormals in this range).
__device__ __forceinline__ float rcp_approx(float b) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(b));
  return r;
}

// sigmoid(g) in the branch-stable form of src/runtime/reference/decode_ops.cpp:334-337, written
// so that both branches share one exponential and one reciprocal: with e = exp(-|g|),
//   g >= 0: 1 / (1 + e)        g < 0: e / (1 + e).
// Nothing can overflow (e <= 1, 1 + e <= 2), so the whole bf16 range of g is handled, including
// gates so negative that the result is a subnormal.  The FP32 error is a few 2^-22, far inside the
// half-ulp of the bf16 rounding that follows, so a result differs from the host op by at most one
// bf16 ulp, and only when the exact value sits within ~1e-6 (relative) of a rounding boundary.
__device__ __forceinline__ float stable_sigmoid(float g) {
  const float e = exp_neg_abs(g);
  const float r = rcp_approx(1.0f + e);
  return (g >= 0.0f ? 1.0f : e) * r;
}

// silu(g) = g / (1 + exp(-g)) (decode_ops.cpp:315-316).
// It is evaluated in exactly that shape, g * (1 / (1 + exp(-g))), with the two fast units: for
// g < -88.72 exp(-g) overflows to +inf, the reciprocal is 0 and the product is -0, just as in the
// host op; for large positive g the exponential vanishes and the result is g.  The exponential may
// flush (1 + tiny == 1), but 1 / (1 + exp(-g)) is subnormal for g in (-88.7, -87.3) and must not be.
// The denominator is carried scaled by 2^-24 so that the single-instruction (flushing) reciprocal never
// sees or produces a subnormal; the scale is folded back into the reciprocal before it meets g, in a
// multiply that keeps subnormals.  Six instructions, none on the integer/logic pipe.
__device__ __forceinline__ float silu(float g) {
  constexpr float kScale = 5.9604644775390625e-08f;  // 2^-24
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(fmaf(e, kScale, kScale)));  // 1 / ((1 + e) * 2^-24)
  return g * (r * kScale);
}

// The same function with the denominator left unscaled and the reciprocal in its subnormal-keeping form
// (MUFU.RCP plus a range fix-up).  Same accuracy class (the two can differ in the last bit of a subnormal
// reciprocal, i.e. for g below -87); measured faster than the form above in
// the HBM-bound SwiGLU kernel and slower in the instruction-bound conv / gated-norm kernels.
__device__ __forceinline__ float silu_unscaled(float g) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
  asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return g * r;
}

// ---------------------------------------------------------------------------- packed FP32 pairs
// sm_100 executes FP32 add / mul / fma on two independent values per instruction (operands in 64-bit
// register pairs).  Each half is the ordinary round-to-nearest IEEE operation with denormals kept, so
// results are bit-identical to the scalar instructions; what halves is the number of issue slots, which
// is what bounds the instruction-heavy kernels here (conv, gated norm, quantiser).
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ float2 unpack_f32x2(uint64_t v) {
  float2 f;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(f.x), "=f"(f.y) : "l"(v));
  return f;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(pack_f32x2(a.x, a.y)), "l"(pack_f32x2(b.x, b.y)),
      "l"(pack_f32x2(c.x, c.y)));
  return unpack_f32x2(d);
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack_f32x2(a.x, a.y)), "l"(pack_f32x2(b.x, b.y)));
  return unpack_f32x2(d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack_f32x2(a.x, a.y)), "l"(pack_f32x2(b.x, b.y)));
  return unpack_f32x2(d);
}
// a[i] += b[i] for eight values, two per instruction
__device__ __forceinline__ void add8(float (&a)[8], const float (&b)[8]) {
#pragma unroll
  for (int i = 0; i < 8; i += 2) {
    const float2 s = add2(make_float2(a[i], a[i + 1]), make_float2(b[i], b[i + 1]));
    a[i] = s.x;
    a[i + 1] = s.y;
  }
}
// silu of two values: the scalar form above with its multiplies and its fma issued pairwise
__device__ __forceinline__ float2 silu2(float2 g) {
  constexpr float kScale = 5.9604644775390625e-08f;  // 2^-24
  const float2 arg = mul2(g, make_float2(-1.4426950408889634f, -1.4426950408889634f));
  float2 e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(arg.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(arg.y));
  const float2 den = fma2(e, make_float2(kScale, kScale), make_float2(kScale, kScale));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.x) : "f"(den.x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.y) : "f"(den.y));
  return mul2(g, mul2(r, make_float2(kScale, kScale)));
}

// ---------------------------------------------------------------------------- bf16 amax

// Magnitude bits of the finite halves of a packed bf16 pair, non-finite halves give 0; bf16
// magnitudes order like their bit patterns, so an unsigned max of these is the amax.
__device__ __forceinline__ uint32_t finite_mag2(uint32_t packed) {
  const uint32_t m = packed & 0x7fff7fffu;
  const uint32_t keep = __vcmpltu2(m, 0x7f807f80u);  // 0xffff per half where finite
  return m & keep;
}
__device__ __forceinline__ uint32_t amax8(const uint4& v) {
  uint32_t m = __vmaxu2(__vmaxu2(finite_mag2(v.x), finite_mag2(v.y)),
                        __vmaxu2(finite_mag2(v.z), finite_mag2(v.w)));
  return max(m & 0xffffu, m >> 16);
}

// The same amax from FP32 values, eight at a time, for kernels that hold the values as floats anyway
// (seven FMNMX instead of the packed-integer sequence).  Two facts make it exact:
//   * fmaxf ignores NaN operands, which is the "finite elements only" rule for NaN;
//   * round-to-nearest-even is monotonic and symmetric, so the largest ROUNDED magnitude equals the
//     rounding of the largest unrounded magnitude.
// What is left is a magnitude that is, or rounds to, infinity: it has to be excluded, and the next
// largest is not known from a running maximum, so that (rare) case is recomputed from the packed
// bf16 bits with the integer sequence above.  `packed` holds the eight values after rounding.
constexpr float kRoundsToBf16Inf = 3.3961775e38f;  // midpoint of the largest finite bf16 and 2^128
__device__ __forceinline__ float amax8_float(const float (&f)[8], const uint4& packed) {
  float t = fmaxf(fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3]))),
                  fmaxf(fmaxf(fabsf(f[4]), fabsf(f[5])), fmaxf(fabsf(f[6]), fabsf(f[7]))));
  if (t >= kRoundsToBf16Inf) t = __uint_as_float(amax8(packed) << 16);
  return t;
}
// bf16 magnitude bits of a non-negative amax accumulated with amax8_float
__device__ __forceinline__ uint32_t amax_bits_of(float t) { return float_to_bf16(t); }

}  // namespace q3x
