// Pointwise operators of the path: residual add, SwiGLU (split and merged layouts), the attention
// sigmoid output gate, FP32 -> bf16 conversion and the q|gate de-interleave.
//
// All are pure HBM streams: three (or two) coalesced 128-bit accesses per eight elements.  A
// thread keeps UNROLL independent 128-bit loads per operand in flight (grid-stride with the
// stride of the whole grid, so every warp access is one contiguous 512-byte segment), and the grid
// is a multiple of the SM count.  Tails that are not a multiple of eight elements, and pointers
// that are not 16-byte aligned, go through a scalar kernel computing the same values.
#include "device_utils.cuh"
#include "host_checks.hpp"
#include "norm_math.cuh"
#include "pointwise_ops.cuh"
#include "q3x_b200.h"

namespace q3x {
namespace {

constexpr int kThreads = 256;

template <class Op>
__device__ __forceinline__ uint4 apply8(const uint4& a, const uint4& b) {
  uint4 o;
  o.x = pack_bf16x2(Op::apply(bf16_lo(a.x), bf16_lo(b.x)), Op::apply(bf16_hi(a.x), bf16_hi(b.x)));
  o.y = pack_bf16x2(Op::apply(bf16_lo(a.y), bf16_lo(b.y)), Op::apply(bf16_hi(a.y), bf16_hi(b.y)));
  o.z = pack_bf16x2(Op::apply(bf16_lo(a.z), bf16_lo(b.z)), Op::apply(bf16_hi(a.z), bf16_hi(b.z)));
  o.w = pack_bf16x2(Op::apply(bf16_lo(a.w), bf16_lo(b.w)), Op::apply(bf16_hi(a.w), bf16_hi(b.w)));
  return o;
}

// kInPlace: the output is exactly one of the inputs, so loads must be coherent ones and the input
// pointers carry no __restrict__ (the out-of-place instantiation reads through ld.global.nc explicitly,
// so it loses nothing by that).
template <class Op, bool kInPlace>
__global__ void __launch_bounds__(kThreads) binary_vec_kernel(const uint4* a, const uint4* b, uint4* out,
                                                              size_t nvec) {
  constexpr int kDepth = Op::kDepth;
  release_next_kernel();
  wait_for_prior_kernels();
  auto store = [](uint4* p, const uint4& v) {
    if (Op::kStreamingStore) st_stream(p, v);
    else st_vec(p, v);
  };
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (kDepth - 1) * stride < nvec; i += kDepth * stride) {
    uint4 va[kDepth], vb[kDepth];
#pragma unroll
    for (int k = 0; k < kDepth; ++k) {
      va[k] = kInPlace ? ld_vec(a + i + k * stride) : ld_stream(a + i + k * stride);
      vb[k] = kInPlace ? ld_vec(b + i + k * stride) : ld_stream(b + i + k * stride);
    }
#pragma unroll
    for (int k = 0; k < kDepth; ++k) store(out + i + k * stride, apply8<Op>(va[k], vb[k]));
  }
  for (; i < nvec; i += stride) {
    const uint4 va = kInPlace ? ld_vec(a + i) : ld_stream(a + i);
    const uint4 vb = kInPlace ? ld_vec(b + i) : ld_stream(b + i);
    store(out + i, apply8<Op>(va, vb));
  }
}

template <class Op>
__global__ void __launch_bounds__(kThreads) binary_scalar_kernel(const uint16_t* a, const uint16_t* b,
                                                                 uint16_t* out, size_t begin, size_t end) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = begin + static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < end; i += stride)
    out[i] = float_to_bf16(Op::apply(bf16_to_float(a[i]), bf16_to_float(b[i])));
}

// Merged SwiGLU: row t holds gate in [0,I) and up in [I,2I).  One thread per output vector;
// vectors_per_row = I/8.
__global__ void __launch_bounds__(kThreads) silu_mul_merged_vec_kernel(const uint4* __restrict__ merged,
                                                                       uint4* __restrict__ out, size_t nvec,
                                                                       unsigned vectors_per_row) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i < nvec; i += SiluMul::kDepth * stride) {
    uint4 g[SiluMul::kDepth], u[SiluMul::kDepth];
#pragma unroll
    for (int k = 0; k < SiluMul::kDepth; ++k) {
      const size_t j = i + k * stride;
      if (j < nvec) {
        const size_t row = j / vectors_per_row;
        const size_t col = j - row * vectors_per_row;
        const uint4* base = merged + row * 2 * vectors_per_row + col;
        g[k] = ld_stream(base);
        u[k] = ld_stream(base + vectors_per_row);
      }
    }
#pragma unroll
    for (int k = 0; k < SiluMul::kDepth; ++k) {
      const size_t j = i + k * stride;
      if (j < nvec) st_stream(out + j, apply8<SiluMul>(g[k], u[k]));
    }
  }
}

__global__ void __launch_bounds__(kThreads) silu_mul_merged_scalar_kernel(const uint16_t* merged, uint16_t* out,
                                                                          size_t count, size_t intermediate) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < count; i += stride) {
    const size_t row = i / intermediate, col = i - row * intermediate;
    const uint16_t* base = merged + row * 2 * intermediate + col;
    out[i] = float_to_bf16(SiluMul::apply(bf16_to_float(base[0]), bf16_to_float(base[intermediate])));
  }
}

__global__ void __launch_bounds__(kThreads) fp32_to_bf16_kernel(const float* __restrict__ in, uint16_t* __restrict__ out,
                                                                size_t count) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < count; i += stride)
    out[i] = float_to_bf16_exact(in[i]);
}

// Diagnostics: the FP32 building blocks of the operators, one value in, one value out, so that tests can
// bound their error against the host reference's libm forms.
__global__ void __launch_bounds__(kThreads) debug_intermediate_kernel(const float* in, size_t count, int function,
                                                                      float p0, float p1, float* out) {
  const size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (i >= count) return;
  const float x = in[i];
  float y;
  switch (function) {
    case 0: y = inverse_rms(x, 1.0f / p0, p1); break;
    case 1: y = inverse_l2(x, p1); break;
    case 2: y = silu(x); break;
    case 3: y = silu_unscaled(x); break;
    case 4: y = stable_sigmoid(x); break;
    default: y = exp_neg_abs(x); break;
  }
  out[i] = y;
}

// q|gate de-interleave: in [heads, 2, dim] -> q [heads, dim], gate [heads, dim]; raw bits.
template <typename T>
__global__ void __launch_bounds__(kThreads) split_q_gate_kernel(const T* __restrict__ in, T* __restrict__ q,
                                                                T* __restrict__ gate, size_t total_out,
                                                                size_t dim_units) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < total_out; i += stride) {
    const size_t head = i / dim_units, d = i - head * dim_units;
    const T* src = in + head * 2 * dim_units + d;
    q[i] = src[0];
    gate[i] = src[dim_units];
  }
}

template <class Op>
int launch_binary(const uint16_t* a, const uint16_t* b, size_t count, uint16_t* out, bool inputs_may_alias,
                  void* stream) {
  using namespace host;
  if (count == 0) return kOk;
  if (a == nullptr || b == nullptr || out == nullptr || mul_overflows(count, sizeof(uint16_t))) return kInvalid;
  const size_t bytes = count * sizeof(uint16_t);
  const Span sa = span(a, bytes), sb = span(b, bytes), so = span(out, bytes);
  if (wraps(sa) || wraps(sb) || wraps(so)) return kInvalid;
  if (!inputs_may_alias && overlap(sa, sb)) return kInvalid;
  if (partial_overlap(so, sa) || partial_overlap(so, sb)) return kInvalid;
  const bool in_place = (out == a) || (out == b);
  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  size_t done = 0;
  if (aligned16(a) && aligned16(b) && aligned16(out) && count >= 8) {
    const size_t nvec = count / 8;
    const unsigned grid = in_place ? wave_grid(binary_vec_kernel<Op, true>, kThreads, nvec, kThreads * Op::kDepth)
                                   : wave_grid(binary_vec_kernel<Op, false>, kThreads, nvec, kThreads * Op::kDepth);
    launch_kernel(in_place ? binary_vec_kernel<Op, true> : binary_vec_kernel<Op, false>, grid, kThreads, 0, s,
                  latency_bound_launch(grid), reinterpret_cast<const uint4*>(a), reinterpret_cast<const uint4*>(b),
                  reinterpret_cast<uint4*>(out), nvec);
    done = nvec * 8;
  }
  if (done < count) {
    const unsigned grid = grid_for(count - done, kThreads, 8);
    binary_scalar_kernel<Op><<<grid, kThreads, 0, s>>>(a, b, out, done, count);
  }
  return launch_status();
}

}  // namespace
}  // namespace q3x

using namespace q3x;
using namespace q3x::host;

extern "C" int q3x_b200_residual_add(const uint16_t* left, const uint16_t* right, size_t count, uint16_t* out,
                                     void* stream) {
  return launch_binary<ResidualAdd>(left, right, count, out, /*inputs_may_alias=*/false, stream);
}

extern "C" int q3x_b200_silu_mul(const uint16_t* gate, const uint16_t* up, size_t count, uint16_t* out,
                                 void* stream) {
  return launch_binary<SiluMul>(gate, up, count, out, /*inputs_may_alias=*/true, stream);
}

extern "C" int q3x_b200_sigmoid_gate(const uint16_t* value, const uint16_t* gate, size_t count, uint16_t* out,
                                     void* stream) {
  return launch_binary<SigmoidGate>(value, gate, count, out, /*inputs_may_alias=*/true, stream);
}

extern "C" int q3x_b200_silu_mul_merged(const uint16_t* merged, size_t tokens, size_t intermediate, uint16_t* out,
                                        void* stream) {
  if (mul3_overflows(tokens, intermediate, 2 * sizeof(uint16_t))) return kInvalid;
  if (tokens == 0 || intermediate == 0) return kOk;
  if (merged == nullptr || out == nullptr) return kInvalid;
  const size_t count = tokens * intermediate;
  const Span sm = span(merged, count * 2 * sizeof(uint16_t)), so = span(out, count * sizeof(uint16_t));
  if (wraps(sm) || wraps(so) || overlap(sm, so)) return kInvalid;
  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  if (intermediate % 8 == 0 && intermediate / 8 <= 0xffffffffu && aligned16(merged) && aligned16(out)) {
    const size_t nvec = count / 8;
    silu_mul_merged_vec_kernel<<<wave_grid(silu_mul_merged_vec_kernel, kThreads, nvec, kThreads * SiluMul::kDepth), kThreads,
                                 0, s>>>(
        reinterpret_cast<const uint4*>(merged), reinterpret_cast<uint4*>(out), nvec,
        static_cast<unsigned>(intermediate / 8));
  } else {
    silu_mul_merged_scalar_kernel<<<grid_for(count, kThreads, 8), kThreads, 0, s>>>(merged, out, count,
                                                                                     intermediate);
  }
  return launch_status();
}

extern "C" int q3x_b200_fp32_to_bf16(const float* in, size_t count, uint16_t* out, void* stream) {
  if (count == 0) return kOk;
  if (in == nullptr || out == nullptr || mul_overflows(count, sizeof(float))) return kInvalid;
  const Span si = span(in, count * sizeof(float)), so = span(out, count * sizeof(uint16_t));
  if (wraps(si) || wraps(so) || overlap(si, so)) return kInvalid;
  clear_stale_error();
  fp32_to_bf16_kernel<<<grid_for(count, kThreads, 8), kThreads, 0, as_stream(stream)>>>(in, out, count);
  return launch_status();
}

extern "C" int q3x_b200_split_interleaved_q_gate(const uint16_t* in, size_t heads, size_t dim, uint16_t* q_out,
                                                 uint16_t* gate_out, void* stream) {
  if (mul3_overflows(heads, dim, 2 * sizeof(uint16_t))) return kInvalid;
  if (heads == 0 || dim == 0) return kOk;
  if (in == nullptr || q_out == nullptr || gate_out == nullptr) return kInvalid;
  const size_t out_bytes = heads * dim * sizeof(uint16_t);
  const Span si = span(in, 2 * out_bytes), sq = span(q_out, out_bytes), sg = span(gate_out, out_bytes);
  if (wraps(si) || wraps(sq) || wraps(sg) || overlap(si, sq) || overlap(si, sg) || overlap(sq, sg)) return kInvalid;
  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  if (dim % 8 == 0 && aligned16(in) && aligned16(q_out) && aligned16(gate_out)) {
    const size_t total = heads * dim / 8;
    split_q_gate_kernel<uint4><<<grid_for(total, kThreads, 8), kThreads, 0, s>>>(
        reinterpret_cast<const uint4*>(in), reinterpret_cast<uint4*>(q_out), reinterpret_cast<uint4*>(gate_out),
        total, dim / 8);
  } else {
    const size_t total = heads * dim;
    split_q_gate_kernel<uint16_t><<<grid_for(total, kThreads, 8), kThreads, 0, s>>>(in, q_out, gate_out, total, dim);
  }
  return launch_status();
}

extern "C" int q3x_b200_debug_intermediate(const float* in, size_t count, int function, float p0, float p1,
                                           float* out, void* stream) {
  if (count == 0) return kOk;
  if (in == nullptr || out == nullptr || function < 0 || function > 5 || mul_overflows(count, sizeof(float)))
    return kInvalid;
  if (function == 0 && !(p0 > 0.0f)) return kInvalid;
  clear_stale_error();
  debug_intermediate_kernel<<<static_cast<unsigned>((count + kThreads - 1) / kThreads), kThreads, 0,
                              as_stream(stream)>>>(in, count, function, p0, p1, out);
  return launch_status();
}
