// Batch-one projections (GEMV): out[r] = sum_c W[r,c] * x[c] for bf16, FP8 (E4M3, per-tensor scale) and NVFP4
// (E2M1 codes, E4M3 block scales per 16 columns, FP32 second-level scale) weights against a bf16 activation,
// FP32 accumulation -- bf16_gemv / fp8_gemv / nvfp4_gemv_reference_cpu
// (src/kernels/reference/gemv_reference.cpp:84-140,179-225).  These are what the decode step runs between the
// fused layer operators; a batch-one projection reads every weight byte once and does two flops with it, so it
// is an HBM stream like the rest of this library and runs on the FP32 pipes (a single activation column is no
// tile for tensor cores).
//
// Layout of the work: a warp owns kRows consecutive output rows and walks their columns together, a lane
// taking one 128-bit vector of each row per trip, so the activation vector (read through L1, it is a few tens
// of KB and shared by every warp of the SM) is unpacked once for kRows rows.  Narrow weights are widened with
// the hardware conversions (cvt e2m1x2 / e4m3x2 -> f16x2 -> f32); NVFP4 rows form each block's 16-term dot
// product first and scale it once by decode(block scale) * scale_2.  Lane partial sums are combined with a
// shuffle tree; the result is written as FP32, as bf16 (round to nearest even), or both.
#include "device_utils.cuh"
#include "host_checks.hpp"
#include "q3x_b200.h"

namespace q3x {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kRows = 2;  // rows per warp

__device__ __forceinline__ float2 half2_to_float2(uint32_t h) {
  float2 f;
  asm("{\n.reg .f16 lo, hi;\nmov.b32 {lo, hi}, %2;\ncvt.f32.f16 %0, lo;\ncvt.f32.f16 %1, hi;\n}"
      : "=f"(f.x), "=f"(f.y)
      : "r"(h));
  return f;
}
// four bytes of E2M1 pairs -> eight floats (low nibble first)
__device__ __forceinline__ void e2m1x8_to_float(uint32_t word, float (&f)[8]) {
  uint32_t h0, h1, h2, h3;
  asm("{\n.reg .b8 b0, b1, b2, b3;\nmov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\ncvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\ncvt.rn.f16x2.e2m1x2 %3, b3;\n}"
      : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3)
      : "r"(word));
  const float2 a = half2_to_float2(h0), b = half2_to_float2(h1), c = half2_to_float2(h2), d = half2_to_float2(h3);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
// two E4M3 bytes -> two floats (low byte first); exact, sign and NaN included
__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t pair) {
  uint32_t h;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"(static_cast<uint16_t>(pair)));
  return half2_to_float2(h);
}
__device__ __forceinline__ void e4m3x4_to_float(uint32_t word, float (&f)[4]) {
  const float2 a = e4m3x2_to_float2(word & 0xffffu), b = e4m3x2_to_float2(word >> 16);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// sum of w[i] * x[i] over eight terms, two per instruction, added to acc
__device__ __forceinline__ float dot8_acc(const float (&w)[8], const float (&x)[8], float acc) {
  float2 s = make_float2(acc, 0.0f);
#pragma unroll
  for (int i = 0; i < 8; i += 2) s = fma2(make_float2(w[i], w[i + 1]), make_float2(x[i], x[i + 1]), s);
  return s.x + s.y;
}

struct Bf16Weights {
  const uint4* w;       // [rows, cols / 8] vectors
  static constexpr int kColsPerVector = 8;
};
struct Fp8Weights {
  const uint4* w;       // [rows, cols / 16]
  float scale;
  static constexpr int kColsPerVector = 16;
};
struct NvFp4Weights {
  const uint4* w;             // [rows, cols / 32]
  const uint16_t* scales;     // [rows, cols / 32] pairs of E4M3 bytes
  float scale_2;
  static constexpr int kColsPerVector = 32;
};

// partial dot product of one weight vector with the matching activation floats
__device__ __forceinline__ float accumulate(const Bf16Weights&, const uint4& w, uint32_t, const float* x, float acc) {
  float wf[8];
  unpack8(w, wf);
  return dot8_acc(wf, *reinterpret_cast<const float(*)[8]>(x), acc);
}
__device__ __forceinline__ float accumulate(const Fp8Weights&, const uint4& w, uint32_t, const float* x, float acc) {
  const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int k = 0; k < 4; k += 2) {
    float a[4], b[4];
    e4m3x4_to_float(words[k], a);
    e4m3x4_to_float(words[k + 1], b);
    const float wf[8] = {a[0], a[1], a[2], a[3], b[0], b[1], b[2], b[3]};
    acc = dot8_acc(wf, *reinterpret_cast<const float(*)[8]>(x + 4 * k), acc);
  }
  return acc;
}
__device__ __forceinline__ float accumulate(const NvFp4Weights& fmt, const uint4& w, uint32_t scale_pair,
                                            const float* x, float acc) {
  const uint32_t words[4] = {w.x, w.y, w.z, w.w};
  const float2 s = e4m3x2_to_float2(scale_pair);
#pragma unroll
  for (int block = 0; block < 2; ++block) {
    float wf[8];
    e2m1x8_to_float(words[2 * block], wf);
    float dot = dot8_acc(wf, *reinterpret_cast<const float(*)[8]>(x + 16 * block), 0.0f);
    e2m1x8_to_float(words[2 * block + 1], wf);
    dot = dot8_acc(wf, *reinterpret_cast<const float(*)[8]>(x + 16 * block + 8), dot);
    acc = fmaf(dot, (block == 0 ? s.x : s.y) * fmt.scale_2, acc);
  }
  return acc;
}

template <class Format>
__global__ void __launch_bounds__(kThreads) gemv_kernel(Format fmt, const uint4* __restrict__ x, size_t rows,
                                                        int row_vectors, float* out_f32, uint16_t* out_bf16) {
  constexpr int kXVectors = Format::kColsPerVector / 8;  // activation vectors per weight vector
  const int lane = threadIdx.x & 31;
  const size_t first_row = (static_cast<size_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5)) * kRows;
  if (first_row >= rows) return;
  const uint4* row_ptr[kRows];
  const uint16_t* scale_ptr[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    const size_t row = min(first_row + r, rows - 1);  // a missing last row repeats the one before (not stored)
    row_ptr[r] = fmt.w + row * static_cast<size_t>(row_vectors);
    if constexpr (std::is_same<Format, NvFp4Weights>::value) scale_ptr[r] = fmt.scales + row * static_cast<size_t>(row_vectors);
    else scale_ptr[r] = nullptr;
  }
  float acc[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) acc[r] = 0.0f;

  // kDepth trips are requested before the first is used: 2 x kDepth 128-bit loads per lane in flight
  constexpr int kDepth = 4;
  for (int base = lane; base < row_vectors; base += 32 * kDepth) {
    uint4 w[kDepth][kRows];
    uint32_t sp[kDepth][kRows];
#pragma unroll
    for (int d = 0; d < kDepth; ++d) {
      const int v = base + 32 * d;
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        w[d][r] = make_uint4(0, 0, 0, 0);
        sp[d][r] = 0;
        if (v < row_vectors) {
          w[d][r] = ld_stream(row_ptr[r] + v);
          if constexpr (std::is_same<Format, NvFp4Weights>::value) sp[d][r] = __ldg(scale_ptr[r] + v);
        }
      }
    }
#pragma unroll
    for (int d = 0; d < kDepth; ++d) {
      const int v = base + 32 * d;
      if (v < row_vectors) {
        float xf[kXVectors * 8];
#pragma unroll
        for (int k = 0; k < kXVectors; ++k)
          unpack8(ld_weight(x + static_cast<size_t>(v) * kXVectors + k), *reinterpret_cast<float(*)[8]>(xf + 8 * k));
#pragma unroll
        for (int r = 0; r < kRows; ++r) acc[r] = accumulate(fmt, w[d][r], sp[d][r], xf, acc[r]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    float total = group_sum<32>(acc[r]);
    if constexpr (std::is_same<Format, Fp8Weights>::value) total *= fmt.scale;
    if (lane == 0 && first_row + r < rows) {
      if (out_f32 != nullptr) out_f32[first_row + r] = total;
      if (out_bf16 != nullptr) out_bf16[first_row + r] = float_to_bf16(total);
    }
  }
}

// Any shape and alignment: one thread per row, the reference's own left-to-right sum.
enum class Kind { kBf16, kFp8, kNvFp4 };
__global__ void __launch_bounds__(128) gemv_scalar_kernel(Kind kind, const void* weights, const uint8_t* block_scales,
                                                          float scale, const uint16_t* x, size_t rows, size_t cols,
                                                          float* out_f32, uint16_t* out_bf16) {
  const size_t row = static_cast<size_t>(blockIdx.x) * 128 + threadIdx.x;
  if (row >= rows) return;
  float sum = 0.0f;
  for (size_t c = 0; c < cols; ++c) {
    float w;
    if (kind == Kind::kBf16) {
      w = bf16_to_float(static_cast<const uint16_t*>(weights)[row * cols + c]);
    } else if (kind == Kind::kFp8) {
      w = e4m3x2_to_float2(static_cast<const uint8_t*>(weights)[row * cols + c]).x * scale;
    } else {
      const uint8_t byte = static_cast<const uint8_t*>(weights)[row * (cols / 2) + c / 2];
      float f[8];
      e2m1x8_to_float((c & 1) ? (byte >> 4) : (byte & 0xfu), f);
      w = f[0] * e4m3x2_to_float2(block_scales[row * (cols / 16) + c / 16]).x * scale;
    }
    sum += w * bf16_to_float(x[c]);
  }
  if (out_f32 != nullptr) out_f32[row] = sum;
  if (out_bf16 != nullptr) out_bf16[row] = float_to_bf16(sum);
}

int launch_gemv(Kind kind, const void* weights, const uint8_t* block_scales, float scale, const uint16_t* x, size_t rows,
                size_t cols, float* out_f32, uint16_t* out_bf16, void* stream) {
  using namespace host;
  if (kind == Kind::kNvFp4 && cols % Q3X_B200_NVFP4_BLOCK != 0) return kInvalid;
  if (kind != Kind::kBf16 && !(std::isfinite(scale) && scale >= 0.0f)) return kInvalid;
  if (mul3_overflows(rows, cols, sizeof(uint16_t))) return kInvalid;
  if (rows == 0 || cols == 0) return kOk;
  if (weights == nullptr || x == nullptr || (out_f32 == nullptr && out_bf16 == nullptr) ||
      (kind == Kind::kNvFp4 && block_scales == nullptr))
    return kInvalid;
  const size_t weight_bytes = kind == Kind::kBf16 ? rows * cols * 2 : kind == Kind::kFp8 ? rows * cols : rows * cols / 2;
  const Span sw = span(weights, weight_bytes), ss = span(block_scales, kind == Kind::kNvFp4 ? rows * cols / 16 : 0),
             sx = span(x, cols * 2), s32 = span(out_f32, out_f32 ? rows * 4 : 0), s16 = span(out_bf16, out_bf16 ? rows * 2 : 0);
  if (wraps(sw) || wraps(ss)) return kInvalid;
  // the outputs are disjoint from every input and from each other; the read-only operands may alias
  for (const Span& o : {s32, s16})
    if (overlap(o, sw) || overlap(o, ss) || overlap(o, sx)) return kInvalid;
  if (overlap(s32, s16)) return kInvalid;
  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  const size_t cols_per_vector = kind == Kind::kBf16 ? 8 : kind == Kind::kFp8 ? 16 : 32;
  const bool vector_ok = cols % cols_per_vector == 0 && cols / cols_per_vector <= 0x7fffffffu && aligned16(weights) &&
                         aligned16(x) && (kind != Kind::kNvFp4 || (reinterpret_cast<uintptr_t>(block_scales) & 1u) == 0);
  const size_t ctas = (rows + kWarps * kRows - 1) / (kWarps * kRows);
  if (vector_ok && ctas <= 0x7fffffffu) {
    const int row_vectors = static_cast<int>(cols / cols_per_vector);
    auto X = reinterpret_cast<const uint4*>(x);
    auto W = reinterpret_cast<const uint4*>(weights);
    const unsigned grid = static_cast<unsigned>(ctas);
    if (kind == Kind::kBf16)
      gemv_kernel<<<grid, kThreads, 0, s>>>(Bf16Weights{W}, X, rows, row_vectors, out_f32, out_bf16);
    else if (kind == Kind::kFp8)
      gemv_kernel<<<grid, kThreads, 0, s>>>(Fp8Weights{W, scale}, X, rows, row_vectors, out_f32, out_bf16);
    else
      gemv_kernel<<<grid, kThreads, 0, s>>>(NvFp4Weights{W, reinterpret_cast<const uint16_t*>(block_scales), scale}, X,
                                            rows, row_vectors, out_f32, out_bf16);
  } else {
    if ((rows + 127) / 128 > 0x7fffffffu) return kNotSupported;
    gemv_scalar_kernel<<<static_cast<unsigned>((rows + 127) / 128), 128, 0, s>>>(kind, weights, block_scales, scale, x,
                                                                                 rows, cols, out_f32, out_bf16);
  }
  return launch_status();
}

}  // namespace
}  // namespace q3x

extern "C" int q3x_b200_bf16_gemv(const uint16_t* weights, const uint16_t* activation, size_t rows, size_t cols,
                                  float* out_f32, uint16_t* out_bf16, void* stream) {
  return q3x::launch_gemv(q3x::Kind::kBf16, weights, nullptr, 1.0f, activation, rows, cols, out_f32, out_bf16, stream);
}

extern "C" int q3x_b200_fp8_gemv(const uint8_t* weights, float weight_scale, const uint16_t* activation, size_t rows,
                                 size_t cols, float* out_f32, uint16_t* out_bf16, void* stream) {
  return q3x::launch_gemv(q3x::Kind::kFp8, weights, nullptr, weight_scale, activation, rows, cols, out_f32, out_bf16,
                          stream);
}

extern "C" int q3x_b200_nvfp4_gemv(const uint8_t* packed_weights, const uint8_t* block_scales, float weight_scale_2,
                                   const uint16_t* activation, size_t rows, size_t cols, float* out_f32,
                                   uint16_t* out_bf16, void* stream) {
  return q3x::launch_gemv(q3x::Kind::kNvFp4, packed_weights, block_scales, weight_scale_2, activation, rows, cols,
                          out_f32, out_bf16, stream);
}
