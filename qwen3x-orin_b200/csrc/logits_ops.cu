// The two operators next to the path that work on logits / scores: row softmax over FP32 scores
// (softmax_reference_cpu, src/runtime/reference/decode_ops.cpp:413-443) and the greedy argmax over a
// bf16 logits vector (bf16_greedy_argmax_kernel, src/kernels/reference/decode_ops.cu:246-345).
#include "device_utils.cuh"
#include "host_checks.hpp"
#include "q3x_b200.h"

namespace q3x {
namespace {

constexpr int kThreads = 256;
constexpr int kArgmaxBlocks = 32;  // partial results 1..32 of the workspace; element 0 is the answer
constexpr uint32_t kNoIndex = 0xffffffffu;

// ---- softmax ---------------------------------------------------------------------------------------
// One CTA per row (grid-stride over rows): maximum, denominator, quotients -- three sweeps over a row that
// is read from L2 after the first.  exp is the accurate one: the result is an FP32 output, not a value on
// its way to a bf16 rounding.
__global__ void __launch_bounds__(kThreads) softmax_rows_kernel(const float* in, size_t rows, size_t cols, float* out) {
  __shared__ float scratch[kThreads / 32];
  __shared__ float broadcast;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* x = in + row * cols;
    float* y = out + row * cols;
    float m = -INFINITY;
    for (size_t c = threadIdx.x; c < cols; c += kThreads) m = fmaxf(m, x[c]);  // fmaxf skips NaN like std::max(m, x)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(kFullMask, m, o));
    if (lane == 0) scratch[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = scratch[0];
      for (int w = 1; w < kThreads / 32; ++w) t = fmaxf(t, scratch[w]);
      broadcast = t;
    }
    __syncthreads();
    m = broadcast;
    float sum = 0.0f;
    for (size_t c = threadIdx.x; c < cols; c += kThreads) sum += expf(x[c] - m);
    __syncthreads();  // scratch and broadcast are reused
    const float total = block_sum<kThreads / 32>(sum, scratch);
    for (size_t c = threadIdx.x; c < cols; c += kThreads) y[c] = __fdiv_rn(expf(x[c] - m), total);
    __syncthreads();
  }
}

// ---- greedy argmax ---------------------------------------------------------------------------------------
struct Best {
  float value;
  uint32_t index;
  uint32_t bits;       // bf16 payload of the selected element
  uint32_t nonfinite;  // any NaN / infinity seen
};
// The reference's selection rule: a candidate replaces the incumbent when the incumbent is empty, when it is
// larger, or when it is equal (signed zeros compare equal) and has the smaller index.
__device__ __forceinline__ Best better(const Best& a, const Best& b) {
  const bool take_b = b.index != kNoIndex && (a.index == kNoIndex || b.value > a.value ||
                                             (b.value == a.value && b.index < a.index));
  Best r = take_b ? b : a;
  r.nonfinite = a.nonfinite | b.nonfinite;
  return r;
}
__device__ __forceinline__ Best shuffle_down(const Best& v, int offset) {
  Best o;
  o.value = __shfl_down_sync(kFullMask, v.value, offset);
  o.index = __shfl_down_sync(kFullMask, v.index, offset);
  o.bits = __shfl_down_sync(kFullMask, v.bits, offset);
  o.nonfinite = __shfl_down_sync(kFullMask, v.nonfinite, offset);
  return o;
}
__device__ __forceinline__ Best block_best(Best mine) {
  __shared__ Best per_warp[kThreads / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mine = better(mine, shuffle_down(mine, o));
  if ((threadIdx.x & 31) == 0) per_warp[threadIdx.x >> 5] = mine;
  __syncthreads();
  Best r = per_warp[0];
  if (threadIdx.x == 0)
    for (int w = 1; w < kThreads / 32; ++w) r = better(r, per_warp[w]);
  return r;  // valid in thread 0
}
struct ArgmaxResult {  // Bf16GreedyArgmaxResult, include/q3x/runtime/decode_ops.h:61-69
  uint32_t index;
  uint16_t value_bits;
  uint16_t has_nonfinite;
};

__global__ void __launch_bounds__(kThreads) argmax_partial_kernel(const uint16_t* __restrict__ in, size_t count,
                                                                  ArgmaxResult* workspace) {
  Best mine{-INFINITY, kNoIndex, 0u, 0u};
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  auto visit = [&](uint32_t bits, size_t i) {
    if ((bits & 0x7f80u) == 0x7f80u) {
      mine.nonfinite = 1u;
    } else {
      const float v = bf16_to_float(static_cast<uint16_t>(bits));
      if (mine.index == kNoIndex || v > mine.value) mine = Best{v, static_cast<uint32_t>(i), bits, mine.nonfinite};
    }
  };
  // eight logits per 128-bit load where the vector is aligned (a thread still meets its indices in increasing
  // order, which is what keeps the earliest of equal maxima); the ragged end one element at a time
  const size_t vectors = (reinterpret_cast<uintptr_t>(in) & 15u) == 0 ? count / 8 : 0;
  for (size_t v = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; v < vectors; v += stride) {
    const uint4 q = ld_stream(reinterpret_cast<const uint4*>(in) + v);
    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      visit(words[k] & 0xffffu, v * 8 + 2 * k);
      visit(words[k] >> 16, v * 8 + 2 * k + 1);
    }
  }
  for (size_t i = vectors * 8 + static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < count; i += stride)
    visit(in[i], i);
  const Best r = block_best(mine);
  if (threadIdx.x == 0)
    workspace[1 + blockIdx.x] = ArgmaxResult{r.index, static_cast<uint16_t>(r.bits), static_cast<uint16_t>(r.nonfinite)};
}

__global__ void __launch_bounds__(32) argmax_final_kernel(ArgmaxResult* workspace, int partials) {
  const int lane = threadIdx.x;
  Best mine{-INFINITY, kNoIndex, 0u, 0u};
  if (lane < partials) {
    const ArgmaxResult p = workspace[1 + lane];
    mine = Best{p.index == kNoIndex ? -INFINITY : bf16_to_float(p.value_bits), p.index, p.value_bits, p.has_nonfinite};
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mine = better(mine, shuffle_down(mine, o));
  if (lane == 0)
    workspace[0] = ArgmaxResult{mine.index, static_cast<uint16_t>(mine.index == kNoIndex ? 0u : mine.bits),
                                static_cast<uint16_t>(mine.nonfinite)};
}

}  // namespace
}  // namespace q3x

using namespace q3x;
using namespace q3x::host;

extern "C" int q3x_b200_softmax(const float* in, size_t rows, size_t cols, float* out, void* stream) {
  if (mul3_overflows(rows, cols, sizeof(float))) return kInvalid;
  if (rows == 0 || cols == 0) return kOk;
  if (in == nullptr || out == nullptr) return kInvalid;
  const Span si = span(in, rows * cols * 4), so = span(out, rows * cols * 4);
  if (wraps(si) || wraps(so) || partial_overlap(si, so)) return kInvalid;
  clear_stale_error();
  softmax_rows_kernel<<<grid_for(rows, 1, 8), kThreads, 0, as_stream(stream)>>>(in, rows, cols, out);
  return launch_status();
}

extern "C" int q3x_b200_bf16_greedy_argmax(const uint16_t* in, size_t count, void* result_workspace, void* stream) {
  if (in == nullptr || result_workspace == nullptr || count == 0 || count > 0xfffffffeu) return kInvalid;
  if (overlap(span(in, count * 2), span(result_workspace, Q3X_B200_ARGMAX_WORKSPACE_RESULTS * sizeof(ArgmaxResult))))
    return kInvalid;
  static_assert(sizeof(ArgmaxResult) == 8, "layout of Bf16GreedyArgmaxResult");
  static_assert(Q3X_B200_ARGMAX_WORKSPACE_RESULTS == 1 + kArgmaxBlocks, "workspace = answer + partials");
  const size_t want = (count + kThreads * 8 - 1) / (kThreads * 8);
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > kArgmaxBlocks ? kArgmaxBlocks : want));
  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  auto ws = static_cast<ArgmaxResult*>(result_workspace);
  argmax_partial_kernel<<<blocks, kThreads, 0, s>>>(in, count, ws);
  argmax_final_kernel<<<1, 32, 0, s>>>(ws, blocks);
  return launch_status();
}
