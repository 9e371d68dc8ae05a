// The bf16 projection of a panel of tokens: out[T, N] (bf16) = X[T, K] (bf16) x W[N, K]^T (bf16), FP32 accumulation,
// one rounding -- bf16_gemv_reference_cpu (src/kernels/reference/gemv_reference.cpp:84-111) per token, which is what
// launch_projection_tile_to_bf16_cuda (include/q3x/runtime/model_weights.h:800-826) computes for Bf16LinearWeight
// (the GDN layers' two gate projections, 48 x 5120, are the model's bf16 weights in the layer loop).
// CUTLASS's sm100 dense collective: tcgen05 MMA with accumulators in tensor memory, TMA loads, 128 x 64 x 64 tiles for
// narrow outputs and 128 x 256 x 64 for wide ones, 1 x 1 x 1 cluster (plain TMA loads of this GPU's own memory).
// The scaled form serves FP8 weights widened to bf16 ONCE at load (E4M3 -> bf16 is exact, the per-tensor scale rides
// in the epilogue as in fp8_gemv_reference_cpu, src/kernels/reference/gemv_reference.cpp:113-141): the same products
// and the same FP32 accumulation as the mixed-input kernel, without its per-tile conversion stage -- memory traded
// for tensor-core time on a part with 180 GB.
#include <cuda_runtime.h>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>

#include "cute/tensor.hpp"
#include "cutlass/cutlass.h"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/numeric_types.h"
#include "cutlass/util/packed_stride.hpp"
#include "host_checks.hpp"
#include "q3x_b200.h"

namespace q3x {
namespace {

using namespace cute;

using Element = cutlass::bfloat16_t;
using ClusterShape = Shape<_1, _1, _1>;

// One instantiation per tile: 128 x 64 for narrow outputs (the 48-row gate projections), 128 x 256 for wide ones.
template <class MmaTileShape>
struct Dense {
  using CollectiveEpilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
      cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, MmaTileShape, ClusterShape,
      cutlass::epilogue::collective::EpilogueTileAuto, float, float, void, cutlass::layout::RowMajor, 8, Element,
      cutlass::layout::RowMajor, 8, cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;
  using CollectiveMainloop = typename cutlass::gemm::collective::CollectiveBuilder<
      cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, Element, cutlass::layout::RowMajor, 8, Element,
      cutlass::layout::ColumnMajor, 8, float, MmaTileShape, ClusterShape,
      cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename CollectiveEpilogue::SharedStorage))>,
      cutlass::gemm::collective::KernelScheduleAuto>::CollectiveOp;
  using GemmKernel =
      cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, CollectiveMainloop, CollectiveEpilogue, void>;
  using Gemm = cutlass::gemm::device::GemmUniversalAdapter<GemmKernel>;
  using StrideA = typename GemmKernel::StrideA;
  using StrideB = typename GemmKernel::StrideB;
  using StrideD = typename GemmKernel::StrideD;

  static typename Gemm::Arguments arguments(const uint16_t* activations, const uint16_t* weights, float scale, int tokens,
                                            int out_features, int in_features, uint16_t* out) {
    const StrideA stride_a = cutlass::make_cute_packed_stride(StrideA{}, make_shape(tokens, in_features, 1));
    const StrideB stride_b = cutlass::make_cute_packed_stride(StrideB{}, make_shape(out_features, in_features, 1));
    const StrideD stride_d = cutlass::make_cute_packed_stride(StrideD{}, make_shape(tokens, out_features, 1));
    typename Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm,
                                  {tokens, out_features, in_features, 1},
                                  {reinterpret_cast<const Element*>(activations), stride_a,
                                   reinterpret_cast<const Element*>(weights), stride_b},
                                  {{scale, 0.0f}, nullptr, stride_d, reinterpret_cast<Element*>(out), stride_d}};
    args.scheduler.max_swizzle_size = 8;
    return args;
  }
  static size_t workspace(int tokens, int out_features, int in_features) {
    return Gemm::get_workspace_size(arguments(nullptr, nullptr, 1.0f, tokens, out_features, in_features, nullptr));
  }
  static int run(const uint16_t* activations, const uint16_t* weights, float scale, int tokens, int out_features,
                 int in_features, uint16_t* out, void* workspace, cudaStream_t s) {
    const auto args = arguments(activations, weights, scale, tokens, out_features, in_features, out);
    Gemm gemm;
    if (gemm.can_implement(args) != cutlass::Status::kSuccess) return host::kNotSupported;
    if (gemm.initialize(args, workspace, s) != cutlass::Status::kSuccess) return host::kNotSupported;
    if (gemm.run(s) != cutlass::Status::kSuccess) {
      const int status = host::launch_status();
      return status != host::kOk ? status : static_cast<int>(cudaErrorLaunchFailure);
    }
    return host::launch_status();
  }
};
using Narrow = Dense<Shape<_128, _64, _64>>;
using Wide = Dense<Shape<_128, _256, _64>>;

bool wide_tile(size_t out_features) { return out_features >= 512; }

// E4M3 -> bf16 is exact (3 mantissa bits, exponents -9 .. 8); 16 codes per thread
__global__ void __launch_bounds__(256) widen_e4m3_kernel(const uint4* __restrict__ codes, size_t vectors, uint4* __restrict__ out) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < vectors;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const uint4 v = __ldg(codes + i);
    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
    uint32_t wide[8];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint16_t pair = static_cast<uint16_t>(words[w] >> (16 * h));
        uint32_t halves;  // two f16 values, exact
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(halves) : "h"(pair));
        const __half2 h2 = *reinterpret_cast<const __half2*>(&halves);
        const float2 f = __half22float2(h2);
        const __nv_bfloat162 b2 = __floats2bfloat162_rn(f.x, f.y);  // exact: at most 4 significant bits
        wide[w * 2 + h] = *reinterpret_cast<const uint32_t*>(&b2);
      }
    }
    out[2 * i] = make_uint4(wide[0], wide[1], wide[2], wide[3]);
    out[2 * i + 1] = make_uint4(wide[4], wide[5], wide[6], wide[7]);
  }
}

}  // namespace
}  // namespace q3x

using namespace q3x;
using namespace q3x::host;

extern "C" size_t q3x_b200_bf16_gemm_workspace_bytes(size_t tokens, size_t out_features, size_t in_features) {
  if (tokens == 0 || out_features == 0 || in_features == 0) return 0;
  if (tokens > 0x7fffffffu || out_features > 0x7fffffffu || in_features > 0x7fffffffu) return 0;
  const int t = static_cast<int>(tokens), n = static_cast<int>(out_features), k = static_cast<int>(in_features);
  const size_t bytes = wide_tile(out_features) ? Wide::workspace(t, n, k) : Narrow::workspace(t, n, k);
  return (bytes + 255) / 256 * 256;  // 0 for these kernels' static tile schedule
}

extern "C" int q3x_b200_bf16_gemm_scaled_bf16(const uint16_t* weights, float weight_scale, const uint16_t* activations,
                                              size_t tokens, size_t out_features, size_t in_features, uint16_t* out,
                                              void* workspace, size_t workspace_bytes, void* stream) {
  if (!std::isfinite(weight_scale)) return kInvalid;
  if (tokens == 0 || out_features == 0) return kOk;
  if (in_features == 0 || in_features % 8 != 0 || out_features % 8 != 0) return kInvalid;
  if (tokens > 0x7fffffffu || out_features > 0x7fffffffu || in_features > 0x7fffffffu) return kInvalid;
  if (weights == nullptr || activations == nullptr || out == nullptr) return kInvalid;
  const size_t need = q3x_b200_bf16_gemm_workspace_bytes(tokens, out_features, in_features);
  if (need != 0 && (workspace == nullptr || workspace_bytes < need || !aligned16(workspace))) return kInvalid;
  if (!aligned16(weights) || !aligned16(activations) || !aligned16(out)) return kNotSupported;
  const Span so = span(out, tokens * out_features * 2), sw = span(need != 0 ? workspace : nullptr, need);
  const Span sweights = span(weights, out_features * in_features * 2), sx = span(activations, tokens * in_features * 2);
  if (overlap(so, sweights) || overlap(so, sx) || overlap(so, sw) || overlap(sw, sweights) || overlap(sw, sx)) return kInvalid;

  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  const int t = static_cast<int>(tokens), n = static_cast<int>(out_features), k = static_cast<int>(in_features);
  void* ws = need != 0 ? workspace : nullptr;
  return wide_tile(out_features) ? Wide::run(activations, weights, weight_scale, t, n, k, out, ws, s)
                                 : Narrow::run(activations, weights, weight_scale, t, n, k, out, ws, s);
}

extern "C" int q3x_b200_bf16_gemm_bf16(const uint16_t* weights, const uint16_t* activations, size_t tokens,
                                       size_t out_features, size_t in_features, uint16_t* out, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  return q3x_b200_bf16_gemm_scaled_bf16(weights, 1.0f, activations, tokens, out_features, in_features, out, workspace,
                                        workspace_bytes, stream);
}

extern "C" int q3x_b200_fp8_weights_to_bf16(const uint8_t* weights, size_t elements, uint16_t* out, void* stream) {
  if (elements == 0) return kOk;
  if (weights == nullptr || out == nullptr || elements % 16 != 0 || mul_overflows(elements, 2)) return kInvalid;
  if (!aligned16(weights) || !aligned16(out)) return kNotSupported;
  if (overlap(span(weights, elements), span(out, elements * 2))) return kInvalid;
  clear_stale_error();
  const size_t vectors = elements / 16;
  const unsigned grid = static_cast<unsigned>(std::min<size_t>((vectors + 255) / 256, static_cast<size_t>(148) * 16));
  widen_e4m3_kernel<<<grid, 256, 0, as_stream(stream)>>>(reinterpret_cast<const uint4*>(weights), vectors,
                                                        reinterpret_cast<uint4*>(out));
  return launch_status();
}
