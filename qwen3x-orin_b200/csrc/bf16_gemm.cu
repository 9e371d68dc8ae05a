// The bf16 projection of a panel of tokens: out[T, N] (bf16) = X[T, K] (bf16) x W[N, K]^T (bf16), FP32 accumulation,
// one rounding -- bf16_gemv_reference_cpu (src/kernels/reference/gemv_reference.cpp:84-111) per token, which is what
// launch_projection_tile_to_bf16_cuda (include/q3x/runtime/model_weights.h:800-826) computes for Bf16LinearWeight
// (the GDN layers' two gate projections, 48 x 5120, are the model's bf16 weights in the layer loop).
// CUTLASS's sm100 dense collective: tcgen05 MMA with accumulators in tensor memory, TMA loads, 128 x 64 x 64 tiles,
// 1 x 1 x 1 cluster (plain TMA loads of this GPU's own memory).
#include <cuda_runtime.h>

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
using MmaTileShape = Shape<_128, _64, _64>;
using ClusterShape = Shape<_1, _1, _1>;

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

Gemm::Arguments make_arguments(const uint16_t* activations, const uint16_t* weights, int tokens, int out_features,
                               int in_features, uint16_t* out) {
  const StrideA stride_a = cutlass::make_cute_packed_stride(StrideA{}, make_shape(tokens, in_features, 1));
  const StrideB stride_b = cutlass::make_cute_packed_stride(StrideB{}, make_shape(out_features, in_features, 1));
  const StrideD stride_d = cutlass::make_cute_packed_stride(StrideD{}, make_shape(tokens, out_features, 1));
  Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm,
                       {tokens, out_features, in_features, 1},
                       {reinterpret_cast<const Element*>(activations), stride_a, reinterpret_cast<const Element*>(weights),
                        stride_b},
                       {{1.0f, 0.0f}, nullptr, stride_d, reinterpret_cast<Element*>(out), stride_d}};
  return args;
}

}  // namespace
}  // namespace q3x

using namespace q3x;
using namespace q3x::host;

extern "C" size_t q3x_b200_bf16_gemm_workspace_bytes(size_t tokens, size_t out_features, size_t in_features) {
  if (tokens == 0 || out_features == 0 || in_features == 0) return 0;
  if (tokens > 0x7fffffffu || out_features > 0x7fffffffu || in_features > 0x7fffffffu) return 0;
  const auto args = make_arguments(nullptr, nullptr, static_cast<int>(tokens), static_cast<int>(out_features),
                                   static_cast<int>(in_features), nullptr);
  return (Gemm::get_workspace_size(args) + 255) / 256 * 256;  // 0 for this kernel's static tile schedule
}

extern "C" int q3x_b200_bf16_gemm_bf16(const uint16_t* weights, const uint16_t* activations, size_t tokens,
                                       size_t out_features, size_t in_features, uint16_t* out, void* workspace,
                                       size_t workspace_bytes, void* stream) {
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
  const auto args = make_arguments(activations, weights, static_cast<int>(tokens), static_cast<int>(out_features),
                                   static_cast<int>(in_features), out);
  Gemm gemm;
  if (gemm.can_implement(args) != cutlass::Status::kSuccess) return kNotSupported;
  if (gemm.initialize(args, need != 0 ? workspace : nullptr, s) != cutlass::Status::kSuccess) return kNotSupported;
  if (gemm.run(s) != cutlass::Status::kSuccess) {
    const int status = launch_status();
    return status != kOk ? status : static_cast<int>(cudaErrorLaunchFailure);
  }
  return launch_status();
}
