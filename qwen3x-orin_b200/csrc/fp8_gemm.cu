// The weight-only FP8 projection of a panel of tokens: out[T, N] (bf16) = X[T, K] (bf16) x W[N, K]^T with W in E4M3
// and one FP32 scale for the whole weight tensor -- the multi-token form of fp8_gemv_reference_cpu
// (src/kernels/reference/gemv_reference.cpp:113-140), which the reference's runner reaches through
// launch_projection_tile_to_bf16_cuda and launch_exact_fp8_whole_chunk_projection_to_bf16_cuda
// (include/q3x/runtime/model_weights.h:800-870) for its attention and GDN projections.  Same numerics as the
// batch-one form: every product decode(w) x x is exact in FP32, the sum is accumulated in FP32, the weight scale is
// applied to the sum, one rounding to bf16.
//
// On sm_100a this is a mixed-input tensor-core GEMM: CUTLASS's sm100 mixed-input collective widens the E4M3 weights
// to bf16 (exact) on their way from shared memory to the MMA's operand and multiplies bf16 x bf16 with tcgen05.  That
// collective wants the narrow operand as A, so the problem is posed transposed -- D^T[N, T] = W[N, K] X[T, K]^T,
// with D^T written column-major, which is out[T, N] row-major.  1 x 1 x 1 cluster: plain TMA loads of this GPU's
// own memory.
#include <cuda_runtime.h>

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

using ElementW = cutlass::float_e4m3_t;  // operand A: weights [N, K], K contiguous
using ElementX = cutlass::bfloat16_t;    // operand B: activations [T, K], K contiguous
using ElementD = cutlass::bfloat16_t;    // D^T [N, T] column-major = out [T, N] row-major
using MmaTileShape = Shape<_128, _128, _128>;
using ClusterShape = Shape<_1, _1, _1>;

using CollectiveEpilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, MmaTileShape, ClusterShape,
    cutlass::epilogue::collective::EpilogueTileAuto, float, float, void, cutlass::layout::ColumnMajor, 8, ElementD,
    cutlass::layout::ColumnMajor, 8, cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;

using CollectiveMainloop = typename cutlass::gemm::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, cute::tuple<ElementW>, cutlass::layout::RowMajor, 16, ElementX,
    cutlass::layout::ColumnMajor, 8, float, MmaTileShape, ClusterShape,
    cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename CollectiveEpilogue::SharedStorage))>,
    cutlass::gemm::KernelTmaWarpSpecialized1SmMixedInputSm100>::CollectiveOp;

using GemmKernel =
    cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, CollectiveMainloop, CollectiveEpilogue, void>;
using Gemm = cutlass::gemm::device::GemmUniversalAdapter<GemmKernel>;
using StrideA = typename GemmKernel::StrideA;
using StrideB = typename GemmKernel::StrideB;
using StrideD = typename GemmKernel::StrideD;

Gemm::Arguments make_arguments(const uint8_t* weights, float weight_scale, const uint16_t* activations, int tokens,
                               int out_features, int in_features, uint16_t* out) {
  // the GEMM's M is out_features, its N is tokens
  const StrideA stride_a = cutlass::make_cute_packed_stride(StrideA{}, make_shape(out_features, in_features, 1));
  const StrideB stride_b = cutlass::make_cute_packed_stride(StrideB{}, make_shape(tokens, in_features, 1));
  const StrideD stride_d = cutlass::make_cute_packed_stride(StrideD{}, make_shape(out_features, tokens, 1));
  Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm,
                       {out_features, tokens, in_features, 1},
                       {reinterpret_cast<const ElementW*>(weights), stride_a, reinterpret_cast<const ElementX*>(activations),
                        stride_b},
                       {{weight_scale, 0.0f}, nullptr, stride_d, reinterpret_cast<ElementD*>(out), stride_d}};
  // consecutive CTAs walk a band of eight tiles of the second dimension: a wave then shares a few weight row blocks and
  // eight token blocks instead of sweeping every weight row block for each token block (measured: the plain order
  // re-read 2.2 GB from HBM for 0.14 GB of operands)
  args.scheduler.max_swizzle_size = 8;
  return args;
}

}  // namespace
}  // namespace q3x

using namespace q3x;
using namespace q3x::host;

extern "C" size_t q3x_b200_fp8_gemm_workspace_bytes(size_t tokens, size_t out_features, size_t in_features) {
  if (tokens == 0 || out_features == 0 || in_features == 0) return 0;
  if (tokens > 0x7fffffffu || out_features > 0x7fffffffu || in_features > 0x7fffffffu) return 0;
  const auto args = make_arguments(nullptr, 1.0f, nullptr, static_cast<int>(tokens), static_cast<int>(out_features),
                                   static_cast<int>(in_features), nullptr);
  return (Gemm::get_workspace_size(args) + 255) / 256 * 256;  // 0 for this kernel's static tile schedule
}

extern "C" int q3x_b200_fp8_gemm_bf16(const uint8_t* weights, float weight_scale, const uint16_t* activations,
                                      size_t tokens, size_t out_features, size_t in_features, uint16_t* out,
                                      void* workspace, size_t workspace_bytes, void* stream) {
  if (tokens == 0 || out_features == 0) return kOk;
  if (in_features == 0 || in_features % 16 != 0 || out_features % 8 != 0) return kInvalid;
  if (tokens > 0x7fffffffu || out_features > 0x7fffffffu || in_features > 0x7fffffffu) return kInvalid;
  if (!(std::isfinite(weight_scale) && weight_scale >= 0.0f)) return kInvalid;
  if (weights == nullptr || activations == nullptr || out == nullptr) return kInvalid;
  const size_t need = q3x_b200_fp8_gemm_workspace_bytes(tokens, out_features, in_features);
  if (need != 0 && (workspace == nullptr || workspace_bytes < need || !aligned16(workspace))) return kInvalid;
  if (!aligned16(weights) || !aligned16(activations) || !aligned16(out)) return kNotSupported;
  const Span so = span(out, tokens * out_features * 2), sw = span(need != 0 ? workspace : nullptr, need);
  const Span sweights = span(weights, out_features * in_features), sx = span(activations, tokens * in_features * 2);
  if (overlap(so, sweights) || overlap(so, sx) || overlap(so, sw) || overlap(sw, sweights) || overlap(sw, sx)) return kInvalid;

  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  const auto args = make_arguments(weights, weight_scale, activations, static_cast<int>(tokens), static_cast<int>(out_features),
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
