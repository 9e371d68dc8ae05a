// The weight-only NVFP4 projection of a panel of tokens: out[T, N] (bf16) = X[T, K] (bf16) x W[N, K]^T with W as
// packed E2M1 codes, one scale per 16 columns (given TRANSPOSED and as bf16, [K / 16, N]: the collective reads the
// scales of a tile with the output dimension contiguous and in the MMA's operand type;
// q3x_b200_nvfp4_transpose_block_scales re-lays a weight's E4M3 scales out once, at load time, and an E4M3 value
// is exact in bf16) and an FP32 second-level scale -- the multi-token form of nvfp4_gemv_reference_cpu
// (src/kernels/reference/gemv_reference.cpp:179-225), which the reference's runner reaches through
// launch_projection_tile_to_bf16_cuda and launch_exact_nvfp4_whole_chunk_branch_to_bf16_cuda
// (include/q3x/runtime/model_weights.h:800-866) for the MLP projections (its kernel:
// src/kernels/sm87/nvfp4_marlin_w4a16.cu).  Same numerics as the batch-one form up to the order of the FP32
// accumulation: code x block scale is exact in bf16 (at most six significant bits), its product with a bf16
// activation is exact in FP32, the second-level scale multiplies the sum, one rounding to bf16.
//
// CUTLASS's sm100 mixed-input collective with block-wise scales (granularity 1 x 16): the transform warps
// widen the codes, multiply them by their block scale and hand bf16 operands to tcgen05.  The narrow operand is A, so
// the problem is posed transposed (D^T[N, T] column-major = out[T, N] row-major).  1 x 1 x 1 cluster: plain TMA loads
// of this GPU's own memory.
#include <cuda_runtime.h>

#include <cmath>
#include <cstddef>
#include <cstdint>

#include "cute/tensor.hpp"
#include "cutlass/cutlass.h"
#include "cutlass/detail/sm100_mixed_dtype_blockwise_layout.hpp"
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

using ElementW = cutlass::float_e2m1_t;  // operand A: weights [N, K], K contiguous, two codes per byte
using ElementS = cutlass::bfloat16_t;    // block scales [K / 16, N], N contiguous
using ElementX = cutlass::bfloat16_t;    // operand B: activations [T, K]
using ElementD = cutlass::bfloat16_t;    // D^T [N, T] column-major = out [T, N] row-major
using MmaTileShape = Shape<_128, _128, _128>;
using ClusterShape = Shape<_1, _1, _1>;
using ScaleConfig = cutlass::detail::Sm100MixedInputBlockwiseScaleConfig<1, 16>;
using LayoutScale = decltype(ScaleConfig::deduce_layout_scale());

using CollectiveEpilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, MmaTileShape, ClusterShape,
    cutlass::epilogue::collective::EpilogueTileAuto, float, float, void, cutlass::layout::ColumnMajor, 8, ElementD,
    cutlass::layout::ColumnMajor, 8, cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;

using CollectiveMainloop = typename cutlass::gemm::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, cute::tuple<ElementW, ElementS>,
    cute::tuple<cutlass::layout::RowMajor, LayoutScale>, 32, ElementX, cutlass::layout::ColumnMajor, 8, float, MmaTileShape,
    ClusterShape,
    cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename CollectiveEpilogue::SharedStorage))>,
    cutlass::gemm::KernelTmaWarpSpecialized1SmMixedInputSm100>::CollectiveOp;

using GemmKernel =
    cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, CollectiveMainloop, CollectiveEpilogue, void>;
using Gemm = cutlass::gemm::device::GemmUniversalAdapter<GemmKernel>;
using StrideA = typename GemmKernel::StrideA;
using StrideB = typename GemmKernel::StrideB;
using StrideD = typename GemmKernel::StrideD;

Gemm::Arguments make_arguments(const uint8_t* codes, const uint16_t* block_scales, float scale_2, const uint16_t* activations,
                               int tokens, int out_features, int in_features, uint16_t* out) {
  const StrideA stride_a = cutlass::make_cute_packed_stride(StrideA{}, make_shape(out_features, in_features, 1));
  const StrideB stride_b = cutlass::make_cute_packed_stride(StrideB{}, make_shape(tokens, in_features, 1));
  const StrideD stride_d = cutlass::make_cute_packed_stride(StrideD{}, make_shape(out_features, tokens, 1));
  const auto layout_s = ScaleConfig::tile_atom_to_shape_scale(make_shape(out_features, in_features, 1));
  Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm,
                       {out_features, tokens, in_features, 1},
                       {reinterpret_cast<const ElementW*>(codes), stride_a, reinterpret_cast<const ElementX*>(activations),
                        stride_b, reinterpret_cast<const ElementS*>(block_scales), layout_s},
                       {{scale_2, 0.0f}, nullptr, stride_d, reinterpret_cast<ElementD*>(out), stride_d}};
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

extern "C" size_t q3x_b200_nvfp4_w4a16_gemm_workspace_bytes(size_t tokens, size_t out_features, size_t in_features) {
  if (tokens == 0 || out_features == 0 || in_features == 0) return 0;
  if (tokens > 0x7fffffffu || out_features > 0x7fffffffu || in_features > 0x7fffffffu) return 0;
  const auto args = make_arguments(nullptr, nullptr, 1.0f, nullptr, static_cast<int>(tokens), static_cast<int>(out_features),
                                   static_cast<int>(in_features), nullptr);
  return (Gemm::get_workspace_size(args) + 255) / 256 * 256;  // 0 for this kernel's static tile schedule
}

extern "C" int q3x_b200_nvfp4_w4a16_gemm_bf16(const uint8_t* packed_weights, const uint16_t* block_scales_transposed,
                                              float weight_scale_2, const uint16_t* activations, size_t tokens,
                                              size_t out_features, size_t in_features, uint16_t* out, void* workspace,
                                              size_t workspace_bytes, void* stream) {
  if (tokens == 0 || out_features == 0) return kOk;
  // TMA units of 16 bytes: 32 codes of a weight row, 8 scales of a scale row
  if (in_features == 0 || in_features % 32 != 0 || out_features % 8 != 0) return kInvalid;
  const uint16_t* const block_scales = block_scales_transposed;
  if (tokens > 0x7fffffffu || out_features > 0x7fffffffu || in_features > 0x7fffffffu) return kInvalid;
  if (!(std::isfinite(weight_scale_2) && weight_scale_2 >= 0.0f)) return kInvalid;
  if (packed_weights == nullptr || block_scales == nullptr || activations == nullptr || out == nullptr) return kInvalid;
  const size_t need = q3x_b200_nvfp4_w4a16_gemm_workspace_bytes(tokens, out_features, in_features);
  if (need != 0 && (workspace == nullptr || workspace_bytes < need || !aligned16(workspace))) return kInvalid;
  if (!aligned16(packed_weights) || !aligned16(block_scales) || !aligned16(activations) || !aligned16(out))
    return kNotSupported;
  const Span so = span(out, tokens * out_features * 2), sw = span(need != 0 ? workspace : nullptr, need);
  const Span inputs[] = {span(packed_weights, out_features * in_features / 2), span(block_scales, out_features * in_features / 16 * 2),
                         span(activations, tokens * in_features * 2)};
  for (const Span& in : inputs)
    if (overlap(so, in) || overlap(sw, in)) return kInvalid;
  if (overlap(so, sw)) return kInvalid;

  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  const auto args = make_arguments(packed_weights, block_scales, weight_scale_2, activations, static_cast<int>(tokens),
                                   static_cast<int>(out_features), static_cast<int>(in_features), out);
  Gemm gemm;
  if (gemm.can_implement(args) != cutlass::Status::kSuccess) return kNotSupported;
  if (gemm.initialize(args, need != 0 ? workspace : nullptr, s) != cutlass::Status::kSuccess) return kNotSupported;
  if (gemm.run(s) != cutlass::Status::kSuccess) {
    const int status = launch_status();
    return status != kOk ? status : static_cast<int>(cudaErrorLaunchFailure);
  }
  return launch_status();
}
