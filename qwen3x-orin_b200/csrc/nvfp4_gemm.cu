// The projection that consumes the NVFP4 activations: out[T, N] (bf16) = A[T, K] x W[N, K]^T with both operands in
// NVFP4 -- E2M1 codes, one E4M3 scale per 16 elements along K, an FP32 second-level scale per activation scale
// group and one for the weight tensor -- on the block-scaled tensor-core path of sm_100a (tcgen05.mma with the
// block scales read from tensor memory, operands brought in by TMA, accumulators in tensor memory).
//
// The reference has no such kernel: its prefill projections multiply bf16 activations with NVFP4 weights
// (src/kernels/sm87/nvfp4_marlin_w4a16.cu, reached through launch_projection_to_bf16_cuda,
// include/q3x/runtime/model_weights.h:794-841).  This is the same projection with the activation operand
// taken from this library's quantiser instead: codes as written by the q3x_b200_*_nvfp4 entry points, block
// scales re-laid out by q3x_b200_nvfp4_swizzle_block_scales, global scales as written per scale group.
//
// The kernel is CUTLASS's sm100 block-scaled collective (mainloop and epilogue builders) instantiated here for
// one tile shape, with a 1 x 1 x 1 cluster: every TMA load is an ordinary one that reads this GPU's own memory.
// An activation scale group has its own second-level scale, so the epilogue's alpha is per ROW: a small kernel
// expands (group scale x weight scale) to one float per token in the workspace, and one persistent GEMM covers
// all tokens.
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "cute/tensor.hpp"
#include "cutlass/cutlass.h"
#include "cutlass/detail/sm100_blockscaled_layout.hpp"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/epilogue/fusion/operations.hpp"
#include "cutlass/epilogue/thread/activation.h"
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

using ElementA = cutlass::nv_float4_t<cutlass::float_e2m1_t>;  // activations [T, K], K contiguous
using ElementB = cutlass::nv_float4_t<cutlass::float_e2m1_t>;  // weights [N, K], K contiguous
using ElementD = cutlass::bfloat16_t;
using ElementAccumulator = float;
using LayoutA = cutlass::layout::RowMajor;
using LayoutB = cutlass::layout::ColumnMajor;
using LayoutD = cutlass::layout::RowMajor;
constexpr int kAlignmentAB = 32;                                        // elements: 16 bytes of codes
constexpr int kAlignmentD = 128 / cutlass::sizeof_bits<ElementD>::value;  // 8 bf16

using MmaTileShape = Shape<_128, _128, _256>;
using ClusterShape = Shape<_1, _1, _1>;

// D = alpha[row] x accumulator, rounded once to bf16 (no source tensor, no bias)
using RowScale = cutlass::epilogue::fusion::PerRowLinCombPerRowBiasEltAct<cutlass::epilogue::thread::Identity, ElementD,
                                                                         ElementAccumulator, ElementD, void,
                                                                         ElementAccumulator>;
using CollectiveEpilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassBlockScaledTensorOp, MmaTileShape, ClusterShape,
    cutlass::epilogue::collective::EpilogueTileAuto, ElementAccumulator, ElementAccumulator, void, LayoutD, kAlignmentD,
    ElementD, LayoutD, kAlignmentD, cutlass::epilogue::collective::EpilogueScheduleAuto, RowScale>::CollectiveOp;

using CollectiveMainloop = typename cutlass::gemm::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassBlockScaledTensorOp, ElementA, LayoutA, kAlignmentAB, ElementB, LayoutB,
    kAlignmentAB, ElementAccumulator, MmaTileShape, ClusterShape,
    cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename CollectiveEpilogue::SharedStorage))>,
    cutlass::gemm::collective::KernelScheduleAuto>::CollectiveOp;

using GemmKernel =
    cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, CollectiveMainloop, CollectiveEpilogue, void>;
using Gemm = cutlass::gemm::device::GemmUniversalAdapter<GemmKernel>;
using ScaleConfig = typename GemmKernel::CollectiveMainloop::Sm1xxBlkScaledConfig;
using ScaleElement = typename GemmKernel::CollectiveMainloop::ElementSF;  // E4M3, unsigned
using StrideA = typename GemmKernel::StrideA;
using StrideB = typename GemmKernel::StrideB;
using StrideD = typename GemmKernel::StrideD;

// alpha[t] = global scale of token t's scale group x the weights' second-level scale
__global__ void row_alpha_kernel(const float* group_scales, float weight_scale_2, size_t tokens, size_t rows_per_scale,
                                 float* alpha) {
  const size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t < tokens) alpha[t] = group_scales[t / rows_per_scale] * weight_scale_2;
}

Gemm::Arguments make_arguments(const uint8_t* a, const uint8_t* a_scales, const uint8_t* w, const uint8_t* w_scales, int m,
                               int n, int k, const float* alpha, uint16_t* out) {
  const StrideA stride_a = cutlass::make_cute_packed_stride(StrideA{}, make_shape(m, k, 1));
  const StrideB stride_b = cutlass::make_cute_packed_stride(StrideB{}, make_shape(n, k, 1));
  const StrideD stride_d = cutlass::make_cute_packed_stride(StrideD{}, make_shape(m, n, 1));
  const auto layout_sfa = ScaleConfig::tile_atom_to_shape_SFA(make_shape(m, n, k, 1));
  const auto layout_sfb = ScaleConfig::tile_atom_to_shape_SFB(make_shape(m, n, k, 1));
  Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm,
                       {m, n, k, 1},
                       {reinterpret_cast<const typename ElementA::DataType*>(a), stride_a,
                        reinterpret_cast<const typename ElementB::DataType*>(w), stride_b,
                        reinterpret_cast<const ScaleElement*>(a_scales), layout_sfa,
                        reinterpret_cast<const ScaleElement*>(w_scales), layout_sfb},
                       {{}, nullptr, stride_d, reinterpret_cast<ElementD*>(out), stride_d}};
  args.epilogue.thread.alpha_ptr = alpha;  // one per row (the default stride of this fusion)
  return args;
}

}  // namespace
}  // namespace q3x

using namespace q3x;
using namespace q3x::host;

namespace {
size_t alpha_bytes(size_t tokens) { return (tokens * sizeof(float) + 255) / 256 * 256; }
}  // namespace

extern "C" size_t q3x_b200_nvfp4_gemm_workspace_bytes(size_t tokens, size_t out_features, size_t in_features,
                                                      size_t /*rows_per_scale*/) {
  if (tokens == 0 || out_features == 0 || in_features == 0) return 0;
  if (tokens > 0x7fffffffu || out_features > 0x7fffffffu || in_features > 0x7fffffffu) return 0;
  const auto args = make_arguments(nullptr, nullptr, nullptr, nullptr, static_cast<int>(tokens), static_cast<int>(out_features),
                                   static_cast<int>(in_features), nullptr, nullptr);
  return alpha_bytes(tokens) + (Gemm::get_workspace_size(args) + 255) / 256 * 256;
}

extern "C" int q3x_b200_nvfp4_gemm_bf16(const uint8_t* activation_codes, const uint8_t* activation_scales_swizzled,
                                        const float* activation_global_scales, size_t rows_per_scale,
                                        const uint8_t* weight_codes, const uint8_t* weight_scales_swizzled,
                                        float weight_scale_2, size_t tokens, size_t out_features, size_t in_features,
                                        uint16_t* out, void* workspace, size_t workspace_bytes, void* stream) {
  if (tokens == 0 || out_features == 0) return kOk;
  if (in_features == 0 || in_features % 64 != 0 || out_features % 8 != 0) return kInvalid;
  if (tokens > 0x7fffffffu || out_features > 0x7fffffffu || in_features > 0x7fffffffu) return kInvalid;
  if (!(std::isfinite(weight_scale_2) && weight_scale_2 >= 0.0f)) return kInvalid;
  if (activation_codes == nullptr || activation_scales_swizzled == nullptr || activation_global_scales == nullptr ||
      weight_codes == nullptr || weight_scales_swizzled == nullptr || out == nullptr)
    return kInvalid;
  const size_t rps = rows_per_scale == 0 || rows_per_scale > tokens ? tokens : rows_per_scale;
  const size_t groups = (tokens + rps - 1) / rps;
  const size_t need = q3x_b200_nvfp4_gemm_workspace_bytes(tokens, out_features, in_features, rows_per_scale);
  if (workspace == nullptr || workspace_bytes < need || !aligned16(workspace)) return kInvalid;
  if (!aligned16(activation_codes) || !aligned16(weight_codes) || !aligned16(activation_scales_swizzled) ||
      !aligned16(weight_scales_swizzled) || !aligned16(out))
    return kNotSupported;
  const Span so = span(out, tokens * out_features * 2), sw = span(workspace, need);
  const Span inputs[] = {span(activation_codes, tokens * in_features / 2), span(weight_codes, out_features * in_features / 2),
                         span(activation_global_scales, groups * sizeof(float)),
                         span(activation_scales_swizzled, q3x_b200_nvfp4_swizzled_scale_bytes(tokens, in_features)),
                         span(weight_scales_swizzled, q3x_b200_nvfp4_swizzled_scale_bytes(out_features, in_features))};
  for (const Span& in : inputs)
    if (overlap(so, in) || overlap(sw, in)) return kInvalid;
  if (overlap(so, sw)) return kInvalid;

  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  float* const alpha = static_cast<float*>(workspace);
  row_alpha_kernel<<<static_cast<unsigned>((tokens + 255) / 256), 256, 0, s>>>(activation_global_scales, weight_scale_2,
                                                                              tokens, rps, alpha);
  const auto args = make_arguments(activation_codes, activation_scales_swizzled, weight_codes, weight_scales_swizzled,
                                   static_cast<int>(tokens), static_cast<int>(out_features), static_cast<int>(in_features),
                                   alpha, out);
  Gemm gemm;
  if (gemm.can_implement(args) != cutlass::Status::kSuccess) return kNotSupported;
  if (gemm.initialize(args, static_cast<uint8_t*>(workspace) + alpha_bytes(tokens), s) != cutlass::Status::kSuccess)
    return kNotSupported;
  if (gemm.run(s) != cutlass::Status::kSuccess) {
    const int status = launch_status();
    return status != kOk ? status : static_cast<int>(cudaErrorLaunchFailure);
  }
  return launch_status();
}
