// Definitions of the projection composites (see q3x_b200_dispatch.hpp): argument checks in the spirit of the
// reference's validators (src/kernels/reference/projection_dispatch.cpp:483-622, 1434-1509 -- every weight
// payload and scale valid, hidden size 5120 where the residual boundary is involved, no writable range
// overlapping any other operand, everything rejected before the first enqueue), then the C ABI.
#include "q3x_b200_dispatch.hpp"

#include <cmath>
#include <string_view>
#include <type_traits>
#include <variant>

#include "q3x_b200.h"

namespace q3x::runtime {
namespace {
constexpr int kInvalidValue = 1;    // cudaErrorInvalidValue
constexpr int kNotSupported = 801;  // cudaErrorNotSupported
constexpr std::size_t kHidden = 5120U;

// Invalid backend -> invalid value; a valid backend this library does not serve -> not supported.
int route_half(const ProjectionBackend backend) noexcept {
  if (!projection_backend_served_by_b200(backend)) return kInvalidValue;
  return backend == kProjectionBackendB200LayerOps ? 0 : kNotSupported;
}

bool valid_scale(const float v) noexcept { return std::isfinite(v) && v >= 0.0F; }

struct Shape {
  std::size_t rows = 0U, cols = 0U;
  const void* payload = nullptr;
  std::size_t payload_bytes = 0U;
  const void* scales = nullptr;
  std::size_t scale_bytes = 0U;
  bool valid = false;
};

// Shape and payload of a weight, with the reference's payload rules (projection_dispatch.cpp:646-690).
Shape describe(const LinearWeight& weight) noexcept {
  return std::visit(
      [](const auto& w) noexcept -> Shape {
        using W = std::decay_t<decltype(w)>;
        Shape s;
        s.rows = w.output_size;
        s.cols = w.input_size;
        if (s.rows == 0U || s.cols == 0U || s.rows > static_cast<std::size_t>(-1) / s.cols / 2U) return s;
        if constexpr (std::is_same_v<W, Bf16LinearWeight>) {
          s.payload = w.weight;
          s.payload_bytes = s.rows * s.cols * 2U;
          s.valid = w.weight != nullptr;
        } else if constexpr (std::is_same_v<W, Fp8LinearWeight>) {
          s.payload = w.weight;
          s.payload_bytes = s.rows * s.cols;
          s.valid = w.weight != nullptr && w.weight_scale_device != nullptr && w.input_scale_device != nullptr &&
                    valid_scale(w.weight_scale) && valid_scale(w.input_scale);
        } else {
          s.payload = w.packed_weight;
          s.payload_bytes = s.rows * s.cols / 2U;
          s.scales = w.block_scale;
          s.scale_bytes = s.rows * s.cols / 16U;
          s.valid = w.packed_weight != nullptr && w.block_scale != nullptr && w.weight_scale_2_device != nullptr &&
                    w.input_scale_device != nullptr && valid_scale(w.weight_scale_2) && valid_scale(w.input_scale) &&
                    s.cols % 16U == 0U;
        }
        return s;
      },
      weight);
}

bool overlaps(const void* a, std::size_t a_bytes, const void* b, std::size_t b_bytes) noexcept {
  if (a == nullptr || b == nullptr || a_bytes == 0U || b_bytes == 0U) return false;
  const auto x = reinterpret_cast<std::uintptr_t>(a), y = reinterpret_cast<std::uintptr_t>(b);
  return x < y + b_bytes && y < x + a_bytes;
}
// a writable range against a weight's payload and block scales
bool touches_weight(const void* p, std::size_t bytes, const Shape& w) noexcept {
  return overlaps(p, bytes, w.payload, w.payload_bytes) || overlaps(p, bytes, w.scales, w.scale_bytes);
}

// out[rows] = bf16(W x): the batch-one projection of any weight kind.
int project(const LinearWeight& weight, const std::uint16_t* input, std::uint16_t* output, void* stream) noexcept {
  return std::visit(
      [&](const auto& w) noexcept -> int {
        using W = std::decay_t<decltype(w)>;
        if constexpr (std::is_same_v<W, Bf16LinearWeight>)
          return q3x_b200_bf16_gemv(w.weight, input, w.output_size, w.input_size, nullptr, output, stream);
        else if constexpr (std::is_same_v<W, Fp8LinearWeight>)
          return q3x_b200_fp8_gemv(w.weight, w.weight_scale, input, w.output_size, w.input_size, nullptr, output, stream);
        else
          return q3x_b200_nvfp4_gemv(w.packed_weight, w.block_scale, w.weight_scale_2, input, w.output_size,
                                     w.input_size, nullptr, output, stream);
      },
      weight);
}

// Shared checks of the gate / up pair: same input width, same output width, outputs disjoint from each
// other, from the input and from both weights.
int check_gate_up(const ProjectionBackend backend, const Shape& gate, const Shape& up, const std::uint16_t* input,
                  const std::uint16_t* gate_output, const std::uint16_t* up_output) noexcept {
  if (!projection_backend_served_by_b200(backend)) return kInvalidValue;
  if (!gate.valid || !up.valid || gate.cols != up.cols || gate.rows != up.rows) return kInvalidValue;
  if (input == nullptr || gate_output == nullptr || up_output == nullptr) return kInvalidValue;
  const std::size_t out_bytes = gate.rows * 2U, in_bytes = gate.cols * 2U;
  if (overlaps(gate_output, out_bytes, up_output, out_bytes) || overlaps(gate_output, out_bytes, input, in_bytes) ||
      overlaps(up_output, out_bytes, input, in_bytes) || touches_weight(gate_output, out_bytes, gate) ||
      touches_weight(gate_output, out_bytes, up) || touches_weight(up_output, out_bytes, gate) ||
      touches_weight(up_output, out_bytes, up))
    return kInvalidValue;
  return 0;
}

int gate_up_silu(const LinearWeight& gate_weight, const LinearWeight& up_weight, const std::size_t rows,
                 const std::uint16_t* input, std::uint16_t* gate_output, std::uint16_t* up_output,
                 void* stream) noexcept {
  int st = project(gate_weight, input, gate_output, stream);
  if (st != 0) return st;
  st = project(up_weight, input, up_output, stream);
  if (st != 0) return st;
  return q3x_b200_silu_mul(gate_output, up_output, rows, gate_output, stream);
}

int post_attention(const ProjectionBackend backend, const LinearWeight& gate_weight, const LinearWeight& up_weight,
                   const std::uint16_t* residual_left, std::uint16_t* residual_right_and_normalized,
                   const std::uint16_t* norm_weight, const float epsilon, std::uint16_t* residual_output,
                   std::uint16_t* gate_output, std::uint16_t* up_output, void* stream) noexcept {
  const Shape gate = describe(gate_weight), up = describe(up_weight);
  if (const int st = check_gate_up(backend, gate, up, residual_right_and_normalized, gate_output, up_output); st != 0)
    return st;
  if (gate.cols != kHidden || residual_left == nullptr || norm_weight == nullptr || residual_output == nullptr ||
      !(std::isfinite(epsilon) && epsilon > 0.0F))
    return kInvalidValue;
  const std::size_t hidden_bytes = kHidden * 2U, out_bytes = gate.rows * 2U;
  if (overlaps(residual_output, hidden_bytes, gate_output, out_bytes) ||
      overlaps(residual_output, hidden_bytes, up_output, out_bytes) ||
      overlaps(residual_left, hidden_bytes, gate_output, out_bytes) ||
      overlaps(residual_left, hidden_bytes, up_output, out_bytes) ||
      overlaps(norm_weight, hidden_bytes, gate_output, out_bytes) ||
      overlaps(norm_weight, hidden_bytes, up_output, out_bytes) ||
      touches_weight(residual_output, hidden_bytes, gate) || touches_weight(residual_output, hidden_bytes, up) ||
      touches_weight(residual_right_and_normalized, hidden_bytes, gate) ||
      touches_weight(residual_right_and_normalized, hidden_bytes, up))
    return kInvalidValue;
  // residual add + centred norm: the normalised row replaces the right operand (its remaining alias rules
  // are the fused operator's own)
  const int st = q3x_b200_residual_add_rms_norm(residual_left, residual_right_and_normalized, norm_weight, 1U, kHidden,
                                                epsilon, residual_output, residual_right_and_normalized, stream);
  if (st != 0) return st;
  return gate_up_silu(gate_weight, up_weight, gate.rows, residual_right_and_normalized, gate_output, up_output, stream);
}

}  // namespace

#if defined(Q3X_B200_USE_REFERENCE_HEADERS)
// declared (not defined) by the reference's header: model_weights.h:389-391
bool is_valid_projection_backend(const ProjectionBackend backend) noexcept {
  return static_cast<std::uint8_t>(backend) <= static_cast<std::uint8_t>(ProjectionBackend::kSm87WeightOnly);
}
std::string_view to_string(const ProjectionBackend backend) noexcept {
  switch (static_cast<std::uint8_t>(backend)) {
    case 0U: return "reference";
    case 1U: return "sm87-weight-only";
    default: return "invalid";
  }
}
#endif

LinearWeightKind linear_weight_kind(const LinearWeight& weight) noexcept {
  return static_cast<LinearWeightKind>(weight.valueless_by_exception() ? 0U : weight.index());
}
std::size_t linear_output_size(const LinearWeight& weight) noexcept {
  return weight.valueless_by_exception() ? 0U : std::visit([](const auto& w) noexcept { return w.output_size; }, weight);
}
std::size_t linear_input_size(const LinearWeight& weight) noexcept {
  return weight.valueless_by_exception() ? 0U : std::visit([](const auto& w) noexcept { return w.input_size; }, weight);
}

namespace {
// "the explicitly selected weight-only backend" of the predicates below; this library's own value counts too
bool weight_only(const ProjectionBackend backend) noexcept {
  return backend == ProjectionBackend::kSm87WeightOnly || backend == kProjectionBackendB200LayerOps;
}
template <class W>
bool shaped(const LinearWeight& weight, const std::size_t rows, const std::size_t cols) noexcept {
  if (weight.valueless_by_exception() || std::get_if<W>(&weight) == nullptr) return false;
  const Shape s = describe(weight);
  return s.valid && s.rows == rows && s.cols == cols;
}
}  // namespace

bool supports_bf16_projection_pair(const ProjectionBackend backend, const LinearWeight& first,
                                   const LinearWeight& second) noexcept {
  return weight_only(backend) && shaped<Bf16LinearWeight>(first, 48U, kHidden) && shaped<Bf16LinearWeight>(second, 48U, kHidden);
}
bool supports_fp8_projection_pair(const ProjectionBackend backend, const LinearWeight& first,
                                  const LinearWeight& second) noexcept {
  return weight_only(backend) && shaped<Fp8LinearWeight>(first, 1024U, kHidden) && shaped<Fp8LinearWeight>(second, 1024U, kHidden);
}
bool supports_fp8_qkv_z_projection_pair(const ProjectionBackend backend, const LinearWeight& qkv,
                                        const LinearWeight& z) noexcept {
  return weight_only(backend) && shaped<Fp8LinearWeight>(qkv, 10240U, kHidden) && shaped<Fp8LinearWeight>(z, 6144U, kHidden);
}
bool supports_linear_attention_qkv_z_ab_projection_fusion(const ProjectionBackend backend, const LinearWeight& qkv,
                                                          const LinearWeight& z, const LinearWeight& a,
                                                          const LinearWeight& b) noexcept {
  return supports_fp8_qkv_z_projection_pair(backend, qkv, z) && supports_bf16_projection_pair(backend, a, b);
}
bool supports_fp8_q_kv_projection_fusion(const ProjectionBackend backend, const LinearWeight& q, const LinearWeight& key,
                                         const LinearWeight& value) noexcept {
  return weight_only(backend) && shaped<Fp8LinearWeight>(q, 12288U, kHidden) && supports_fp8_projection_pair(backend, key, value);
}
bool supports_nvfp4_gate_up_silu_fusion(const ProjectionBackend backend, const LinearWeight& gate,
                                        const LinearWeight& up) noexcept {
  return weight_only(backend) && shaped<NvFp4LinearWeight>(gate, 17408U, kHidden) && shaped<NvFp4LinearWeight>(up, 17408U, kHidden);
}
bool supports_nvfp4_down_residual_norm_fusion(const ProjectionBackend backend, const LinearWeight& down) noexcept {
  return weight_only(backend) && shaped<NvFp4LinearWeight>(down, kHidden, 17408U);
}

int launch_projection_reference_cuda(const LinearWeight& weight, const std::uint16_t* input, float* output,
                                     void* cuda_stream) noexcept {
  const Shape s = describe(weight);
  if (!s.valid || input == nullptr || output == nullptr) return kInvalidValue;
  if (overlaps(output, s.rows * 4U, input, s.cols * 2U) || touches_weight(output, s.rows * 4U, s)) return kInvalidValue;
  return std::visit(
      [&](const auto& w) noexcept -> int {
        using W = std::decay_t<decltype(w)>;
        if constexpr (std::is_same_v<W, Bf16LinearWeight>)
          return q3x_b200_bf16_gemv(w.weight, input, w.output_size, w.input_size, output, nullptr, cuda_stream);
        else if constexpr (std::is_same_v<W, Fp8LinearWeight>)
          return q3x_b200_fp8_gemv(w.weight, w.weight_scale, input, w.output_size, w.input_size, output, nullptr, cuda_stream);
        else
          return q3x_b200_nvfp4_gemv(w.packed_weight, w.block_scale, w.weight_scale_2, input, w.output_size, w.input_size,
                                     output, nullptr, cuda_stream);
      },
      weight);
}

int launch_projection_to_bf16_reference_cuda(const LinearWeight& weight, const std::uint16_t* input, float* fp32_scratch,
                                             const std::size_t scratch_elements, std::uint16_t* output,
                                             void* cuda_stream) noexcept {
  // the two-stage path: the FP32 result lands in the caller's scratch, its rounding in `output` (one kernel here)
  const Shape s = describe(weight);
  if (!s.valid || input == nullptr || output == nullptr || fp32_scratch == nullptr || scratch_elements < s.rows)
    return kInvalidValue;
  if (overlaps(output, s.rows * 2U, input, s.cols * 2U) || touches_weight(output, s.rows * 2U, s) ||
      overlaps(fp32_scratch, s.rows * 4U, input, s.cols * 2U) || touches_weight(fp32_scratch, s.rows * 4U, s) ||
      overlaps(fp32_scratch, s.rows * 4U, output, s.rows * 2U))
    return kInvalidValue;
  return std::visit(
      [&](const auto& w) noexcept -> int {
        using W = std::decay_t<decltype(w)>;
        if constexpr (std::is_same_v<W, Bf16LinearWeight>)
          return q3x_b200_bf16_gemv(w.weight, input, w.output_size, w.input_size, fp32_scratch, output, cuda_stream);
        else if constexpr (std::is_same_v<W, Fp8LinearWeight>)
          return q3x_b200_fp8_gemv(w.weight, w.weight_scale, input, w.output_size, w.input_size, fp32_scratch, output,
                                   cuda_stream);
        else
          return q3x_b200_nvfp4_gemv(w.packed_weight, w.block_scale, w.weight_scale_2, input, w.output_size, w.input_size,
                                     fp32_scratch, output, cuda_stream);
      },
      weight);
}

int launch_projection_to_bf16_cuda(const ProjectionBackend backend, const LinearWeight& weight,
                                   const std::uint16_t* input, float* /*fp32_scratch*/,
                                   std::size_t /*scratch_elements*/, std::uint16_t* output, void* cuda_stream) noexcept {
  // (the FP32 scratch of the reference's two-step path is not needed: the GEMV rounds its own result)
  if (!projection_backend_served_by_b200(backend)) return kInvalidValue;
  const Shape s = describe(weight);
  if (!s.valid || input == nullptr || output == nullptr) return kInvalidValue;
  if (overlaps(output, s.rows * 2U, input, s.cols * 2U) || touches_weight(output, s.rows * 2U, s)) return kInvalidValue;
  return project(weight, input, output, cuda_stream);
}

int launch_projection_tile_to_bf16_cuda(const ProjectionBackend backend, const LinearWeight& weight,
                                        const std::uint16_t* input, const std::size_t token_count,
                                        float* /*fp32_scratch*/, std::size_t /*scratch_elements*/, std::uint16_t* output,
                                        void* cuda_stream) noexcept {
  // The whole tile is validated before anything is enqueued (model_weights.h:824-825).  FP8 and bf16 weights of two
  // or more tokens go to the tensor-core GEMMs (one pass over the weights); everything else runs as ordered
  // batch-one projections.
  if (!projection_backend_served_by_b200(backend)) return kInvalidValue;
  const Shape s = describe(weight);
  if (!s.valid || input == nullptr || output == nullptr || token_count == 0U ||
      token_count > kMaximumProjectionTileTokenCount)
    return kInvalidValue;
  const std::size_t in_bytes = token_count * s.cols * 2U, out_bytes = token_count * s.rows * 2U;
  if (overlaps(output, out_bytes, input, in_bytes) || touches_weight(output, out_bytes, s)) return kInvalidValue;
  if (const auto* fp8 = std::get_if<Fp8LinearWeight>(&weight);
      fp8 != nullptr && token_count >= 2U && s.cols % 16U == 0U && s.rows % 8U == 0U) {
    const int st = q3x_b200_fp8_gemm_bf16(fp8->weight, fp8->weight_scale, input, token_count, s.rows, s.cols, output,
                                          nullptr, 0U, cuda_stream);
    if (st != kNotSupported) return st;  // a shape or alignment the GEMM does not take: token by token below
  }
  if (const auto* dense = std::get_if<Bf16LinearWeight>(&weight);
      dense != nullptr && token_count >= 2U && s.cols % 8U == 0U && s.rows % 8U == 0U) {
    const int st = q3x_b200_bf16_gemm_bf16(dense->weight, input, token_count, s.rows, s.cols, output, nullptr, 0U, cuda_stream);
    if (st != kNotSupported) return st;
  }
  for (std::size_t t = 0U; t < token_count; ++t)
    if (const int st = project(weight, input + t * s.cols, output + t * s.rows, cuda_stream); st != 0) return st;
  return 0;
}

namespace {
// Validation of several projections over one shared activation: every weight valid, the same input width, every
// output disjoint from the input, from every weight and from every other output -- all before the first enqueue.
struct SharedInputProjection {
  const LinearWeight* weight;
  std::uint16_t* output;
};
template <std::size_t N>
int check_shared_input(const ProjectionBackend backend, const SharedInputProjection (&p)[N], const std::uint16_t* input,
                       const std::size_t token_count) noexcept {
  if (!projection_backend_served_by_b200(backend) || input == nullptr || token_count == 0U) return kInvalidValue;
  Shape shapes[N];
  for (std::size_t i = 0; i < N; ++i) {
    if (p[i].weight->valueless_by_exception() || p[i].output == nullptr) return kInvalidValue;
    shapes[i] = describe(*p[i].weight);
    if (!shapes[i].valid || shapes[i].cols != shapes[0].cols) return kInvalidValue;
  }
  const std::size_t in_bytes = token_count * shapes[0].cols * 2U;
  for (std::size_t i = 0; i < N; ++i) {
    const std::size_t out_bytes = token_count * shapes[i].rows * 2U;
    if (overlaps(p[i].output, out_bytes, input, in_bytes)) return kInvalidValue;
    for (std::size_t j = 0; j < N; ++j) {
      if (touches_weight(p[i].output, out_bytes, shapes[j])) return kInvalidValue;
      if (j != i && overlaps(p[i].output, out_bytes, p[j].output, token_count * shapes[j].rows * 2U)) return kInvalidValue;
    }
  }
  return 0;
}
}  // namespace

int launch_projection_pair_tile_to_bf16_cuda(const ProjectionBackend backend, const LinearWeight& first_weight,
                                             const LinearWeight& second_weight, const std::uint16_t* input,
                                             const std::size_t token_count, float* fp32_scratch,
                                             const std::size_t scratch_elements, std::uint16_t* first_output,
                                             std::uint16_t* second_output, void* cuda_stream) noexcept {
  if (token_count > kMaximumProjectionTileTokenCount) return kInvalidValue;
  const SharedInputProjection pair[] = {{&first_weight, first_output}, {&second_weight, second_output}};
  if (const int st = check_shared_input(backend, pair, input, token_count); st != 0) return st;
  if (const int st = launch_projection_tile_to_bf16_cuda(backend, first_weight, input, token_count, fp32_scratch,
                                                         scratch_elements, first_output, cuda_stream);
      st != 0)
    return st;
  return launch_projection_tile_to_bf16_cuda(backend, second_weight, input, token_count, fp32_scratch, scratch_elements,
                                             second_output, cuda_stream);
}

int launch_linear_attention_qkv_z_ab_to_bf16_cuda(const ProjectionBackend backend, const LinearWeight& qkv_weight,
                                                  const LinearWeight& z_weight, const LinearWeight& a_weight,
                                                  const LinearWeight& b_weight, const std::uint16_t* input,
                                                  std::uint16_t* qkv_output, std::uint16_t* z_output,
                                                  std::uint16_t* a_output, std::uint16_t* b_output,
                                                  void* cuda_stream) noexcept {
  // structurally ineligible calls are "not supported" so that the caller keeps its two-call route (model_weights.h:892-897)
  if (!supports_linear_attention_qkv_z_ab_projection_fusion(backend, qkv_weight, z_weight, a_weight, b_weight))
    return kNotSupported;
  const SharedInputProjection group[] = {{&qkv_weight, qkv_output}, {&z_weight, z_output}, {&a_weight, a_output}, {&b_weight, b_output}};
  if (const int st = check_shared_input(backend, group, input, 1U); st != 0) return st;
  for (const SharedInputProjection& p : group)
    if (const int st = project(*p.weight, input, p.output, cuda_stream); st != 0) return st;
  return 0;
}

int launch_full_attention_q_kv_to_bf16_cuda(const ProjectionBackend backend, const LinearWeight& q_weight,
                                            const LinearWeight& key_weight, const LinearWeight& value_weight,
                                            const std::uint16_t* input, float* /*fp32_scratch*/,
                                            std::size_t /*scratch_elements*/, std::uint16_t* q_output,
                                            std::uint16_t* key_output, std::uint16_t* value_output,
                                            void* cuda_stream) noexcept {
  const SharedInputProjection group[] = {{&q_weight, q_output}, {&key_weight, key_output}, {&value_weight, value_output}};
  if (const int st = check_shared_input(backend, group, input, 1U); st != 0) return st;
  for (const SharedInputProjection& p : group)
    if (const int st = project(*p.weight, input, p.output, cuda_stream); st != 0) return st;
  return 0;
}

int launch_exact_fp8_whole_chunk_projection_to_bf16_cuda(const ProjectionBackend backend, const LinearWeight& weight,
                                                         const std::uint16_t* input, const std::size_t token_count,
                                                         std::uint16_t* output, void* cuda_stream) noexcept {
  // the reference's structural gate (projection_dispatch.cpp:1000-1024): weight-only backend, FP8 weight, a chunk
  // of 256 or 512 tokens, one of the five attention / GDN projection shapes
  const bool backend_ok = backend == ProjectionBackend::kSm87WeightOnly || backend == kProjectionBackendB200LayerOps;
  if (!backend_ok || weight.valueless_by_exception() || (token_count != 256U && token_count != 512U)) return kNotSupported;
  const auto* fp8 = std::get_if<Fp8LinearWeight>(&weight);
  if (fp8 == nullptr) return kNotSupported;
  const std::size_t n = fp8->output_size, k = fp8->input_size;
  const bool shape_ok = (k == 5120U && (n == 10240U || n == 6144U || n == 12288U || n == 1024U)) || (n == 5120U && k == 6144U);
  if (!shape_ok) return kNotSupported;
  const Shape s = describe(weight);
  if (!s.valid || input == nullptr || output == nullptr) return kInvalidValue;
  const std::size_t in_bytes = token_count * k * 2U, out_bytes = token_count * n * 2U;
  if (overlaps(output, out_bytes, input, in_bytes) || touches_weight(output, out_bytes, s)) return kInvalidValue;
  // (a pointer that misses the GEMM's 16-byte alignment comes back as cudaErrorNotSupported, as a near miss does there)
  return q3x_b200_fp8_gemm_bf16(fp8->weight, fp8->weight_scale, input, token_count, n, k, output, nullptr, 0U, cuda_stream);
}

int launch_mlp_gate_up_silu_to_bf16_cuda(const ProjectionBackend backend, const LinearWeight& gate_weight,
                                         const LinearWeight& up_weight, const std::uint16_t* input,
                                         float* /*fp32_scratch*/, std::size_t /*scratch_elements*/,
                                         std::uint16_t* gate_output, std::uint16_t* up_output,
                                         void* cuda_stream) noexcept {
  const Shape gate = describe(gate_weight), up = describe(up_weight);
  if (const int st = check_gate_up(backend, gate, up, input, gate_output, up_output); st != 0) return st;
  return gate_up_silu(gate_weight, up_weight, gate.rows, input, gate_output, up_output, cuda_stream);
}

int launch_post_attention_residual_norm_mlp_gate_up_silu_to_bf16_cuda(
    const ProjectionBackend backend, const LinearWeight& gate_weight, const LinearWeight& up_weight,
    const std::uint16_t* residual_left, std::uint16_t* residual_right_and_normalized, const std::uint16_t* norm_weight,
    const float epsilon, float* /*fp32_scratch*/, std::size_t /*scratch_elements*/, std::uint16_t* residual_output,
    std::uint16_t* gate_output, std::uint16_t* up_output, void* cuda_stream) noexcept {
  return post_attention(backend, gate_weight, up_weight, residual_left, residual_right_and_normalized, norm_weight,
                        epsilon, residual_output, gate_output, up_output, cuda_stream);
}

int launch_decode_runner_post_attention_residual_norm_mlp_gate_up_silu_dead_up_to_bf16_cuda(
    const ProjectionBackend backend, const LinearWeight& gate_weight, const LinearWeight& up_weight,
    const std::uint16_t* residual_left, std::uint16_t* residual_right_and_normalized, const std::uint16_t* norm_weight,
    const float epsilon, float* /*fp32_scratch*/, std::size_t /*scratch_elements*/, std::uint16_t* residual_output,
    std::uint16_t* gate_output, std::uint16_t* up_workspace, void* cuda_stream) noexcept {
  // same work: here the rounded up projection is written to up_workspace, which the caller treats as dead
  return post_attention(backend, gate_weight, up_weight, residual_left, residual_right_and_normalized, norm_weight,
                        epsilon, residual_output, gate_output, up_workspace, cuda_stream);
}

int launch_mlp_down_residual_norm_to_bf16_cuda(const ProjectionBackend backend, const LinearWeight& down_weight,
                                               const std::uint16_t* activation, const std::uint16_t* residual_left,
                                               const std::uint16_t* norm_weight, const float epsilon,
                                               float* /*fp32_scratch*/, std::size_t /*scratch_elements*/,
                                               std::uint16_t* raw_down_output, std::uint16_t* residual_output,
                                               std::uint16_t* normalized_output, void* cuda_stream) noexcept {
  if (!projection_backend_served_by_b200(backend)) return kInvalidValue;
  const Shape down = describe(down_weight);
  if (!down.valid || down.rows != kHidden || activation == nullptr || residual_left == nullptr ||
      norm_weight == nullptr || raw_down_output == nullptr || residual_output == nullptr ||
      normalized_output == nullptr || !(std::isfinite(epsilon) && epsilon > 0.0F))
    return kInvalidValue;
  // three distinct output boundaries (model_weights.h:977-988); no writable range overlaps any other operand
  const std::size_t hidden_bytes = kHidden * 2U, in_bytes = down.cols * 2U;
  std::uint16_t* const outs[] = {raw_down_output, residual_output, normalized_output};
  for (int i = 0; i < 3; ++i) {
    for (int j = i + 1; j < 3; ++j)
      if (overlaps(outs[i], hidden_bytes, outs[j], hidden_bytes)) return kInvalidValue;
    if (overlaps(outs[i], hidden_bytes, activation, in_bytes) || overlaps(outs[i], hidden_bytes, residual_left, hidden_bytes) ||
        overlaps(outs[i], hidden_bytes, norm_weight, hidden_bytes) || touches_weight(outs[i], hidden_bytes, down))
      return kInvalidValue;
  }
  const int st = project(down_weight, activation, raw_down_output, cuda_stream);
  if (st != 0) return st;
  return q3x_b200_residual_add_rms_norm(residual_left, raw_down_output, norm_weight, 1U, kHidden, epsilon, residual_output,
                                        normalized_output, cuda_stream);
}

// ---- the elementwise halves ----------------------------------------------------------------------------

int launch_mlp_gate_up_silu_epilogue_cuda(const ProjectionBackend backend, std::uint16_t* gate_output,
                                          const std::uint16_t* up_output, const std::size_t token_count,
                                          const std::size_t intermediate_size, void* cuda_stream) noexcept {
  if (const int r = route_half(backend); r != 0) return r;
  if (intermediate_size != 0U && token_count > static_cast<std::size_t>(-1) / intermediate_size) return kInvalidValue;
  return q3x_b200_silu_mul(gate_output, up_output, token_count * intermediate_size, gate_output, cuda_stream);
}

int launch_post_attention_residual_norm_prologue_cuda(const ProjectionBackend backend,
                                                      const std::uint16_t* residual_left,
                                                      std::uint16_t* residual_right_and_normalized,
                                                      const std::uint16_t* norm_weight, const float epsilon,
                                                      const std::size_t token_count, const std::size_t hidden_size,
                                                      std::uint16_t* residual_output, void* cuda_stream) noexcept {
  if (const int r = route_half(backend); r != 0) return r;
  if (hidden_size != kHidden || token_count == 0U) return kInvalidValue;  // projection_dispatch.cpp:483-534
  return q3x_b200_residual_add_rms_norm(residual_left, residual_right_and_normalized, norm_weight, token_count,
                                        hidden_size, epsilon, residual_output, residual_right_and_normalized,
                                        cuda_stream);
}

int launch_mlp_down_residual_norm_epilogue_cuda(const ProjectionBackend backend, const std::uint16_t* raw_down_output,
                                                const std::uint16_t* residual_left, const std::uint16_t* norm_weight,
                                                const float epsilon, const std::size_t token_count,
                                                const std::size_t hidden_size, std::uint16_t* residual_output,
                                                std::uint16_t* normalized_output, void* cuda_stream) noexcept {
  if (const int r = route_half(backend); r != 0) return r;
  // three distinct boundaries (model_weights.h:977-983): raw down stays observable
  if (hidden_size != kHidden || token_count == 0U || normalized_output == nullptr ||
      normalized_output == raw_down_output)
    return kInvalidValue;
  return q3x_b200_residual_add_rms_norm(residual_left, raw_down_output, norm_weight, token_count, hidden_size, epsilon,
                                        residual_output, normalized_output, cuda_stream);
}

}  // namespace q3x::runtime
