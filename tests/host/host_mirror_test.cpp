// Host-side checks of the C++ mirror (no GPU needed: every call below must be answered by the
// argument checks before any device work).  Mirrors the style of the reference's own plain test
// executables: counts failures, prints them, returns non-zero when any check failed.
#include <cstdint>
#include <cstdio>

#include "q3x_b200_nvfp4.hpp"
#include "q3x_b200_ops.hpp"

namespace rt = q3x::runtime;

static int failures = 0;
#define EXPECT(cond)                                                  \
  do {                                                                \
    if (!(cond)) {                                                    \
      ++failures;                                                     \
      std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);     \
    }                                                                 \
  } while (0)

static void test_launcher_limits() {
  auto* p = reinterpret_cast<std::uint16_t*>(0x100000);  // never dereferenced on these paths
  auto* f = reinterpret_cast<float*>(0x900000);
  constexpr int kInvalid = 1;
  // M32 entry admits exactly 32 tokens; the prefill entry 1..512 tokens of width 5120
  EXPECT(rt::launch_residual_add_headwise_centered_rms_norm_m32_5120_cuda(p, p + 0x100000, p + 0x200000, 31, 5120, 1e-6F,
                                                                        p + 0x300000, p + 0x400000) == kInvalid);
  EXPECT(rt::launch_residual_add_headwise_centered_rms_norm_prefill_5120_cuda(p, p + 0x100000, p + 0x200000, 513, 5120,
                                                                            1e-6F, p + 0x300000,
                                                                            p + 0x400000) == kInvalid);
  EXPECT(rt::launch_residual_add_headwise_centered_rms_norm_prefill_5120_cuda(p, p + 0x100000, p + 0x200000, 0, 5120,
                                                                            1e-6F, p + 0x300000,
                                                                            p + 0x400000) == kInvalid);
  EXPECT(rt::launch_residual_add_headwise_centered_rms_norm_prefill_5120_cuda(p, p + 0x100000, p + 0x200000, 8, 4096,
                                                                            1e-6F, p + 0x300000,
                                                                            p + 0x400000) == kInvalid);
  EXPECT(rt::launch_qk_partial_neox_rope_tile_24_4_256_64_cuda(p, p + 0x100000, f, f + 0x1000, 0, 17) == kInvalid);
  EXPECT(rt::launch_qk_partial_neox_rope_tile_24_4_256_64_cuda(p, p + 0x100000, f, f + 0x1000, 0, 0) == kInvalid);
  EXPECT(rt::launch_full_attention_preprocess_24_4_256_64_cuda(p, p + 0x100000, p + 0x200000, p + 0x210000, 1e-6F,
                                                               p + 0x300000, p + 0x800000, f, f + 0x100000, 0,
                                                               513) == kInvalid);
  EXPECT(rt::launch_full_attention_preprocess_24_4_256_64_prompt_wide_p8000_cuda(
             p, p + 0x100000, p + 0x200000, p + 0x210000, 1e-6F, p + 0x300000, p + 0x800000, f, f + 0x100000, 4000,
             8000) == kInvalid);
  EXPECT(rt::can_launch_full_attention_preprocess_prompt_wide_p8000(32000, 8000));
  EXPECT(!rt::can_launch_full_attention_preprocess_prompt_wide_p8000(40000, 8000));
  rt::GdnDimensions wrong;
  wrong.value_head_count = 32;
  EXPECT(rt::launch_causal_conv1d_silu_update_reference_cuda(p, p + 0x100000, p + 0x200000, p + 0x300000, wrong) ==
         kInvalid);
  EXPECT(rt::launch_causal_conv1d_silu_update_tile_reference_cuda(p, 17, p + 0x100000, p + 0x200000, p + 0x300000) ==
         kInvalid);
  namespace conv = rt::gdn_prefill_whole_span_conv_detail;
  EXPECT(conv::launch_causal_conv1d_silu_update_whole_span_exact_cuda(p, 513, p + 0x1000000, p + 0x2000000,
                                                                      p + 0x3000000) == kInvalid);
  EXPECT(conv::launch_causal_conv1d_silu_update_token_parallel_exact_cuda(p, 8, p + 0x1000000, p + 0x2000000, p) ==
         kInvalid);  // this form needs a disjoint output
  // empty shapes are successful no-ops even with null pointers; a bad epsilon is not
  EXPECT(rt::launch_residual_add_reference_cuda(nullptr, nullptr, 0, nullptr) == 0);
  EXPECT(rt::launch_silu_mul_reference_cuda(nullptr, nullptr, 0, nullptr) == 0);
  EXPECT(rt::launch_centered_rms_norm_reference_cuda(nullptr, nullptr, 0, 1e-6F, nullptr) == 0);
  EXPECT(rt::launch_centered_rms_norm_reference_cuda(p, p + 0x1000, 8, 0.0F, p + 0x2000) == kInvalid);
  EXPECT(rt::launch_embedding_gather_reference_cuda(p, 100, 8, 100, p + 0x100000) == kInvalid);  // id out of range
  EXPECT(rt::launch_embedding_gather_prompt_reference_cuda(p, 100, 8, nullptr, 0, p + 0x100000) == kInvalid);
  // chunked GDN prefill: 1 to 512 tokens, the whole workspace, both norm operands, a valid norm epsilon
  {
    namespace chunked = rt::gdn_prefill_chunk64_native_detail;
    const std::size_t bytes = chunked::workspace_bytes();
    EXPECT(bytes > 0 && bytes % 16 == 0);
    auto* ws = reinterpret_cast<std::uint8_t*>(0x40000000);
    auto call = [&](void* w, std::size_t cap, std::size_t tokens, const std::uint16_t* nw, float norm_eps) {
      return chunked::launch(w, cap, p, tokens, p + 0x1000000, p + 0x1100000, p + 0x1200000, p + 0x1300000, p + 0x2000000,
                             p + 0x2000000, 1e-6F, nw, p + 0x3000000, norm_eps, p + 0x5000000);
    };
    EXPECT(call(ws, bytes, 0, p + 0x1400000, 1e-6F) == kInvalid);
    EXPECT(call(ws, bytes, 513, p + 0x1400000, 1e-6F) == kInvalid);
    EXPECT(call(nullptr, bytes, 64, p + 0x1400000, 1e-6F) == kInvalid);
    EXPECT(call(ws, bytes - 16, 64, p + 0x1400000, 1e-6F) == kInvalid);
    EXPECT(call(ws, bytes, 64, nullptr, 1e-6F) == kInvalid);
    EXPECT(call(ws, bytes, 64, p + 0x1400000, 0.0F) == kInvalid);
  }
}

static void test_dispatch() {
  using B = rt::ProjectionBackend;
  auto* p = reinterpret_cast<std::uint16_t*>(0x100000);
  EXPECT(rt::is_valid_projection_backend(B::kReference) && rt::is_valid_projection_backend(B::kSm87WeightOnly) &&
         rt::is_valid_projection_backend(B::kB200LayerOps) && !rt::is_valid_projection_backend(static_cast<B>(7)));
  EXPECT(static_cast<int>(B::kReference) == 0 && static_cast<int>(B::kSm87WeightOnly) == 1);
  // other backends are told "not supported" so the caller falls back; junk is invalid
  EXPECT(rt::launch_mlp_gate_up_silu_epilogue_cuda(B::kReference, p, p + 0x100000, 1, 17408) == 801);
  EXPECT(rt::launch_mlp_gate_up_silu_epilogue_cuda(B::kSm87WeightOnly, p, p + 0x100000, 1, 17408) == 801);
  EXPECT(rt::launch_mlp_gate_up_silu_epilogue_cuda(static_cast<B>(9), p, p + 0x100000, 1, 17408) == 1);
  EXPECT(rt::launch_mlp_gate_up_silu_epilogue_cuda(B::kB200LayerOps, nullptr, nullptr, 0, 17408) == 0);
  EXPECT(rt::launch_post_attention_residual_norm_prologue_cuda(B::kB200LayerOps, p, p + 0x100000, p + 0x200000, 1e-6F,
                                                               1, 4096, p + 0x300000) == 1);
  EXPECT(rt::launch_mlp_down_residual_norm_epilogue_cuda(B::kB200LayerOps, p, p + 0x100000, p + 0x200000, 1e-6F, 1,
                                                         5120, p + 0x300000, nullptr) == 1);
  EXPECT(rt::launch_mlp_down_residual_norm_epilogue_cuda(B::kB200LayerOps, p, p + 0x100000, p + 0x200000, 1e-6F, 1,
                                                         5120, p + 0x300000, p) == 1);  // normalized == raw down
  // eligibility predicates of the fused projection routes: backend, weight type, the model's exact shapes, payload
  auto* b8 = reinterpret_cast<std::uint8_t*>(0x4000000);
  auto* sc = reinterpret_cast<float*>(0x9000000);
  auto fp8 = [&](std::size_t rows) {
    rt::Fp8LinearWeight w{};
    w.weight = b8; w.weight_scale_device = sc; w.input_scale_device = sc;
    w.weight_scale = 0.02F; w.input_scale = 1.0F; w.output_size = rows; w.input_size = 5120;
    return rt::LinearWeight{w};
  };
  auto bf = [&](std::size_t rows) {
    rt::Bf16LinearWeight w{};
    w.weight = p; w.output_size = rows; w.input_size = 5120;
    return rt::LinearWeight{w};
  };
  auto fp4 = [&](std::size_t rows, std::size_t cols) {
    rt::NvFp4LinearWeight w{};
    w.packed_weight = b8; w.block_scale = b8 + 0x8000000; w.weight_scale_2_device = sc; w.input_scale_device = sc;
    w.weight_scale_2 = 0.01F; w.input_scale = 1.0F; w.output_size = rows; w.input_size = cols;
    return rt::LinearWeight{w};
  };
  EXPECT(rt::linear_weight_kind(fp8(1024)) == rt::LinearWeightKind::kFp8 && rt::linear_output_size(fp8(1024)) == 1024 &&
         rt::linear_input_size(bf(48)) == 5120 && rt::linear_weight_kind(bf(48)) == rt::LinearWeightKind::kBf16 &&
         rt::linear_weight_kind(fp4(17408, 5120)) == rt::LinearWeightKind::kNvFp4);
  EXPECT(rt::supports_bf16_projection_pair(B::kSm87WeightOnly, bf(48), bf(48)));
  EXPECT(!rt::supports_bf16_projection_pair(B::kReference, bf(48), bf(48)));       // not the selected fast backend
  EXPECT(!rt::supports_bf16_projection_pair(B::kSm87WeightOnly, bf(48), bf(64)));  // wrong rows
  EXPECT(!rt::supports_bf16_projection_pair(B::kSm87WeightOnly, bf(48), fp8(48))); // wrong type
  EXPECT(rt::supports_fp8_projection_pair(B::kSm87WeightOnly, fp8(1024), fp8(1024)) &&
         !rt::supports_fp8_projection_pair(B::kSm87WeightOnly, fp8(1024), fp8(2048)));
  EXPECT(rt::supports_fp8_qkv_z_projection_pair(B::kB200LayerOps, fp8(10240), fp8(6144)) &&
         !rt::supports_fp8_qkv_z_projection_pair(B::kSm87WeightOnly, fp8(6144), fp8(10240)));
  EXPECT(rt::supports_linear_attention_qkv_z_ab_projection_fusion(B::kSm87WeightOnly, fp8(10240), fp8(6144), bf(48), bf(48)) &&
         !rt::supports_linear_attention_qkv_z_ab_projection_fusion(B::kSm87WeightOnly, fp8(10240), fp8(6144), bf(48), bf(32)));
  EXPECT(rt::supports_fp8_q_kv_projection_fusion(B::kSm87WeightOnly, fp8(12288), fp8(1024), fp8(1024)) &&
         !rt::supports_fp8_q_kv_projection_fusion(B::kSm87WeightOnly, fp8(6144), fp8(1024), fp8(1024)));
  EXPECT(rt::supports_nvfp4_gate_up_silu_fusion(B::kSm87WeightOnly, fp4(17408, 5120), fp4(17408, 5120)) &&
         !rt::supports_nvfp4_gate_up_silu_fusion(B::kSm87WeightOnly, fp4(17408, 5120), fp8(17408)));
  EXPECT(rt::supports_nvfp4_down_residual_norm_fusion(B::kSm87WeightOnly, fp4(5120, 17408)) &&
         !rt::supports_nvfp4_down_residual_norm_fusion(B::kSm87WeightOnly, fp4(17408, 5120)));
  {
    rt::Fp8LinearWeight hollow = std::get<rt::Fp8LinearWeight>(fp8(1024));
    hollow.weight_scale_device = nullptr;  // incomplete payload
    EXPECT(!rt::supports_fp8_projection_pair(B::kSm87WeightOnly, rt::LinearWeight{hollow}, fp8(1024)));
  }
  // the fused four-projection call is "not supported" off its exact group, before anything else is looked at
  EXPECT(rt::launch_linear_attention_qkv_z_ab_to_bf16_cuda(B::kSm87WeightOnly, fp8(10240), fp8(6144), bf(48), bf(32), p, p, p,
                                                           p, p) == 801);
  EXPECT(rt::launch_linear_attention_qkv_z_ab_to_bf16_cuda(B::kReference, fp8(10240), fp8(6144), bf(48), bf(48), p, p, p, p,
                                                           p) == 801);
  // the eligible group still validates its buffers: every output here aliases the input
  EXPECT(rt::launch_linear_attention_qkv_z_ab_to_bf16_cuda(B::kSm87WeightOnly, fp8(10240), fp8(6144), bf(48), bf(48), p, p, p,
                                                           p, p) == 1);
  auto* f = reinterpret_cast<float*>(0x20000000);
  EXPECT(rt::launch_projection_reference_cuda(fp8(1024), nullptr, f) == 1);
  EXPECT(rt::launch_projection_to_bf16_reference_cuda(fp8(1024), p, f, 1023, p + 0x800000) == 1);  // scratch too small
  EXPECT(rt::launch_projection_to_bf16_reference_cuda(fp8(1024), p, nullptr, 1024, p + 0x800000) == 1);
  EXPECT(rt::launch_projection_pair_tile_to_bf16_cuda(B::kSm87WeightOnly, fp8(1024), fp8(1024), p, 65, nullptr, 0,
                                                      p + 0x800000, p + 0xa00000) == 1);  // above the tile limit
  EXPECT(rt::launch_projection_pair_tile_to_bf16_cuda(B::kSm87WeightOnly, fp8(1024), fp8(1024), p, 4, nullptr, 0,
                                                      p + 0x800000, p + 0x800000) == 1);  // the outputs alias
  EXPECT(rt::launch_full_attention_q_kv_to_bf16_cuda(B::kSm87WeightOnly, fp8(12288), fp8(1024), fp8(1024), p, nullptr, 0,
                                                     p + 0x800000, p + 0xa00000, p + 0xa00100) == 1);  // k and v overlap
}

static void test_bindings() {
  using Issue = rt::PrefillOperatorBindingIssue;
  auto has = [](const rt::PrefillOperatorBindingValidation& v, Issue i) {
    return rt::has_prefill_operator_binding_issue(v, i);
  };
  const auto design = rt::make_unbound_layer_major_c8192_operator_bindings();
  EXPECT(design.binding_count == 17);
  auto v = rt::validate_layer_major_c8192_operator_bindings(design);
  EXPECT(v.role_coverage_complete && v.logical_capacity_complete && v.exact_numerics_complete &&
         v.native_provider_complete && v.forbidden_boundaries_satisfied);
  EXPECT(!v.aot_tactics_complete && !v.launcher_bindings_complete && !v.attestation_complete && !v.complete() &&
         !v.executable());
  EXPECT(has(v, Issue::kTacticIdentityUnbound) && has(v, Issue::kLauncherBindingIncomplete) &&
         has(v, Issue::kC8192AttestationUnbound) && !has(v, Issue::kMissingRole));

  const auto legacy = rt::make_legacy_c512_prefill_launcher_inventory();
  v = rt::validate_layer_major_c8192_operator_bindings(legacy);
  EXPECT(has(v, Issue::kInsufficientLogicalPanelCapacity) && has(v, Issue::kLegacyC512InventoryOnly) &&
         !v.logical_capacity_complete);

  // a fully bound, authenticated set validates (and is still not executable)
  auto full = design;
  std::uint64_t next = 100;
  for (auto& b : full.bindings) {
    const auto need = rt::prefill_operator_role_requirements(b.role);
    b.tactic.identity = next++;
    auto bind = [&](rt::PrefillResourceBinding& r, bool required) {
      if (required) r = {rt::PrefillResourceBindingState::kBound, next++};
    };
    bind(b.weight, need.weight);
    bind(b.sidecar, need.sidecar);
    bind(b.workspace, need.workspace);
    bind(b.launcher, need.launcher);
    bind(b.completion_event, need.completion_event);
    b.attestation = rt::PrefillBindingAttestation::kAuthenticatedC8192;
  }
  v = rt::validate_layer_major_c8192_operator_bindings(full);
  EXPECT(v.issue_mask == 0 && v.complete() && !v.executable());

  auto broken = full;
  broken.bindings[1].tactic.identity = broken.bindings[0].tactic.identity;  // gate/up and down share a tactic
  EXPECT(has(rt::validate_layer_major_c8192_operator_bindings(broken), Issue::kGateDownTacticAlias));
  broken = full;
  broken.bindings[3].role = rt::PrefillBindingRole::kLinearFp8Qkv;  // duplicate + missing
  v = rt::validate_layer_major_c8192_operator_bindings(broken);
  EXPECT(has(v, Issue::kDuplicateRole) && has(v, Issue::kMissingRole) && !v.role_coverage_complete && !v.complete());
  broken = full;
  broken.bindings[5].provider = rt::PrefillOperatorProvider::kCuBlasLtReference;
  broken.bindings[6].numerical_mode = rt::PrefillNumericalMode::kApproximate;
  broken.bindings[7].uses_mtp = true;
  broken.bindings[8].weight = {rt::PrefillResourceBindingState::kUnbound, 5};  // identity without a binding
  broken.bindings[9].role = static_cast<rt::PrefillBindingRole>(40);
  v = rt::validate_layer_major_c8192_operator_bindings(broken);
  EXPECT(has(v, Issue::kCuBlasLtForbidden) && has(v, Issue::kNonNativeProvider) &&
         has(v, Issue::kApproximateNumericsForbidden) && has(v, Issue::kMtpForbidden) &&
         has(v, Issue::kMalformedBindingIdentity) && has(v, Issue::kWeightBindingIncomplete) &&
         has(v, Issue::kInvalidRole) && !v.forbidden_boundaries_satisfied);
  broken = full;
  broken.binding_count = 18;
  EXPECT(has(rt::validate_layer_major_c8192_operator_bindings(broken), Issue::kInvalidRole));

  // requirements table (prefill_operator_bindings.cpp:107-146)
  auto need = rt::prefill_operator_role_requirements(rt::PrefillBindingRole::kResidual);
  EXPECT(!need.weight && !need.sidecar && need.workspace && need.launcher && need.completion_event);
  need = rt::prefill_operator_role_requirements(rt::PrefillBindingRole::kNvfp4Down);
  EXPECT(need.weight && need.sidecar && need.workspace);
  need = rt::prefill_operator_role_requirements(rt::PrefillBindingRole::kFinalHandoff);
  EXPECT(!need.weight && !need.workspace && need.launcher);
  need = rt::prefill_operator_role_requirements(rt::PrefillBindingRole::kInvalid);
  EXPECT(!need.launcher && !need.completion_event);

  // this library's contribution: three roles get launcher + tactic identities, nothing else
  const auto ours = rt::make_b200_layer_op_bindings();
  int bound = 0;
  for (const auto& b : ours.bindings) {
    const bool mine = b.role == rt::PrefillBindingRole::kResidual || b.role == rt::PrefillBindingRole::kNormalization ||
                      b.role == rt::PrefillBindingRole::kEmbedding;
    EXPECT(b.launcher.bound() == mine && b.tactic.aot_bound() == mine);
    bound += b.launcher.bound() ? 1 : 0;
  }
  EXPECT(bound == 3);
  v = rt::validate_layer_major_c8192_operator_bindings(ours);
  EXPECT(!has(v, Issue::kMalformedBindingIdentity) && !v.complete() && has(v, Issue::kC8192AttestationUnbound));
}

static void test_nvfp4_front_end() {
  namespace qz = q3x::quantization;
  auto* p = reinterpret_cast<std::uint16_t*>(0x100000);
  qz::NvFp4ActivationBuffers b{reinterpret_cast<std::uint32_t*>(0x40000000), reinterpret_cast<float*>(0x41000000),
                               reinterpret_cast<std::uint8_t*>(0x42000000), reinterpret_cast<std::uint8_t*>(0x48000000)};
  EXPECT(qz::nvfp4_activation_scale_groups(16384, 512) == 32 && qz::nvfp4_activation_scale_groups(513, 512) == 2 &&
         qz::nvfp4_activation_scale_groups(7, 0) == 1 && qz::nvfp4_activation_scale_groups(0, 512) == 0);
  EXPECT(qz::nvfp4_activation_scratch_words(16384, 512) >= 2 * 32 + 2);
  auto* p8 = reinterpret_cast<std::uint8_t*>(0x50000000);
  // the reference's status vocabulary (include/q3x/quantization/nvfp4.h:41-46)
  EXPECT(static_cast<int>(qz::NvFp4Status::kInvalidColumnCount) == 2 && static_cast<int>(qz::NvFp4Status::kSizeOverflow) == 3);
  EXPECT(qz::validate_nvfp4_activation_shape(512, 5120) == qz::NvFp4Status::kSuccess);
  EXPECT(qz::validate_nvfp4_activation_shape(512, 5128) == qz::NvFp4Status::kInvalidColumnCount);
  EXPECT(qz::validate_nvfp4_activation_shape(static_cast<std::size_t>(-1) / 32, 64) == qz::NvFp4Status::kSizeOverflow);
  EXPECT(qz::nvfp4_status_string(qz::NvFp4Status::kSuccess)[0] == 's');
  // 128 x 4 scale tiles: 512 rows x 5120 columns = 4 row tiles x 80 block tiles; ragged edges round up
  EXPECT(qz::nvfp4_swizzled_block_scale_bytes(512, 5120) == 4 * 80 * 512);
  EXPECT(qz::nvfp4_swizzled_block_scale_bytes(130, 48) == 2 * 1 * 512);
  EXPECT(qz::launch_nvfp4_swizzle_block_scales_cuda(p8, 4, 24, p8 + 0x100000) == 1);  // not a block multiple
  // the projection on those operands: host-side refusals (shape, scale, workspace), empty problem, workspace query
  {
    qz::NvFp4ProjectionWeight weight{p8 + 0x1000000, p8 + 0x2000000, 0.5F, 64, 128};
    EXPECT(qz::nvfp4_projection_workspace_bytes(256, 64, 128, 0) >= 256 * sizeof(float));
    EXPECT(qz::nvfp4_projection_workspace_bytes(0, 64, 128, 0) == 0);
    const auto fp = reinterpret_cast<const float*>(p8 + 0x3000000);
    auto out = reinterpret_cast<std::uint16_t*>(p8 + 0x4000000);
    EXPECT(qz::launch_nvfp4_projection_to_bf16_cuda(weight, p8, p8 + 0x100000, fp, 0, 0, out, nullptr, 0) == 0);
    EXPECT(qz::launch_nvfp4_projection_to_bf16_cuda(weight, p8, p8 + 0x100000, fp, 0, 256, out, p8 + 0x5000000, 8) == 1);
    weight.in_features = 96;
    EXPECT(qz::launch_nvfp4_projection_to_bf16_cuda(weight, p8, p8 + 0x100000, fp, 0, 256, out, p8 + 0x5000000, 1 << 20) == 1);
    weight.in_features = 128;
    weight.scale_2 = -1.0F;
    EXPECT(qz::launch_nvfp4_projection_to_bf16_cuda(weight, p8, p8 + 0x100000, fp, 0, 256, out, p8 + 0x5000000, 1 << 20) == 1);
  }
  // empty shapes succeed with null buffers; bad shapes and missing buffers are refused on the host
  EXPECT(qz::launch_silu_mul_nvfp4_cuda(nullptr, nullptr, 0, 17408, 512, nullptr, {}) == 0);
  EXPECT(qz::launch_silu_mul_nvfp4_cuda(p, p + 0x1000000, 4, 17400, 512, p + 0x2000000, b) == 1);   // not a block multiple
  EXPECT(qz::launch_silu_mul_nvfp4_cuda(p, p + 0x1000000, 4, 17408, 512, p + 0x2000000, {}) == 1);  // no buffers
  EXPECT(qz::launch_residual_add_centered_rms_norm_nvfp4_cuda(p, p + 0x1000000, p + 0x2000000, 4, 5120, 0.0F, 512,
                                                              p + 0x3000000, p + 0x4000000, b) == 1);  // epsilon
  EXPECT(qz::launch_residual_add_centered_rms_norm_nvfp4_cuda(p, p + 0x1000000, p + 0x2000000, 4, 5120, 1e-6F, 512,
                                                              p + 0x3000000, nullptr, b) == 1);  // normalised rows required
  EXPECT(qz::launch_headwise_plain_rms_norm_silu_gate_nvfp4_cuda(p, p + 0x1000000, p + 0x2000000, 4, 48, 128, 1e-6F, 512,
                                                                 p + 0x2000008, b) == 1);  // partial overlap with the gate
  EXPECT(qz::launch_nvfp4_quantize_activations_cuda(p, 4, 5128, 512, b) == 1);             // not a block multiple
  EXPECT(qz::launch_sigmoid_gate_nvfp4_cuda(nullptr, nullptr, 0, 6144, 512, nullptr, {}) == 0);
  EXPECT(qz::launch_sigmoid_gate_nvfp4_cuda(p, p + 0x1000000, 4, 6144, 512, p + 8, b) == 1);  // partial overlap
}

int main() {
  test_launcher_limits();
  test_nvfp4_front_end();
  test_dispatch();
  test_bindings();
  if (failures == 0) std::printf("host mirror tests passed\n");
  return failures == 0 ? 0 : 1;
}
