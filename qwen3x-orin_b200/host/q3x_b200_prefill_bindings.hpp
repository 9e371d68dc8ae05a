// Prefill operator binding descriptors: the host-only value types and validator of
// include/q3x/runtime/prefill_operator_roles.h and prefill_operator_bindings.h, kept source-compatible
// (same type names, enumerator values, field names and function names) so that planning code written
// against the reference compiles against this library.  Nothing here touches the GPU; as in the
// reference a validated descriptor is never "executable" by itself.
//
// Added on top: make_b200_layer_op_bindings(), which fills in the roles this library actually
// provides kernels for (kResidual, kNormalization, kEmbedding) with its own launcher identities.
#pragma once

#include <array>
#include <cstddef>
#include <cstdint>

namespace q3x::runtime {

// prefill_operator_roles.h:11-31 -- enumerator order is ABI
enum class PrefillBindingRole : std::uint8_t {
  kNvfp4GateUp = 0, kNvfp4Down, kLinearFp8Qkv, kLinearFp8Z, kLinearFp8O, kFullFp8Q, kFullFp8K, kFullFp8V, kFullFp8O,
  kLinearBf16A, kLinearBf16B, kExactGdn, kExactCausalAttention, kResidual, kNormalization, kEmbedding, kFinalHandoff,
  kCount,
  kInvalid = 0xffU,
};
inline constexpr std::size_t kPrefillRequiredOperatorRoleCount = static_cast<std::size_t>(PrefillBindingRole::kCount);
inline constexpr std::size_t kLayerMajorPrefillRequiredOperatorRoleCount = kPrefillRequiredOperatorRoleCount;
static_assert(kPrefillRequiredOperatorRoleCount == 17U);

enum class PrefillNumericalMode : std::uint8_t { kUnbound = 0, kExact, kApproximate };
enum class PrefillOperatorProvider : std::uint8_t { kUnbound = 0, kNative, kCuBlasLtReference, kExternalRuntime };
enum class PrefillTacticMode : std::uint8_t { kUnbound = 0, kAheadOfTime, kJit, kRequestTimeSelected };

// prefill_execution_plan.h:22-24
inline constexpr std::uint32_t kLayerMajorPrefillLegacyPublicTileTokens = 512U;
inline constexpr std::uint32_t kLayerMajorPrefillOperatorPanelTokens = 8'192U;

// prefill_operator_bindings.h:23-38
enum class PrefillBindingAttestation : std::uint8_t { kUnboundDesign = 0, kLegacyC512InventoryOnly, kAuthenticatedC8192 };
enum class PrefillResourceBindingState : std::uint8_t { kNotRequired = 0, kUnbound, kBound };

struct PrefillResourceBinding {
  PrefillResourceBindingState state = PrefillResourceBindingState::kUnbound;
  std::uint64_t identity = 0U;  // opaque non-zero id, never an address or a callable
  [[nodiscard]] constexpr bool bound() const noexcept {
    return state == PrefillResourceBindingState::kBound && identity != 0U;
  }
};
struct PrefillTacticBinding {
  PrefillTacticMode mode = PrefillTacticMode::kUnbound;
  std::uint64_t identity = 0U;
  [[nodiscard]] constexpr bool aot_bound() const noexcept {
    return mode == PrefillTacticMode::kAheadOfTime && identity != 0U;
  }
};
struct PrefillOperatorRoleRequirements {  // which resources a role must have bound
  bool weight = false, sidecar = false, workspace = false;
  bool launcher = true, completion_event = true;
};
struct PrefillOperatorBinding {
  PrefillBindingRole role = PrefillBindingRole::kInvalid;
  std::uint32_t maximum_logical_panel_m = 0U;
  PrefillNumericalMode numerical_mode = PrefillNumericalMode::kUnbound;
  PrefillOperatorProvider provider = PrefillOperatorProvider::kUnbound;
  PrefillTacticBinding tactic;
  PrefillResourceBinding weight, sidecar, workspace, launcher, completion_event;  // in this order
  PrefillBindingAttestation attestation = PrefillBindingAttestation::kUnboundDesign;
  bool uses_mtp = false;
};
struct PrefillOperatorBindingSet {
  std::array<PrefillOperatorBinding, kLayerMajorPrefillRequiredOperatorRoleCount> bindings{};
  std::size_t binding_count = 0U;
};

// prefill_operator_bindings.h:86-110 -- bit positions are ABI
enum class PrefillOperatorBindingIssue : std::uint64_t {
  kNone = 0U,
  // roles and capacity
  kInvalidRole = 1ULL << 0U, kMissingRole = 1ULL << 1U, kDuplicateRole = 1ULL << 2U,
  kInsufficientLogicalPanelCapacity = 1ULL << 3U,
  // numerics, provider, forbidden boundaries
  kNumericalModeUnbound = 1ULL << 4U, kApproximateNumericsForbidden = 1ULL << 5U, kProviderUnbound = 1ULL << 6U,
  kNonNativeProvider = 1ULL << 7U, kCuBlasLtForbidden = 1ULL << 8U, kMtpForbidden = 1ULL << 9U,
  // tactics
  kTacticNotAot = 1ULL << 10U, kTacticIdentityUnbound = 1ULL << 11U, kGateDownTacticAlias = 1ULL << 12U,
  // resources
  kWeightBindingIncomplete = 1ULL << 13U, kSidecarBindingIncomplete = 1ULL << 14U,
  kWorkspaceBindingIncomplete = 1ULL << 15U, kLauncherBindingIncomplete = 1ULL << 16U,
  kCompletionEventBindingIncomplete = 1ULL << 17U, kMalformedBindingIdentity = 1ULL << 18U,
  // attestation and encoding
  kC8192AttestationUnbound = 1ULL << 19U, kLegacyC512InventoryOnly = 1ULL << 20U, kMalformedEnumEncoding = 1ULL << 21U,
};

struct PrefillOperatorBindingValidation {
  std::uint64_t issue_mask = 0U;
  std::array<std::uint8_t, kLayerMajorPrefillRequiredOperatorRoleCount> role_counts{};
  // one verdict per aspect; operator_bindings_complete is their conjunction
  bool role_coverage_complete = false, logical_capacity_complete = false, exact_numerics_complete = false;
  bool native_provider_complete = false, aot_tactics_complete = false, artifact_bindings_complete = false;
  bool workspace_bindings_complete = false, launcher_bindings_complete = false, completion_events_complete = false;
  bool forbidden_boundaries_satisfied = false, attestation_complete = false, operator_bindings_complete = false;
  [[nodiscard]] constexpr bool complete() const noexcept { return operator_bindings_complete; }
  // a descriptor is never a launchable plan (prefill_operator_bindings.h:139-142)
  [[nodiscard]] constexpr bool executable() const noexcept { return false; }
};

[[nodiscard]] constexpr bool has_prefill_operator_binding_issue(const PrefillOperatorBindingValidation& validation,
                                                                const PrefillOperatorBindingIssue issue) noexcept {
  return (validation.issue_mask & static_cast<std::uint64_t>(issue)) != 0U;
}

[[nodiscard]] PrefillOperatorRoleRequirements prefill_operator_role_requirements(PrefillBindingRole role) noexcept;
[[nodiscard]] PrefillOperatorBindingSet make_unbound_layer_major_c8192_operator_bindings() noexcept;
[[nodiscard]] PrefillOperatorBindingSet make_legacy_c512_prefill_launcher_inventory() noexcept;
[[nodiscard]] PrefillOperatorBindingValidation validate_layer_major_c8192_operator_bindings(
    const PrefillOperatorBindingSet& binding_set) noexcept;

// ---- this library's contribution to a binding set ---------------------------------------------------
// Launcher identities of the C-ABI entry points that serve the three roles on this path.  They are
// opaque ids (FNV-1a of the entry point's name), stable across builds, never addresses.
[[nodiscard]] std::uint64_t b200_launcher_identity(PrefillBindingRole role) noexcept;
// The unbound C8192 design with kResidual / kNormalization / kEmbedding given this library's tactic
// and launcher identities (panel capacity 8192, exact numerics, native provider, ahead-of-time
// tactic).  Weights, workspaces, events and the attestation stay unbound: they belong to the
// deployment, so the set still does not validate as complete.
[[nodiscard]] PrefillOperatorBindingSet make_b200_layer_op_bindings() noexcept;

}  // namespace q3x::runtime
