// Role requirements, inventories and the C8192 validator.  The rules are those of the reference's
// src/runtime/prefill_operator_bindings.cpp (requirements :107-146, validation :158-385), restated
// with a per-role requirement table and one pass over the bindings that fills a set of "family"
// flags, each of which can only be cleared.
#include "q3x_b200_prefill_bindings.hpp"

namespace q3x::runtime {
namespace {

using Issue = PrefillOperatorBindingIssue;
using State = PrefillResourceBindingState;

constexpr bool known_role(const PrefillBindingRole role) noexcept {
  return static_cast<std::uint8_t>(role) < static_cast<std::uint8_t>(PrefillBindingRole::kCount);
}

// weight, sidecar, workspace, launcher, completion event -- indexed by role
constexpr PrefillOperatorRoleRequirements kQuantisedProjection{true, true, true, true, true};
constexpr PrefillOperatorRoleRequirements kWeightedOperator{true, false, true, true, true};
constexpr PrefillOperatorRoleRequirements kWeightlessOperator{false, false, true, true, true};
constexpr PrefillOperatorRoleRequirements kHandoff{false, false, false, true, true};
constexpr PrefillOperatorRoleRequirements kNothing{false, false, false, false, false};

constexpr PrefillOperatorRoleRequirements kByRole[kPrefillRequiredOperatorRoleCount] = {
    kQuantisedProjection,  // kNvfp4GateUp
    kQuantisedProjection,  // kNvfp4Down
    kQuantisedProjection,  // kLinearFp8Qkv
    kQuantisedProjection,  // kLinearFp8Z
    kQuantisedProjection,  // kLinearFp8O
    kQuantisedProjection,  // kFullFp8Q
    kQuantisedProjection,  // kFullFp8K
    kQuantisedProjection,  // kFullFp8V
    kQuantisedProjection,  // kFullFp8O
    kWeightedOperator,     // kLinearBf16A
    kWeightedOperator,     // kLinearBf16B
    kWeightedOperator,     // kExactGdn
    kWeightlessOperator,   // kExactCausalAttention
    kWeightlessOperator,   // kResidual
    kWeightedOperator,     // kNormalization
    kWeightedOperator,     // kEmbedding
    kHandoff,              // kFinalHandoff
};

constexpr PrefillResourceBinding open_slot(const bool required) noexcept {
  return PrefillResourceBinding{required ? State::kUnbound : State::kNotRequired, 0U};
}

PrefillOperatorBindingSet inventory(const std::uint32_t panel_tokens,
                                    const PrefillBindingAttestation attestation) noexcept {
  PrefillOperatorBindingSet set;
  set.binding_count = set.bindings.size();
  for (std::size_t i = 0; i < set.bindings.size(); ++i) {
    PrefillOperatorBinding& b = set.bindings[i];
    const PrefillOperatorRoleRequirements need = kByRole[i];
    b.role = static_cast<PrefillBindingRole>(i);
    b.maximum_logical_panel_m = panel_tokens;
    b.numerical_mode = PrefillNumericalMode::kExact;
    b.provider = PrefillOperatorProvider::kNative;
    b.tactic = PrefillTacticBinding{PrefillTacticMode::kAheadOfTime, 0U};  // required mode, not yet chosen
    b.weight = open_slot(need.weight);
    b.sidecar = open_slot(need.sidecar);
    b.workspace = open_slot(need.workspace);
    b.launcher = open_slot(need.launcher);
    b.completion_event = open_slot(need.completion_event);
    b.attestation = attestation;
    b.uses_mtp = false;
  }
  return set;
}

// identity must be zero unless bound, non-zero when bound
constexpr bool well_formed(const PrefillResourceBinding& r) noexcept {
  switch (r.state) {
    case State::kNotRequired:
    case State::kUnbound:
      return r.identity == 0U;
    case State::kBound:
      return r.identity != 0U;
  }
  return false;
}

struct Verdict {
  std::uint64_t mask = 0U;
  void raise(const Issue issue) noexcept { mask |= static_cast<std::uint64_t>(issue); }
  // one resource slot against its requirement; clears `family` when the slot falls short
  void slot(const PrefillResourceBinding& r, const bool required, const Issue shortfall, bool& family) noexcept {
    const bool formed = well_formed(r);
    if (!formed) raise(Issue::kMalformedBindingIdentity);
    const bool satisfied = formed && (required ? r.bound() : r.state == State::kNotRequired);
    if (!satisfied) {
      raise(shortfall);
      family = false;
    }
  }
};

}  // namespace

PrefillOperatorRoleRequirements prefill_operator_role_requirements(const PrefillBindingRole role) noexcept {
  return known_role(role) ? kByRole[static_cast<std::size_t>(role)] : kNothing;
}

PrefillOperatorBindingSet make_unbound_layer_major_c8192_operator_bindings() noexcept {
  return inventory(kLayerMajorPrefillOperatorPanelTokens, PrefillBindingAttestation::kUnboundDesign);
}

PrefillOperatorBindingSet make_legacy_c512_prefill_launcher_inventory() noexcept {
  return inventory(kLayerMajorPrefillLegacyPublicTileTokens, PrefillBindingAttestation::kLegacyC512InventoryOnly);
}

PrefillOperatorBindingValidation validate_layer_major_c8192_operator_bindings(
    const PrefillOperatorBindingSet& set) noexcept {
  PrefillOperatorBindingValidation out;
  Verdict v;
  const std::size_t capacity = set.bindings.size();
  const std::size_t inspected = set.binding_count < capacity ? set.binding_count : capacity;
  if (set.binding_count > capacity) v.raise(Issue::kInvalidRole);

  // role census
  for (std::size_t i = 0; i < inspected; ++i) {
    const PrefillBindingRole role = set.bindings[i].role;
    if (!known_role(role)) {
      v.raise(Issue::kInvalidRole);
      continue;
    }
    std::uint8_t& seen = out.role_counts[static_cast<std::size_t>(role)];
    if (seen != 0U) v.raise(Issue::kDuplicateRole);
    if (seen != 0xffU) ++seen;
  }
  bool coverage = set.binding_count == capacity;
  for (const std::uint8_t seen : out.role_counts) {
    if (seen == 0U) v.raise(Issue::kMissingRole);
    if (seen != 1U) coverage = false;
  }

  // families: each starts satisfied and can only be cleared
  bool capacity_ok = true, exact = true, native = true, aot = true, artifacts = true, workspaces = true,
       launchers = true, events = true, boundaries = true, attested = true;
  std::uint64_t gate_up_tactic = 0U, down_tactic = 0U;
  for (std::size_t i = 0; i < inspected; ++i) {
    const PrefillOperatorBinding& b = set.bindings[i];
    if (!known_role(b.role)) {
      capacity_ok = exact = native = aot = artifacts = workspaces = launchers = events = boundaries = attested = false;
      continue;
    }
    if (b.role == PrefillBindingRole::kNvfp4GateUp) gate_up_tactic = b.tactic.identity;
    if (b.role == PrefillBindingRole::kNvfp4Down) down_tactic = b.tactic.identity;

    if (b.maximum_logical_panel_m < kLayerMajorPrefillOperatorPanelTokens) {
      v.raise(Issue::kInsufficientLogicalPanelCapacity);
      capacity_ok = false;
    }
    switch (b.numerical_mode) {
      case PrefillNumericalMode::kExact:
        break;
      case PrefillNumericalMode::kUnbound:
        v.raise(Issue::kNumericalModeUnbound);
        exact = false;
        break;
      case PrefillNumericalMode::kApproximate:
        v.raise(Issue::kApproximateNumericsForbidden);
        exact = boundaries = false;
        break;
      default:
        v.raise(Issue::kMalformedEnumEncoding);
        exact = boundaries = false;
        break;
    }
    switch (b.provider) {
      case PrefillOperatorProvider::kNative:
        break;
      case PrefillOperatorProvider::kUnbound:
        v.raise(Issue::kProviderUnbound);
        native = false;
        break;
      case PrefillOperatorProvider::kCuBlasLtReference:
        v.raise(Issue::kCuBlasLtForbidden);
        v.raise(Issue::kNonNativeProvider);
        native = boundaries = false;
        break;
      case PrefillOperatorProvider::kExternalRuntime:
        v.raise(Issue::kNonNativeProvider);
        native = boundaries = false;
        break;
      default:
        v.raise(Issue::kMalformedEnumEncoding);
        native = boundaries = false;
        break;
    }
    if (b.uses_mtp) {
      v.raise(Issue::kMtpForbidden);
      boundaries = false;
    }
    if (b.tactic.mode != PrefillTacticMode::kAheadOfTime) {
      v.raise(Issue::kTacticNotAot);
      aot = false;
    }
    if (b.tactic.identity == 0U) {
      v.raise(Issue::kTacticIdentityUnbound);
      aot = false;
    }
    const PrefillOperatorRoleRequirements need = kByRole[static_cast<std::size_t>(b.role)];
    v.slot(b.weight, need.weight, Issue::kWeightBindingIncomplete, artifacts);
    v.slot(b.sidecar, need.sidecar, Issue::kSidecarBindingIncomplete, artifacts);
    v.slot(b.workspace, need.workspace, Issue::kWorkspaceBindingIncomplete, workspaces);
    v.slot(b.launcher, need.launcher, Issue::kLauncherBindingIncomplete, launchers);
    v.slot(b.completion_event, need.completion_event, Issue::kCompletionEventBindingIncomplete, events);
    switch (b.attestation) {
      case PrefillBindingAttestation::kAuthenticatedC8192:
        break;
      case PrefillBindingAttestation::kUnboundDesign:
        v.raise(Issue::kC8192AttestationUnbound);
        attested = false;
        break;
      case PrefillBindingAttestation::kLegacyC512InventoryOnly:
        v.raise(Issue::kLegacyC512InventoryOnly);
        attested = false;
        break;
      default:
        v.raise(Issue::kMalformedEnumEncoding);
        attested = false;
        break;
    }
  }
  // gate/up and down must not share one tactic artifact
  if (gate_up_tactic != 0U && gate_up_tactic == down_tactic) {
    v.raise(Issue::kGateDownTacticAlias);
    aot = false;
  }

  out.issue_mask = v.mask;
  out.role_coverage_complete = coverage;
  out.logical_capacity_complete = coverage && capacity_ok;
  out.exact_numerics_complete = coverage && exact;
  out.native_provider_complete = coverage && native;
  out.aot_tactics_complete = coverage && aot;
  out.artifact_bindings_complete = coverage && artifacts;
  out.workspace_bindings_complete = coverage && workspaces;
  out.launcher_bindings_complete = coverage && launchers;
  out.completion_events_complete = coverage && events;
  out.forbidden_boundaries_satisfied = coverage && boundaries;
  out.attestation_complete = coverage && attested;
  out.operator_bindings_complete =
      coverage && capacity_ok && exact && native && aot && artifacts && workspaces && launchers && events &&
      boundaries && attested && v.mask == 0U;
  return out;
}

namespace {
constexpr std::uint64_t fnv1a(const char* text) noexcept {
  std::uint64_t h = 0xcbf29ce484222325ULL;
  for (; *text != '\0'; ++text) h = (h ^ static_cast<unsigned char>(*text)) * 0x100000001b3ULL;
  return h == 0U ? 1U : h;
}
}  // namespace

std::uint64_t b200_launcher_identity(const PrefillBindingRole role) noexcept {
  switch (role) {
    case PrefillBindingRole::kResidual:
      return fnv1a("q3x_b200_residual_add_rms_norm");
    case PrefillBindingRole::kNormalization:
      return fnv1a("q3x_b200_rms_norm");
    case PrefillBindingRole::kEmbedding:
      return fnv1a("q3x_b200_embedding_gather");
    default:
      return 0U;
  }
}

PrefillOperatorBindingSet make_b200_layer_op_bindings() noexcept {
  PrefillOperatorBindingSet set = make_unbound_layer_major_c8192_operator_bindings();
  for (PrefillOperatorBinding& b : set.bindings) {
    const std::uint64_t id = b200_launcher_identity(b.role);
    if (id == 0U) continue;
    b.tactic = PrefillTacticBinding{PrefillTacticMode::kAheadOfTime, id ^ 0x5a5a5a5a5a5a5a5aULL};
    b.launcher = PrefillResourceBinding{PrefillResourceBindingState::kBound, id};
  }
  return set;
}

}  // namespace q3x::runtime
