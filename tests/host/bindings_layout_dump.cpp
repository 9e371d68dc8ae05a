// Prints every ABI-relevant number of the prefill operator binding types -- enumerator values, struct sizes,
// alignments and field offsets, the issue bit positions, the role requirements the library reports -- one
// "name value" line each.  Compiled twice by the test: once against this library's mirror
// (q3x_b200_prefill_bindings.hpp) and once, with -DUSE_REFERENCE_HEADERS, against the reference project's own
// prefill_operator_roles.h / prefill_operator_bindings.h; the two outputs must be identical.
#include <cstddef>
#include <cstdint>
#include <cstdio>

#if defined(USE_REFERENCE_HEADERS)
#include "q3x/runtime/prefill_operator_bindings.h"
#include "q3x/runtime/prefill_operator_roles.h"
#else
#include "q3x_b200_prefill_bindings.hpp"
#endif

using namespace q3x::runtime;

#define VALUE(expr) std::printf("%s %llu\n", #expr, static_cast<unsigned long long>(expr))
#define ENUM(e) std::printf("%s %llu\n", #e, static_cast<unsigned long long>(e))
#define LAYOUT(T) std::printf("sizeof(%s) %zu\nalignof(%s) %zu\n", #T, sizeof(T), #T, alignof(T))
#define OFFSET(T, f) std::printf("offsetof(%s,%s) %zu\n", #T, #f, offsetof(T, f))

int main() {
  ENUM(PrefillBindingRole::kNvfp4GateUp); ENUM(PrefillBindingRole::kNvfp4Down); ENUM(PrefillBindingRole::kLinearFp8Qkv);
  ENUM(PrefillBindingRole::kLinearFp8Z); ENUM(PrefillBindingRole::kLinearFp8O); ENUM(PrefillBindingRole::kFullFp8Q);
  ENUM(PrefillBindingRole::kFullFp8K); ENUM(PrefillBindingRole::kFullFp8V); ENUM(PrefillBindingRole::kFullFp8O);
  ENUM(PrefillBindingRole::kLinearBf16A); ENUM(PrefillBindingRole::kLinearBf16B); ENUM(PrefillBindingRole::kExactGdn);
  ENUM(PrefillBindingRole::kExactCausalAttention); ENUM(PrefillBindingRole::kResidual);
  ENUM(PrefillBindingRole::kNormalization); ENUM(PrefillBindingRole::kEmbedding); ENUM(PrefillBindingRole::kFinalHandoff);
  ENUM(PrefillBindingRole::kCount); ENUM(PrefillBindingRole::kInvalid);
  VALUE(kPrefillRequiredOperatorRoleCount); VALUE(kLayerMajorPrefillRequiredOperatorRoleCount);
  ENUM(PrefillNumericalMode::kUnbound); ENUM(PrefillNumericalMode::kExact); ENUM(PrefillNumericalMode::kApproximate);
  ENUM(PrefillOperatorProvider::kUnbound); ENUM(PrefillOperatorProvider::kNative);
  ENUM(PrefillOperatorProvider::kCuBlasLtReference); ENUM(PrefillOperatorProvider::kExternalRuntime);
  ENUM(PrefillTacticMode::kUnbound); ENUM(PrefillTacticMode::kAheadOfTime); ENUM(PrefillTacticMode::kJit);
  ENUM(PrefillTacticMode::kRequestTimeSelected);
  ENUM(PrefillBindingAttestation::kUnboundDesign); ENUM(PrefillBindingAttestation::kLegacyC512InventoryOnly);
  ENUM(PrefillBindingAttestation::kAuthenticatedC8192);
  ENUM(PrefillResourceBindingState::kNotRequired); ENUM(PrefillResourceBindingState::kUnbound);
  ENUM(PrefillResourceBindingState::kBound);
  ENUM(PrefillOperatorBindingIssue::kNone); ENUM(PrefillOperatorBindingIssue::kInvalidRole);
  ENUM(PrefillOperatorBindingIssue::kMissingRole); ENUM(PrefillOperatorBindingIssue::kDuplicateRole);
  ENUM(PrefillOperatorBindingIssue::kInsufficientLogicalPanelCapacity);
  ENUM(PrefillOperatorBindingIssue::kNumericalModeUnbound); ENUM(PrefillOperatorBindingIssue::kApproximateNumericsForbidden);
  ENUM(PrefillOperatorBindingIssue::kProviderUnbound); ENUM(PrefillOperatorBindingIssue::kNonNativeProvider);
  ENUM(PrefillOperatorBindingIssue::kCuBlasLtForbidden); ENUM(PrefillOperatorBindingIssue::kMtpForbidden);
  ENUM(PrefillOperatorBindingIssue::kTacticNotAot); ENUM(PrefillOperatorBindingIssue::kTacticIdentityUnbound);
  ENUM(PrefillOperatorBindingIssue::kGateDownTacticAlias); ENUM(PrefillOperatorBindingIssue::kWeightBindingIncomplete);
  ENUM(PrefillOperatorBindingIssue::kSidecarBindingIncomplete); ENUM(PrefillOperatorBindingIssue::kWorkspaceBindingIncomplete);
  ENUM(PrefillOperatorBindingIssue::kLauncherBindingIncomplete);
  ENUM(PrefillOperatorBindingIssue::kCompletionEventBindingIncomplete);
  ENUM(PrefillOperatorBindingIssue::kMalformedBindingIdentity); ENUM(PrefillOperatorBindingIssue::kC8192AttestationUnbound);
  ENUM(PrefillOperatorBindingIssue::kLegacyC512InventoryOnly); ENUM(PrefillOperatorBindingIssue::kMalformedEnumEncoding);

  LAYOUT(PrefillResourceBinding); OFFSET(PrefillResourceBinding, state); OFFSET(PrefillResourceBinding, identity);
  LAYOUT(PrefillTacticBinding); OFFSET(PrefillTacticBinding, mode); OFFSET(PrefillTacticBinding, identity);
  LAYOUT(PrefillOperatorRoleRequirements); OFFSET(PrefillOperatorRoleRequirements, weight);
  OFFSET(PrefillOperatorRoleRequirements, sidecar); OFFSET(PrefillOperatorRoleRequirements, workspace);
  OFFSET(PrefillOperatorRoleRequirements, launcher); OFFSET(PrefillOperatorRoleRequirements, completion_event);
  LAYOUT(PrefillOperatorBinding); OFFSET(PrefillOperatorBinding, role); OFFSET(PrefillOperatorBinding, maximum_logical_panel_m);
  OFFSET(PrefillOperatorBinding, numerical_mode); OFFSET(PrefillOperatorBinding, provider);
  OFFSET(PrefillOperatorBinding, tactic); OFFSET(PrefillOperatorBinding, weight); OFFSET(PrefillOperatorBinding, sidecar);
  OFFSET(PrefillOperatorBinding, workspace); OFFSET(PrefillOperatorBinding, launcher);
  OFFSET(PrefillOperatorBinding, completion_event); OFFSET(PrefillOperatorBinding, attestation);
  OFFSET(PrefillOperatorBinding, uses_mtp);
  LAYOUT(PrefillOperatorBindingSet); OFFSET(PrefillOperatorBindingSet, bindings); OFFSET(PrefillOperatorBindingSet, binding_count);
  LAYOUT(PrefillOperatorBindingValidation); OFFSET(PrefillOperatorBindingValidation, issue_mask);
  OFFSET(PrefillOperatorBindingValidation, role_counts); OFFSET(PrefillOperatorBindingValidation, role_coverage_complete);
  OFFSET(PrefillOperatorBindingValidation, logical_capacity_complete);
  OFFSET(PrefillOperatorBindingValidation, exact_numerics_complete);
  OFFSET(PrefillOperatorBindingValidation, native_provider_complete); OFFSET(PrefillOperatorBindingValidation, aot_tactics_complete);
  OFFSET(PrefillOperatorBindingValidation, artifact_bindings_complete);
  OFFSET(PrefillOperatorBindingValidation, workspace_bindings_complete);
  OFFSET(PrefillOperatorBindingValidation, launcher_bindings_complete);
  OFFSET(PrefillOperatorBindingValidation, completion_events_complete);
  OFFSET(PrefillOperatorBindingValidation, forbidden_boundaries_satisfied);
  OFFSET(PrefillOperatorBindingValidation, attestation_complete);
  OFFSET(PrefillOperatorBindingValidation, operator_bindings_complete);
  return 0;
}
