// Compiled against the REFERENCE project's own headers (only where a reference checkout exists) and
// linked against libq3x_b200_host.so: taking the address of every launcher through the reference's
// declarations proves that the mirror defines exactly those symbols (same mangled names, i.e. same
// namespaces, names and parameter types).
#include <cstdio>

#include "q3x/runtime/decode_ops.h"
#include "q3x/runtime/gdn_decode.h"
#include "q3x/runtime/layout_ops.h"

namespace rt = q3x::runtime;

int main() {
  const void* symbols[] = {
      reinterpret_cast<const void*>(&rt::launch_embedding_gather_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_embedding_gather_prompt_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_centered_rms_norm_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_plain_rms_norm_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_headwise_centered_rms_norm_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_headwise_plain_rms_norm_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_headwise_plain_rms_norm_silu_gate_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_residual_add_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_residual_add_centered_rms_norm_5120_cuda),
      reinterpret_cast<const void*>(&rt::launch_residual_add_headwise_centered_rms_norm_m32_5120_cuda),
      reinterpret_cast<const void*>(&rt::launch_residual_add_headwise_centered_rms_norm_prefill_5120_cuda),
      reinterpret_cast<const void*>(&rt::launch_fp32_to_bf16_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_silu_mul_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_sigmoid_gate_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_l2_normalize_heads_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_partial_neox_rope_256_64_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_qk_partial_neox_rope_tile_24_4_256_64_cuda),
      reinterpret_cast<const void*>(&rt::launch_full_attention_preprocess_24_4_256_64_reference_256_cuda),
      reinterpret_cast<const void*>(&rt::launch_full_attention_preprocess_24_4_256_64_prompt_wide_p8000_cuda),
      reinterpret_cast<const void*>(&rt::launch_full_attention_preprocess_24_4_256_64_cuda),
      reinterpret_cast<const void*>(&rt::launch_split_interleaved_q_gate_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_causal_conv1d_silu_update_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_causal_conv1d_silu_update_tile_reference_cuda),
  };
  int missing = 0;
  for (const void* s : symbols) missing += s == nullptr ? 1 : 0;
  std::printf("%zu reference launcher symbols resolved\n", sizeof(symbols) / sizeof(symbols[0]));
  return missing;
}
