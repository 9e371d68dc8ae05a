// Compiled against the REFERENCE project's own headers (only where a reference checkout exists) and
// linked against libq3x_b200_host.so: taking the address of every launcher through the reference's
// declarations proves that the mirror defines exactly those symbols (same mangled names, i.e. same
// namespaces, names and parameter types).  The projection composites take the reference's LinearWeight; the
// test links them from q3x_b200_dispatch.cpp compiled against the reference's model_weights.h
// (-DQ3X_B200_USE_REFERENCE_HEADERS), the way a reference build would compile that file.
#include <cstdio>

#include "gdn_prefill_whole_span_conv_sm87.h"  // src/kernels/reference (source-private header)
#include "../sm87/gdn_prefill_chunk64_native_sm87.h"  // src/kernels/sm87 (source-private header)
#include "q3x/kernels/reference_gemv.h"
#include "q3x/runtime/decode_ops.h"
#include "q3x/runtime/gdn_decode.h"
#include "q3x/runtime/layout_ops.h"
#include "q3x/runtime/model_weights.h"

namespace rt = q3x::runtime;
namespace kn = q3x::kernels;
namespace conv = q3x::runtime::gdn_prefill_whole_span_conv_detail;
namespace chunked = q3x::runtime::gdn_prefill_chunk64_native_detail;

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
      // the prefill conv forms (source-private header of the reference)
      reinterpret_cast<const void*>(static_cast<std::size_t (*)() noexcept>(&chunked::workspace_bytes)),
      reinterpret_cast<const void*>(&chunked::launch),
      reinterpret_cast<const void*>(&chunked::launch_fixed_production),
      reinterpret_cast<const void*>(&conv::launch_causal_conv1d_silu_update_whole_span_exact_cuda),
      reinterpret_cast<const void*>(&conv::launch_causal_conv1d_silu_update_token_parallel_exact_cuda),
      reinterpret_cast<const void*>(&conv::launch_causal_conv1d_silu_update_token_parallel_compact_qk_exact_cuda),
      reinterpret_cast<const void*>(&conv::launch_causal_conv1d_silu_update_prompt_wide_p40_compact_qk_exact_cuda),
      // the operators between the fused layer ops
      reinterpret_cast<const void*>(&rt::launch_gated_delta_net_update_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_gated_delta_net_update_tile_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_gated_delta_net_update_warp_parallel_cuda),
      reinterpret_cast<const void*>(&rt::launch_gated_delta_net_update_tile_warp_parallel_cuda),
      reinterpret_cast<const void*>(&rt::launch_gated_delta_net_update_plain_rms_norm_silu_gate_cuda),
      reinterpret_cast<const void*>(
          &rt::gdn_decode_detail::launch_gated_delta_net_update_plain_rms_norm_silu_gate_exact_cuda),
      reinterpret_cast<const void*>(&rt::supports_gated_delta_net_update_plain_rms_norm_silu_gate_fusion),
      reinterpret_cast<const void*>(&rt::launch_softmax_reference_cuda),
      reinterpret_cast<const void*>(&rt::gqa_attention_splitkv_sigmoid_gate_24_4_256_workspace_elements),
      reinterpret_cast<const void*>(&rt::launch_gqa_attention_splitkv_sigmoid_gate_24_4_256_cuda),
      reinterpret_cast<const void*>(&rt::launch_bf16_greedy_argmax_cuda),
      reinterpret_cast<const void*>(&rt::launch_bulk_causal_gqa_sigmoid_gate_24_4_256_cuda),
      reinterpret_cast<const void*>(&rt::launch_bulk_causal_gqa_sigmoid_gate_24_4_256_fixed_cuda),
      reinterpret_cast<const void*>(&rt::launch_bulk_causal_gqa_sigmoid_gate_24_4_256_group_q64_panel_fixed_cuda),
      reinterpret_cast<const void*>(&kn::launch_bf16_gemv_reference_cuda),
      reinterpret_cast<const void*>(&kn::launch_bf16_gemv_bf16_cuda),
      reinterpret_cast<const void*>(&kn::launch_fp8_gemv_reference_cuda),
      reinterpret_cast<const void*>(&kn::launch_nvfp4_gemv_reference_cuda),
      // the projection composites, declared by the reference's model_weights.h with its own LinearWeight
      reinterpret_cast<const void*>(&rt::launch_projection_to_bf16_cuda),
      reinterpret_cast<const void*>(&rt::launch_projection_tile_to_bf16_cuda),
      reinterpret_cast<const void*>(&rt::launch_projection_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_projection_to_bf16_reference_cuda),
      reinterpret_cast<const void*>(&rt::launch_projection_pair_tile_to_bf16_cuda),
      reinterpret_cast<const void*>(&rt::launch_linear_attention_qkv_z_ab_to_bf16_cuda),
      reinterpret_cast<const void*>(&rt::launch_full_attention_q_kv_to_bf16_cuda),
      reinterpret_cast<const void*>(&rt::supports_bf16_projection_pair),
      reinterpret_cast<const void*>(&rt::supports_fp8_projection_pair),
      reinterpret_cast<const void*>(&rt::supports_fp8_qkv_z_projection_pair),
      reinterpret_cast<const void*>(&rt::supports_linear_attention_qkv_z_ab_projection_fusion),
      reinterpret_cast<const void*>(&rt::supports_fp8_q_kv_projection_fusion),
      reinterpret_cast<const void*>(&rt::supports_nvfp4_gate_up_silu_fusion),
      reinterpret_cast<const void*>(&rt::supports_nvfp4_down_residual_norm_fusion),
      reinterpret_cast<const void*>(&rt::linear_weight_kind),
      reinterpret_cast<const void*>(&rt::linear_output_size),
      reinterpret_cast<const void*>(&rt::linear_input_size),
      reinterpret_cast<const void*>(&rt::is_valid_projection_backend),
      reinterpret_cast<const void*>(&rt::launch_exact_fp8_whole_chunk_projection_to_bf16_cuda),
      reinterpret_cast<const void*>(&rt::launch_mlp_gate_up_silu_to_bf16_cuda),
      reinterpret_cast<const void*>(&rt::launch_post_attention_residual_norm_mlp_gate_up_silu_to_bf16_cuda),
      reinterpret_cast<const void*>(
          &rt::launch_decode_runner_post_attention_residual_norm_mlp_gate_up_silu_dead_up_to_bf16_cuda),
      reinterpret_cast<const void*>(&rt::launch_mlp_down_residual_norm_to_bf16_cuda),
  };
  int missing = 0;
  for (const void* s : symbols) missing += s == nullptr ? 1 : 0;
  std::printf("%zu reference launcher symbols resolved\n", sizeof(symbols) / sizeof(symbols[0]));
  return missing;
}
