/*
 * q3x_b200.h -- C ABI of libq3x_b200.so: the B200 (sm_100a) implementation of the fused
 * per-layer elementwise / normalisation operators of the Qwen3.6-27B hybrid model
 * (gated-delta-net + full-attention layers).
 *
 * Each entry point is what a binding of the reference project's operator API for this path
 * would call; the comment above it names the reference declaration it stands in for (path
 * inside the reference project : line).
 *
 * Conventions (those of the reference launchers, include/q3x/runtime/decode_ops.h:172-176):
 *   - every tensor pointer is device-accessible memory; bf16 tensors are raw bfloat16 bits in
 *     uint16_t, row-major; arithmetic is FP32, outputs are rounded to nearest-even;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *   - the return value is a cudaError_t as int; 0 = the work was enqueued;
 *   - a call allocates nothing, copies nothing to the host and never synchronises;
 *   - invalid host-visible arguments return cudaErrorInvalidValue (1) BEFORE anything is
 *     enqueued; a valid shape this build has no kernel for returns cudaErrorNotSupported (801);
 *   - an empty shape is a successful no-op, even with NULL pointers;
 *   - a stale CUDA last-error of the calling thread is cleared before the first launch, and the
 *     value returned is the status of this call's own launches.
 * Aliasing: an output may be EXACTLY an input where stated; every partial overlap is rejected.
 * Any alignment is accepted; 16-byte aligned pointers with widths that are multiples of 8
 * elements take the 128-bit fast paths, everything else a scalar path with identical results.
 * Exceptions, which have 128-bit kernels only and return cudaErrorNotSupported for a pointer that is
 * not 16-byte aligned: the causal conv, the full-attention pre-processing, and the operators fused
 * with NVFP4 quantisation.
 */
#ifndef Q3X_B200_H_
#define Q3X_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define Q3X_B200_ABI_VERSION 1

/* Model constants of the path (include/q3x/runtime/decode_ops.h:8-9,39;
 * include/q3x/runtime/gdn_decode.h:8-22). */
#define Q3X_B200_HIDDEN 5120
#define Q3X_B200_Q_HEADS 24
#define Q3X_B200_KV_HEADS 4
#define Q3X_B200_ATTN_HEAD_DIM 256
#define Q3X_B200_ROTARY_DIM 64
#define Q3X_B200_GDN_QK_HEADS 16
#define Q3X_B200_GDN_V_HEADS 48
#define Q3X_B200_GDN_HEAD_DIM 128
#define Q3X_B200_GDN_CHANNELS 10240
#define Q3X_B200_NVFP4_BLOCK 16

int q3x_b200_abi_version(void);
/* cudaGetErrorString of a value returned by any entry point (diagnostics only). */
const char* q3x_b200_error_string(int status);

/* ---------------------------------------------------------------- embedding */

/* launch_embedding_gather_prompt_reference_cuda (include/q3x/runtime/decode_ops.h:192-196);
 * with token_count == 1 also launch_embedding_gather_reference_cuda (:178-181) once the id is
 * on the device.  out[t,:] = table[ids[t],:], a bitwise copy.  An id >= vocab leaves its
 * output row untouched.  table, ids and out must be pairwise disjoint. */
int q3x_b200_embedding_gather(const uint16_t* table, size_t vocab, size_t hidden,
                              const uint32_t* token_ids, size_t token_count, uint16_t* out,
                              void* stream);

/* launch_embedding_gather_reference_cuda (decode_ops.h:178-181): the single-token decode form with
 * the id passed by value; an id >= vocab is rejected on the host (cudaErrorInvalidValue). */
int q3x_b200_embedding_gather_one(const uint16_t* table, size_t vocab, size_t hidden,
                                  size_t token_id, uint16_t* out, void* stream);

/* ---------------------------------------------------------------- RMS norms */

/* launch_centered_rms_norm_reference_cuda / launch_plain_rms_norm_reference_cuda (rows = 1)
 * and launch_headwise_centered_/plain_rms_norm_reference_cuda (decode_ops.h:198-216):
 * y = bf16(x * 1/sqrt(mean(x^2)+eps) * (w [+1 if centered])) for each of `rows` rows of
 * `width` elements sharing one weight vector.  out may be exactly in. */
int q3x_b200_rms_norm(const uint16_t* in, const uint16_t* weight, size_t rows, size_t width,
                      float eps, int centered, uint16_t* out, void* stream);

/* launch_headwise_plain_rms_norm_silu_gate_reference_cuda (decode_ops.h:218-222): plain norm
 * times silu(gate) in FP32, one rounding.  out may be exactly in or exactly gate. */
int q3x_b200_rms_norm_silu_gate(const uint16_t* in, const uint16_t* weight, const uint16_t* gate,
                                size_t rows, size_t width, float eps, uint16_t* out,
                                void* stream);

/* launch_l2_normalize_heads_reference_cuda (decode_ops.h:300-303): y = bf16(x * s) with
 * s = scale / sqrt(sum(x^2)+eps) (scale folded into the factor first).  scale = 1 is the
 * reference op; 1/sqrt(128) is the q form of the prefill compact layout
 * (src/kernels/reference/gdn_prefill_whole_span_conv_sm87.cu:344-371). */
int q3x_b200_l2_normalize_heads(const uint16_t* in, size_t heads, size_t dim, float eps,
                                float scale, uint16_t* out, void* stream);

/* ---------------------------------------------------------------- residual stream */

/* launch_residual_add_reference_cuda (decode_ops.h:228-231): out = bf16(left+right).
 * left/right disjoint; out may be exactly left or exactly right. */
int q3x_b200_residual_add(const uint16_t* left, const uint16_t* right, size_t count,
                          uint16_t* out, void* stream);

/* launch_residual_add_centered_rms_norm_5120_cuda (decode_ops.h:238-243, tokens = 1),
 * launch_residual_add_headwise_centered_rms_norm_m32_5120_cuda (:252-259) and
 * ..._prefill_5120_cuda (:265-272), for any token count and any hidden size:
 * residual = bf16(left+right); normalized = centred RMSNorm of the ROUNDED residual, bit-equal
 * to the two-op chain.  residual_out must be disjoint from everything; normalized_out may be
 * exactly `right`, NULL skips it. */
int q3x_b200_residual_add_rms_norm(const uint16_t* left, const uint16_t* right,
                                   const uint16_t* weight, size_t tokens, size_t hidden,
                                   float eps, uint16_t* residual_out, uint16_t* normalized_out,
                                   void* stream);

/* ---------------------------------------------------------------- NVFP4 activations
 * No counterpart in the reference, which only decodes NVFP4 weights
 * (include/q3x/quantization/nvfp4.h:28-34 gives the scale convention this follows:
 * real = E2M1(code) * E4M3(block scale) * global scale, global = amax / 2688; 16-element blocks;
 * even column in the low nibble).  Rows are grouped `rows_per_scale` at a time (0 = one group);
 * group g owns global_scales[g].  codes [rows, cols/2], scales [rows, cols/16] row-major. */

/* Number of scale groups of a [rows, *] tensor. */
size_t q3x_b200_nvfp4_group_count(size_t rows, size_t rows_per_scale);
/* Size, in uint32 words, of the `scratch` argument of the entry points below (group amax words and
 * group arrival counters, plus an error word at the end).  The caller owns the memory and ZEROES IT
 * ONCE, when it is allocated (cudaMemsetAsync); every call leaves the words it used zero again, so one
 * buffer serves any sequence of calls, of any shapes, with no clearing in between (the single-kernel
 * forms put no memset node in front of their kernel).  Calls that share one scratch buffer must not
 * overlap on the GPU (same stream, or ordered by events).
 * The LAST word is a sticky error flag: the library only ever sets bits in it, and only when a bounded
 * wait inside a single-kernel form gave up (the outputs of that call are then not valid and the scratch
 * must be zeroed again).  Clear it once, run any number of calls, read it once. */
size_t q3x_b200_nvfp4_scratch_words(size_t rows, size_t rows_per_scale);

/* amax_bits[g] = largest finite |x| of group g as bf16 magnitude bits (uint32), group_count words.
 * The call zeroes amax_bits itself. */
int q3x_b200_group_amax(const uint16_t* in, size_t rows, size_t cols, size_t rows_per_scale,
                        uint32_t* amax_bits, void* stream);
/* global_scales[g] = amax == 0 ? 1 : amax / 2688. */
int q3x_b200_amax_to_global_scale(const uint32_t* amax_bits, size_t groups, float* global_scales,
                                  void* stream);
/* Quantise with the given global scales. */
int q3x_b200_nvfp4_quantize(const uint16_t* in, size_t rows, size_t cols, size_t rows_per_scale,
                            const float* global_scales, uint8_t* codes, uint8_t* scales,
                            void* stream);
/* The three steps above in one call. */
int q3x_b200_nvfp4_quantize_dynamic(const uint16_t* in, size_t rows, size_t cols,
                                    size_t rows_per_scale, uint32_t* scratch,
                                    float* global_scales_out, uint8_t* codes, uint8_t* scales,
                                    void* stream);

/* The block scales of a [rows, cols] tensor re-laid out for block-scaled tensor-core MMA (tcgen05.mma with
 * 16-element E4M3 scale vectors): 512-byte tiles of 128 rows x 4 blocks, the byte of (row r, block b) at
 * tile (r / 128, b / 4), offset (r % 32) * 16 + (r % 128 / 32) * 4 + b % 4, tiles row-tile major, ragged edges
 * padded with zero bytes.  Every quantiser entry point writes the canonical row-major view
 * (include/q3x/quantization/nvfp4.h:50-55); this call converts it (a bit-exact permutation).
 * q3x_b200_nvfp4_swizzled_scale_bytes gives the size of `swizzled`.  No counterpart in the reference. */
size_t q3x_b200_nvfp4_swizzled_scale_bytes(size_t rows, size_t cols);
int q3x_b200_nvfp4_swizzle_block_scales(const uint8_t* row_major, size_t rows, size_t cols, uint8_t* swizzled,
                                        void* stream);

/* The projection that consumes the NVFP4 activations: out[tokens, out_features] (bf16, row-major) =
 * A x W^T with A = [tokens, in_features] and W = [out_features, in_features] both NVFP4 -- packed E2M1
 * codes (in_features / 2 bytes per row, even column in the low nibble), block scales in the swizzled layout
 * above, FP32 second-level scales: one per activation scale group of rows_per_scale rows (0 = one group), as
 * the quantiser entry points write them, and one for the weights.  Runs on the block-scaled tensor cores (FP32 accumulation, one rounding to bf16).
 * in_features must be a multiple of 64, out_features of 8; pointers 16-byte aligned.  `workspace` holds
 * q3x_b200_nvfp4_gemm_workspace_bytes(...) bytes (never 0 for a non-empty problem); nothing is allocated.
 * The reference's prefill projection multiplies bf16 activations with NVFP4 weights
 * (launch_projection_to_bf16_cuda, include/q3x/runtime/model_weights.h:794-841, kernel
 * src/kernels/sm87/nvfp4_marlin_w4a16.cu); this is that projection with the activation operand taken from
 * this library's quantiser, so it has the reference's shape contract but not its numerics. */
/* The bf16 projection of a panel of tokens: out[tokens, out_features] = activations[tokens, in_features] x W^T with
 * W = [out_features, in_features] bf16 -- q3x_b200_bf16_gemv for many tokens (bf16_gemv_reference_cpu,
 * src/kernels/reference/gemv_reference.cpp:84-111, per token; launch_projection_tile_to_bf16_cuda for
 * Bf16LinearWeight, include/q3x/runtime/model_weights.h:800-826).  Tensor cores, FP32 accumulation, one rounding.
 * in_features and out_features must be multiples of 8; pointers 16-byte aligned; workspace as for
 * q3x_b200_fp8_gemm_bf16. */
size_t q3x_b200_bf16_gemm_workspace_bytes(size_t tokens, size_t out_features, size_t in_features);
int q3x_b200_bf16_gemm_bf16(const uint16_t* weights, const uint16_t* activations, size_t tokens, size_t out_features,
                            size_t in_features, uint16_t* out, void* workspace, size_t workspace_bytes, void* stream);
/* The same projection with a per-tensor scale in the epilogue, out = bf16(scale * sum), and the exact widening of
 * FP8 (E4M3) weights to bf16 that feeds it: a runner that keeps a bf16 copy of its FP8 projection weights (made once
 * at load; `elements` a multiple of 16) gets the products and the FP32 accumulation of q3x_b200_fp8_gemm_bf16 --
 * fp8_gemv_reference_cpu per token (src/kernels/reference/gemv_reference.cpp:113-141) -- on the dense tensor-core
 * path, without a conversion stage inside the GEMM.  Outputs 512 or more columns wide use 128 x 256 tiles. */
int q3x_b200_bf16_gemm_scaled_bf16(const uint16_t* weights, float weight_scale, const uint16_t* activations,
                                   size_t tokens, size_t out_features, size_t in_features, uint16_t* out,
                                   void* workspace, size_t workspace_bytes, void* stream);
int q3x_b200_fp8_weights_to_bf16(const uint8_t* weights, size_t elements, uint16_t* out, void* stream);
/* The same for an NVFP4 weight: packed E2M1 codes [rows, cols / 2] times their row-major E4M3 block scales
 * [rows, cols / 16] -> bf16 [rows, cols], exactly (a code has two significant bits, a scale four); the second-level
 * FP32 scale then rides as `weight_scale` of q3x_b200_bf16_gemm_scaled_bf16, which gives the products and the FP32
 * accumulation of q3x_b200_nvfp4_w4a16_gemm_bf16 (nvfp4_gemv_reference_cpu per token,
 * src/kernels/reference/gemv_reference.cpp:179-225).  cols must be a multiple of 16. */
int q3x_b200_nvfp4_weights_to_bf16(const uint8_t* packed_weights, const uint8_t* block_scales, size_t rows,
                                   size_t cols, uint16_t* out, void* stream);


/* The weight-only FP8 projection of a panel of tokens: out[tokens, out_features] (bf16, row-major) =
 * activations[tokens, in_features] (bf16) x W^T with W = [out_features, in_features] E4M3 bytes and one FP32
 * scale for the tensor -- q3x_b200_fp8_gemv for many tokens (fp8_gemv_reference_cpu,
 * src/kernels/reference/gemv_reference.cpp:113-140, per token), which is what
 * launch_projection_tile_to_bf16_cuda and launch_exact_fp8_whole_chunk_projection_to_bf16_cuda
 * (include/q3x/runtime/model_weights.h:800-870) compute for Fp8LinearWeight.  Tensor cores (the weights are
 * widened to bf16, exactly, inside the kernel), FP32 accumulation, the scale applied to the sum, one rounding.
 * in_features must be a multiple of 16, out_features of 8; pointers 16-byte aligned; `workspace` holds
 * q3x_b200_fp8_gemm_workspace_bytes(...) bytes and may be NULL when that is 0.  Nothing is allocated. */
size_t q3x_b200_fp8_gemm_workspace_bytes(size_t tokens, size_t out_features, size_t in_features);
int q3x_b200_fp8_gemm_bf16(const uint8_t* weights, float weight_scale, const uint16_t* activations, size_t tokens,
                           size_t out_features, size_t in_features, uint16_t* out, void* workspace,
                           size_t workspace_bytes, void* stream);

/* The weight-only NVFP4 projection of a panel of tokens: q3x_b200_nvfp4_gemv for many tokens
 * (nvfp4_gemv_reference_cpu, src/kernels/reference/gemv_reference.cpp:179-225, per token) -- bf16 activations
 * [tokens, in_features], packed E2M1 weights [out_features, in_features / 2] as the checkpoint holds them, block
 * scales TRANSPOSED to [in_features / 16, out_features] and widened to bf16 (exact;
 * q3x_b200_nvfp4_transpose_block_scales re-lays a weight's row-major E4M3 scales out, once, when the weight is
 * loaded), FP32 second-level scale; what
 * launch_projection_tile_to_bf16_cuda and
 * launch_exact_nvfp4_whole_chunk_branch_to_bf16_cuda (include/q3x/runtime/model_weights.h:800-866) compute for
 * NvFp4LinearWeight.  Tensor cores (codes x block scales become bf16 operands, exactly, inside the kernel), FP32
 * accumulation, the second-level scale applied to the sum, one rounding.  in_features must be a multiple of 32,
 * out_features of 8; pointers 16-byte aligned; workspace as for q3x_b200_fp8_gemm_bf16. */
int q3x_b200_nvfp4_transpose_block_scales(const uint8_t* row_major, size_t rows, size_t cols, uint16_t* transposed,
                                          void* stream);
size_t q3x_b200_nvfp4_w4a16_gemm_workspace_bytes(size_t tokens, size_t out_features, size_t in_features);
int q3x_b200_nvfp4_w4a16_gemm_bf16(const uint8_t* packed_weights, const uint16_t* block_scales_transposed,
                                   float weight_scale_2,
                                   const uint16_t* activations, size_t tokens, size_t out_features,
                                   size_t in_features, uint16_t* out, void* workspace, size_t workspace_bytes,
                                   void* stream);

size_t q3x_b200_nvfp4_gemm_workspace_bytes(size_t tokens, size_t out_features, size_t in_features,
                                           size_t rows_per_scale);
int q3x_b200_nvfp4_gemm_bf16(const uint8_t* activation_codes, const uint8_t* activation_scales_swizzled,
                             const float* activation_global_scales, size_t rows_per_scale,
                             const uint8_t* weight_codes, const uint8_t* weight_scales_swizzled,
                             float weight_scale_2, size_t tokens, size_t out_features, size_t in_features,
                             uint16_t* out, void* workspace, size_t workspace_bytes, void* stream);

/* Residual add + centred RMSNorm + NVFP4 of the normalised rows, global scale from the group
 * amax.  normalized_out is required (it is the operand the codes are derived from, bit for
 * bit); it may be exactly `right`.  One kernel that crosses HBM once where a scale group is short
 * enough to wait in L2 (see the _single_pass form), else two kernels: the norm, which also reduces
 * each group's amax, then the quantiser, which derives the scales from it.  Same bytes either way.
 * codes, scales, global_scales_out and scratch must not overlap each other nor any other operand. */
int q3x_b200_residual_add_rms_norm_nvfp4(const uint16_t* left, const uint16_t* right,
                                         const uint16_t* weight, size_t tokens, size_t hidden,
                                         float eps, size_t rows_per_scale, uint16_t* residual_out,
                                         uint16_t* normalized_out, uint32_t* scratch,
                                         float* global_scales_out, uint8_t* codes, uint8_t* scales,
                                         void* stream);
/* The same result, insisting on ONE pass over HBM: a single kernel whose CTAs alternate between
 * normalising a row and quantising the row written `lag` rows earlier, which still sits in L2 and
 * whose scale group is complete by then.  Returns cudaErrorNotSupported, with nothing enqueued,
 * when a scale group is too long to stay in L2 (group rows x row bytes beyond a few tens of MB,
 * e.g. rows_per_scale == 0 on a long tensor). */
int q3x_b200_residual_add_rms_norm_nvfp4_single_pass(const uint16_t* left, const uint16_t* right,
                                                     const uint16_t* weight, size_t tokens,
                                                     size_t hidden, float eps, size_t rows_per_scale,
                                                     uint16_t* residual_out, uint16_t* normalized_out,
                                                     uint32_t* scratch, float* global_scales_out,
                                                     uint8_t* codes, uint8_t* scales, void* stream);

/* Gated RMSNorm * silu(z) + NVFP4 of its output rows.  `heads_per_row` heads of `dim` form one
 * quantisation row (48 x 128 = 6144 for the GDN output).  One kernel or two, as above. */
int q3x_b200_rms_norm_silu_gate_nvfp4(const uint16_t* in, const uint16_t* weight,
                                      const uint16_t* gate, size_t tokens, size_t heads_per_row,
                                      size_t dim, float eps, size_t rows_per_scale, uint16_t* out,
                                      uint32_t* scratch, float* global_scales_out,
                                      uint8_t* codes, uint8_t* scales, void* stream);
/* Single-pass form (dim must be 128). */
int q3x_b200_rms_norm_silu_gate_nvfp4_single_pass(const uint16_t* in, const uint16_t* weight,
                                                  const uint16_t* gate, size_t tokens,
                                                  size_t heads_per_row, size_t dim, float eps,
                                                  size_t rows_per_scale, uint16_t* out,
                                                  uint32_t* scratch, float* global_scales_out,
                                                  uint8_t* codes, uint8_t* scales, void* stream);

/* SwiGLU (launch_silu_mul_reference_cuda, decode_ops.h:290-293) + NVFP4 of its output, the operand
 * of the MLP down projection: out = bf16(silu(gate) * up) over [tokens, intermediate], then codes
 * [tokens, intermediate / 2], block scales [tokens, intermediate / 16] and one global scale per
 * rows_per_scale rows, derived from `out` bit for bit.  out may be exactly gate or exactly up.
 * One kernel where a scale group is a whole number of 4096-element chunks and short enough to wait
 * in L2 (17408 x 512 is), else three (SwiGLU, group amax, quantiser).  Scratch and error word as
 * above.  The quantisation half has no counterpart in the reference. */
int q3x_b200_silu_mul_nvfp4(const uint16_t* gate, const uint16_t* up, size_t tokens,
                            size_t intermediate, size_t rows_per_scale, uint16_t* out,
                            uint32_t* scratch, float* global_scales_out, uint8_t* codes,
                            uint8_t* scales, void* stream);

/* The attention sigmoid output gate (launch_sigmoid_gate_reference_cuda, decode_ops.h:295-298) +
 * NVFP4 of its output, the operand of the attention output projection: out = bf16(value *
 * sigmoid(gate)) over [tokens, width], codes, block scales and global scales as above.  out may be
 * exactly value or exactly gate.  One kernel or three, as for q3x_b200_silu_mul_nvfp4. */
int q3x_b200_sigmoid_gate_nvfp4(const uint16_t* value, const uint16_t* gate, size_t tokens,
                                size_t width, size_t rows_per_scale, uint16_t* out,
                                uint32_t* scratch, float* global_scales_out, uint8_t* codes,
                                uint8_t* scales, void* stream);

/* No counterpart in the reference.  q3x_b200_residual_add_rms_norm_nvfp4 for callers that cannot
 * hand over scratch memory because they cannot allocate any: code that runs inside a stream
 * callback, a plugin whose host gives it the input and output tensors and nothing more, a service
 * whose device allocator is closed once it is serving.  The scratch words are a fixed array inside the library (64 KB of device memory on
 * every GPU that loads the library, held until the process exits), so there is no `scratch`
 * argument; inputs and outputs are still the caller's.
 *   - tokens must not exceed Q3X_B200_STATIC_SCRATCH_MAX_TOKENS (and the scale groups must fit the
 *     same array, which they do for rows_per_scale = 0 or >= 2): larger calls return
 *     cudaErrorInvalidValue before anything is enqueued.  q3x_b200_static_scratch_max_tokens()
 *     returns the limit of the library actually loaded.
 *   - The call allocates nothing and frees nothing.  The FIRST call on a device looks up the
 *     array's device address (once per device, with that device current).
 *   - All calls share the one array and it keeps the previous call's contents; each call clears
 *     the words it uses, on `stream`, before its kernels.  Two calls that overlap on the GPU
 *     (different streams, or graphs replayed concurrently) race on it: keep them ordered.
 * Outputs are bit-identical to q3x_b200_residual_add_rms_norm_nvfp4 on the same inputs. */
#define Q3X_B200_STATIC_SCRATCH_MAX_TOKENS 16384
size_t q3x_b200_static_scratch_max_tokens(void);
int q3x_b200_residual_add_rms_norm_nvfp4_static_scratch(
    const uint16_t* left, const uint16_t* right, const uint16_t* weight, size_t tokens, size_t hidden,
    float eps, size_t rows_per_scale, uint16_t* residual_out, uint16_t* normalized_out,
    float* global_scales_out, uint8_t* codes, uint8_t* scales, void* stream);

/* Diagnostics (no counterpart in the reference): the two narrow conversions the quantiser uses,
 * one value per output byte.  format 0 = E4M3 round-to-nearest-even with saturation at 448,
 * format 1 = E2M1 (code in the low nibble). */
int q3x_b200_debug_encode(const float* in, size_t count, int format, uint8_t* out, void* stream);
/* Diagnostics (no counterpart in the reference): the FP32 building blocks of the operators, out[i] =
 * f(in[i]), so that their error against the host reference's libm expressions can be measured.
 * function 0 = inverse RMS 1/sqrt(in/p0 + p1) (p0 = row width, p1 = epsilon), 1 = inverse L2 norm
 * 1/sqrt(in + p1), 2 = silu, 3 = silu in the form the SwiGLU stream uses, 4 = branch-stable sigmoid,
 * 5 = exp(-|in|). */
int q3x_b200_debug_intermediate(const float* in, size_t count, int function, float p0, float p1,
                                float* out, void* stream);
/* Diagnostics: returns the CUDA last-error pending in this library's runtime without clearing it;
 * with plant != 0 first leaves a stale host-side argument error there (nothing reaches the GPU),
 * which the next entry point must clear before its own launch
 * (the stale-error rule the reference tests with launch_after_stale,
 * tests/decode_ops_cuda_test.cu:374-387). */
int q3x_b200_debug_stale_error(int plant);

/* ---------------------------------------------------------------- full attention */

/* launch_split_interleaved_q_gate_reference_cuda (include/q3x/runtime/layout_ops.h:35-38) */
int q3x_b200_split_interleaved_q_gate(const uint16_t* in, size_t heads, size_t dim,
                                      uint16_t* q_out, uint16_t* gate_out, void* stream);

/* launch_partial_neox_rope_256_64_reference_cuda (decode_ops.h:305-308): one position,
 * cos/sin [32] FP32; out may be exactly in. */
int q3x_b200_partial_neox_rope_256_64(const uint16_t* in, const float* cosines,
                                      const float* sines, size_t heads, uint16_t* out,
                                      void* stream);

/* launch_qk_partial_neox_rope_tile_24_4_256_64_cuda (decode_ops.h:314-317): in-place rotation of
 * query [tokens,24,256] and key [tokens,4,256] with [position,32] tables; any tokens >= 1. */
int q3x_b200_qk_partial_neox_rope(uint16_t* query, uint16_t* key, const float* cosines,
                                  const float* sines, size_t first_position, size_t tokens,
                                  void* stream);

/* launch_full_attention_preprocess_24_4_256_64_cuda and its _reference_256 / _prompt_wide_p8000
 * forms (decode_ops.h:333-377): split q|gate, centred head norm of q and (in place) k, partial
 * RoPE of both at positions first_position + t.  Any tokens >= 1 (the reference admits <= 512
 * or exactly 8000).  Writable tensors must not overlap each other or any input. */
int q3x_b200_full_attention_preprocess(const uint16_t* interleaved_q_gate, uint16_t* key,
                                       const uint16_t* q_weight, const uint16_t* k_weight,
                                       float eps, uint16_t* q_out, uint16_t* gate_out,
                                       const float* cosines, const float* sines,
                                       size_t first_position, size_t tokens, void* stream);

/* launch_sigmoid_gate_reference_cuda (decode_ops.h:295-298): out = bf16(value * sigmoid(gate));
 * out may be exactly value or exactly gate. */
int q3x_b200_sigmoid_gate(const uint16_t* value, const uint16_t* gate, size_t count,
                          uint16_t* out, void* stream);

/* ---------------------------------------------------------------- MLP */

/* launch_silu_mul_reference_cuda (decode_ops.h:290-293): out = bf16(silu(gate) * up);
 * out may be exactly gate or exactly up. */
int q3x_b200_silu_mul(const uint16_t* gate, const uint16_t* up, size_t count, uint16_t* out,
                      void* stream);
/* The merged-projection layout of src/kernels/sm87/nvfp4_marlin_w4a16.cu:211-227:
 * merged [tokens, 2*intermediate], gate first; out [tokens, intermediate], disjoint. */
int q3x_b200_silu_mul_merged(const uint16_t* merged, size_t tokens, size_t intermediate,
                             uint16_t* out, void* stream);

/* launch_fp32_to_bf16_reference_cuda (decode_ops.h:274-276) */
int q3x_b200_fp32_to_bf16(const float* in, size_t count, uint16_t* out, void* stream);

/* ---------------------------------------------------------------- gated delta net */

/* launch_causal_conv1d_silu_update_reference_cuda (tokens = 1), ..._tile_reference_cuda
 * (include/q3x/runtime/gdn_decode.h:75-93) and the prefill whole-span / token-parallel launchers
 * (src/kernels/reference/gdn_prefill_whole_span_conv_sm87.h), for any token count:
 * out[t,c] = bf16(silu(fma chain over raw[t-3..t,c] and w[c,0..3])), history [channels,3]
 * (oldest first) supplies rows before t = 0 and receives the last three RAW rows.
 * channels must be 10240 (else cudaErrorInvalidValue: it is the reference's only geometry) and every
 * pointer 16-byte aligned (else cudaErrorNotSupported).
 * raw may be exactly out (serial path: one token run per channel block). */
int q3x_b200_causal_conv1d_silu(const uint16_t* raw, size_t tokens, size_t channels,
                                const uint16_t* conv_weight, uint16_t* history_in_out,
                                uint16_t* out, void* stream);

/* The conv above with the q/k L2 norm applied to its rounded output in the same pass
 * (channels [0,2048) = q heads, [2048,4096) = k heads of 128; q additionally times q_scale):
 * the prefill fusion of gdn_prefill_whole_span_conv_sm87.cu:210-373, written token-major in
 * place of the compact chunk layout.  raw and out must be disjoint. */
int q3x_b200_causal_conv1d_silu_l2norm(const uint16_t* raw, size_t tokens,
                                       const uint16_t* conv_weight, uint16_t* history_in_out,
                                       float l2_eps, float q_scale, uint16_t* out, void* stream);

/* launch_causal_conv1d_silu_update_token_parallel_compact_qk_exact_cuda
 * (src/kernels/reference/gdn_prefill_whole_span_conv_sm87.h:59-67), for any token count: the conv as above,
 * `out` receiving the plain conv output of EVERY channel, plus the L2-normalised q and k heads (q additionally
 * times q_scale; the reference uses 1/sqrt(128)) in the operand layout of the chunked GDN prefill:
 * compact_q / compact_k [ceil(tokens / 64), 16 heads, 64, 128] bf16, the rows of the last chunk beyond `tokens`
 * zeroed.  raw and out must be disjoint; the compact tensors must be disjoint from every other operand. */
int q3x_b200_causal_conv1d_silu_compact_qk(const uint16_t* raw, size_t tokens, const uint16_t* conv_weight,
                                           uint16_t* history_in_out, uint16_t* out, float l2_eps, float q_scale,
                                           uint16_t* compact_q, uint16_t* compact_k, void* stream);

/* ---------------------------------------------------------------- between the fused operators
 * The stateful / contracting steps that sit between the operators above in a layer, in their batch-one
 * (decode) and short-tile forms, which are HBM-bound streams like the rest of this library. */

/* launch_gated_delta_net_update_reference_cuda (tokens = 1) and ..._tile_reference_cuda / the
 * warp-parallel forms (include/q3x/runtime/gdn_decode.h:85-140), for any token count: the gated-delta-net
 * recurrence, token by token.  conv_qkv [tokens, 10240] (the conv output: q 2048 | k 2048 | v 6144), a and b
 * [tokens, 48], A_log and dt_bias [48], state [48, 128(v), 128(k)] bf16, out [tokens, 48 * 128].  The q / k L2
 * norm (q additionally times 1/sqrt(128)), the gates and the sums are FP32; the state is rounded to bf16 after
 * every token, the output uses the state before that rounding.  state_out may be exactly state_in; every other
 * overlap of a written range is rejected.  Pointers must be 16-byte aligned (else cudaErrorNotSupported). */
int q3x_b200_gated_delta_net_update(const uint16_t* conv_qkv, size_t tokens, const uint16_t* a,
                                    const uint16_t* b, const uint16_t* A_log, const uint16_t* dt_bias,
                                    const uint16_t* state_in, uint16_t* state_out, float l2_eps,
                                    uint16_t* out, void* stream);
/* launch_gated_delta_net_update_plain_rms_norm_silu_gate_cuda (gdn_decode.h:171-188): the recurrence with the
 * GDN output's gated RMSNorm as its epilogue -- the raw output is rounded to bf16, then
 * out = bf16(rmsnorm_128(raw) * norm_weight * silu(silu_gate)); norm_weight [128], silu_gate [tokens, 6144]. */
int q3x_b200_gated_delta_net_update_rms_norm_silu_gate(
    const uint16_t* conv_qkv, size_t tokens, const uint16_t* a, const uint16_t* b, const uint16_t* A_log,
    const uint16_t* dt_bias, const uint16_t* state_in, uint16_t* state_out, float l2_eps,
    const uint16_t* norm_weight, const uint16_t* silu_gate, float norm_eps, uint16_t* out, void* stream);

/* gdn_prefill_chunk64_native_detail::launch without its norm epilogue
 * (src/kernels/sm87/gdn_prefill_chunk64_native_sm87.h:98-109), for any token count: the same recurrence over a
 * prefill span in chunks of 64 tokens (the WY form).  Everything that does not depend on the running state -- q / k
 * normalisation, the chunk's Gram matrices, the triangular solves -- runs for all chunks at once; three small
 * tensor-core products per chunk remain sequential.  Operands and result as q3x_b200_gated_delta_net_update.
 * Products take bf16 operands with FP32 accumulation and the state stays FP32 between the chunks of a call
 * (rounded to bf16 once, in state_out), so against the token-by-token entry, which rounds the state after every
 * token, the result agrees to the level of that rounding and is not bit-identical.  workspace: caller-owned, at
 * least q3x_b200_gated_delta_net_chunked_workspace_bytes(tokens) bytes (about 2.4 MB per 64 tokens), 16-byte
 * aligned, disjoint from every operand; stale contents do not matter. */
size_t q3x_b200_gated_delta_net_chunked_workspace_bytes(size_t tokens);
/* The sequential half of the chunked form exists twice: path 0 keeps the state in the accumulators of mma.sync
 * products (two CTAs per head; the default, the faster one today), path 1 keeps it in tensor memory and issues
 * tcgen05 products from shared-memory descriptors (one CTA per head).  Same operands, same roundings, sums in another
 * order.  Process-wide switch (initially from the environment variable Q3X_B200_GDN_CHUNK_PATH = "tcgen05");
 * cudaErrorInvalidValue for any other value.  The last 256 bytes of the workspace hold a word that path 1 raises
 * when one of its bounded waits on the tensor cores runs out (the results of that call are then invalid); every call
 * of path 1 clears it first. */
int q3x_b200_gated_delta_net_chunked_select_path(int path);
int q3x_b200_gated_delta_net_update_chunked(const uint16_t* conv_qkv, size_t tokens, const uint16_t* a,
                                            const uint16_t* b, const uint16_t* A_log, const uint16_t* dt_bias,
                                            const uint16_t* state_in, uint16_t* state_out, float l2_eps,
                                            uint16_t* out, void* workspace, size_t workspace_bytes, void* stream);

/* launch_gqa_attention_splitkv_sigmoid_gate_24_4_256_cuda and
 * gqa_attention_splitkv_sigmoid_gate_24_4_256_workspace_elements (include/q3x/runtime/decode_ops.h:397-423),
 * for any sequence_length >= 1: one query token [24, 256] against key / value caches [sequence_length, 4, 256],
 * softmax in FP32, attention rounded to bf16, times sigmoid(gate) [24, 256], rounded again.  gate == NULL gives
 * the attention output itself (launch_gqa_attention_reference_cuda without its probabilities).  workspace is
 * caller-owned FP32 scratch of at least q3x_b200_gqa_decode_workspace_floats(sequence_length) elements;
 * stale contents do not matter. */
size_t q3x_b200_gqa_decode_workspace_floats(size_t sequence_length);
int q3x_b200_gqa_attention_decode_sigmoid_gate(const uint16_t* query, const uint16_t* key_cache,
                                               const uint16_t* value_cache, size_t sequence_length,
                                               float attention_scale, float* workspace, size_t workspace_floats,
                                               const uint16_t* gate, uint16_t* out, void* stream);

/* Bulk causal GQA attention of a tile of `tokens` tokens appended at position `first_position`, with the sigmoid
 * output gate: for token t and query head h, attention over cache positions 0 .. first_position + t (the caches
 * [position, 4, 256] already hold the tile's own keys and values), rounded to bf16, times sigmoid(gate[t, h]),
 * rounded again (gate may be NULL: plain attention).  query / gate / out are tile-local [tokens, 24, 256].
 * gqa_attention_reference_cpu + sigmoid_gate_reference_cpu per token
 * (src/runtime/reference/decode_ops.cpp:302-342,445-508); replaces
 * launch_bulk_causal_gqa_sigmoid_gate_24_4_256[_fixed]_cuda and the panel form
 * (include/q3x/runtime/decode_ops.h:419-505).  Any tokens and first_position; no scratch; pointers 16-byte aligned;
 * out must not overlap an input. */
int q3x_b200_gqa_attention_prefill_sigmoid_gate(const uint16_t* query, const uint16_t* key_cache,
                                                const uint16_t* value_cache, const uint16_t* gate,
                                                size_t first_position, size_t tokens, float scale, uint16_t* out,
                                                void* stream);
/* The prefill attention exists twice: path 1 on tcgen05 (the default: 128 tokens of one head per CTA, scores and
 * output in tensor memory, the probabilities as two bf16 operands), path 0 on mma.sync.  Process-wide switch
 * (the environment variable Q3X_B200_GQA_PREFILL_PATH = "mma" starts on path 0).  Path 1 bounds every wait on the
 * tensor cores; q3x_b200_gqa_prefill_tcgen05_error synchronises and returns its sticky error word (0 = no wait ever
 * ran out, -1 = the word could not be read). */
int q3x_b200_gqa_prefill_select_path(int path);
int q3x_b200_gqa_prefill_tcgen05_error(void);

/* launch_bf16_gemv_reference_cuda / launch_bf16_gemv_bf16_cuda, launch_fp8_gemv_reference_cuda and
 * launch_nvfp4_gemv_reference_cuda (include/q3x/kernels/reference_gemv.h:64-130): batch-one projections
 * out[r] = sum_c W[r,c] * x[c], FP32 accumulation, x [cols] bf16.  The result is written as FP32 (out_f32), as
 * bf16 rounded to nearest even (out_bf16), or both; at least one must be given.  bf16 weights [rows, cols];
 * FP8 weights E4M3 [rows, cols] with a per-tensor weight_scale; NVFP4 weights in the canonical layout (packed
 * [rows, cols / 2], even column in the low nibble; E4M3 block scales [rows, cols / 16]; FP32 weight_scale_2).
 * Outputs must be disjoint from every input; read-only operands may alias.  Any shape and alignment. */
int q3x_b200_bf16_gemv(const uint16_t* weights, const uint16_t* activation, size_t rows, size_t cols,
                       float* out_f32, uint16_t* out_bf16, void* stream);
int q3x_b200_fp8_gemv(const uint8_t* weights, float weight_scale, const uint16_t* activation, size_t rows,
                      size_t cols, float* out_f32, uint16_t* out_bf16, void* stream);
int q3x_b200_nvfp4_gemv(const uint8_t* packed_weights, const uint8_t* block_scales, float weight_scale_2,
                        const uint16_t* activation, size_t rows, size_t cols, float* out_f32,
                        uint16_t* out_bf16, void* stream);

/* launch_softmax_reference_cuda (decode_ops.h:372-374), the FP32 row softmax of softmax_reference_cpu
 * (src/runtime/reference/decode_ops.cpp:413-443): out may be exactly in. */
int q3x_b200_softmax(const float* in, size_t rows, size_t cols, float* out, void* stream);

/* launch_bf16_greedy_argmax_cuda (decode_ops.h:277-280): result_workspace holds
 * Q3X_B200_ARGMAX_WORKSPACE_RESULTS records of {uint32 index, uint16 value_bits, uint16 has_nonfinite}
 * (Bf16GreedyArgmaxResult, decode_ops.h:61-69); record 0 receives the answer, the rest is scratch.  Non-finite
 * logits are skipped and flagged; equal maxima (signed zeros included) select the smallest index; no finite
 * logit at all gives index 0xffffffff. */
#define Q3X_B200_ARGMAX_WORKSPACE_RESULTS 33
int q3x_b200_bf16_greedy_argmax(const uint16_t* in, size_t count, void* result_workspace, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* Q3X_B200_H_ */
