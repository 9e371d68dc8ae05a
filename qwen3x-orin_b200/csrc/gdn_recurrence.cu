// Gated-delta-net recurrence (the step between the conv / q-k L2 norm and the gated RMSNorm of a GDN
// layer), token-sequential, with the reference's numerics
// (gated_delta_net_update_reference_cpu, src/runtime/reference/gdn_decode.cpp:186-293):
//   per value head h (48), with q / k taken from qk head h / 3 of the conv output:
//     qn = q * (1 / sqrt(sum q^2 + eps)) * (1 / sqrt(128))        kn = k * (1 / sqrt(sum k^2 + eps))   (FP32)
//     g = -exp(A_log[h]) * softplus(a[h] + dt_bias[h])            alpha = exp(g)    beta = sigmoid(b[h])
//     per state row v (128):  pred  = sum_k (alpha * S[v,k]) * kn[k]
//                             delta = (value[v] - pred) * beta
//                             S'[v,k] = fma(delta, kn[k], alpha * S[v,k])     -> persisted as bf16
//                             out[v]  = bf16(sum_k S'[v,k] * qn[k])           (FP32 S', before its rounding)
// The state [48, 128(v), 128(k)] is bf16; a step reads the bf16 state the previous step persisted.
//
// Work layout: one CTA of 1024 threads per value head.  A group of 16 lanes owns one state row, a lane
// eight consecutive k (one 128-bit vector), so a CTA covers 64 rows per pass and a head takes two
// passes; both rows of a thread stay in registers across the tokens of a call, rounded to bf16 after
// every step exactly as if they had gone through memory, and are stored once at the end.  Every
// 16-lane group derives qn, kn and the gates for itself (a few shuffles and two libm calls on
// L2-resident operands), so the recurrence itself needs no shared memory and no barrier.  The only HBM
// traffic that matters is the state: 1.5 MB in, 1.5 MB out per call.
//
// With the norm epilogue (launch_gated_delta_net_update_plain_rms_norm_silu_gate_cuda,
// include/q3x/runtime/gdn_decode.h:171-188) the 128 rounded outputs of the head go through shared memory
// once: plain RMSNorm over the head, times weight, times silu(z), one more rounding.
#include "device_utils.cuh"
#include "host_checks.hpp"
#include "norm_math.cuh"
#include "q3x_b200.h"

namespace q3x {
namespace {

constexpr int kHead = Q3X_B200_GDN_HEAD_DIM;                 // 128
constexpr int kValueHeads = Q3X_B200_GDN_V_HEADS;            // 48
constexpr int kChannels = Q3X_B200_GDN_CHANNELS;             // 10240
constexpr int kKOffset = Q3X_B200_GDN_QK_HEADS * kHead;      // 2048
constexpr int kVOffset = 2 * kKOffset;                       // 4096
constexpr int kLanesPerRow = kHead / 8;                      // 16
constexpr int kThreads = 1024;
constexpr int kRowsPerPass = kThreads / kLanesPerRow;        // 64
constexpr int kPasses = kHead / kRowsPerPass;                // 2

// softplus and sigmoid in the branch forms of src/runtime/reference/gdn_decode.cpp:62-73 (libm calls:
// they run once per token and lane, far off the critical path)
__device__ __forceinline__ float softplus_ref(float v) { return v > 20.0f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float sigmoid_ref(float v) {
  if (v >= 0.0f) return __fdiv_rn(1.0f, 1.0f + expf(-v));
  const float e = expf(v);
  return __fdiv_rn(e, 1.0f + e);
}

__device__ __forceinline__ float dot8(const float (&a)[8], const float (&b)[8]) {
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s = fmaf(a[i], b[i], s);
  return s;
}

template <bool kNorm>
__global__ void __launch_bounds__(kThreads, 1) gdn_recurrence_kernel(
    const uint16_t* __restrict__ conv_qkv, size_t tokens, const uint16_t* __restrict__ a,
    const uint16_t* __restrict__ b, const uint16_t* __restrict__ A_log, const uint16_t* __restrict__ dt_bias,
    const uint4* state_in, uint4* state_out, float l2_eps, const uint4* __restrict__ norm_weight,
    const uint16_t* __restrict__ norm_gate, float norm_eps, uint16_t* out) {
  __shared__ float head_out[kNorm ? kHead : 1];
  const int head = blockIdx.x;
  const int lane = threadIdx.x & (kLanesPerRow - 1);
  const int row0 = threadIdx.x / kLanesPerRow;  // rows row0 and row0 + 64
  const int qk_head = head / 3;

  float S[kPasses][8];
#pragma unroll
  for (int p = 0; p < kPasses; ++p) {
    const size_t vec = (static_cast<size_t>(head) * kHead + row0 + p * kRowsPerPass) * kLanesPerRow + lane;
    unpack8(ld_vec(state_in + vec), S[p]);
  }
  const float a_decay = -expf(bf16_to_float(A_log[head]));
  const float bias = bf16_to_float(dt_bias[head]);
  const float inv_sqrt_dim = __fdiv_rn(1.0f, sqrtf(static_cast<float>(kHead)));

  for (size_t t = 0; t < tokens; ++t) {
    const uint16_t* row = conv_qkv + t * kChannels;
    float q[8], k[8];
    unpack8(ld_weight(reinterpret_cast<const uint4*>(row + qk_head * kHead) + lane), q);
    unpack8(ld_weight(reinterpret_cast<const uint4*>(row + kKOffset + qk_head * kHead) + lane), k);
    const float q_sum = group_sum<kLanesPerRow>(dot8(q, q));
    const float k_sum = group_sum<kLanesPerRow>(dot8(k, k));
    // 1 / sqrt(sum + eps), then the extra 1 / sqrt(128) for q: the reference's two-step product
    const float q_scale = __fdiv_rn(1.0f, sqrtf(q_sum + l2_eps)) * inv_sqrt_dim;
    const float k_scale = __fdiv_rn(1.0f, sqrtf(k_sum + l2_eps));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      q[i] *= q_scale;
      k[i] *= k_scale;
    }
    const float g = a_decay * softplus_ref(bf16_to_float(a[t * kValueHeads + head]) + bias);
    const float alpha = expf(g);
    const float beta = sigmoid_ref(bf16_to_float(b[t * kValueHeads + head]));

#pragma unroll
    for (int p = 0; p < kPasses; ++p) {
      const int v = row0 + p * kRowsPerPass;
      float decayed[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) decayed[i] = alpha * S[p][i];
      const float pred = group_sum<kLanesPerRow>(dot8(decayed, k));
      const float value = bf16_to_float(row[kVOffset + head * kHead + v]);
      const float delta = (value - pred) * beta;
      float updated[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) updated[i] = fmaf(delta, k[i], decayed[i]);
      const float result = group_sum<kLanesPerRow>(dot8(updated, q));
      // the state crosses a bf16 boundary after every step
      const uint4 packed = pack8(updated);
      unpack8(packed, S[p]);
      if (lane == 0) {
        if (kNorm) head_out[v] = bf16_to_float(float_to_bf16(result));
        else out[(t * kValueHeads + head) * kHead + v] = float_to_bf16(result);
      }
    }
    if (kNorm) {
      // plain RMSNorm over the head's 128 rounded outputs, times weight, times silu(z); one rounding
      __syncthreads();
      if (threadIdx.x < 32) {  // a whole warp (the shuffles name all 32 lanes); its two halves do the same work
        float x[8], w[8], z[8], y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = head_out[lane * 8 + i];
        const size_t base = (t * kValueHeads + head) * kHead;
        unpack8(ld_weight(norm_weight + lane), w);
        unpack8(ld_weight(reinterpret_cast<const uint4*>(norm_gate + base) + lane), z);
        const float inv = inverse_rms(group_sum<kLanesPerRow>(dot8(x, x)), 1.0f / kHead, norm_eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = x[i] * inv * w[i] * silu(z[i]);
        if (threadIdx.x < kLanesPerRow) st_vec(reinterpret_cast<uint4*>(out + base) + lane, pack8(y));
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int p = 0; p < kPasses; ++p) {
    const size_t vec = (static_cast<size_t>(head) * kHead + row0 + p * kRowsPerPass) * kLanesPerRow + lane;
    st_vec(state_out + vec, pack8(S[p]));
  }
}

// ---- many tokens in one call ---------------------------------------------------------------------------------
// The loop above pays, for every token, the L2 round trips of its inputs and the libm chains of its gates before the
// state arithmetic can start.  None of that depends on the state, so for a tile of tokens it is done kGdnBatch tokens
// at a time and in parallel: half-warps normalise q and k and derive alpha and beta of one token each (the same
// 16-lane sums and the same expressions as above, so the same bits), every thread stages the value rows, all into
// shared memory; then the 1024 threads run the state arithmetic of those tokens back to back out of shared memory,
// and the rounded outputs leave as one coalesced block.  Two barriers per batch instead of a dozen dependent
// latencies per token.
constexpr int kGdnBatch = 16;

__global__ void __launch_bounds__(kThreads, 1) gdn_recurrence_tile_kernel(
    const uint16_t* __restrict__ conv_qkv, size_t tokens, const uint16_t* __restrict__ a,
    const uint16_t* __restrict__ b, const uint16_t* __restrict__ A_log, const uint16_t* __restrict__ dt_bias,
    const uint4* state_in, uint4* state_out, float l2_eps, uint16_t* out) {
  __shared__ __align__(16) float sq[kGdnBatch][kHead];
  __shared__ __align__(16) float sk[kGdnBatch][kHead];
  __shared__ float sv[kGdnBatch][kHead];
  __shared__ float s_alpha[kGdnBatch], s_beta[kGdnBatch];
  __shared__ __align__(16) uint16_t s_out[kGdnBatch][kHead];
  const int head = blockIdx.x;
  const int lane = threadIdx.x & (kLanesPerRow - 1);
  const int group = threadIdx.x / kLanesPerRow;  // 64 groups of 16 lanes
  const int row0 = group;                        // state rows row0 and row0 + 64
  const int qk_head = head / 3;

  float S[kPasses][8];
#pragma unroll
  for (int p = 0; p < kPasses; ++p) {
    const size_t vec = (static_cast<size_t>(head) * kHead + row0 + p * kRowsPerPass) * kLanesPerRow + lane;
    unpack8(ld_vec(state_in + vec), S[p]);
  }
  const float a_decay = -expf(bf16_to_float(A_log[head]));
  const float bias = bf16_to_float(dt_bias[head]);
  const float inv_sqrt_dim = __fdiv_rn(1.0f, sqrtf(static_cast<float>(kHead)));

  for (size_t t0 = 0; t0 < tokens; t0 += kGdnBatch) {
    const int count = static_cast<int>(min(static_cast<size_t>(kGdnBatch), tokens - t0));
    // ---- prepare: group i < 16 takes token t0 + i (whole warps, so the 16-lane shuffles name live lanes)
    if (group < kGdnBatch) {
      const bool live = group < count;
      const uint16_t* row = conv_qkv + (t0 + (live ? group : 0)) * kChannels;
      float q[8], k[8];
      unpack8(live ? ld_weight(reinterpret_cast<const uint4*>(row + qk_head * kHead) + lane) : make_uint4(0, 0, 0, 0), q);
      unpack8(live ? ld_weight(reinterpret_cast<const uint4*>(row + kKOffset + qk_head * kHead) + lane) : make_uint4(0, 0, 0, 0), k);
      const float q_sum = group_sum<kLanesPerRow>(dot8(q, q));
      const float k_sum = group_sum<kLanesPerRow>(dot8(k, k));
      const float q_scale = __fdiv_rn(1.0f, sqrtf(q_sum + l2_eps)) * inv_sqrt_dim;
      const float k_scale = __fdiv_rn(1.0f, sqrtf(k_sum + l2_eps));
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sq[group][lane * 8 + i] = q[i] * q_scale;
        sk[group][lane * 8 + i] = k[i] * k_scale;
      }
      if (lane == 0 && live) {
        const float g = a_decay * softplus_ref(bf16_to_float(a[(t0 + group) * kValueHeads + head]) + bias);
        s_alpha[group] = expf(g);
        s_beta[group] = sigmoid_ref(bf16_to_float(b[(t0 + group) * kValueHeads + head]));
      }
    }
    for (int i = threadIdx.x; i < count * kHead; i += kThreads) {
      const int t = i / kHead, v = i % kHead;
      sv[t][v] = bf16_to_float(conv_qkv[(t0 + t) * kChannels + kVOffset + head * kHead + v]);
    }
    __syncthreads();
    // ---- the recurrence over the prepared tokens
    for (int t = 0; t < count; ++t) {
      float q[8], k[8];
      *reinterpret_cast<float4*>(q) = *reinterpret_cast<const float4*>(&sq[t][lane * 8]);
      *reinterpret_cast<float4*>(q + 4) = *reinterpret_cast<const float4*>(&sq[t][lane * 8 + 4]);
      *reinterpret_cast<float4*>(k) = *reinterpret_cast<const float4*>(&sk[t][lane * 8]);
      *reinterpret_cast<float4*>(k + 4) = *reinterpret_cast<const float4*>(&sk[t][lane * 8 + 4]);
      const float alpha = s_alpha[t], beta = s_beta[t];
#pragma unroll
      for (int p = 0; p < kPasses; ++p) {
        const int v = row0 + p * kRowsPerPass;
        float decayed[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) decayed[i] = alpha * S[p][i];
        const float pred = group_sum<kLanesPerRow>(dot8(decayed, k));
        const float delta = (sv[t][v] - pred) * beta;
        float updated[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) updated[i] = fmaf(delta, k[i], decayed[i]);
        const float result = group_sum<kLanesPerRow>(dot8(updated, q));
        const uint4 packed = pack8(updated);  // the state crosses a bf16 boundary after every step
        unpack8(packed, S[p]);
        if (lane == 0) s_out[t][v] = float_to_bf16(result);
      }
    }
    __syncthreads();
    // ---- the batch's outputs: count x 128 bf16 of this head, 16 bytes per thread
    for (int i = threadIdx.x; i < count * (kHead / 8); i += kThreads) {
      const int t = i / (kHead / 8), c = i % (kHead / 8);
      st_vec(out + ((t0 + t) * kValueHeads + head) * kHead + c * 8, *reinterpret_cast<const uint4*>(&s_out[t][c * 8]));
    }
    // (the next batch's preparation writes sq / sk / sv, which every thread has finished reading at the barrier
    // above; s_out is rewritten only after the next batch's first barrier)
  }
#pragma unroll
  for (int p = 0; p < kPasses; ++p) {
    const size_t vec = (static_cast<size_t>(head) * kHead + row0 + p * kRowsPerPass) * kLanesPerRow + lane;
    st_vec(state_out + vec, pack8(S[p]));
  }
}

int launch_gdn(const uint16_t* conv_qkv, size_t tokens, const uint16_t* a, const uint16_t* b, const uint16_t* A_log,
               const uint16_t* dt_bias, const uint16_t* state_in, uint16_t* state_out, float l2_eps,
               const uint16_t* norm_weight, const uint16_t* norm_gate, float norm_eps, bool norm, uint16_t* out,
               void* stream) {
  using namespace host;
  if (!valid_epsilon(l2_eps) || (norm && !valid_epsilon(norm_eps))) return kInvalid;
  if (mul3_overflows(tokens, kChannels, sizeof(uint16_t))) return kInvalid;
  if (tokens == 0) return kOk;
  if (conv_qkv == nullptr || a == nullptr || b == nullptr || A_log == nullptr || dt_bias == nullptr ||
      state_in == nullptr || state_out == nullptr || out == nullptr || (norm && (!norm_weight || !norm_gate)))
    return kInvalid;
  constexpr size_t kStateBytes = static_cast<size_t>(kValueHeads) * kHead * kHead * 2;
  const size_t out_bytes = tokens * kValueHeads * kHead * 2;
  const Span sc = span(conv_qkv, tokens * kChannels * 2), sa = span(a, tokens * kValueHeads * 2),
             sb = span(b, tokens * kValueHeads * 2), sl = span(A_log, kValueHeads * 2),
             sd = span(dt_bias, kValueHeads * 2), si = span(state_in, kStateBytes), so = span(state_out, kStateBytes),
             sy = span(out, out_bytes), sw = span(norm_weight, norm ? kHead * 2 : 0),
             sz = span(norm_gate, norm ? out_bytes : 0);
  // exact state_in == state_out is the one alias allowed (include/q3x/runtime/gdn_decode.h:60-64); every
  // writable range is otherwise disjoint from every other operand
  if (partial_overlap(si, so)) return kInvalid;
  const Span readers[] = {sc, sa, sb, sl, sd, sw, sz};
  for (const Span& r : readers)
    if (overlap(so, r) || overlap(sy, r) || wraps(r)) return kInvalid;
  if (overlap(sy, so) || overlap(sy, si) || wraps(sy) || wraps(so) || wraps(si)) return kInvalid;
  if (!aligned16(conv_qkv) || !aligned16(state_in) || !aligned16(state_out) || !aligned16(out) ||
      (norm && (!aligned16(norm_weight) || !aligned16(norm_gate))))
    return kNotSupported;
  clear_stale_error();
  auto SI = reinterpret_cast<const uint4*>(state_in);
  auto SO = reinterpret_cast<uint4*>(state_out);
  cudaStream_t s = as_stream(stream);
  if (norm)
    gdn_recurrence_kernel<true><<<kValueHeads, kThreads, 0, s>>>(conv_qkv, tokens, a, b, A_log, dt_bias, SI, SO,
                                                                 l2_eps, reinterpret_cast<const uint4*>(norm_weight),
                                                                 norm_gate, norm_eps, out);
  else if (tokens >= 4)
    gdn_recurrence_tile_kernel<<<kValueHeads, kThreads, 0, s>>>(conv_qkv, tokens, a, b, A_log, dt_bias, SI, SO, l2_eps, out);
  else
    gdn_recurrence_kernel<false><<<kValueHeads, kThreads, 0, s>>>(conv_qkv, tokens, a, b, A_log, dt_bias, SI, SO,
                                                                  l2_eps, nullptr, nullptr, 1.0f, out);
  return launch_status();
}

}  // namespace
}  // namespace q3x

extern "C" int q3x_b200_gated_delta_net_update(const uint16_t* conv_qkv, size_t tokens, const uint16_t* a,
                                               const uint16_t* b, const uint16_t* A_log, const uint16_t* dt_bias,
                                               const uint16_t* state_in, uint16_t* state_out, float l2_eps,
                                               uint16_t* out, void* stream) {
  return q3x::launch_gdn(conv_qkv, tokens, a, b, A_log, dt_bias, state_in, state_out, l2_eps, nullptr, nullptr, 1.0f,
                         false, out, stream);
}

extern "C" int q3x_b200_gated_delta_net_update_rms_norm_silu_gate(
    const uint16_t* conv_qkv, size_t tokens, const uint16_t* a, const uint16_t* b, const uint16_t* A_log,
    const uint16_t* dt_bias, const uint16_t* state_in, uint16_t* state_out, float l2_eps, const uint16_t* norm_weight,
    const uint16_t* silu_gate, float norm_eps, uint16_t* out, void* stream) {
  return q3x::launch_gdn(conv_qkv, tokens, a, b, A_log, dt_bias, state_in, state_out, l2_eps, norm_weight, silu_gate,
                         norm_eps, true, out, stream);
}
