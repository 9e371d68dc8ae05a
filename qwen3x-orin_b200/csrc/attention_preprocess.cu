// Full-attention pre-processing for Q = 24 heads, KV = 4 heads, head_dim 256, rotary 64:
//   split the interleaved [q|gate] projection, centred per-head RMSNorm of q and (in place) k,
//   partial NeoX RoPE of both -- one pass over HBM -- plus the stand-alone RoPE forms.
//
// One warp owns one 256-wide head: each lane holds one 128-bit vector (8 dims), the sum of squares
// is a five-step shuffle tree, and the rotation pairs dim d (lanes 0..3) with dim d+32 (lanes 4..7)
// through one lane exchange.  The normalised values are rounded to bf16 BEFORE the rotation reads
// them and the rotation is computed as separate multiplies and an add/subtract (no FMA), which is
// the arithmetic of the host reference (src/runtime/reference/decode_ops.cpp:392-404).
#include "device_utils.cuh"
#include "host_checks.hpp"
#include "norm_math.cuh"
#include "q3x_b200.h"

namespace q3x {
namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerCta = kThreads / 32;
constexpr int kQHeads = Q3X_B200_Q_HEADS;
constexpr int kKvHeads = Q3X_B200_KV_HEADS;
constexpr int kHeadsPerToken = kQHeads + kKvHeads;
constexpr int kVecPerHead = Q3X_B200_ATTN_HEAD_DIM / 8;  // 32: one vector per lane
constexpr int kPairs = Q3X_B200_ROTARY_DIM / 2;          // 32 cos/sin values per position

__device__ __forceinline__ uint4 shfl_xor_vec(const uint4& v, int mask) {
  uint4 o;
  o.x = __shfl_xor_sync(kFullMask, v.x, mask);
  o.y = __shfl_xor_sync(kFullMask, v.y, mask);
  o.z = __shfl_xor_sync(kFullMask, v.z, mask);
  o.w = __shfl_xor_sync(kFullMask, v.w, mask);
  return o;
}

// Rotation of the eight dims a lane (< 8) holds.  `own` are this lane's rounded values, `other`
// the partner lane's (lane ^ 4).  Lanes 0..3 hold the first half of each pair, lanes 4..7 the second.
__device__ __forceinline__ uint4 rotate8(const uint4& own, const uint4& other, const float* __restrict__ cos_row,
                                         const float* __restrict__ sin_row, int lane) {
  const int pair0 = (lane & 3) * 8;
  const float4 c0 = __ldg(reinterpret_cast<const float4*>(cos_row + pair0));
  const float4 c1 = __ldg(reinterpret_cast<const float4*>(cos_row + pair0 + 4));
  const float4 s0 = __ldg(reinterpret_cast<const float4*>(sin_row + pair0));
  const float4 s1 = __ldg(reinterpret_cast<const float4*>(sin_row + pair0 + 4));
  const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  float a[8], b[8], y[8];
  unpack8(own, a);
  unpack8(other, b);
  const bool first_half = lane < 4;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float ac = __fmul_rn(a[i], c[i]);
    const float bs = __fmul_rn(b[i], s[i]);
    // first half:  x[d]    * cos - x[d+32] * sin      second half: x[d+32] * cos + x[d] * sin
    y[i] = first_half ? __fsub_rn(ac, bs) : __fadd_rn(ac, bs);
  }
  return pack8(y);
}

__device__ __forceinline__ uint4 centered_norm_head(const uint4& x, const uint4& w, float eps) {
  float f[8], g[8], y[8];
  unpack8(x, f);
  float partial = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) partial = fmaf(f[i], f[i], partial);
  const float sum = group_sum<32>(partial);
  const float inv = inverse_rms(sum, 1.0f / 256.0f, eps);
  unpack8(w, g);
#pragma unroll
  for (int i = 0; i < 8; ++i) y[i] = f[i] * inv * (g[i] + 1.0f);
  return pack8(y);
}

// One CTA of seven warps owns one token per iteration: warps 0..5 take four q heads each (with their
// gates), warp 6 the four k heads, so the q / k choice is warp-uniform and no index division is
// needed.  A lane issues the eight (q, gate) or four (k) 128-bit loads of its heads back to back.
constexpr int kPreWarps = 7;
constexpr int kPreThreads = kPreWarps * 32;
constexpr int kHeadsPerWarp = 4;
static_assert(kPreWarps * kHeadsPerWarp == kHeadsPerToken, "28 heads = 7 warps x 4");

__global__ void __launch_bounds__(kPreThreads) attention_preprocess_kernel(
    const uint4* __restrict__ q_gate, uint4* key, const uint4* __restrict__ q_weight,
    const uint4* __restrict__ k_weight, float eps, uint4* __restrict__ q_out, uint4* __restrict__ gate_out,
    const float* __restrict__ cosines, const float* __restrict__ sines, size_t first_position, size_t tokens) {
  release_next_kernel();
  wait_for_prior_kernels();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const bool is_q = warp < kPreWarps - 1;
  const uint4 w = ld_weight((is_q ? q_weight : k_weight) + lane);

  for (size_t token = blockIdx.x; token < tokens; token += gridDim.x) {
    uint4 x[kHeadsPerWarp], g[kHeadsPerWarp];
    if (is_q) {
      const uint4* src = q_gate + (token * (2 * kQHeads) + 2 * (warp * kHeadsPerWarp)) * kVecPerHead + lane;
#pragma unroll
      for (int h = 0; h < kHeadsPerWarp; ++h) {
        x[h] = ld_stream(src + (2 * h) * kVecPerHead);
        g[h] = ld_stream(src + (2 * h + 1) * kVecPerHead);
      }
    } else {
#pragma unroll
      for (int h = 0; h < kHeadsPerWarp; ++h) x[h] = ld_vec(key + (token * kKvHeads + h) * kVecPerHead + lane);
    }
    const size_t table = (first_position + token) * kPairs;
#pragma unroll
    for (int h = 0; h < kHeadsPerWarp; ++h) {
      uint4 y = centered_norm_head(x[h], w, eps);
      const uint4 partner = shfl_xor_vec(y, 4);
      if (lane < 8) y = rotate8(y, partner, cosines + table, sines + table, lane);
      if (is_q) {
        const size_t dst = (token * kQHeads + warp * kHeadsPerWarp + h) * kVecPerHead + lane;
        st_vec(q_out + dst, y);
        st_vec(gate_out + dst, g[h]);
      } else {
        st_vec(key + (token * kKvHeads + h) * kVecPerHead + lane, y);
      }
    }
  }
}

// Stand-alone rotation, one warp per head.  kTable: the cos/sin row is chosen per token
// (item / heads_per_token + first_position), else one row serves every head.
// in == out is allowed; then only the rotary lanes touch memory.
__global__ void __launch_bounds__(kThreads) rope_heads_kernel(const uint4* in, uint4* out,
                                                              const float* __restrict__ cosines,
                                                              const float* __restrict__ sines, size_t heads,
                                                              size_t heads_per_token, size_t first_position,
                                                              bool per_token_table) {
  const int lane = threadIdx.x & 31;
  const size_t warp = static_cast<size_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  const size_t stride = static_cast<size_t>(gridDim.x) * kWarpsPerCta;
  const bool in_place = in == out;
  for (size_t head = warp; head < heads; head += stride) {
    uint4 x = make_uint4(0, 0, 0, 0);
    if (lane < 8 || !in_place) x = ld_vec(in + head * kVecPerHead + lane);
    const uint4 partner = shfl_xor_vec(x, 4);
    if (lane < 8) {
      const size_t table = per_token_table ? (first_position + head / heads_per_token) * kPairs : 0;
      x = rotate8(x, partner, cosines + table, sines + table, lane);
    }
    if (lane < 8 || !in_place) st_vec(out + head * kVecPerHead + lane, x);
  }
}

// Scalar rotation for unaligned buffers: one thread per (head, pair).
__global__ void __launch_bounds__(kThreads) rope_heads_scalar_kernel(const uint16_t* in, uint16_t* out,
                                                                     const float* cosines, const float* sines,
                                                                     size_t heads, size_t heads_per_token,
                                                                     size_t first_position, bool per_token_table) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  const size_t total = heads * 128;  // 32 rotary pairs + 96 pass-through pairs of dims
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < total; i += stride) {
    const size_t head = i / 128;
    const int slot = static_cast<int>(i - head * 128);
    const uint16_t* x = in + head * 256;
    uint16_t* y = out + head * 256;
    if (slot < kPairs) {
      const size_t table = per_token_table ? (first_position + head / heads_per_token) * kPairs : 0;
      const float a = bf16_to_float(x[slot]), b = bf16_to_float(x[slot + kPairs]);
      const float c = cosines[table + slot], s = sines[table + slot];
      const uint16_t lo = float_to_bf16(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)));
      const uint16_t hi = float_to_bf16(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s)));
      y[slot] = lo;
      y[slot + kPairs] = hi;
    } else if (in != out) {
      const int d = 64 + (slot - kPairs) * 2;
      y[d] = x[d];
      y[d + 1] = x[d + 1];
    }
  }
}

}  // namespace
}  // namespace q3x

using namespace q3x;
using namespace q3x::host;

extern "C" int q3x_b200_full_attention_preprocess(const uint16_t* interleaved_q_gate, uint16_t* key,
                                                  const uint16_t* q_weight, const uint16_t* k_weight, float eps,
                                                  uint16_t* q_out, uint16_t* gate_out, const float* cosines,
                                                  const float* sines, size_t first_position, size_t tokens,
                                                  void* stream) {
  if (!valid_epsilon(eps)) return kInvalid;
  if (tokens == 0) return kOk;
  if (interleaved_q_gate == nullptr || key == nullptr || q_weight == nullptr || k_weight == nullptr ||
      q_out == nullptr || gate_out == nullptr || cosines == nullptr || sines == nullptr)
    return kInvalid;
  constexpr size_t kHead = Q3X_B200_ATTN_HEAD_DIM * sizeof(uint16_t);
  if (mul_overflows(tokens, 2 * kQHeads * kHead)) return kInvalid;
  // last table row read is first_position + tokens - 1
  if (first_position > std::numeric_limits<size_t>::max() - tokens ||
      mul_overflows(first_position + tokens, kPairs * sizeof(float)))
    return kInvalid;
  const size_t table_bytes = (first_position + tokens) * kPairs * sizeof(float);
  const Span in = span(interleaved_q_gate, tokens * 2 * kQHeads * kHead), k = span(key, tokens * kKvHeads * kHead),
             qw = span(q_weight, kHead), kw = span(k_weight, kHead), q = span(q_out, tokens * kQHeads * kHead),
             g = span(gate_out, tokens * kQHeads * kHead), c = span(cosines, table_bytes),
             s = span(sines, table_bytes);
  const Span all[] = {in, k, qw, kw, q, g, c, s};
  for (const Span& x : all)
    if (wraps(x)) return kInvalid;
  // every writable range is disjoint from every other operand
  const int writable[] = {1, 4, 5};
  for (int wi : writable)
    for (int j = 0; j < 8; ++j)
      if (j != wi && overlap(all[wi], all[j])) return kInvalid;
  if (!aligned16(interleaved_q_gate) || !aligned16(key) || !aligned16(q_weight) || !aligned16(k_weight) ||
      !aligned16(q_out) || !aligned16(gate_out) || !aligned16(cosines) || !aligned16(sines))
    return kNotSupported;
  clear_stale_error();
  const unsigned grid = wave_grid(attention_preprocess_kernel, kPreThreads, tokens, 1);
  launch_kernel(attention_preprocess_kernel, grid, kPreThreads, 0, as_stream(stream), latency_bound_launch(grid),
                reinterpret_cast<const uint4*>(interleaved_q_gate), reinterpret_cast<uint4*>(key),
                reinterpret_cast<const uint4*>(q_weight), reinterpret_cast<const uint4*>(k_weight), eps,
                reinterpret_cast<uint4*>(q_out), reinterpret_cast<uint4*>(gate_out), cosines, sines, first_position,
                tokens);
  return launch_status();
}

namespace {

int launch_rope(const uint16_t* in, uint16_t* out, const float* cosines, const float* sines, size_t heads,
                size_t heads_per_token, size_t first_position, bool per_token, void* stream) {
  clear_stale_error();
  cudaStream_t s = as_stream(stream);
  if (aligned16(in) && aligned16(out) && aligned16(cosines) && aligned16(sines)) {
    rope_heads_kernel<<<grid_for(heads, kWarpsPerCta, 8), kThreads, 0, s>>>(
        reinterpret_cast<const uint4*>(in), reinterpret_cast<uint4*>(out), cosines, sines, heads, heads_per_token,
        first_position, per_token);
  } else {
    rope_heads_scalar_kernel<<<grid_for(heads * 128, kThreads, 8), kThreads, 0, s>>>(
        in, out, cosines, sines, heads, heads_per_token, first_position, per_token);
  }
  return launch_status();
}

}  // namespace

extern "C" int q3x_b200_partial_neox_rope_256_64(const uint16_t* in, const float* cosines, const float* sines,
                                                 size_t heads, uint16_t* out, void* stream) {
  if (mul_overflows(heads, Q3X_B200_ATTN_HEAD_DIM * sizeof(uint16_t))) return kInvalid;
  if (heads == 0) return kOk;
  if (in == nullptr || cosines == nullptr || sines == nullptr || out == nullptr) return kInvalid;
  const size_t bytes = heads * Q3X_B200_ATTN_HEAD_DIM * sizeof(uint16_t);
  const Span si = span(in, bytes), so = span(out, bytes), sc = span(cosines, kPairs * 4), ss = span(sines, kPairs * 4);
  if (wraps(si) || wraps(so) || partial_overlap(so, si) || overlap(so, sc) || overlap(so, ss)) return kInvalid;
  return launch_rope(in, out, cosines, sines, heads, 1, 0, false, stream);
}

extern "C" int q3x_b200_qk_partial_neox_rope(uint16_t* query, uint16_t* key, const float* cosines,
                                             const float* sines, size_t first_position, size_t tokens,
                                             void* stream) {
  if (tokens == 0) return kOk;
  if (query == nullptr || key == nullptr || cosines == nullptr || sines == nullptr) return kInvalid;
  constexpr size_t kHead = Q3X_B200_ATTN_HEAD_DIM * sizeof(uint16_t);
  if (mul_overflows(tokens, kQHeads * kHead) || first_position > std::numeric_limits<size_t>::max() - tokens ||
      mul_overflows(first_position + tokens, kPairs * sizeof(float)))
    return kInvalid;
  const size_t table_bytes = (first_position + tokens) * kPairs * sizeof(float);
  const Span q = span(query, tokens * kQHeads * kHead), k = span(key, tokens * kKvHeads * kHead),
             c = span(cosines, table_bytes), s = span(sines, table_bytes);
  if (wraps(q) || wraps(k) || overlap(q, k) || overlap(q, c) || overlap(q, s) || overlap(k, c) || overlap(k, s))
    return kInvalid;
  int st = launch_rope(query, query, cosines, sines, tokens * kQHeads, kQHeads, first_position, true, stream);
  if (st != kOk) return st;
  return launch_rope(key, key, cosines, sines, tokens * kKvHeads, kKvHeads, first_position, true, stream);
}
