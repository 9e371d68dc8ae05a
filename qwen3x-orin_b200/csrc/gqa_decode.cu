// Batch-one (decode) grouped-query attention for Q = 24 heads, KV = 4 heads, head_dim 256 against a
// KV cache of any length, with the attention sigmoid output gate as its epilogue:
//   s[h,p] = (q[h] . K[p, h/6]) * scale;  P = softmax_p(s);  o[h] = bf16(sum_p P[h,p] * V[p, h/6]);
//   out[h] = bf16(o[h] * sigmoid(gate[h]))
// (gqa_attention_reference_cpu, src/runtime/reference/decode_ops.cpp:445-508, followed by
// sigmoid_gate_reference_cpu across a bf16 boundary, the contract of
// launch_gqa_attention_splitkv_sigmoid_gate_24_4_256_cuda, include/q3x/runtime/decode_ops.h:397-423).
//
// The work is a single pass over the cache -- 4 KB per position for K and V together -- so the kernel is
// HBM-bound by design and runs on the FP32 pipes: six query heads share a KV head, which is far too thin
// a tile for tensor cores to matter.  Split-KV with online softmax:
//   * grid = (splits, 4 KV heads); a CTA of eight warps walks its share of the positions in batches of
//     eight; within a warp a lane owns eight of the 256 dims (one 128-bit load per cache row), so a row is
//     one fully coalesced 512-byte access;
//   * per batch a lane forms its 8 x 6 partial dot products (q for its dims lives in registers), the warp
//     sums them with a reduce-scatter butterfly (48 shuffles for 48 sums) that leaves position p's six
//     scores with the lanes whose upper three index bits are p, those lanes update the running maximum /
//     denominator of their heads and turn scores into probabilities, and the probabilities go back to all
//     lanes through shared memory for the P.V accumulation (6 heads x 8 dims of FP32 accumulators per lane);
//   * the V rows of the batch and the K rows of the NEXT batch are requested before the reduction starts,
//     so sixteen 512-byte loads per warp are in flight while the arithmetic runs;
//   * at the end a CTA merges its warps' (max, denominator, accumulator) states through shared memory and
//     writes one partial state per head to the workspace; a second small kernel merges the splits of each
//     head, rounds, applies the gate and rounds again.
#include "device_utils.cuh"
#include "host_checks.hpp"
#include "q3x_b200.h"

namespace q3x {
namespace {

constexpr int kQHeads = Q3X_B200_Q_HEADS;          // 24
constexpr int kKvHeads = Q3X_B200_KV_HEADS;        // 4
constexpr int kGroup = kQHeads / kKvHeads;         // 6 query heads per KV head
constexpr int kDim = Q3X_B200_ATTN_HEAD_DIM;       // 256
constexpr int kRowVectors = kDim / 8;              // 32: one vector per lane
#ifndef Q3X_GQA_WARPS
#define Q3X_GQA_WARPS 8
#endif
#ifndef Q3X_GQA_BATCH
#define Q3X_GQA_BATCH 8
#endif
constexpr int kWarps = Q3X_GQA_WARPS;
constexpr int kThreads = kWarps * 32;
constexpr int kBatch = Q3X_GQA_BATCH;              // positions per warp iteration (8 or 4)
static_assert(kBatch == 8 || kBatch == 4, "the reduce-scatter below is written for 8 or 4 positions");
constexpr int kSums = kBatch * kGroup;             // partial sums a lane holds before the reduction
// After the reduce-scatter a lane's top log2(kBatch) index bits name its position, the next bit the half of the
// heads (three each), and the remaining low bits are replicas.
constexpr int kHalfMask = 16 / kBatch;             // 2 (batch 8) or 4 (batch 4)
constexpr int kPosShift = kBatch == 8 ? 2 : 3;
constexpr int kMaxSplits = 37;                     // 37 x 4 KV heads = 148 CTAs, one per SM
constexpr int kPartialFloats = 2 + kDim;           // max, denominator, accumulator
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Sums v[0..N) across the warp so that afterwards v[0..N/2) of a lane holds the totals of one half,
// chosen by the lane's bit `mask`: lanes with the bit clear keep the lower half, lanes with it set the
// upper half.  One shuffle per surviving value.
template <int N>
__device__ __forceinline__ void halve(float (&v)[kSums], int mask) {
  const bool upper = (threadIdx.x & mask) != 0;
#pragma unroll
  for (int i = 0; i < N / 2; ++i) {
    const float keep = upper ? v[i + N / 2] : v[i];
    const float send = upper ? v[i] : v[i + N / 2];
    v[i] = keep + __shfl_xor_sync(kFullMask, send, mask);
  }
}

// Partial attention state of one KV head over positions [first, last), one CTA; warp w takes the batches
// w, w + 8, ... of that range.  workspace: [kv head][split][query head in group][kPartialFloats].
__global__ void __launch_bounds__(kThreads, 1) gqa_decode_partial_kernel(
    const uint16_t* __restrict__ query, const uint4* __restrict__ key_cache, const uint4* __restrict__ value_cache,
    size_t length, size_t positions_per_split, float scale, float* __restrict__ workspace) {
  __shared__ __align__(16) float probs[kWarps][kBatch * kGroup + 8];  // 48 probabilities + 6 rescale factors
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int kv = blockIdx.y;
  const size_t first = static_cast<size_t>(blockIdx.x) * positions_per_split;
  const size_t last = min(length, first + positions_per_split);

  // q of this KV head's six query heads for the lane's eight dims, pre-multiplied by nothing: the scale is
  // applied to the finished sum, as the host op does
  float q[kGroup][8];
#pragma unroll
  for (int h = 0; h < kGroup; ++h)
    unpack8(ld_weight(reinterpret_cast<const uint4*>(query + (kv * kGroup + h) * kDim) + lane), q[h]);

  float acc[kGroup][8];
#pragma unroll
  for (int h = 0; h < kGroup; ++h)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[h][i] = 0.0f;
  // running maximum (in the scaled-score domain) and denominator of the three heads this lane looks after
  // during the softmax step: heads 3 * (bit kHalfMask of the lane) + {0, 1, 2}
  float run_max[3] = {-INFINITY, -INFINITY, -INFINITY};
  float run_sum[3] = {0.0f, 0.0f, 0.0f};

  const size_t row_stride = static_cast<size_t>(kKvHeads) * kRowVectors;  // vectors between positions
  const uint4* k_base = key_cache + static_cast<size_t>(kv) * kRowVectors + lane;
  const uint4* v_base = value_cache + static_cast<size_t>(kv) * kRowVectors + lane;
  auto load_rows = [&](const uint4* base, size_t start, uint4 (&rows)[kBatch]) {
#pragma unroll
    for (int p = 0; p < kBatch; ++p) {
      const size_t pos = min(start + p, last - 1);  // a position past the end re-reads the last row (masked later)
      rows[p] = ld_stream(base + pos * row_stride);
    }
  };

  const size_t stride = static_cast<size_t>(kWarps) * kBatch;
  size_t start = first + static_cast<size_t>(warp) * kBatch;
  uint4 k_rows[kBatch], v_rows[kBatch];
  if (start < last) load_rows(k_base, start, k_rows);
  for (; start < last; start += stride) {
    // ---- partial dot products: sums[p * 6 + h] over the lane's eight dims ------------------------------
    float sums[kSums];
#pragma unroll
    for (int p = 0; p < kBatch; ++p) {
      float k[8];
      unpack8(k_rows[p], k);
#pragma unroll
      for (int h = 0; h < kGroup; ++h) {
        float2 s = mul2(make_float2(q[h][0], q[h][1]), make_float2(k[0], k[1]));
#pragma unroll
        for (int i = 2; i < 8; i += 2) s = fma2(make_float2(q[h][i], q[h][i + 1]), make_float2(k[i], k[i + 1]), s);
        sums[p * kGroup + h] = s.x + s.y;
      }
    }
    // the loads the arithmetic below hides: this batch's V rows and the next batch's K rows
    load_rows(v_base, start, v_rows);
    if (start + stride < last) load_rows(k_base, start + stride, k_rows);

    // ---- reduce-scatter: lane bits 4..2 select the position, bit 1 the half of the heads -----------------
    if constexpr (kBatch == 8) {
      halve<48>(sums, 16);
      halve<24>(sums, 8);
      halve<12>(sums, 4);
      halve<6>(sums, 2);
#pragma unroll
      for (int i = 0; i < 3; ++i) sums[i] += __shfl_xor_sync(kFullMask, sums[i], 1);
    } else {
      halve<24>(sums, 16);
      halve<12>(sums, 8);
      halve<6>(sums, 4);
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        sums[i] += __shfl_xor_sync(kFullMask, sums[i], 2);
        sums[i] += __shfl_xor_sync(kFullMask, sums[i], 1);
      }
    }
    const int my_pos = lane >> kPosShift;
    const bool valid = start + my_pos < last;
    // ---- online softmax for the lane's three heads ----------------------------------------------------------
    float p_val[3], rescale[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const float s = valid ? sums[i] * scale : -INFINITY;
      float batch_max = s;
      if (kBatch == 8) batch_max = fmaxf(batch_max, __shfl_xor_sync(kFullMask, batch_max, 4));
      batch_max = fmaxf(batch_max, __shfl_xor_sync(kFullMask, batch_max, 8));
      batch_max = fmaxf(batch_max, __shfl_xor_sync(kFullMask, batch_max, 16));
      const float new_max = fmaxf(run_max[i], batch_max);  // finite: every batch has a valid position
      rescale[i] = ex2((run_max[i] - new_max) * kLog2e);   // 0 on the first batch (run_max = -inf)
      p_val[i] = ex2((s - new_max) * kLog2e);              // 0 for a masked position
      float batch_sum = p_val[i];
      if (kBatch == 8) batch_sum += __shfl_xor_sync(kFullMask, batch_sum, 4);
      batch_sum += __shfl_xor_sync(kFullMask, batch_sum, 8);
      batch_sum += __shfl_xor_sync(kFullMask, batch_sum, 16);
      run_sum[i] = fmaf(run_sum[i], rescale[i], batch_sum);
      run_max[i] = new_max;
    }
    // ---- probabilities and rescale factors to every lane ---------------------------------------------------------
    __syncwarp();  // the previous batch's readers are done
    if ((lane & (kHalfMask - 1)) == 0) {
      const int half = (lane & kHalfMask) ? 1 : 0;
#pragma unroll
      for (int i = 0; i < 3; ++i) probs[warp][my_pos * kGroup + half * 3 + i] = p_val[i];
      if (my_pos == 0) {
#pragma unroll
        for (int i = 0; i < 3; ++i) probs[warp][kBatch * kGroup + half * 3 + i] = rescale[i];
      }
    }
    __syncwarp();
    float factor[kGroup];
#pragma unroll
    for (int h = 0; h < kGroup; ++h) factor[h] = probs[warp][kBatch * kGroup + h];
#pragma unroll
    for (int h = 0; h < kGroup; ++h)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[h][i] *= factor[h];
    // ---- P.V ----------------------------------------------------------------------------------------------------------
#pragma unroll
    for (int p = 0; p < kBatch; ++p) {
      float v[8];
      unpack8(v_rows[p], v);
#pragma unroll
      for (int h = 0; h < kGroup; ++h) {
        const float w = probs[warp][p * kGroup + h];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          const float2 r = fma2(make_float2(w, w), make_float2(v[i], v[i + 1]), make_float2(acc[h][i], acc[h][i + 1]));
          acc[h][i] = r.x;
          acc[h][i + 1] = r.y;
        }
      }
    }
  }

  // ---- the CTA's partial state: its warps' (max, denominator, accumulator) merged through shared memory ----
  // (three heads per round, so that the staging fits the static 48 KB: 8 warps x 3 heads x 256 floats)
  __shared__ float warp_max[kWarps][kGroup], warp_sum[kWarps][kGroup];
  __shared__ float stage[kWarps][3][kDim];
  if (lane == 0 || lane == kHalfMask) {  // position slot 0, both head halves
    const int half = lane == 0 ? 0 : 1;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      warp_max[warp][half * 3 + i] = run_max[i];
      warp_sum[warp][half * 3 + i] = run_sum[i];
    }
  }
  __syncthreads();
  float* out = workspace + (static_cast<size_t>(kv) * gridDim.x + blockIdx.x) * kGroup * kPartialFloats;
#pragma unroll
  for (int round = 0; round < 2; ++round) {
    // this warp's accumulators of the round's three heads, rescaled to the CTA-wide maximum of each head
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int h = round * 3 + j;
      float top = warp_max[0][h];
#pragma unroll
      for (int w = 1; w < kWarps; ++w) top = fmaxf(top, warp_max[w][h]);
      // an idle warp holds (-inf, 0, zeros); a CTA with no position at all keeps top = -inf and writes zeros
      const float f = warp_sum[warp][h] == 0.0f ? 0.0f : ex2((warp_max[warp][h] - top) * kLog2e);
#pragma unroll
      for (int i = 0; i < 8; ++i) stage[warp][j][lane * 8 + i] = acc[h][i] * f;
    }
    __syncthreads();
    for (int item = threadIdx.x; item < 3 * kDim; item += kThreads) {
      const int j = item / kDim, d = item - j * kDim;
      float total = 0.0f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) total += stage[w][j][d];
      out[(round * 3 + j) * kPartialFloats + 2 + d] = total;
    }
    if (threadIdx.x < 3) {
      const int h = round * 3 + threadIdx.x;
      float top = warp_max[0][h];
      for (int w = 1; w < kWarps; ++w) top = fmaxf(top, warp_max[w][h]);
      float den = 0.0f;
      for (int w = 0; w < kWarps; ++w)
        den += warp_sum[w][h] == 0.0f ? 0.0f : warp_sum[w][h] * ex2((warp_max[w][h] - top) * kLog2e);
      out[h * kPartialFloats + 0] = top;
      out[h * kPartialFloats + 1] = den;
    }
    __syncthreads();
  }
}

// Merges the per-split states of one query head, rounds to bf16, applies the sigmoid gate (when given) and
// rounds again.  One CTA per query head, one thread per dim.
__global__ void __launch_bounds__(kDim) gqa_decode_merge_kernel(const float* __restrict__ workspace, int splits,
                                                               const uint16_t* __restrict__ gate,
                                                               uint16_t* __restrict__ out) {
  const int head = blockIdx.x;
  const int kv = head / kGroup, h = head % kGroup;
  const int d = threadIdx.x;
  const int partials = splits;
  const float* base = workspace + (static_cast<size_t>(kv) * partials * kGroup + h) * kPartialFloats;
  const size_t step = static_cast<size_t>(kGroup) * kPartialFloats;
  float top = -INFINITY;
  for (int s = 0; s < partials; ++s) top = fmaxf(top, base[s * step]);
  float den = 0.0f, num = 0.0f;
  for (int s = 0; s < partials; ++s) {
    const float* p = base + s * step;
    const float w = p[1] == 0.0f ? 0.0f : ex2((p[0] - top) * kLog2e);  // an empty split left (-inf, 0, zeros)
    den = fmaf(p[1], w, den);
    num = fmaf(p[2 + d], w, num);
  }
  const float attention = __fdiv_rn(num, den);
  const uint16_t rounded = float_to_bf16(attention);
  uint16_t result = rounded;
  if (gate != nullptr)
    result = float_to_bf16(bf16_to_float(rounded) * stable_sigmoid(bf16_to_float(gate[head * kDim + d])));
  out[head * kDim + d] = result;
}

int plan_splits(size_t length) {
  // at least two batches per warp and split, at most one CTA per SM and KV head
  const size_t per_split_min = static_cast<size_t>(kWarps) * kBatch * 2;
  const size_t want = (length + per_split_min - 1) / per_split_min;
  return static_cast<int>(want < 1 ? 1 : (want > kMaxSplits ? kMaxSplits : want));
}

}  // namespace
}  // namespace q3x

using namespace q3x;
using namespace q3x::host;

extern "C" size_t q3x_b200_gqa_decode_workspace_floats(size_t sequence_length) {
  return static_cast<size_t>(plan_splits(sequence_length)) * kQHeads * kPartialFloats;
}

extern "C" int q3x_b200_gqa_attention_decode_sigmoid_gate(const uint16_t* query, const uint16_t* key_cache,
                                                          const uint16_t* value_cache, size_t sequence_length,
                                                          float attention_scale, float* workspace,
                                                          size_t workspace_floats, const uint16_t* gate,
                                                          uint16_t* out, void* stream) {
  if (!std::isfinite(attention_scale)) return kInvalid;
  if (sequence_length == 0 || mul_overflows(sequence_length, static_cast<size_t>(kKvHeads) * kDim * 2)) return kInvalid;
  if (query == nullptr || key_cache == nullptr || value_cache == nullptr || workspace == nullptr || out == nullptr)
    return kInvalid;
  const size_t need = q3x_b200_gqa_decode_workspace_floats(sequence_length);
  if (workspace_floats < need) return kInvalid;
  const size_t cache_bytes = sequence_length * kKvHeads * kDim * 2, head_bytes = static_cast<size_t>(kQHeads) * kDim * 2;
  const Span sq = span(query, head_bytes), sk = span(key_cache, cache_bytes), sv = span(value_cache, cache_bytes),
             sw = span(workspace, need * sizeof(float)), sg = span(gate, gate ? head_bytes : 0), so = span(out, head_bytes);
  if (wraps(sk) || wraps(sv) || wraps(sw)) return kInvalid;
  const Span readers[] = {sq, sk, sv, sg};
  for (const Span& r : readers)
    if (overlap(so, r) || overlap(sw, r)) return kInvalid;
  if (overlap(so, sw)) return kInvalid;
  if (!aligned16(query) || !aligned16(key_cache) || !aligned16(value_cache) || !aligned16(workspace)) return kNotSupported;
  const int splits = plan_splits(sequence_length);
  const size_t per_split = ((sequence_length + splits - 1) / splits + kBatch - 1) / kBatch * kBatch;
  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  gqa_decode_partial_kernel<<<dim3(splits, kKvHeads), kThreads, 0, s>>>(
      query, reinterpret_cast<const uint4*>(key_cache), reinterpret_cast<const uint4*>(value_cache), sequence_length,
      per_split, attention_scale, workspace);
  gqa_decode_merge_kernel<<<kQHeads, kDim, 0, s>>>(workspace, splits, gate, out);
  return launch_status();
}
