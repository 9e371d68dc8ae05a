// Causal depthwise conv1d (4 taps) + SiLU over the GDN projection [tokens, 10240], with the
// optional q/k L2 norm of its rounded output in the same pass.
//
// Layout of the work: a thread owns eight adjacent channels (one 128-bit vector per token row) and
// walks a run of consecutive tokens, keeping the three previous RAW rows in registers, so every
// input row is fetched once per run (plus a three-row halo at the start of a run) with fully
// coalesced 128-bit accesses.  A CTA is 128 threads = 1024 channels = 8 heads of 128, which makes
// the L2 norm of a head a 16-lane shuffle reduction with no shared memory.  grid = (channel
// blocks, token runs).
//
// The accumulation is the reference's fused chain, oldest tap first
// (src/runtime/reference/gdn_decode.cpp:163-175):
//   acc = fma(h0,w0,0); acc = fma(h1,w1,acc); acc = fma(h2,w2,acc); acc = fma(x,w3,acc)
// history [channels,3] holds RAW inputs, oldest first; the CTA of the first run reads it before any
// write and is also the one that publishes the new history, so the update is race-free in place.
#include <type_traits>

#include "device_utils.cuh"
#include "host_checks.hpp"
#include "norm_math.cuh"
#include "q3x_b200.h"

namespace q3x {
namespace {

constexpr int kThreads = 128;
constexpr int kBatch = 8;        // token rows staged per cp.async group
constexpr int kRunTokens = 64;   // aimed-at token run per CTA on the parallel path (halo overhead 3/64)

// Input rows reach the SM through cp.async into shared memory, two batches of kBatch rows deep: the
// next batch is in flight while the current one is computed, so a warp keeps 8 x 512 bytes of loads
// outstanding at all times.  A thread copies, reads and later overwrites only its own 16-byte slots,
// so the staging needs no barrier, only the per-thread cp.async wait.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* global_src) {
  const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(global_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
constexpr int kHeadVectors = Q3X_B200_GDN_HEAD_DIM / 8;                               // 16 lanes per head
constexpr int kQkVectors = 2 * Q3X_B200_GDN_QK_HEADS * Q3X_B200_GDN_HEAD_DIM / 8;     // 512: q then k

__device__ __forceinline__ uint32_t half_of(const uint4& v, int i) {
  const uint32_t w = i < 2 ? v.x : i < 4 ? v.y : i < 6 ? v.z : v.w;
  return (i & 1) ? (w >> 16) : (w & 0xffffu);
}

// history vectors (channel-major: element 3j + r = channel j, slot r) -> row r as a packed vector
__device__ __forceinline__ uint4 history_row(const uint4 (&h)[3], int r) {
  uint32_t e[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int idx = 3 * j + r;
    e[j] = half_of(h[idx / 8], idx % 8);
  }
  return make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
}

// How one launch cuts [channel blocks] x [token runs] into CTAs.  The channel blocks whose heads also
// get the L2 norm ("norm blocks": q and k, the first 512 channel vectors) cost about half as much again
// per token as the rest, so their CTAs come first in the grid: the hardware starts CTAs in index order,
// the long jobs are all under way before the short ones fill in behind them, and the launch ends
// without a tail of slow CTAs (measured 145 -> 130 us at 16384 tokens against a channel-major grid).
struct ConvPlan {
  unsigned norm_blocks, plain_blocks;  // channel blocks of either kind
  unsigned norm_ctas;                  // CTAs [0, norm_ctas) work on norm blocks
  size_t run_tokens;                   // tokens per CTA
};

// kInPlace: raw == out with a single token run; the last three raw rows are then kept as bits in
// registers because memory no longer holds them when the history is published.
// kCompact (with kL2): `out` receives the plain conv output for every channel, and the normalised q / k heads
// go to compact_q / compact_k instead, laid out [chunk of 64 tokens, qk head (16), token in chunk (64), 128]
// with the rows of the last chunk beyond `tokens` zeroed -- the operand layout of the reference's chunked
// GDN prefill (src/kernels/reference/gdn_prefill_whole_span_conv_sm87.cu:210-373).
constexpr int kCompactChunk = 64;
template <bool kL2, bool kInPlace, bool kCompact = false>
__global__ void __launch_bounds__(kThreads, kInPlace ? 1 : 4)
    causal_conv_kernel(const uint4* raw, size_t tokens, int channel_vectors, const uint4* __restrict__ weight,
                       uint4* history, uint4* out, ConvPlan plan, float l2_eps, float q_scale,
                       uint4* compact_q = nullptr, uint4* compact_k = nullptr) {
  release_next_kernel();
  wait_for_prior_kernels();
  // CTA index -> (channel block, token run); the blocks that carry the L2 norm come first
  unsigned channel_block, run;
  if (blockIdx.x < plan.norm_ctas) {
    channel_block = blockIdx.x % plan.norm_blocks;
    run = blockIdx.x / plan.norm_blocks;
  } else {
    const unsigned rest = blockIdx.x - plan.norm_ctas;
    channel_block = plan.norm_blocks + rest % plan.plain_blocks;
    run = rest / plan.plain_blocks;
  }
  const size_t run_tokens = plan.run_tokens;
  // channel vector: channels 8cv .. 8cv+7 (the launcher admits only widths that fill every CTA)
  const int cv = channel_block * kThreads + threadIdx.x;
  const size_t t0 = static_cast<size_t>(run) * run_tokens;
  const size_t t1 = min(tokens, t0 + run_tokens);

  float w[8][4];   // taps: weight[(8cv + j) * 4 + tap]: four vectors, vector k = channels 2k, 2k+1
  float win[3][8]; // the three rows before the current token (exact bf16 values), win[0] oldest
  uint4 keep[3];   // their bits (in-place path only)
#pragma unroll
  for (int r = 0; r < 3; ++r) keep[r] = make_uint4(0, 0, 0, 0);
  {
    uint4 rows[3];
#pragma unroll
    for (int r = 0; r < 3; ++r) rows[r] = make_uint4(0, 0, 0, 0);
    {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float f[8];
        unpack8(ld_weight(weight + static_cast<size_t>(cv) * 4 + k), f);
#pragma unroll
        for (int tap = 0; tap < 4; ++tap) {
          w[2 * k][tap] = f[tap];
          w[2 * k + 1][tap] = f[4 + tap];
        }
      }
      if (t0 == 0) {
        uint4 h[3];
#pragma unroll
        for (int k = 0; k < 3; ++k) h[k] = ld_vec(history + static_cast<size_t>(cv) * 3 + k);
#pragma unroll
        for (int r = 0; r < 3; ++r) rows[r] = history_row(h, r);
      } else {
#pragma unroll
        for (int r = 0; r < 3; ++r)  // t0 >= run_tokens >= kBatch > 3
          rows[r] = ld_vec(raw + (t0 - 3 + r) * channel_vectors + cv);
      }
    }
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      unpack8(rows[r], win[r]);
      if (kInPlace) keep[r] = rows[r];
    }
  }

  // uniform per CTA: 128 vectors per CTA divide the 256 of q and the 256 of k
  const bool is_qk = kL2 && cv < kQkVectors;
  const float head_scale = (kL2 && cv < kQkVectors / 2) ? q_scale : 1.0f;  // q heads carry the extra scale
  const size_t row_stride = static_cast<size_t>(channel_vectors);
  const uint4* raw_col = raw + cv;
  uint4* out_col = out + cv;

  __shared__ __align__(16) uint4 stage[2][kBatch][kThreads];
  auto issue_batch = [&](size_t first_token, int buffer) {
    const uint4* src = raw_col + first_token * row_stride;
    if (first_token + kBatch <= t1) {
#pragma unroll
      for (int u = 0; u < kBatch; ++u) cp_async16(&stage[buffer][u][threadIdx.x], src + u * row_stride);
    } else {
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
        if (first_token + u < t1) cp_async16(&stage[buffer][u][threadIdx.x], src + u * row_stride);
    }
    cp_async_commit();
  };
  // One token: the four-tap chain on rows h0 (oldest) .. h2 and x, SiLU, rounding, optional L2 norm
  // (kNorm is a compile-time copy of is_qk, so the token loop carries no branch for it).
  // compact layout: the lane's vector of head `cv / 16` (q heads first, then k heads) for token t
  uint4* const compact_base = kCompact ? (cv < kQkVectors / 2 ? compact_q : compact_k) : nullptr;
  const int compact_head = (cv % (kQkVectors / 2)) / kHeadVectors, compact_lane = cv % kHeadVectors;
  auto compact_slot = [&](size_t t) {
    return compact_base + ((t / kCompactChunk * Q3X_B200_GDN_QK_HEADS + compact_head) * kCompactChunk +
                           t % kCompactChunk) * kHeadVectors + compact_lane;
  };
  auto emit_token = [&](auto norm_tag, const float (&h0)[8], const float (&h1)[8], const float (&h2)[8],
                        const float (&x)[8], uint4* dst, size_t t) {
    constexpr bool kNorm = decltype(norm_tag)::value;
    float y[8];
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      float2 acc = fma2(make_float2(h0[j], h0[j + 1]), make_float2(w[j][0], w[j + 1][0]), make_float2(0.0f, 0.0f));
      acc = fma2(make_float2(h1[j], h1[j + 1]), make_float2(w[j][1], w[j + 1][1]), acc);
      acc = fma2(make_float2(h2[j], h2[j + 1]), make_float2(w[j][2], w[j + 1][2]), acc);
      acc = fma2(make_float2(x[j], x[j + 1]), make_float2(w[j][3], w[j + 1][3]), acc);
      const float2 s2 = silu2(acc);
      y[j] = s2.x;
      y[j + 1] = s2.y;
    }
    uint4 packed = pack8(y);
    if (kNorm && kCompact) st_vec(dst, packed);  // the conv output itself stays un-normalised in `out`
    if (kNorm) {
      // L2 norm of the ROUNDED conv output over the 128 channels of this head (16 lanes)
      float r[8];
      unpack8(packed, r);
      float partial = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) partial = fmaf(r[j], r[j], partial);
      const float sum = group_sum<kHeadVectors>(partial);
      const float inv = inverse_l2(sum, l2_eps) * head_scale;  // (* 1.0f is exact for the k heads)
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const float2 p = mul2(make_float2(r[j], r[j + 1]), make_float2(inv, inv));
        r[j] = p.x;
        r[j + 1] = p.y;
      }
      packed = pack8(r);
      if (kCompact) {
        st_vec(compact_slot(t), packed);
        return;
      }
    }
    st_vec(dst, packed);
  };

  auto run_tokens_loop = [&](auto norm_tag) {
    issue_batch(t0, 0);
    int buffer = 0;
    for (size_t t = t0; t < t1; t += kBatch, buffer ^= 1) {
      if (t + kBatch < t1) {
        issue_batch(t + kBatch, buffer ^ 1);
        cp_async_wait<1>();  // everything but the batch just issued has landed
      } else {
        cp_async_wait<0>();
      }
      uint4* dst = out_col + t * row_stride;
      if (t + kBatch <= t1) {
        // A full batch: rows[0..2] are the carried window, rows[3 + u] the batch's tokens.  Every index
        // is a compile-time constant, so the sliding window costs no register moves inside the batch.
        float rows[kBatch + 3][8];
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
          for (int j = 0; j < 8; ++j) rows[r][j] = win[r][j];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const uint4 x_bits = stage[buffer][u][threadIdx.x];
          unpack8(x_bits, rows[u + 3]);
          emit_token(norm_tag, rows[u], rows[u + 1], rows[u + 2], rows[u + 3], dst + u * row_stride, t + u);
          if (kInPlace && u >= kBatch - 3) keep[u - (kBatch - 3)] = x_bits;
        }
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
          for (int j = 0; j < 8; ++j) win[r][j] = rows[kBatch + r][j];
      } else {
        // the ragged last batch of the last run: one token at a time, shifting the window
        for (int u = 0; u < kBatch && t + u < t1; ++u) {
          const uint4 x_bits = stage[buffer][u][threadIdx.x];
          float x[8];
          unpack8(x_bits, x);
          emit_token(norm_tag, win[0], win[1], win[2], x, dst + u * row_stride, t + u);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            win[0][j] = win[1][j];
            win[1][j] = win[2][j];
            win[2][j] = x[j];
          }
          if (kInPlace) {
            keep[0] = keep[1];
            keep[1] = keep[2];
            keep[2] = x_bits;
          }
        }
      }
    }
  };
  if (is_qk) run_tokens_loop(std::true_type{});
  else run_tokens_loop(std::false_type{});
  if (kCompact && is_qk && t1 == tokens) {  // the run that ends the span zeroes the tail of the last chunk
    const size_t padded = (tokens + kCompactChunk - 1) / kCompactChunk * kCompactChunk;
    for (size_t t = tokens; t < padded; ++t) st_vec(compact_slot(t), make_uint4(0, 0, 0, 0));
  }

  // New history = the last three rows of (old history ++ raw), published by the first run's CTA.
  if (run == 0) {
    uint4 rows[3];
    if (kInPlace) {
#pragma unroll
      for (int r = 0; r < 3; ++r) rows[r] = keep[r];
    } else {
      uint4 h[3];
      if (tokens < 3) {
#pragma unroll
        for (int k = 0; k < 3; ++k) h[k] = ld_vec(history + static_cast<size_t>(cv) * 3 + k);
      }
#pragma unroll
      for (int r = 0; r < 3; ++r) {
        // row index in the concatenation, counted from the first raw row (negative = old history)
        const long long idx = static_cast<long long>(tokens) - 3 + r;
        if (idx >= 0) {
          rows[r] = ld_vec(raw + static_cast<size_t>(idx) * channel_vectors + cv);
        } else {
          rows[r] = idx == -1 ? history_row(h, 2) : idx == -2 ? history_row(h, 1) : history_row(h, 0);
        }
      }
    }
    uint32_t flat[24];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int r = 0; r < 3; ++r) flat[j * 3 + r] = half_of(rows[r], j);
#pragma unroll
    for (int k = 0; k < 3; ++k)
      st_vec(history + static_cast<size_t>(cv) * 3 + k,
             make_uint4(flat[k * 8 + 0] | (flat[k * 8 + 1] << 16), flat[k * 8 + 2] | (flat[k * 8 + 3] << 16),
                        flat[k * 8 + 4] | (flat[k * 8 + 5] << 16), flat[k * 8 + 6] | (flat[k * 8 + 7] << 16)));
  }
}

int launch_conv(const uint16_t* raw, size_t tokens, size_t channels, const uint16_t* weight, uint16_t* history,
                uint16_t* out, bool l2, float l2_eps, float q_scale, void* stream, uint16_t* compact_q = nullptr,
                uint16_t* compact_k = nullptr) {
  using namespace host;
  if (mul3_overflows(tokens, channels, sizeof(uint16_t))) return kInvalid;
  if (tokens == 0 || channels == 0) return kOk;
  if (raw == nullptr || weight == nullptr || history == nullptr || out == nullptr) return kInvalid;
  if (channels != Q3X_B200_GDN_CHANNELS) return kInvalid;  // the reference's only geometry
  static_assert(Q3X_B200_GDN_CHANNELS % (8 * kThreads) == 0, "every CTA must be filled with channel vectors");
  const size_t bytes = tokens * channels * sizeof(uint16_t);
  const Span sr = span(raw, bytes), so = span(out, bytes), sw = span(weight, channels * 4 * 2),
             sh = span(history, channels * 3 * 2);
  if (wraps(sr) || wraps(so)) return kInvalid;
  // exact raw == out is the one alias allowed (src/runtime/reference/gdn_decode.cpp:80-88)
  if (overlap(sr, sw) || overlap(sr, sh) || overlap(sw, sh) || overlap(sw, so) || overlap(sh, so) ||
      partial_overlap(sr, so))
    return kInvalid;
  if (l2 && raw == out) return kInvalid;
  const bool compact = compact_q != nullptr || compact_k != nullptr;
  if (compact) {
    if (!l2 || compact_q == nullptr || compact_k == nullptr) return kInvalid;
    const size_t chunks = (tokens + kCompactChunk - 1) / kCompactChunk;
    if (mul3_overflows(chunks, static_cast<size_t>(kCompactChunk) * Q3X_B200_GDN_QK_HEADS, Q3X_B200_GDN_HEAD_DIM * 2))
      return kInvalid;
    const size_t compact_bytes = chunks * kCompactChunk * Q3X_B200_GDN_QK_HEADS * Q3X_B200_GDN_HEAD_DIM * 2;
    const Span cq = span(compact_q, compact_bytes), ck = span(compact_k, compact_bytes);
    if (wraps(cq) || wraps(ck) || overlap(cq, ck)) return kInvalid;
    for (const Span& other : {sr, so, sw, sh})
      if (overlap(cq, other) || overlap(ck, other)) return kInvalid;
    if (!aligned16(compact_q) || !aligned16(compact_k)) return kNotSupported;
  }
  if (!aligned16(raw) || !aligned16(out) || !aligned16(weight) || !aligned16(history)) return kNotSupported;
  const int channel_vectors = static_cast<int>(channels / 8);
  const bool serial = raw == out;  // in place: one run, each thread reads a row before overwriting it
  const unsigned channel_blocks = static_cast<unsigned>((channel_vectors + kThreads - 1) / kThreads);
  ConvPlan plan{0, channel_blocks, 0, tokens};
  if (!serial) {
    // token runs sized so that the grid is a whole number of resident waves (no idle tail wave), about
    // kRunTokens long, in multiples of the staging batch
    const unsigned resident = compact ? resident_grid(causal_conv_kernel<true, false, true>, kThreads)
                              : l2    ? resident_grid(causal_conv_kernel<true, false>, kThreads)
                                      : resident_grid(causal_conv_kernel<false, false>, kThreads);
    if (l2) plan.norm_blocks = channel_blocks < kQkVectors / kThreads ? channel_blocks : kQkVectors / kThreads;
    plan.plain_blocks = channel_blocks - plan.norm_blocks;
    const size_t waves = tokens * channel_blocks / (static_cast<size_t>(resident) * kRunTokens) + 1;
    const size_t want_runs = (static_cast<size_t>(resident) * waves + channel_blocks - 1) / channel_blocks;
    size_t run = (tokens + want_runs - 1) / want_runs;
    run = (run + kBatch - 1) / kBatch * kBatch;
    plan.run_tokens = run < static_cast<size_t>(kBatch) ? static_cast<size_t>(kBatch) : run;
  }
  const size_t runs = (tokens + plan.run_tokens - 1) / plan.run_tokens;
  if (runs * channel_blocks > 0x7fffffffu) return kNotSupported;
  plan.norm_ctas = static_cast<unsigned>(runs * plan.norm_blocks);
  const dim3 grid(static_cast<unsigned>(runs * channel_blocks));
  clear_stale_error();
  auto R = reinterpret_cast<const uint4*>(raw);
  auto W = reinterpret_cast<const uint4*>(weight);
  auto H = reinterpret_cast<uint4*>(history);
  auto O = reinterpret_cast<uint4*>(out);
  cudaStream_t s = as_stream(stream);
  auto kernel = compact ? causal_conv_kernel<true, false, true>
                : l2    ? causal_conv_kernel<true, false>
                : serial ? causal_conv_kernel<false, true>
                         : causal_conv_kernel<false, false>;
  launch_kernel(kernel, grid, kThreads, 0, s, latency_bound_launch(grid.x), R, tokens, channel_vectors, W, H, O, plan,
                l2 ? l2_eps : 0.0f, l2 ? q_scale : 1.0f, reinterpret_cast<uint4*>(compact_q),
                reinterpret_cast<uint4*>(compact_k));
  return launch_status();
}

}  // namespace
}  // namespace q3x

extern "C" int q3x_b200_causal_conv1d_silu(const uint16_t* raw, size_t tokens, size_t channels,
                                           const uint16_t* conv_weight, uint16_t* history_in_out, uint16_t* out,
                                           void* stream) {
  return q3x::launch_conv(raw, tokens, channels, conv_weight, history_in_out, out, false, 0.0f, 1.0f, stream);
}

extern "C" int q3x_b200_causal_conv1d_silu_l2norm(const uint16_t* raw, size_t tokens, const uint16_t* conv_weight,
                                                  uint16_t* history_in_out, float l2_eps, float q_scale,
                                                  uint16_t* out, void* stream) {
  if (!q3x::host::valid_epsilon(l2_eps) || !std::isfinite(q_scale)) return q3x::host::kInvalid;
  return q3x::launch_conv(raw, tokens, Q3X_B200_GDN_CHANNELS, conv_weight, history_in_out, out, true, l2_eps,
                          q_scale, stream);
}

extern "C" int q3x_b200_causal_conv1d_silu_compact_qk(const uint16_t* raw, size_t tokens, const uint16_t* conv_weight,
                                                      uint16_t* history_in_out, uint16_t* out, float l2_eps,
                                                      float q_scale, uint16_t* compact_q, uint16_t* compact_k,
                                                      void* stream) {
  if (!q3x::host::valid_epsilon(l2_eps) || !std::isfinite(q_scale)) return q3x::host::kInvalid;
  if (tokens != 0 && (compact_q == nullptr || compact_k == nullptr)) return q3x::host::kInvalid;
  return q3x::launch_conv(raw, tokens, Q3X_B200_GDN_CHANNELS, conv_weight, history_in_out, out, true, l2_eps, q_scale,
                          stream, compact_q, compact_k);
}
