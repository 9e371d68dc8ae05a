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
#include "device_utils.cuh"
#include "host_checks.hpp"
#include "q3x_b200.h"

namespace q3x {
namespace {

constexpr int kThreads = 128;
constexpr int kTokenUnroll = 4;
constexpr int kRunTokens = 32;  // tokens per CTA on the parallel path (multiple of kTokenUnroll)
constexpr int kHeadVectors = Q3X_B200_GDN_HEAD_DIM / 8;                               // 16 lanes per head
constexpr int kQkVectors = 2 * Q3X_B200_GDN_QK_HEADS * Q3X_B200_GDN_HEAD_DIM / 8;     // 512: q then k

__device__ __forceinline__ uint16_t half_of(const uint4& v, int i) {
  const uint32_t w = i < 2 ? v.x : i < 4 ? v.y : i < 6 ? v.z : v.w;
  return static_cast<uint16_t>((i & 1) ? (w >> 16) : (w & 0xffffu));
}

template <bool kL2>
__global__ void __launch_bounds__(kThreads) causal_conv_kernel(const uint4* raw, size_t tokens, int channel_vectors,
                                                               const uint4* __restrict__ weight, uint4* history,
                                                               uint4* out, size_t run_tokens, float l2_eps,
                                                               float q_scale) {
  const int cv = blockIdx.x * kThreads + threadIdx.x;  // channel vector: channels 8cv .. 8cv+7
  const bool active = cv < channel_vectors;
  const size_t t0 = static_cast<size_t>(blockIdx.y) * run_tokens;
  const size_t t1 = min(tokens, t0 + run_tokens);

  // taps: weight[(8cv + j) * 4 + tap]  ->  four vectors, vector k = channels 2k and 2k+1
  float w[8][4];
  // the three rows before t0, per channel, as floats (exact bf16 values): win[r][j], r = 0 oldest
  float win[3][8];
  uint4 win_bits[3];
#pragma unroll
  for (int r = 0; r < 3; ++r) win_bits[r] = make_uint4(0, 0, 0, 0);
  if (active) {
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
      // history[(8cv + j) * 3 + r]: 24 bf16 = three vectors, channel-major -> transpose to rows
      uint4 h[3];
#pragma unroll
      for (int k = 0; k < 3; ++k) h[k] = ld_vec(history + static_cast<size_t>(cv) * 3 + k);
      uint16_t rows[3][8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int r = 0; r < 3; ++r) {
          const int e = j * 3 + r;
          rows[r][j] = half_of(h[e / 8], e % 8);
        }
#pragma unroll
      for (int r = 0; r < 3; ++r) {
        win_bits[r].x = rows[r][0] | (static_cast<uint32_t>(rows[r][1]) << 16);
        win_bits[r].y = rows[r][2] | (static_cast<uint32_t>(rows[r][3]) << 16);
        win_bits[r].z = rows[r][4] | (static_cast<uint32_t>(rows[r][5]) << 16);
        win_bits[r].w = rows[r][6] | (static_cast<uint32_t>(rows[r][7]) << 16);
      }
    } else {
#pragma unroll
      for (int r = 0; r < 3; ++r)  // t0 >= run_tokens >= 3
        win_bits[r] = ld_vec(raw + (t0 - 3 + r) * channel_vectors + cv);
    }
  }
#pragma unroll
  for (int r = 0; r < 3; ++r) unpack8(win_bits[r], win[r]);

  const bool is_q = kL2 && cv < kQkVectors / 2;
  const bool is_qk = kL2 && cv < kQkVectors;  // uniform per CTA: 128 vectors per CTA divide 256

  for (size_t t = t0; t < t1; t += kTokenUnroll) {
    uint4 x_bits[kTokenUnroll];
#pragma unroll
    for (int u = 0; u < kTokenUnroll; ++u) {
      x_bits[u] = make_uint4(0, 0, 0, 0);
      if (active && t + u < t1) x_bits[u] = ld_vec(raw + (t + u) * channel_vectors + cv);
    }
#pragma unroll
    for (int u = 0; u < kTokenUnroll; ++u) {
      if (t + u >= t1) break;  // uniform across the CTA
      float x[8], y[8];
      unpack8(x_bits[u], x);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float acc = fmaf(win[0][j], w[j][0], 0.0f);
        acc = fmaf(win[1][j], w[j][1], acc);
        acc = fmaf(win[2][j], w[j][2], acc);
        acc = fmaf(x[j], w[j][3], acc);
        y[j] = silu(acc);
        win[0][j] = win[1][j];
        win[1][j] = win[2][j];
        win[2][j] = x[j];
      }
      win_bits[0] = win_bits[1];
      win_bits[1] = win_bits[2];
      win_bits[2] = x_bits[u];
      uint4 packed = pack8(y);
      if (is_qk) {
        // L2 norm of the ROUNDED conv output over the 128 channels of this head (16 lanes)
        float r[8];
        unpack8(packed, r);
        float partial = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) partial = fmaf(r[j], r[j], partial);
        const float sum = group_sum<kHeadVectors>(partial);
        float inv = 1.0f / sqrtf(__fadd_rn(sum, l2_eps));
        if (is_q && q_scale != 1.0f) inv = inv * q_scale;
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = r[j] * inv;
        packed = pack8(r);
      }
      if (active) st_vec(out + (t + u) * channel_vectors + cv, packed);
    }
  }

  // new history = the last three raw rows of (old history ++ raw); published by the first run's CTA
  if (blockIdx.y == 0 && active) {
    if (gridDim.y > 1) {  // tokens > run_tokens >= 3: the rows come straight from raw
#pragma unroll
      for (int r = 0; r < 3; ++r) win_bits[r] = ld_vec(raw + (tokens - 3 + r) * channel_vectors + cv);
    }  // else the register window already is that sequence (also when tokens < 3)
    uint16_t flat[24];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int r = 0; r < 3; ++r) flat[j * 3 + r] = half_of(win_bits[r], j);
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      uint4 v;
      v.x = flat[k * 8 + 0] | (static_cast<uint32_t>(flat[k * 8 + 1]) << 16);
      v.y = flat[k * 8 + 2] | (static_cast<uint32_t>(flat[k * 8 + 3]) << 16);
      v.z = flat[k * 8 + 4] | (static_cast<uint32_t>(flat[k * 8 + 5]) << 16);
      v.w = flat[k * 8 + 6] | (static_cast<uint32_t>(flat[k * 8 + 7]) << 16);
      st_vec(history + static_cast<size_t>(cv) * 3 + k, v);
    }
  }
}

int launch_conv(const uint16_t* raw, size_t tokens, size_t channels, const uint16_t* weight, uint16_t* history,
                uint16_t* out, bool l2, float l2_eps, float q_scale, void* stream) {
  using namespace host;
  if (mul3_overflows(tokens, channels, sizeof(uint16_t))) return kInvalid;
  if (tokens == 0 || channels == 0) return kOk;
  if (raw == nullptr || weight == nullptr || history == nullptr || out == nullptr) return kInvalid;
  if (channels != Q3X_B200_GDN_CHANNELS) return kInvalid;  // the reference's only geometry
  const size_t bytes = tokens * channels * sizeof(uint16_t);
  const Span sr = span(raw, bytes), so = span(out, bytes), sw = span(weight, channels * 4 * 2),
             sh = span(history, channels * 3 * 2);
  if (wraps(sr) || wraps(so)) return kInvalid;
  // exact raw == out is the one alias allowed (src/runtime/reference/gdn_decode.cpp:80-88)
  if (overlap(sr, sw) || overlap(sr, sh) || overlap(sw, sh) || overlap(sw, so) || overlap(sh, so) ||
      partial_overlap(sr, so))
    return kInvalid;
  if (l2 && raw == out) return kInvalid;
  if (!aligned16(raw) || !aligned16(out) || !aligned16(weight) || !aligned16(history)) return kNotSupported;
  const int channel_vectors = static_cast<int>(channels / 8);
  const bool serial = raw == out;  // in place: one run, each thread reads a row before overwriting it
  const size_t run = serial ? tokens : static_cast<size_t>(kRunTokens);
  const size_t runs = (tokens + run - 1) / run;
  if (runs > 65535u) {
    // grid.y limit: longer spans are cut into launches that hand the history over in order
    const size_t span_tokens = static_cast<size_t>(65535u) * run;
    for (size_t first = 0; first < tokens; first += span_tokens) {
      const size_t n = tokens - first < span_tokens ? tokens - first : span_tokens;
      const int st = launch_conv(raw + first * channels, n, channels, weight, history, out + first * channels, l2,
                                 l2_eps, q_scale, stream);
      if (st != kOk) return st;
    }
    return kOk;
  }
  const dim3 grid((channel_vectors + kThreads - 1) / kThreads, static_cast<unsigned>(runs));
  clear_stale_error();
  auto R = reinterpret_cast<const uint4*>(raw);
  auto W = reinterpret_cast<const uint4*>(weight);
  auto H = reinterpret_cast<uint4*>(history);
  auto O = reinterpret_cast<uint4*>(out);
  if (l2)
    causal_conv_kernel<true><<<grid, kThreads, 0, as_stream(stream)>>>(R, tokens, channel_vectors, W, H, O, run,
                                                                      l2_eps, q_scale);
  else
    causal_conv_kernel<false><<<grid, kThreads, 0, as_stream(stream)>>>(R, tokens, channel_vectors, W, H, O, run,
                                                                       0.0f, 1.0f);
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
