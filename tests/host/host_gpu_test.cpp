// Drives the C++ mirror of the reference operator API (libq3x_b200_host.so) ON A GPU: one launcher of
// every family is called through its q3x::runtime name with real device buffers, and its output bytes
// are compared with the same operation requested straight from the C ABI (libq3x_b200.so), whose
// parity with the CPU oracle the Python tests establish.  A wrong argument order or a dropped argument
// in the mirror's forwarding code shows up here as a byte mismatch.
//
// Plain executable in the style of the reference's own tests: prints failures, returns their count;
// exit code 77 = no sm_100 device (skipped).
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "q3x_b200.h"
#include "q3x_b200_nvfp4.hpp"
#include "q3x_b200_ops.hpp"

namespace rt = q3x::runtime;

static int failures = 0;
#define EXPECT(cond)                                              \
  do {                                                            \
    if (!(cond)) {                                                \
      ++failures;                                                 \
      std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond); \
    }                                                             \
  } while (0)
#define CUDA_OK(call) EXPECT((call) == cudaSuccess)

// deterministic pseudo-random bf16 bits: N(0,1)-like magnitudes, both signs, no specials
static std::uint16_t bf16_of(float v) {
  std::uint32_t u;
  std::memcpy(&u, &v, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<std::uint16_t>(u >> 16);
}
static std::uint32_t lcg_state = 12345u;
static float uniform() {
  lcg_state = lcg_state * 1664525u + 1013904223u;
  return static_cast<float>(lcg_state >> 8) / 16777216.0f;
}
static std::vector<std::uint16_t> random_bf16(std::size_t n, float scale) {
  std::vector<std::uint16_t> v(n);
  for (auto& x : v) x = bf16_of((uniform() + uniform() + uniform() - 1.5f) * 2.0f * scale);
  return v;
}

template <typename T>
struct DeviceBuffer {
  T* p = nullptr;
  std::size_t n = 0;
  explicit DeviceBuffer(std::size_t count, int fill = 0x5a) : n(count) {
    CUDA_OK(cudaMalloc(&p, count * sizeof(T)));
    CUDA_OK(cudaMemset(p, fill, count * sizeof(T)));
  }
  explicit DeviceBuffer(const std::vector<T>& host) : n(host.size()) {
    CUDA_OK(cudaMalloc(&p, n * sizeof(T)));
    CUDA_OK(cudaMemcpy(p, host.data(), n * sizeof(T), cudaMemcpyHostToDevice));
  }
  ~DeviceBuffer() { cudaFree(p); }
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;
  std::vector<T> get() const {
    std::vector<T> h(n);
    CUDA_OK(cudaMemcpy(h.data(), p, n * sizeof(T), cudaMemcpyDeviceToHost));
    return h;
  }
};
using Bf16 = DeviceBuffer<std::uint16_t>;

template <typename T>
static bool same(const DeviceBuffer<T>& a, const DeviceBuffer<T>& b) {
  CUDA_OK(cudaDeviceSynchronize());
  const auto x = a.get(), y = b.get();
  return x.size() == y.size() && std::memcmp(x.data(), y.data(), x.size() * sizeof(T)) == 0;
}
// not everything still the fill pattern: the launcher really wrote
template <typename T>
static bool written(const DeviceBuffer<T>& a) {
  const auto x = a.get();
  std::size_t untouched = 0;
  for (const T& v : x) {
    T fill;
    std::memset(&fill, 0x5a, sizeof(T));
    untouched += std::memcmp(&v, &fill, sizeof(T)) == 0 ? 1 : 0;
  }
  return untouched * 10 < x.size();
}

static void test_pointwise_and_embedding(cudaStream_t s) {
  const std::size_t n = 3 * 17408 + 5;  // not a multiple of eight: vector body and scalar tail
  Bf16 gate(random_bf16(n, 2.0f)), up(random_bf16(n, 1.0f)), a(n), b(n);
  EXPECT(rt::launch_silu_mul_reference_cuda(gate.p, up.p, n, a.p, s) == 0);
  EXPECT(q3x_b200_silu_mul(gate.p, up.p, n, b.p, s) == 0);
  EXPECT(same(a, b) && written(a));
  EXPECT(rt::launch_sigmoid_gate_reference_cuda(up.p, gate.p, n, a.p, s) == 0);
  EXPECT(q3x_b200_sigmoid_gate(up.p, gate.p, n, b.p, s) == 0);
  EXPECT(same(a, b));
  EXPECT(rt::launch_residual_add_reference_cuda(gate.p, up.p, n, a.p, s) == 0);
  EXPECT(q3x_b200_residual_add(gate.p, up.p, n, b.p, s) == 0);
  EXPECT(same(a, b));

  const std::size_t vocab = 300, hidden = 5120, tokens = 37;
  Bf16 table(random_bf16(vocab * hidden, 0.02f));
  std::vector<std::uint32_t> ids(tokens);
  for (std::size_t t = 0; t < tokens; ++t) ids[t] = static_cast<std::uint32_t>((t * 97u + 11u) % vocab);
  DeviceBuffer<std::uint32_t> d_ids(ids);
  Bf16 e1(tokens * hidden), e2(tokens * hidden);
  EXPECT(rt::launch_embedding_gather_prompt_reference_cuda(table.p, vocab, hidden, d_ids.p, tokens, e1.p, s) == 0);
  EXPECT(q3x_b200_embedding_gather(table.p, vocab, hidden, d_ids.p, tokens, e2.p, s) == 0);
  EXPECT(same(e1, e2) && written(e1));
  // by-value form: one row, against the table itself
  Bf16 one(hidden);
  EXPECT(rt::launch_embedding_gather_reference_cuda(table.p, vocab, hidden, 123, one.p, s) == 0);
  CUDA_OK(cudaDeviceSynchronize());
  const auto row = one.get(), tab = table.get();
  EXPECT(std::memcmp(row.data(), tab.data() + 123 * hidden, hidden * 2) == 0);

  std::vector<float> f(4099);
  for (auto& x : f) x = (uniform() - 0.5f) * 100.0f;
  DeviceBuffer<float> d_f(f);
  Bf16 c1(f.size()), c2(f.size());
  EXPECT(rt::launch_fp32_to_bf16_reference_cuda(d_f.p, f.size(), c1.p, s) == 0);
  EXPECT(q3x_b200_fp32_to_bf16(d_f.p, f.size(), c2.p, s) == 0);
  EXPECT(same(c1, c2) && written(c1));
}

static void test_norms(cudaStream_t s) {
  const float eps = 1e-6f;
  const std::size_t tokens = 77, hidden = 5120;
  Bf16 left(random_bf16(tokens * hidden, 1.0f)), right(random_bf16(tokens * hidden, 1.0f)),
      w(random_bf16(hidden, 0.02f));
  Bf16 r1(tokens * hidden), n1(tokens * hidden), r2(tokens * hidden), n2(tokens * hidden);
  EXPECT(rt::launch_residual_add_headwise_centered_rms_norm_prefill_5120_cuda(left.p, right.p, w.p, tokens, hidden, eps,
                                                                            r1.p, n1.p, s) == 0);
  EXPECT(q3x_b200_residual_add_rms_norm(left.p, right.p, w.p, tokens, hidden, eps, r2.p, n2.p, s) == 0);
  EXPECT(same(r1, r2) && same(n1, n2) && written(n1));
  // decode form: one token, weight and epsilon in their own positions
  Bf16 r3(hidden), n3(hidden), r4(hidden), n4(hidden);
  EXPECT(rt::launch_residual_add_centered_rms_norm_5120_cuda(left.p, right.p, w.p, eps, r3.p, n3.p, s) == 0);
  EXPECT(q3x_b200_residual_add_rms_norm(left.p, right.p, w.p, 1, hidden, eps, r4.p, n4.p, s) == 0);
  EXPECT(same(r3, r4) && same(n3, n4));
  // M32 form
  Bf16 r5(32 * hidden), n5(32 * hidden), r6(32 * hidden), n6(32 * hidden);
  EXPECT(rt::launch_residual_add_headwise_centered_rms_norm_m32_5120_cuda(left.p, right.p, w.p, 32, hidden, eps, r5.p,
                                                                        n5.p, s) == 0);
  EXPECT(q3x_b200_residual_add_rms_norm(left.p, right.p, w.p, 32, hidden, eps, r6.p, n6.p, s) == 0);
  EXPECT(same(r5, r6) && same(n5, n6));

  // single-row and head-wise norms, centred and plain; gated; L2
  Bf16 o1(tokens * hidden), o2(tokens * hidden);
  EXPECT(rt::launch_centered_rms_norm_reference_cuda(left.p, w.p, hidden, eps, o1.p, s) == 0);
  EXPECT(q3x_b200_rms_norm(left.p, w.p, 1, hidden, eps, 1, o2.p, s) == 0);
  EXPECT(same(o1, o2));
  EXPECT(rt::launch_plain_rms_norm_reference_cuda(left.p, w.p, hidden, eps, o1.p, s) == 0);
  EXPECT(q3x_b200_rms_norm(left.p, w.p, 1, hidden, eps, 0, o2.p, s) == 0);
  EXPECT(same(o1, o2));
  const std::size_t heads = 24 * 9, dim = 256;
  Bf16 hw(random_bf16(dim, 0.02f));
  EXPECT(rt::launch_headwise_centered_rms_norm_reference_cuda(left.p, hw.p, heads, dim, eps, o1.p, s) == 0);
  EXPECT(q3x_b200_rms_norm(left.p, hw.p, heads, dim, eps, 1, o2.p, s) == 0);
  EXPECT(same(o1, o2));
  EXPECT(rt::launch_headwise_plain_rms_norm_reference_cuda(left.p, hw.p, 48 * 5, 128, eps, o1.p, s) == 0);
  EXPECT(q3x_b200_rms_norm(left.p, hw.p, 48 * 5, 128, eps, 0, o2.p, s) == 0);
  EXPECT(same(o1, o2));
  EXPECT(rt::launch_headwise_plain_rms_norm_silu_gate_reference_cuda(left.p, hw.p, right.p, 48 * 5, 128, eps, o1.p,
                                                                     s) == 0);
  EXPECT(q3x_b200_rms_norm_silu_gate(left.p, hw.p, right.p, 48 * 5, 128, eps, o2.p, s) == 0);
  EXPECT(same(o1, o2));
  EXPECT(rt::launch_l2_normalize_heads_reference_cuda(left.p, 16 * 7, 128, eps, o1.p, s) == 0);
  EXPECT(q3x_b200_l2_normalize_heads(left.p, 16 * 7, 128, eps, 1.0f, o2.p, s) == 0);
  EXPECT(same(o1, o2));
}

static void test_full_attention(cudaStream_t s) {
  const float eps = 1e-6f;
  const std::size_t tokens = 19, first = 40, positions = first + tokens;
  std::vector<float> cosv(positions * 32), sinv(positions * 32);
  for (std::size_t p = 0; p < positions; ++p)
    for (std::size_t i = 0; i < 32; ++i) {
      const float angle = static_cast<float>(p) / std::pow(1.0e7f, 2.0f * static_cast<float>(i) / 64.0f);
      cosv[p * 32 + i] = std::cos(angle);
      sinv[p * 32 + i] = std::sin(angle);
    }
  DeviceBuffer<float> cosd(cosv), sind(sinv);
  const auto qg_host = random_bf16(tokens * 24 * 2 * 256, 1.0f);
  const auto key_host = random_bf16(tokens * 4 * 256, 1.0f);
  Bf16 qg(qg_host), k1(key_host), k2(key_host), qw(random_bf16(256, 0.02f)), kw(random_bf16(256, 0.02f));
  Bf16 q1(tokens * 24 * 256), g1(tokens * 24 * 256), q2(tokens * 24 * 256), g2(tokens * 24 * 256);
  EXPECT(rt::launch_full_attention_preprocess_24_4_256_64_cuda(qg.p, k1.p, qw.p, kw.p, eps, q1.p, g1.p, cosd.p, sind.p,
                                                               first, tokens, s) == 0);
  EXPECT(q3x_b200_full_attention_preprocess(qg.p, k2.p, qw.p, kw.p, eps, q2.p, g2.p, cosd.p, sind.p, first, tokens,
                                            s) == 0);
  EXPECT(same(q1, q2) && same(g1, g2) && same(k1, k2) && written(q1));
  // the split and the stand-alone rotations
  Bf16 sq1(tokens * 24 * 256), sg1(tokens * 24 * 256), sq2(tokens * 24 * 256), sg2(tokens * 24 * 256);
  EXPECT(rt::launch_split_interleaved_q_gate_reference_cuda(qg.p, tokens * 24, 256, sq1.p, sg1.p, s) == 0);
  EXPECT(q3x_b200_split_interleaved_q_gate(qg.p, tokens * 24, 256, sq2.p, sg2.p, s) == 0);
  EXPECT(same(sq1, sq2) && same(sg1, sg2) && same(sg1, g1));
  Bf16 k3(key_host), k4(key_host);
  const std::size_t tile = 16;
  EXPECT(rt::launch_qk_partial_neox_rope_tile_24_4_256_64_cuda(sq1.p, k3.p, cosd.p, sind.p, first, tile, s) == 0);
  EXPECT(q3x_b200_qk_partial_neox_rope(sq2.p, k4.p, cosd.p, sind.p, first, tile, s) == 0);
  EXPECT(same(sq1, sq2) && same(k3, k4));
  Bf16 ro1(24 * 256), ro2(24 * 256);
  EXPECT(rt::launch_partial_neox_rope_256_64_reference_cuda(sg1.p, cosd.p + 32 * first, sind.p + 32 * first, 24, ro1.p,
                                                            s) == 0);
  EXPECT(q3x_b200_partial_neox_rope_256_64(sg1.p, cosd.p + 32 * first, sind.p + 32 * first, 24, ro2.p, s) == 0);
  EXPECT(same(ro1, ro2) && written(ro1));
}

static void test_conv(cudaStream_t s) {
  const std::size_t channels = 10240;
  const auto raw_host = random_bf16(16 * channels, 1.0f);
  const auto hist_host = random_bf16(channels * 3, 1.0f);
  Bf16 raw(raw_host), w(random_bf16(channels * 4, 0.5f));
  for (std::size_t tokens : {std::size_t{1}, std::size_t{7}, std::size_t{16}}) {
    Bf16 h1(hist_host), h2(hist_host), o1(tokens * channels), o2(tokens * channels);
    if (tokens == 1)
      EXPECT(rt::launch_causal_conv1d_silu_update_reference_cuda(raw.p, w.p, h1.p, o1.p, rt::GdnDimensions{}, s) == 0);
    else
      EXPECT(rt::launch_causal_conv1d_silu_update_tile_reference_cuda(raw.p, tokens, w.p, h1.p, o1.p,
                                                                      rt::GdnDimensions{}, s) == 0);
    EXPECT(q3x_b200_causal_conv1d_silu(raw.p, tokens, channels, w.p, h2.p, o2.p, s) == 0);
    EXPECT(same(o1, o2) && same(h1, h2) && written(o1));
  }
  namespace conv = rt::gdn_prefill_whole_span_conv_detail;
  Bf16 h1(hist_host), h2(hist_host), h3(hist_host), o1(16 * channels), o2(16 * channels), o3(16 * channels);
  EXPECT(conv::launch_causal_conv1d_silu_update_whole_span_exact_cuda(raw.p, 16, w.p, h1.p, o1.p, s) == 0);
  EXPECT(conv::launch_causal_conv1d_silu_update_token_parallel_exact_cuda(raw.p, 16, w.p, h2.p, o2.p, s) == 0);
  EXPECT(q3x_b200_causal_conv1d_silu(raw.p, 16, channels, w.p, h3.p, o3.p, s) == 0);
  EXPECT(same(o1, o3) && same(o2, o3) && same(h1, h3) && same(h2, h3));
}

static void test_dispatch_halves(cudaStream_t s) {
  const float eps = 1e-6f;
  const std::size_t tokens = 9, hidden = 5120, inter = 17408;
  const auto gate_host = random_bf16(tokens * inter, 1.5f);
  Bf16 g1(gate_host), g2(gate_host), up(random_bf16(tokens * inter, 1.0f));
  EXPECT(rt::launch_mlp_gate_up_silu_epilogue_cuda(rt::ProjectionBackend::kB200LayerOps, g1.p, up.p, tokens, inter,
                                                   s) == 0);
  EXPECT(q3x_b200_silu_mul(g2.p, up.p, tokens * inter, g2.p, s) == 0);
  EXPECT(same(g1, g2));
  EXPECT(rt::launch_mlp_gate_up_silu_epilogue_cuda(rt::ProjectionBackend::kReference, g1.p, up.p, tokens, inter, s) ==
         static_cast<int>(cudaErrorNotSupported));
  const auto right_host = random_bf16(tokens * hidden, 1.0f);
  Bf16 left(random_bf16(tokens * hidden, 1.0f)), w(random_bf16(hidden, 0.02f)), ra(right_host), rb(right_host);
  Bf16 res1(tokens * hidden), res2(tokens * hidden);
  EXPECT(rt::launch_post_attention_residual_norm_prologue_cuda(rt::ProjectionBackend::kB200LayerOps, left.p, ra.p, w.p,
                                                               eps, tokens, hidden, res1.p, s) == 0);
  EXPECT(q3x_b200_residual_add_rms_norm(left.p, rb.p, w.p, tokens, hidden, eps, res2.p, rb.p, s) == 0);
  EXPECT(same(res1, res2) && same(ra, rb));
  Bf16 n1(tokens * hidden), n2(tokens * hidden);
  EXPECT(rt::launch_mlp_down_residual_norm_epilogue_cuda(rt::ProjectionBackend::kB200LayerOps, ra.p, left.p, w.p, eps,
                                                         tokens, hidden, res1.p, n1.p, s) == 0);
  EXPECT(q3x_b200_residual_add_rms_norm(left.p, ra.p, w.p, tokens, hidden, eps, res2.p, n2.p, s) == 0);
  EXPECT(same(res1, res2) && same(n1, n2));
}

// The projection composites with real weights: outputs must equal the GEMV + fused-operator sequence requested
// from the C ABI, for the three weight kinds.
static std::vector<std::uint8_t> random_bytes(std::size_t n, std::uint8_t lo, std::uint8_t hi) {
  std::vector<std::uint8_t> v(n);
  for (auto& x : v) x = static_cast<std::uint8_t>(lo + static_cast<unsigned>(uniform() * (hi - lo)));
  return v;
}

static void test_composites(cudaStream_t s) {
  const float eps = 1e-6f;
  const std::size_t hidden = 5120, inter = 1024;  // a narrow MLP keeps the test quick; hidden is the model's
  DeviceBuffer<float> dev_scalar(std::vector<float>{0.01f});
  // NVFP4 gate / up [inter, hidden], bf16 down [hidden, inter]
  DeviceBuffer<std::uint8_t> gate_w(random_bytes(inter * hidden / 2, 0, 255)), up_w(random_bytes(inter * hidden / 2, 0, 255));
  DeviceBuffer<std::uint8_t> gate_s(random_bytes(inter * hidden / 16, 0x20, 0x48)), up_s(random_bytes(inter * hidden / 16, 0x20, 0x48));
  rt::NvFp4LinearWeight gate{}, up{};
  gate.packed_weight = gate_w.p; gate.block_scale = gate_s.p; gate.weight_scale_2_device = dev_scalar.p;
  gate.input_scale_device = dev_scalar.p; gate.weight_scale_2 = 0.01f; gate.input_scale = 1.0f;
  gate.output_size = inter; gate.input_size = hidden;
  up = gate; up.packed_weight = up_w.p; up.block_scale = up_s.p;
  const rt::LinearWeight gate_lw = gate, up_lw = up;
  Bf16 left(random_bf16(hidden, 1.0f)), w(random_bf16(hidden, 0.02f));
  const auto right_host = random_bf16(hidden, 1.0f);
  Bf16 ra(right_host), rb(right_host), res1(hidden), res2(hidden);
  Bf16 g1(inter), u1(inter), g2(inter), u2(inter);
  EXPECT(rt::launch_post_attention_residual_norm_mlp_gate_up_silu_to_bf16_cuda(
             rt::ProjectionBackend::kSm87WeightOnly, gate_lw, up_lw, left.p, ra.p, w.p, eps, nullptr, 0, res1.p, g1.p, u1.p,
             s) == 0);
  EXPECT(q3x_b200_residual_add_rms_norm(left.p, rb.p, w.p, 1, hidden, eps, res2.p, rb.p, s) == 0);
  EXPECT(q3x_b200_nvfp4_gemv(gate_w.p, gate_s.p, 0.01f, rb.p, inter, hidden, nullptr, g2.p, s) == 0);
  EXPECT(q3x_b200_nvfp4_gemv(up_w.p, up_s.p, 0.01f, rb.p, inter, hidden, nullptr, u2.p, s) == 0);
  EXPECT(q3x_b200_silu_mul(g2.p, u2.p, inter, g2.p, s) == 0);
  EXPECT(same(res1, res2) && same(ra, rb) && same(g1, g2) && same(u1, u2) && written(g1));
  // the decode-runner twin and the plain gate / up composite give the same gate output
  Bf16 rc(right_host), res3(hidden), g3(inter), u3(inter), g4(inter), u4(inter);
  EXPECT(rt::launch_decode_runner_post_attention_residual_norm_mlp_gate_up_silu_dead_up_to_bf16_cuda(
             rt::kProjectionBackendB200LayerOps, gate_lw, up_lw, left.p, rc.p, w.p, eps, nullptr, 0, res3.p, g3.p, u3.p, s) == 0);
  EXPECT(rt::launch_mlp_gate_up_silu_to_bf16_cuda(rt::ProjectionBackend::kReference, gate_lw, up_lw, rb.p, nullptr, 0, g4.p,
                                                  u4.p, s) == 0);
  EXPECT(same(g3, g1) && same(res3, res1) && same(g4, g1) && same(u4, u1));
  // down projection (bf16 weights) + residual + norm: three distinct boundaries
  Bf16 down_w(random_bf16(hidden * inter, 0.03f));
  rt::Bf16LinearWeight down{};
  down.weight = down_w.p; down.output_size = hidden; down.input_size = inter;
  const rt::LinearWeight down_lw = down;
  Bf16 raw1(hidden), r1(hidden), n1(hidden), raw2(hidden), r2(hidden), n2(hidden);
  EXPECT(rt::launch_mlp_down_residual_norm_to_bf16_cuda(rt::ProjectionBackend::kReference, down_lw, g1.p, left.p, w.p, eps,
                                                        nullptr, 0, raw1.p, r1.p, n1.p, s) == 0);
  EXPECT(q3x_b200_bf16_gemv(down_w.p, g1.p, hidden, inter, nullptr, raw2.p, s) == 0);
  EXPECT(q3x_b200_residual_add_rms_norm(left.p, raw2.p, w.p, 1, hidden, eps, r2.p, n2.p, s) == 0);
  EXPECT(same(raw1, raw2) && same(r1, r2) && same(n1, n2) && written(n1));
  // FP8 weights through the single projection entry
  DeviceBuffer<std::uint8_t> fp8_w(random_bytes(inter * hidden, 0x10, 0x60));
  rt::Fp8LinearWeight f8{};
  f8.weight = fp8_w.p; f8.weight_scale_device = dev_scalar.p; f8.input_scale_device = dev_scalar.p;
  f8.weight_scale = 0.02f; f8.input_scale = 1.0f; f8.output_size = inter; f8.input_size = hidden;
  const rt::LinearWeight f8_lw = f8;
  Bf16 p1(inter), p2(inter);
  EXPECT(rt::launch_projection_to_bf16_cuda(rt::ProjectionBackend::kSm87WeightOnly, f8_lw, left.p, nullptr, 0, p1.p, s) == 0);
  EXPECT(q3x_b200_fp8_gemv(fp8_w.p, 0.02f, left.p, inter, hidden, nullptr, p2.p, s) == 0);
  EXPECT(same(p1, p2) && written(p1));
  // the sequence-tile form: FP8 weights of several tokens go through the weight-only tensor-core GEMM (same bytes
  // as the C-ABI call), one token through the batch-one kernel; bf16 weights likewise
  {
    Bf16 xs3(random_bf16(3 * hidden, 1.0f)), t1(3 * inter), t2(3 * inter), t3(inter);
    EXPECT(rt::launch_projection_tile_to_bf16_cuda(rt::ProjectionBackend::kSm87WeightOnly, f8_lw, xs3.p, 3, nullptr, 0, t1.p,
                                                   s) == 0);
    EXPECT(q3x_b200_fp8_gemm_bf16(fp8_w.p, 0.02f, xs3.p, 3, inter, hidden, t2.p, nullptr, 0, s) == 0);
    EXPECT(same(t1, t2) && written(t1));
    EXPECT(rt::launch_projection_tile_to_bf16_cuda(rt::ProjectionBackend::kSm87WeightOnly, f8_lw, xs3.p, 1, nullptr, 0, t3.p,
                                                   s) == 0);
    EXPECT(q3x_b200_fp8_gemv(fp8_w.p, 0.02f, xs3.p, inter, hidden, nullptr, t2.p, s) == 0);
    EXPECT(cudaStreamSynchronize(static_cast<cudaStream_t>(s)) == cudaSuccess);
    {
      std::vector<std::uint16_t> a(inter), b(inter);
      cudaMemcpy(a.data(), t3.p, inter * 2, cudaMemcpyDeviceToHost);
      cudaMemcpy(b.data(), t2.p, inter * 2, cudaMemcpyDeviceToHost);
      EXPECT(a == b);
    }
    Bf16 d1(3 * hidden), d2(3 * hidden), acts(random_bf16(3 * inter, 0.5f));
    EXPECT(rt::launch_projection_tile_to_bf16_cuda(rt::ProjectionBackend::kReference, down_lw, acts.p, 3, nullptr, 0, d1.p,
                                                   s) == 0);
    EXPECT(q3x_b200_bf16_gemm_bf16(down_w.p, acts.p, 3, hidden, inter, d2.p, nullptr, 0, s) == 0);
    EXPECT(same(d1, d2) && written(d1));
    EXPECT(rt::launch_projection_tile_to_bf16_cuda(rt::ProjectionBackend::kSm87WeightOnly, f8_lw, xs3.p, 65, nullptr, 0, t1.p,
                                                   s) == 1);
    EXPECT(rt::launch_projection_tile_to_bf16_cuda(rt::ProjectionBackend::kSm87WeightOnly, f8_lw, xs3.p, 0, nullptr, 0, t1.p,
                                                   s) == 1);
  }
  // one FP8 projection over a whole prefill chunk: the reference's structural gate, then the same GEMM
  {
    const std::size_t kv = 1024, chunk = 256;
    DeviceBuffer<std::uint8_t> kv_w(random_bytes(kv * hidden, 0x10, 0x60));
    rt::Fp8LinearWeight kvw = f8;
    kvw.weight = kv_w.p; kvw.output_size = kv; kvw.input_size = hidden;
    const rt::LinearWeight kv_lw = kvw;
    Bf16 xc(random_bf16(chunk * hidden, 1.0f)), c1(chunk * kv), c2(chunk * kv);
    EXPECT(rt::launch_exact_fp8_whole_chunk_projection_to_bf16_cuda(rt::ProjectionBackend::kSm87WeightOnly, kv_lw, xc.p, chunk,
                                                                    c1.p, s) == 0);
    EXPECT(q3x_b200_fp8_gemm_bf16(kv_w.p, 0.02f, xc.p, chunk, kv, hidden, c2.p, nullptr, 0, s) == 0);
    EXPECT(same(c1, c2) && written(c1));
    constexpr int kUnsupported = 801;
    EXPECT(rt::launch_exact_fp8_whole_chunk_projection_to_bf16_cuda(rt::ProjectionBackend::kSm87WeightOnly, kv_lw, xc.p, 128,
                                                                    c1.p, s) == kUnsupported);
    EXPECT(rt::launch_exact_fp8_whole_chunk_projection_to_bf16_cuda(rt::ProjectionBackend::kReference, kv_lw, xc.p, chunk,
                                                                    c1.p, s) == kUnsupported);
    rt::Fp8LinearWeight odd = kvw;
    odd.output_size = 512;  // [512, 5120] is none of the five shapes
    EXPECT(rt::launch_exact_fp8_whole_chunk_projection_to_bf16_cuda(rt::ProjectionBackend::kSm87WeightOnly, rt::LinearWeight{odd},
                                                                    xc.p, chunk, c1.p, s) == kUnsupported);
    EXPECT(rt::launch_exact_fp8_whole_chunk_projection_to_bf16_cuda(rt::ProjectionBackend::kSm87WeightOnly, kv_lw, xc.p, chunk,
                                                                    xc.p, s) == 1);             // output on the input
  }
  // FP32 output, and the two-step form that leaves the FP32 result in the scratch as well
  {
    DeviceBuffer<float> y1(inter), y2(inter), y3(inter);
    Bf16 b1(inter);
    EXPECT(rt::launch_projection_reference_cuda(f8_lw, left.p, y1.p, s) == 0);
    EXPECT(q3x_b200_fp8_gemv(fp8_w.p, 0.02f, left.p, inter, hidden, y2.p, nullptr, s) == 0);
    EXPECT(rt::launch_projection_to_bf16_reference_cuda(f8_lw, left.p, y3.p, inter, b1.p, s) == 0);
    EXPECT(cudaStreamSynchronize(static_cast<cudaStream_t>(s)) == cudaSuccess);
    std::vector<float> a(inter), b(inter), c(inter);
    cudaMemcpy(a.data(), y1.p, inter * 4, cudaMemcpyDeviceToHost);
    cudaMemcpy(b.data(), y2.p, inter * 4, cudaMemcpyDeviceToHost);
    cudaMemcpy(c.data(), y3.p, inter * 4, cudaMemcpyDeviceToHost);
    EXPECT(std::memcmp(a.data(), b.data(), inter * 4) == 0 && std::memcmp(a.data(), c.data(), inter * 4) == 0);
    EXPECT(same(b1, p1));
  }
  // two, three and four projections of one activation equal the single calls
  {
    const std::size_t kv = 1024;
    DeviceBuffer<std::uint8_t> k_w(random_bytes(kv * hidden, 0x10, 0x60)), v_w(random_bytes(kv * hidden, 0x10, 0x60));
    rt::Fp8LinearWeight kw = f8, vw = f8;
    kw.weight = k_w.p; kw.output_size = kv;
    vw.weight = v_w.p; vw.output_size = kv;
    const rt::LinearWeight k_lw = kw, v_lw = vw;
    Bf16 xs3(random_bf16(3 * hidden, 1.0f)), k1(3 * kv), v1(3 * kv), k2(3 * kv), v2(3 * kv);
    EXPECT(rt::launch_projection_pair_tile_to_bf16_cuda(rt::ProjectionBackend::kSm87WeightOnly, k_lw, v_lw, xs3.p, 3, nullptr, 0,
                                                        k1.p, v1.p, s) == 0);
    EXPECT(q3x_b200_fp8_gemm_bf16(k_w.p, 0.02f, xs3.p, 3, kv, hidden, k2.p, nullptr, 0, s) == 0);
    EXPECT(q3x_b200_fp8_gemm_bf16(v_w.p, 0.02f, xs3.p, 3, kv, hidden, v2.p, nullptr, 0, s) == 0);
    EXPECT(same(k1, k2) && same(v1, v2) && written(k1) && written(v1));
    Bf16 q1(inter), q2(inter), k3(kv), v3(kv), k4(kv), v4(kv);
    EXPECT(rt::launch_full_attention_q_kv_to_bf16_cuda(rt::ProjectionBackend::kSm87WeightOnly, f8_lw, k_lw, v_lw, left.p, nullptr,
                                                       0, q1.p, k3.p, v3.p, s) == 0);
    EXPECT(q3x_b200_fp8_gemv(fp8_w.p, 0.02f, left.p, inter, hidden, nullptr, q2.p, s) == 0);
    EXPECT(q3x_b200_fp8_gemv(k_w.p, 0.02f, left.p, kv, hidden, nullptr, k4.p, s) == 0);
    EXPECT(q3x_b200_fp8_gemv(v_w.p, 0.02f, left.p, kv, hidden, nullptr, v4.p, s) == 0);
    EXPECT(same(q1, q2) && same(k3, k4) && same(v3, v4) && written(q1));
    // the linear-attention group at its exact shapes
    const std::size_t qkv = 10240, zr = 6144, ab = 48;
    DeviceBuffer<std::uint8_t> qkv_w(random_bytes(qkv * hidden, 0x10, 0x60)), z_w(random_bytes(zr * hidden, 0x10, 0x60));
    Bf16 a_w(random_bf16(ab * hidden, 0.03f)), b_w(random_bf16(ab * hidden, 0.03f));
    rt::Fp8LinearWeight qkvw = f8, zw = f8;
    qkvw.weight = qkv_w.p; qkvw.output_size = qkv;
    zw.weight = z_w.p; zw.output_size = zr;
    rt::Bf16LinearWeight aw{}, bw{};
    aw.weight = a_w.p; aw.output_size = ab; aw.input_size = hidden;
    bw = aw; bw.weight = b_w.p;
    Bf16 o_qkv(qkv), o_z(zr), o_a(ab), o_b(ab), e_qkv(qkv), e_z(zr), e_a(ab), e_b(ab);
    EXPECT(rt::launch_linear_attention_qkv_z_ab_to_bf16_cuda(rt::ProjectionBackend::kSm87WeightOnly, rt::LinearWeight{qkvw},
                                                             rt::LinearWeight{zw}, rt::LinearWeight{aw}, rt::LinearWeight{bw},
                                                             left.p, o_qkv.p, o_z.p, o_a.p, o_b.p, s) == 0);
    EXPECT(q3x_b200_fp8_gemv(qkv_w.p, 0.02f, left.p, qkv, hidden, nullptr, e_qkv.p, s) == 0);
    EXPECT(q3x_b200_fp8_gemv(z_w.p, 0.02f, left.p, zr, hidden, nullptr, e_z.p, s) == 0);
    EXPECT(q3x_b200_bf16_gemv(a_w.p, left.p, ab, hidden, nullptr, e_a.p, s) == 0);
    EXPECT(q3x_b200_bf16_gemv(b_w.p, left.p, ab, hidden, nullptr, e_b.p, s) == 0);
    EXPECT(same(o_qkv, e_qkv) && same(o_z, e_z) && same(o_a, e_a) && same(o_b, e_b) && written(o_qkv) && written(o_a));
    EXPECT(rt::launch_linear_attention_qkv_z_ab_to_bf16_cuda(rt::ProjectionBackend::kSm87WeightOnly, rt::LinearWeight{zw},
                                                             rt::LinearWeight{qkvw}, rt::LinearWeight{aw}, rt::LinearWeight{bw},
                                                             left.p, o_qkv.p, o_z.p, o_a.p, o_b.p, s) == 801);
  }
  // rejections, all before any enqueue
  constexpr int kInvalid = 1;
  EXPECT(rt::launch_projection_to_bf16_cuda(static_cast<rt::ProjectionBackend>(9), f8_lw, left.p, nullptr, 0, p1.p, s) == kInvalid);
  EXPECT(rt::launch_projection_to_bf16_cuda(rt::ProjectionBackend::kReference, f8_lw, left.p, nullptr, 0, left.p, s) == kInvalid);
  rt::NvFp4LinearWeight broken = gate;
  broken.block_scale = nullptr;
  EXPECT(rt::launch_mlp_gate_up_silu_to_bf16_cuda(rt::ProjectionBackend::kReference, rt::LinearWeight{broken}, up_lw, rb.p,
                                                  nullptr, 0, g4.p, u4.p, s) == kInvalid);
  EXPECT(rt::launch_mlp_gate_up_silu_to_bf16_cuda(rt::ProjectionBackend::kReference, gate_lw, up_lw, rb.p, nullptr, 0, g4.p,
                                                  g4.p, s) == kInvalid);  // gate and up outputs alias
  EXPECT(rt::launch_mlp_down_residual_norm_to_bf16_cuda(rt::ProjectionBackend::kReference, down_lw, g1.p, left.p, w.p, eps,
                                                        nullptr, 0, raw1.p, raw1.p, n1.p, s) == kInvalid);
  EXPECT(rt::launch_mlp_down_residual_norm_to_bf16_cuda(rt::ProjectionBackend::kReference, gate_lw, g1.p, left.p, w.p, eps,
                                                        nullptr, 0, raw1.p, r1.p, n1.p, s) == kInvalid);  // rows != 5120
}

// The launchers of the operators between the fused layer ops, through their q3x::runtime / q3x::kernels names.
static void test_core_launchers(cudaStream_t s) {
  const float eps = 1e-6f;
  Bf16 conv(random_bf16(16 * 10240, 1.0f)), a(random_bf16(16 * 48, 1.0f)), b(random_bf16(16 * 48, 1.0f)),
      A_log(random_bf16(48, 1.0f)), dt(random_bf16(48, 1.0f));
  const auto state_host = random_bf16(48 * 128 * 128, 0.05f);
  Bf16 s1(state_host), s2(state_host), o1(16 * 6144), o2(16 * 6144);
  EXPECT(rt::launch_gated_delta_net_update_tile_reference_cuda(conv.p, 16, a.p, b.p, A_log.p, dt.p, s1.p, s1.p, eps, o1.p,
                                                               rt::GdnDimensions{}, s) == 0);
  EXPECT(q3x_b200_gated_delta_net_update(conv.p, 16, a.p, b.p, A_log.p, dt.p, s2.p, s2.p, eps, o2.p, s) == 0);
  EXPECT(same(s1, s2) && same(o1, o2) && written(o1));
  EXPECT(rt::launch_gated_delta_net_update_tile_reference_cuda(conv.p, 17, a.p, b.p, A_log.p, dt.p, s1.p, s1.p, eps, o1.p,
                                                               rt::GdnDimensions{}, s) == 1);
  Bf16 z(random_bf16(6144, 1.0f)), nw(random_bf16(128, 1.0f)), f1(6144), f2(6144), s3(state_host), s4(state_host);
  EXPECT(rt::launch_gated_delta_net_update_plain_rms_norm_silu_gate_cuda(conv.p, a.p, b.p, A_log.p, dt.p, s3.p, s3.p, eps, nw.p,
                                                                         z.p, 48, 128, eps, f1.p, rt::GdnDimensions{}, s) == 0);
  EXPECT(q3x_b200_gated_delta_net_update_rms_norm_silu_gate(conv.p, 1, a.p, b.p, A_log.p, dt.p, s4.p, s4.p, eps, nw.p, z.p, eps,
                                                            f2.p, s) == 0);
  EXPECT(same(f1, f2) && same(s3, s4) && written(f1));
  // the chunked prefill form with its norm epilogue: the C-ABI recurrence, then the gated norm in place
  {
    namespace chunked = rt::gdn_prefill_chunk64_native_detail;
    const std::size_t tile = 100, bytes = chunked::workspace_bytes();
    EXPECT(bytes == q3x_b200_gated_delta_net_chunked_workspace_bytes(512) && bytes > 0);
    Bf16 cconv(random_bf16(tile * 10240, 1.0f)), ca(random_bf16(tile * 48, 1.0f)), cb(random_bf16(tile * 48, 1.0f)),
        cz(random_bf16(tile * 6144, 1.0f)), c1(tile * 6144), c2(tile * 6144), cs1(state_host), cs2(state_host);
    DeviceBuffer<std::uint8_t> cws(bytes);
    EXPECT(chunked::launch(cws.p, bytes, cconv.p, tile, ca.p, cb.p, A_log.p, dt.p, cs1.p, cs1.p, eps, nw.p, cz.p, eps, c1.p, s) == 0);
    EXPECT(q3x_b200_gated_delta_net_update_chunked(cconv.p, tile, ca.p, cb.p, A_log.p, dt.p, cs2.p, cs2.p, eps, c2.p, cws.p, bytes,
                                                   s) == 0);
    EXPECT(q3x_b200_rms_norm_silu_gate(c2.p, nw.p, cz.p, tile * 48, 128, eps, c2.p, s) == 0);
    EXPECT(same(c1, c2) && same(cs1, cs2) && written(c1));
    EXPECT(chunked::launch_fixed_production(cws.p, bytes, cconv.p, tile, ca.p, cb.p, A_log.p, dt.p, cs1.p, cs1.p, eps, nw.p,
                                            cz.p, eps, c1.p, s) == 0);
    EXPECT(chunked::launch(cws.p, bytes, cconv.p, 513, ca.p, cb.p, A_log.p, dt.p, cs1.p, cs1.p, eps, nw.p, cz.p, eps, c1.p, s) == 1);
    EXPECT(chunked::launch(cws.p, bytes - 1, cconv.p, tile, ca.p, cb.p, A_log.p, dt.p, cs1.p, cs1.p, eps, nw.p, cz.p, eps, c1.p,
                           s) == 1);
    EXPECT(chunked::launch(cws.p, bytes, cconv.p, tile, ca.p, cb.p, A_log.p, dt.p, cs1.p, cs1.p, eps, nullptr, cz.p, eps, c1.p,
                           s) == 1);
  }
  // decode attention
  const std::size_t length = 300;
  Bf16 q(random_bf16(24 * 256, 1.0f)), kc(random_bf16(length * 1024, 1.0f)), vc(random_bf16(length * 1024, 1.0f)),
      gate(random_bf16(24 * 256, 2.0f)), a1(24 * 256), a2(24 * 256);
  const std::size_t need = rt::gqa_attention_splitkv_sigmoid_gate_24_4_256_workspace_elements(length);
  EXPECT(need == q3x_b200_gqa_decode_workspace_floats(length) && need > 0);
  DeviceBuffer<float> ws(need);
  EXPECT(rt::launch_gqa_attention_splitkv_sigmoid_gate_24_4_256_cuda(q.p, kc.p, vc.p, length, 0.0625f, ws.p, need, gate.p, a1.p,
                                                                     s) == 0);
  CUDA_OK(cudaStreamSynchronize(s));
  EXPECT(q3x_b200_gqa_attention_decode_sigmoid_gate(q.p, kc.p, vc.p, length, 0.0625f, ws.p, need, gate.p, a2.p, s) == 0);
  EXPECT(same(a1, a2) && written(a1));
  EXPECT(rt::launch_gqa_attention_splitkv_sigmoid_gate_24_4_256_cuda(q.p, kc.p, vc.p, 64, 0.0625f, ws.p, need, gate.p, a1.p, s) == 1);
  // bulk causal attention of a prefill tile: 40 tokens appended at position 260 of the same caches
  {
    const std::size_t tile = 40, first = length - tile;
    Bf16 qt(random_bf16(tile * 24 * 256, 1.0f)), gt(random_bf16(tile * 24 * 256, 2.0f)), o1(tile * 24 * 256), o2(tile * 24 * 256),
        o3(tile * 24 * 256);
    EXPECT(rt::launch_bulk_causal_gqa_sigmoid_gate_24_4_256_cuda(qt.p, kc.p, vc.p, gt.p, first, tile, o1.p, s) == 0);
    EXPECT(rt::launch_bulk_causal_gqa_sigmoid_gate_24_4_256_group_q64_panel_fixed_cuda(qt.p, kc.p, vc.p, gt.p, first, tile, o3.p,
                                                                                     s) == 0);
    EXPECT(q3x_b200_gqa_attention_prefill_sigmoid_gate(qt.p, kc.p, vc.p, gt.p, first, tile, 0.0625f, o2.p, s) == 0);
    EXPECT(same(o1, o2) && same(o3, o2) && written(o1));
    EXPECT(rt::launch_bulk_causal_gqa_sigmoid_gate_24_4_256_fixed_cuda(qt.p, kc.p, vc.p, gt.p, first, 1, o1.p, s) == 1);
    EXPECT(rt::launch_bulk_causal_gqa_sigmoid_gate_24_4_256_fixed_cuda(qt.p, kc.p, vc.p, gt.p, first, 513, o1.p, s) == 1);
    EXPECT(rt::launch_bulk_causal_gqa_sigmoid_gate_24_4_256_cuda(qt.p, kc.p, vc.p, nullptr, first, tile, o1.p, s) == 1);
  }
  // argmax and the FP32 GEMV launchers
  DeviceBuffer<rt::Bf16GreedyArgmaxResult> r1(rt::kBf16GreedyArgmaxWorkspaceResults), r2(rt::kBf16GreedyArgmaxWorkspaceResults);
  EXPECT(rt::launch_bf16_greedy_argmax_cuda(kc.p, length * 1024, r1.p, s) == 0);
  EXPECT(q3x_b200_bf16_greedy_argmax(kc.p, length * 1024, r2.p, s) == 0);
  CUDA_OK(cudaDeviceSynchronize());
  EXPECT(std::memcmp(r1.get().data(), r2.get().data(), 8) == 0);
  DeviceBuffer<float> y1(24), y2(24);
  EXPECT(q3x::kernels::launch_bf16_gemv_reference_cuda(q.p, gate.p, 24, 256, y1.p, s) == 0);
  EXPECT(q3x_b200_bf16_gemv(q.p, gate.p, 24, 256, y2.p, nullptr, s) == 0);
  EXPECT(same(y1, y2) && written(y1));
}

int main() {
  int device_count = 0;
  if (cudaGetDeviceCount(&device_count) != cudaSuccess || device_count == 0) {
    std::printf("no CUDA device: skipped\n");
    return 77;
  }
  cudaDeviceProp prop{};
  CUDA_OK(cudaGetDeviceProperties(&prop, 0));
  if (prop.major != 10) {
    std::printf("device is sm_%d%d, the library is built for sm_100a: skipped\n", prop.major, prop.minor);
    return 77;
  }
  cudaStream_t s = nullptr;
  CUDA_OK(cudaStreamCreate(&s));
  test_pointwise_and_embedding(s);
  test_norms(s);
  test_full_attention(s);
  test_conv(s);
  test_dispatch_halves(s);
  test_composites(s);
  test_core_launchers(s);
  CUDA_OK(cudaStreamSynchronize(s));
  CUDA_OK(cudaGetLastError());
  CUDA_OK(cudaStreamDestroy(s));
  if (failures == 0) std::printf("host mirror GPU tests passed\n");
  return failures;
}
