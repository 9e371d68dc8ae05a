// Row-wise normalisations: centred / plain RMSNorm (single row, head-wise and token-wise), the
// GDN output's gated RMSNorm * silu(z), the q/k L2 norm, and the residual add fused with the
// centred RMSNorm of the rounded residual.
//
// Three kernels cover every shape:
//   * head_rows_kernel  -- rows of 64 / 128 / 256 elements (GDN heads, q/k heads): 8, 16 or 32
//     lanes own one row, one 128-bit vector per lane, shuffle reduction, two rows in flight per
//     lane group.  CTAs take contiguous row ranges.
//   * hidden_rows_kernel -- rows of up to 8192 elements (the 5120-wide residual stream): one
//     128-thread CTA per row, the whole row lives in registers between the reduction and the
//     scaling, so each element crosses HBM once per tensor.
//   * generic_rows_kernel -- any width / alignment, scalar accesses; same arithmetic.
// Reductions are FP32: per-lane sequential partial sums, then a shuffle / shared-memory tree with a
// fixed order, so results do not depend on the launch geometry.
#include "device_utils.cuh"
#include "host_checks.hpp"
#include "internal.hpp"
#include "norm_math.cuh"
#include "q3x_b200.h"

namespace q3x {
namespace {

// Accumulates a running group amax in registers and flushes it with one atomic when the group
// changes; rows are visited in increasing order so a thread flushes a handful of times at most.
struct AmaxTracker {
  float value = 0.0f;  // running amax (see amax8_float); converted to bf16 bits when flushed
  size_t group = 0;
  size_t boundary = 0;  // first row of the next group; rows arrive in increasing order
  bool live = false;
  // call BEFORE accumulating the values of `row`
  __device__ __forceinline__ void enter_row(uint32_t* amax_bits, size_t row, size_t rows_per_group) {
    if (!live || row >= boundary) {  // the division runs once per group a thread visits, not per row
      if (live && value != 0.0f) atomicMax(amax_bits + group, amax_bits_of(value));
      value = 0.0f;
      group = row / rows_per_group;
      boundary = (group + 1) * rows_per_group;
      live = true;
    }
  }
  __device__ __forceinline__ void flush(uint32_t* amax_bits) {
    // fast path: the whole warp ends in the same group -> one atomic per warp
    const size_t g0 = static_cast<size_t>(__shfl_sync(kFullMask, static_cast<unsigned long long>(group), 0));
    const bool uniform = __all_sync(kFullMask, live && group == g0);
    const uint32_t bits = amax_bits_of(value);
    if (uniform) {
      const uint32_t m = group_max_u32<32>(bits);
      if ((threadIdx.x & 31) == 0 && m != 0) atomicMax(amax_bits + g0, m);
    } else if (live && bits != 0) {
      atomicMax(amax_bits + group, bits);
    }
  }
};

// ------------------------------------------------------------------------------------------
// Rows of LANES * 8 elements.
template <int LANES, NormMode MODE, bool kAmax>
__global__ void __launch_bounds__(256) head_rows_kernel(const uint4* in, const uint4* __restrict__ weight,
                                                        const uint4* gate, size_t rows, size_t rows_per_cta,
                                                        float eps, float l2_scale, uint4* out, bool coherent,
                                                        uint32_t* amax_bits, size_t rows_per_amax_group) {
  constexpr int kRowsPerPass = 256 / LANES;
  const int lane = threadIdx.x % LANES;
  const int slot = threadIdx.x / LANES;
  const size_t begin = static_cast<size_t>(blockIdx.x) * rows_per_cta;
  const size_t end = min(rows, begin + rows_per_cta);
  uint4 w = make_uint4(0, 0, 0, 0);
  if (MODE != NormMode::kL2) w = ld_weight(weight + lane);
  AmaxTracker tracker;

  // two row passes in flight: pass p covers rows base + p * kRowsPerPass + slot
  for (size_t base = begin; base < end; base += 2 * kRowsPerPass) {
    uint4 x[2], z[2];
    bool valid[2];
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      const size_t row = base + p * kRowsPerPass + slot;
      valid[p] = row < end;
      x[p] = z[p] = make_uint4(0, 0, 0, 0);
      if (valid[p]) {
        const size_t v = row * LANES + lane;
        x[p] = coherent ? ld_vec(in + v) : ld_stream(in + v);
        if (MODE == NormMode::kPlainSiluGate) z[p] = coherent ? ld_vec(gate + v) : ld_stream(gate + v);
      }
    }
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      const float sum = group_sum<LANES>(sum_squares8(x[p]));
      float inv;
      if (MODE == NormMode::kL2) {
        inv = inverse_l2(sum, eps);
        if (l2_scale != 1.0f) inv = inv * l2_scale;
      } else {
        inv = inverse_rms(sum, 1.0f / static_cast<float>(LANES * 8), eps);
      }
      if (valid[p]) {
        const size_t row = base + p * kRowsPerPass + slot;
        if (kAmax) tracker.enter_row(amax_bits, row, rows_per_amax_group);
        const uint4 y = scale8<MODE, kAmax>(x[p], w, z[p], inv, &tracker.value);
        st_vec(out + row * LANES + lane, y);
      }
    }
  }
  if (kAmax) tracker.flush(amax_bits);
}

// ------------------------------------------------------------------------------------------
// One 128-thread CTA per row of up to 128 * VPT vectors.  kResidual: x = bf16(a + b) is formed
// first, stored to residual_out, and the norm runs on the rounded value.
template <int VPT, bool kResidual, NormMode MODE, bool kAmax>
__global__ void __launch_bounds__(128) hidden_rows_kernel(const uint4* a, const uint4* b,
                                                          const uint4* __restrict__ weight, int row_vectors,
                                                          float width, float eps, uint4* residual_out,
                                                          uint4* normalized_out, bool coherent,
                                                          uint32_t* amax_bits, size_t rows_per_amax_group) {
  __shared__ float scratch[4];
  __shared__ uint32_t amax_scratch[4];
  const size_t row = blockIdx.x;
  const size_t row_base = row * static_cast<size_t>(row_vectors);
  uint4 x[VPT];
  float partial = 0.0f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * 128;
    x[k] = make_uint4(0, 0, 0, 0);
    if (v < row_vectors) x[k] = coherent ? ld_vec(a + row_base + v) : ld_stream(a + row_base + v);
  }
  if (kResidual) {
    uint4 r[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = threadIdx.x + k * 128;
      r[k] = make_uint4(0, 0, 0, 0);
      if (v < row_vectors) r[k] = coherent ? ld_vec(b + row_base + v) : ld_stream(b + row_base + v);
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      float l[8], rr[8];
      unpack8(x[k], l);
      unpack8(r[k], rr);
      add8(l, rr);
      x[k] = pack8(l);
      const int v = threadIdx.x + k * 128;
      if (v < row_vectors) st_vec(residual_out + row_base + v, x[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < VPT; ++k) partial += sum_squares8(x[k]);
  if (normalized_out == nullptr) return;
  const float total = block_sum<4>(partial, scratch);
  const float inv = inverse_rms(total, 1.0f / width, eps);
  float top_f = 0.0f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * 128;
    if (v < row_vectors) {
      const uint4 y = scale8<MODE, kAmax>(x[k], ld_weight(weight + v), make_uint4(0, 0, 0, 0), inv, &top_f);
      st_vec(normalized_out + row_base + v, y);
    }
  }
  if (kAmax) {
    uint32_t top = group_max_u32<32>(amax_bits_of(top_f));
    if ((threadIdx.x & 31) == 0) amax_scratch[threadIdx.x >> 5] = top;
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t m = max(max(amax_scratch[0], amax_scratch[1]), max(amax_scratch[2], amax_scratch[3]));
      if (m != 0) atomicMax(amax_bits + row / rows_per_amax_group, m);
    }
  }
}

// ------------------------------------------------------------------------------------------
// Any width, any alignment: one 256-thread CTA per row, scalar accesses, two sweeps.
template <bool kResidual, NormMode MODE>
__global__ void __launch_bounds__(256) generic_rows_kernel(const uint16_t* a, const uint16_t* b,
                                                           const uint16_t* weight, const uint16_t* gate,
                                                           size_t width, float eps, float l2_scale,
                                                           uint16_t* residual_out, uint16_t* out) {
  __shared__ float scratch[8];
  const size_t base = static_cast<size_t>(blockIdx.x) * width;
  const uint16_t* x = kResidual ? residual_out + base : a + base;
  float partial = 0.0f;
  for (size_t i = threadIdx.x; i < width; i += 256) {
    float v;
    if (kResidual) {
      const uint16_t r = float_to_bf16(bf16_to_float(a[base + i]) + bf16_to_float(b[base + i]));
      residual_out[base + i] = r;
      v = bf16_to_float(r);
    } else {
      v = bf16_to_float(x[i]);
    }
    partial = fmaf(v, v, partial);
  }
  if (out == nullptr) return;
  const float total = block_sum<8>(partial, scratch);
  float inv;
  if (MODE == NormMode::kL2) {
    inv = inverse_l2(total, eps);
    if (l2_scale != 1.0f) inv = inv * l2_scale;
  } else {
    inv = inverse_rms(total, 1.0f / static_cast<float>(width), eps);
  }
  for (size_t i = threadIdx.x; i < width; i += 256) {
    const float v = bf16_to_float(x[i]);  // a thread re-reads only what it wrote itself
    float y;
    if (MODE == NormMode::kL2) {
      y = v * inv;
    } else {
      const float gamma = bf16_to_float(weight[i]) + (MODE == NormMode::kCentered ? 1.0f : 0.0f);
      y = v * inv * gamma;
      if (MODE == NormMode::kPlainSiluGate) y *= silu(bf16_to_float(gate[base + i]));
    }
    out[base + i] = float_to_bf16(y);
  }
}

template <int LANES, NormMode MODE>
void launch_head_rows(const uint16_t* in, const uint16_t* weight, const uint16_t* gate, size_t rows, float eps,
                      float l2_scale, uint16_t* out, bool coherent, uint32_t* amax_bits, size_t rows_per_amax_group,
                      cudaStream_t s) {
  constexpr size_t kRowsPerIter = 2 * (256 / LANES);
  // contiguous row ranges, a whole number of resident waves (at most four) so no partial wave idles
  const unsigned resident = amax_bits ? host::resident_grid(head_rows_kernel<LANES, MODE, true>, 256)
                                      : host::resident_grid(head_rows_kernel<LANES, MODE, false>, 256);
  const size_t iterations = (rows + kRowsPerIter - 1) / kRowsPerIter;
  size_t waves = iterations / (static_cast<size_t>(resident) * 8);  // >= 8 iterations per CTA
  waves = waves < 1 ? 1 : (waves > 4 ? 4 : waves);
  const size_t grid = iterations < resident * waves ? iterations : resident * waves;
  size_t rows_per_cta = (rows + grid - 1) / grid;
  rows_per_cta = (rows_per_cta + kRowsPerIter - 1) / kRowsPerIter * kRowsPerIter;
  const unsigned ctas = static_cast<unsigned>((rows + rows_per_cta - 1) / rows_per_cta);
  auto i = reinterpret_cast<const uint4*>(in);
  auto w = reinterpret_cast<const uint4*>(weight);
  auto g = reinterpret_cast<const uint4*>(gate);
  auto o = reinterpret_cast<uint4*>(out);
  if (amax_bits)
    head_rows_kernel<LANES, MODE, true><<<ctas, 256, 0, s>>>(i, w, g, rows, rows_per_cta, eps, l2_scale, o, coherent,
                                                             amax_bits, rows_per_amax_group);
  else
    head_rows_kernel<LANES, MODE, false><<<ctas, 256, 0, s>>>(i, w, g, rows, rows_per_cta, eps, l2_scale, o,
                                                              coherent, nullptr, 1);
}

template <bool kResidual, NormMode MODE, bool kAmax>
void launch_hidden_rows_vpt(int vpt, dim3 grid, cudaStream_t s, const uint4* a, const uint4* b, const uint4* w,
                            int row_vectors, float width, float eps, uint4* residual_out, uint4* normalized_out,
                            bool coherent, uint32_t* amax_bits, size_t rows_per_amax_group) {
#define Q3X_CASE(V)                                                                                              \
  case V:                                                                                                        \
    hidden_rows_kernel<V, kResidual, MODE, kAmax><<<grid, 128, 0, s>>>(a, b, w, row_vectors, width, eps,        \
                                                                       residual_out, normalized_out, coherent,   \
                                                                       amax_bits, rows_per_amax_group);          \
    break;
  switch (vpt) {
    Q3X_CASE(1) Q3X_CASE(2) Q3X_CASE(3) Q3X_CASE(4) Q3X_CASE(5) Q3X_CASE(6) Q3X_CASE(7) Q3X_CASE(8)
  }
#undef Q3X_CASE
}

}  // namespace

// Internal launcher shared with the NVFP4 entry points.  Arguments are already validated.
// a: input (or left); b: right when residual_out != nullptr; out may be nullptr only with residual.
void launch_norm_rows(NormMode mode, const uint16_t* a, const uint16_t* b, const uint16_t* weight,
                      const uint16_t* gate, size_t rows, size_t width, float eps, float l2_scale,
                      uint16_t* residual_out, uint16_t* out, bool coherent, uint32_t* amax_bits,
                      size_t rows_per_amax_group, cudaStream_t s) {
  const bool residual = residual_out != nullptr;
  bool vector_ok = width % 8 == 0 && host::aligned16(a) && (out == nullptr || host::aligned16(out)) &&
                   (mode == NormMode::kL2 || host::aligned16(weight)) &&
                   (mode != NormMode::kPlainSiluGate || host::aligned16(gate)) &&
                   (!residual || (host::aligned16(b) && host::aligned16(residual_out)));
  // amax tracking exists on the vector kernels only; the entry points that need it check alignment
  if (vector_ok && !residual && out != nullptr && (width == 64 || width == 128 || width == 256)) {
#define Q3X_HEAD(L, M) \
  launch_head_rows<L, M>(a, weight, gate, rows, eps, l2_scale, out, coherent, amax_bits, rows_per_amax_group, s)
#define Q3X_HEAD_MODE(L)                                                      \
  switch (mode) {                                                             \
    case NormMode::kCentered: Q3X_HEAD(L, NormMode::kCentered); break;        \
    case NormMode::kPlain: Q3X_HEAD(L, NormMode::kPlain); break;              \
    case NormMode::kPlainSiluGate: Q3X_HEAD(L, NormMode::kPlainSiluGate); break; \
    case NormMode::kL2: Q3X_HEAD(L, NormMode::kL2); break;                    \
  }
    if (width == 64) { Q3X_HEAD_MODE(8) } else if (width == 128) { Q3X_HEAD_MODE(16) } else { Q3X_HEAD_MODE(32) }
#undef Q3X_HEAD_MODE
#undef Q3X_HEAD
    return;
  }
  if (vector_ok && width <= 8192 && mode != NormMode::kPlainSiluGate && mode != NormMode::kL2 &&
      rows <= 0x7fffffffu) {
    const int row_vectors = static_cast<int>(width / 8);
    const int vpt = (row_vectors + 127) / 128;
    const dim3 grid(static_cast<unsigned>(rows));
    auto A = reinterpret_cast<const uint4*>(a);
    auto B = reinterpret_cast<const uint4*>(b);
    auto W = reinterpret_cast<const uint4*>(weight);
    auto R = reinterpret_cast<uint4*>(residual_out);
    auto O = reinterpret_cast<uint4*>(out);
    const float fw = static_cast<float>(width);
#define Q3X_HID(RES, M, AM) \
  launch_hidden_rows_vpt<RES, M, AM>(vpt, grid, s, A, B, W, row_vectors, fw, eps, R, O, coherent, amax_bits, \
                                     rows_per_amax_group)
    if (residual) {
      if (amax_bits) Q3X_HID(true, NormMode::kCentered, true); else Q3X_HID(true, NormMode::kCentered, false);
    } else if (mode == NormMode::kCentered) {
      if (amax_bits) Q3X_HID(false, NormMode::kCentered, true); else Q3X_HID(false, NormMode::kCentered, false);
    } else {
      if (amax_bits) Q3X_HID(false, NormMode::kPlain, true); else Q3X_HID(false, NormMode::kPlain, false);
    }
#undef Q3X_HID
    return;
  }
  // generic path (rows are capped per launch by the grid limit)
  const size_t kMaxGrid = 0x7fffffffu;
  for (size_t first = 0; first < rows; first += kMaxGrid) {
    const unsigned grid = static_cast<unsigned>(rows - first < kMaxGrid ? rows - first : kMaxGrid);
    const size_t off = first * width;
    const uint16_t* g = gate ? gate + off : nullptr;
    uint16_t* o = out ? out + off : nullptr;
    if (residual) {
      generic_rows_kernel<true, NormMode::kCentered><<<grid, 256, 0, s>>>(a + off, b + off, weight, g, width, eps,
                                                                          l2_scale, residual_out + off, o);
    } else {
      switch (mode) {
        case NormMode::kCentered:
          generic_rows_kernel<false, NormMode::kCentered><<<grid, 256, 0, s>>>(a + off, nullptr, weight, g, width,
                                                                               eps, l2_scale, nullptr, o);
          break;
        case NormMode::kPlain:
          generic_rows_kernel<false, NormMode::kPlain><<<grid, 256, 0, s>>>(a + off, nullptr, weight, g, width, eps,
                                                                            l2_scale, nullptr, o);
          break;
        case NormMode::kPlainSiluGate:
          generic_rows_kernel<false, NormMode::kPlainSiluGate><<<grid, 256, 0, s>>>(a + off, nullptr, weight, g,
                                                                                    width, eps, l2_scale, nullptr, o);
          break;
        case NormMode::kL2:
          generic_rows_kernel<false, NormMode::kL2><<<grid, 256, 0, s>>>(a + off, nullptr, weight, g, width, eps,
                                                                         l2_scale, nullptr, o);
          break;
      }
    }
  }
}

// True when launch_norm_rows would take a 128-bit kernel that can also track the amax.
bool norm_rows_vector_path(const void* a, const void* b, const void* weight, const void* gate, size_t width,
                           const void* residual_out, const void* out, NormMode mode) {
  const bool residual = residual_out != nullptr;
  const bool aligned = width % 8 == 0 && host::aligned16(a) && host::aligned16(out) && host::aligned16(weight) &&
                       (mode != NormMode::kPlainSiluGate || host::aligned16(gate)) &&
                       (!residual || (host::aligned16(b) && host::aligned16(residual_out)));
  if (!aligned) return false;
  if (!residual && (width == 64 || width == 128 || width == 256)) return true;
  return width <= 8192 && mode != NormMode::kPlainSiluGate && mode != NormMode::kL2;
}

}  // namespace q3x

using namespace q3x;
using namespace q3x::host;

namespace {

// Shared checks of the row-norm entry points.  Returns kOk to proceed, or the status to return
// (*done = true when the call is a finished no-op).
int check_rows(const void* in, const void* weight, const void* gate, bool needs_gate, size_t rows, size_t width,
               float eps, const void* out, bool needs_weight, bool* done) {
  *done = false;
  if (!valid_epsilon(eps)) return kInvalid;
  if (mul3_overflows(rows, width, sizeof(uint16_t))) return kInvalid;
  if (rows == 0 || width == 0) {
    *done = true;
    return kOk;
  }
  if (in == nullptr || out == nullptr || (needs_weight && weight == nullptr) || (needs_gate && gate == nullptr))
    return kInvalid;
  const size_t bytes = rows * width * sizeof(uint16_t);
  const Span si = span(in, bytes), so = span(out, bytes), sw = span(weight, needs_weight ? width * 2 : 0);
  if (wraps(si) || wraps(so)) return kInvalid;
  if (partial_overlap(so, si) || overlap(so, sw)) return kInvalid;
  if (needs_gate) {
    const Span sg = span(gate, bytes);
    if (wraps(sg) || partial_overlap(so, sg)) return kInvalid;
  }
  return kOk;
}

}  // namespace

extern "C" int q3x_b200_rms_norm(const uint16_t* in, const uint16_t* weight, size_t rows, size_t width, float eps,
                                 int centered, uint16_t* out, void* stream) {
  bool done;
  const int st = check_rows(in, weight, nullptr, false, rows, width, eps, out, true, &done);
  if (st != kOk || done) return st;
  clear_stale_error();
  launch_norm_rows(centered ? NormMode::kCentered : NormMode::kPlain, in, nullptr, weight, nullptr, rows, width, eps,
                   1.0f, nullptr, out, /*coherent=*/out == in, nullptr, 1, as_stream(stream));
  return launch_status();
}

extern "C" int q3x_b200_rms_norm_silu_gate(const uint16_t* in, const uint16_t* weight, const uint16_t* gate,
                                           size_t rows, size_t width, float eps, uint16_t* out, void* stream) {
  bool done;
  const int st = check_rows(in, weight, gate, true, rows, width, eps, out, true, &done);
  if (st != kOk || done) return st;
  clear_stale_error();
  launch_norm_rows(NormMode::kPlainSiluGate, in, nullptr, weight, gate, rows, width, eps, 1.0f, nullptr, out,
                   /*coherent=*/out == in || out == gate, nullptr, 1, as_stream(stream));
  return launch_status();
}

extern "C" int q3x_b200_l2_normalize_heads(const uint16_t* in, size_t heads, size_t dim, float eps, float scale,
                                           uint16_t* out, void* stream) {
  bool done;
  if (!std::isfinite(scale)) return kInvalid;
  const int st = check_rows(in, nullptr, nullptr, false, heads, dim, eps, out, false, &done);
  if (st != kOk || done) return st;
  clear_stale_error();
  launch_norm_rows(NormMode::kL2, in, nullptr, nullptr, nullptr, heads, dim, eps, scale, nullptr, out,
                   /*coherent=*/out == in, nullptr, 1, as_stream(stream));
  return launch_status();
}

namespace q3x {
// Argument rules of the fused residual boundary (src/kernels/reference/decode_ops.cu:1913-1953,
// :2945-2968): residual_out disjoint from everything, normalized_out exactly `right` or disjoint.
int check_residual_norm(const uint16_t* left, const uint16_t* right, const uint16_t* weight, size_t tokens,
                        size_t hidden, float eps, const uint16_t* residual_out, const uint16_t* normalized_out,
                        bool* done) {
  *done = false;
  if (!valid_epsilon(eps)) return kInvalid;
  if (mul3_overflows(tokens, hidden, sizeof(uint16_t))) return kInvalid;
  if (tokens == 0 || hidden == 0) {
    *done = true;
    return kOk;
  }
  if (left == nullptr || right == nullptr || weight == nullptr || residual_out == nullptr) return kInvalid;
  const size_t bytes = tokens * hidden * sizeof(uint16_t);
  const Span sl = span(left, bytes), sr = span(right, bytes), sw = span(weight, hidden * 2),
             so = span(residual_out, bytes), sn = span(normalized_out, normalized_out ? bytes : 0);
  if (wraps(sl) || wraps(sr) || wraps(so) || wraps(sn)) return kInvalid;
  if (overlap(sl, sr)) return kInvalid;
  if (overlap(so, sl) || overlap(so, sr) || overlap(so, sw) || overlap(so, sn)) return kInvalid;
  if (overlap(sn, sl) || overlap(sn, sw) || partial_overlap(sn, sr)) return kInvalid;
  return kOk;
}
}  // namespace q3x

extern "C" int q3x_b200_residual_add_rms_norm(const uint16_t* left, const uint16_t* right, const uint16_t* weight,
                                              size_t tokens, size_t hidden, float eps, uint16_t* residual_out,
                                              uint16_t* normalized_out, void* stream) {
  bool done;
  const int st = check_residual_norm(left, right, weight, tokens, hidden, eps, residual_out, normalized_out, &done);
  if (st != kOk || done) return st;
  clear_stale_error();
  launch_norm_rows(NormMode::kCentered, left, right, weight, nullptr, tokens, hidden, eps, 1.0f, residual_out,
                   normalized_out, /*coherent=*/normalized_out == right, nullptr, 1, as_stream(stream));
  return launch_status();
}
