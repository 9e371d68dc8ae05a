// NVFP4 activation quantisation: 16-element blocks, one E4M3 scale per block, one FP32 global
// scale per group of rows.  real = E2M1(code) * E4M3(scale) * global; global = amax / (448 * 6).
//
// The arithmetic, step for step (all IEEE binary32, no contraction):
//   A      = largest finite |x| of the group          (exact: unsigned max of bf16 magnitude bits)
//   global = A == 0 ? 1 : A / 2688
//   k      = 1 / (global * 6)
//   per block: s   = amax_b == 0 ? 0 : e4m3_rn_satfinite(amax_b * k)
//              d   = e4m3_decode(s) * global
//              inv = d == 0 ? 0 : min(1 / d, FLT_MAX)
//              code_i = e2m1_rn_satfinite(x_i * inv), even column in the low nibble.
// The two narrow conversions are the hardware ones (cvt.rn.satfinite.e4m3x2.f32 /
// cvt.rn.satfinite.e2m1x2.f32): round-to-nearest-even onto the format's grid with saturation to
// its largest finite value.
//
// Work layout of the stand-alone quantiser: one 128-thread CTA per row, so the row's group, its
// global scale and k are computed once per CTA; a lane owns eight elements (one 128-bit load),
// lane pairs share a block's amax through one shuffle, each lane stores its four code bytes as one
// 32-bit word (a warp writes 512 contiguous bytes) and the row's block scales are collected in
// shared memory and written as 128-bit stores.
#include "device_utils.cuh"
#include "host_checks.hpp"
#include "internal.hpp"
#include "nvfp4_math.cuh"
#include "q3x_b200.h"

namespace q3x {
namespace {

constexpr int kThreads = 256;
constexpr int kRowThreads = 128;
constexpr int kMaxRowScaleBytes = 8192;  // shared-memory staging of one row's block scales

// ---- group amax -------------------------------------------------------------------------

__global__ void __launch_bounds__(kThreads) group_amax_vec_kernel(const uint4* __restrict__ in, size_t nvec,
                                                                  size_t chunk, size_t group_vectors,
                                                                  uint32_t* amax_bits) {
  const size_t begin = static_cast<size_t>(blockIdx.x) * chunk;
  const size_t end = min(nvec, begin + chunk);
  size_t v = begin + threadIdx.x;
  size_t group = v / group_vectors;
  size_t boundary = (group + 1) * group_vectors;
  uint32_t top = 0;
  for (; v < end; v += kThreads) {
    while (v >= boundary) {
      if (top != 0) atomicMax(amax_bits + group, top);
      top = 0;
      ++group;
      boundary += group_vectors;
    }
    top = max(top, amax8(ld_stream(in + v)));
  }
  // one atomic per warp when the warp ends inside a single group
  const size_t g0 = static_cast<size_t>(__shfl_sync(kFullMask, static_cast<unsigned long long>(group), 0));
  if (__all_sync(kFullMask, group == g0)) {
    top = group_max_u32<32>(top);
    if ((threadIdx.x & 31) == 0 && top != 0) atomicMax(amax_bits + g0, top);
  } else if (top != 0) {
    atomicMax(amax_bits + group, top);
  }
}

__global__ void __launch_bounds__(kThreads) group_amax_scalar_kernel(const uint16_t* in, size_t count,
                                                                     size_t group_elements, uint32_t* amax_bits) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < count; i += stride) {
    const uint32_t m = in[i] & 0x7fffu;
    if (m != 0 && m < 0x7f80u) atomicMax(amax_bits + i / group_elements, m);
  }
}

__global__ void amax_to_scale_kernel(const uint32_t* amax_bits, size_t groups, float* global_scales) {
  const size_t g = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (g < groups) global_scales[g] = global_scale_from_amax_bits(amax_bits[g]);
}

// ---- quantiser --------------------------------------------------------------------------

// One CTA per row (grid-stride over rows).  kWideScales: the row's scale bytes are a multiple of 16
// and 16-byte aligned, so they go out as 128-bit stores from shared memory.
template <bool kWideScales>
__global__ void __launch_bounds__(kRowThreads) nvfp4_quantize_rows_kernel(const uint4* __restrict__ in, size_t rows,
                                                                          int row_vectors, size_t rows_per_scale,
                                                                          const float* __restrict__ global_scales,
                                                                          const uint32_t* __restrict__ amax_bits,
                                                                          float* global_scales_out,
                                                                          uint32_t* __restrict__ codes,
                                                                          uint8_t* __restrict__ scales) {
  __shared__ __align__(16) uint8_t scale_bytes[kWideScales ? kMaxRowScaleBytes : 16];
  __shared__ float inv_table[kRowThreads];  // indexed by E4M3 code 0..127
  static_assert(kRowThreads == 128, "one thread per non-negative E4M3 code");
  const int tid = threadIdx.x;
  for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t group = rows_per_scale ? row / rows_per_scale : 0;
    float global;
    if (amax_bits != nullptr) {
      // the scale is derived here from the group amax; the group's first row also publishes it
      global = global_scale_from_amax_bits(__ldg(amax_bits + group));
      if (tid == 0 && row == group * rows_per_scale) global_scales_out[group] = global;
    } else {
      global = __ldg(global_scales + group);
    }
    const float k = block_scale_factor(global);
    // 1 / (decode(s) * global) for every scale code, once per row instead of once per lane and block
    __syncthreads();  // the previous row's readers of inv_table / scale_bytes are done
    inv_table[tid] = block_inverse(static_cast<uint32_t>(tid), global);
    __syncthreads();
    const uint4* src = in + row * static_cast<size_t>(row_vectors);
    uint32_t* dst = codes + row * static_cast<size_t>(row_vectors);
    uint8_t* srow = scales + row * static_cast<size_t>(row_vectors / 2);
    // the bound is the same for all lanes of a warp, so the pair shuffle always has its partner
    for (int base = 0; base < row_vectors; base += 2 * kRowThreads) {
      uint4 x[2];
      bool valid[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int v = base + u * kRowThreads + tid;
        valid[u] = v < row_vectors;  // lane pairs are valid together (row_vectors is even)
        x[u] = valid[u] ? ld_stream(src + v) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int v = base + u * kRowThreads + tid;
        float f[8];
        unpack8(x[u], f);
        float m = amax8_float(f, x[u]);
        m = fmaxf(m, __shfl_xor_sync(kFullMask, m, 1));
        const uint32_t s = block_scale_code(m, k);
        if (valid[u]) {
          dst[v] = quantize8(f, inv_table[s]);
          if ((tid & 1) == 0) {
            if (kWideScales) scale_bytes[v >> 1] = static_cast<uint8_t>(s);
            else srow[v >> 1] = static_cast<uint8_t>(s);
          }
        }
      }
    }
    if (kWideScales) {
      __syncthreads();
      for (int i = tid; i < row_vectors / 32; i += kRowThreads)
        reinterpret_cast<uint4*>(srow)[i] = reinterpret_cast<const uint4*>(scale_bytes)[i];
    }
  }
}

// Any alignment: one thread per 16-element block.
__global__ void __launch_bounds__(kThreads) nvfp4_quantize_scalar_kernel(const uint16_t* in, size_t blocks,
                                                                         size_t row_blocks, size_t rows_per_scale,
                                                                         const float* global_scales, uint8_t* codes,
                                                                         uint8_t* scales) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t b = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; b < blocks; b += stride) {
    const uint16_t* x = in + b * 16;
    uint32_t m = 0;
    for (int i = 0; i < 16; ++i) {
      const uint32_t mag = x[i] & 0x7fffu;
      if (mag < 0x7f80u) m = max(m, mag);
    }
    const size_t row = b / row_blocks;
    const float global = global_scales[rows_per_scale ? row / rows_per_scale : 0];
    const uint32_t s = block_scale_code(m, block_scale_factor(global));
    const float inv = block_inverse(s, global);
    scales[b] = static_cast<uint8_t>(s);
    for (int h = 0; h < 2; ++h) {
      float f[8];
      for (int i = 0; i < 8; ++i) f[i] = __fmul_rn(bf16_to_float(x[h * 8 + i]), inv);
      const uint32_t word = encode_e2m1x8(f);
      for (int i = 0; i < 4; ++i) codes[b * 8 + h * 4 + i] = static_cast<uint8_t>(word >> (8 * i));
    }
  }
}

// ---- block scales in the tiled layout of block-scaled tensor-core MMA ------------------------------------
// A block-scaled tcgen05.mma reads its scale factors from 512-byte tiles that cover 128 rows x 4 blocks
// (64 columns): inside a tile the byte of (row r, block b) sits at (r % 32) * 16 + (r % 128 / 32) * 4 + b % 4,
// tiles are ordered row-tile major, and a ragged edge is padded with zero bytes to whole tiles.  The quantiser
// writes the canonical row-major [rows, cols / 16] view (the checkpoint layout,
// include/q3x/quantization/nvfp4.h:50-55); this kernel re-lays it out, one thread per destination byte.
__global__ void __launch_bounds__(kThreads) swizzle_scales_kernel(const uint8_t* __restrict__ row_major, size_t rows,
                                                                  size_t row_blocks, size_t block_tiles,
                                                                  size_t out_bytes, uint8_t* __restrict__ swizzled) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t o = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; o < out_bytes; o += stride) {
    const size_t tile = o / 512, in_tile = o % 512;
    const size_t row = tile / block_tiles * 128 + in_tile % 16 / 4 * 32 + in_tile / 16;
    const size_t block = tile % block_tiles * 4 + in_tile % 4;
    swizzled[o] = (row < rows && block < row_blocks) ? row_major[row * row_blocks + block] : uint8_t{0};
  }
}

// Block scales [rows, row_blocks] E4M3 -> [row_blocks, rows] bf16: the order and the type in which the weight-only
// tensor-core projection reads a weight's block scales (an E4M3 value is exact in bf16; one thread per destination
// element; a weight is re-laid out once, when it is loaded).
__global__ void __launch_bounds__(kThreads) transpose_scales_kernel(const uint8_t* __restrict__ row_major, size_t rows,
                                                                    size_t row_blocks, uint16_t* __restrict__ transposed) {
  const size_t total = rows * row_blocks;
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t o = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; o < total; o += stride) {
    const uint32_t code = row_major[(o % rows) * row_blocks + o / rows];
    const uint16_t magnitude = float_to_bf16(decode_e4m3_positive(code & 0x7fu));
    transposed[o] = static_cast<uint16_t>(magnitude | ((code & 0x80u) << 8));
  }
}

// Packed E2M1 codes x their E4M3 block scale -> bf16, one block of 16 weights per thread.  The product of a code
// (values 0, 0.5 .. 6: two significant bits) and a scale (four) has at most six significant bits: exact in bf16.
__global__ void __launch_bounds__(kThreads) widen_weights_kernel(const uint2* __restrict__ packed, const uint8_t* __restrict__ scales,
                                                                 size_t blocks, uint4* __restrict__ out) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < blocks; i += stride) {
    const uint2 codes = __ldg(packed + i);
    const uint32_t scale_code = scales[i];
    const float magnitude = decode_e4m3_positive(scale_code & 0x7fu);
    const float scale = (scale_code & 0x80u) ? -magnitude : magnitude;
    const uint32_t words[2] = {codes.x, codes.y};
    float f[16];
#pragma unroll
    for (int w = 0; w < 2; ++w)
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const uint32_t code = (words[w] >> (4 * n)) & 0xfu;
        // E2M1: exponent field e (2 bits), mantissa m: value = e == 0 ? 0.5 m : (1 + 0.5 m) * 2^(e - 1)
        const uint32_t e = (code >> 1) & 3u, m = code & 1u;
        const float value = e == 0 ? 0.5f * static_cast<float>(m) : (1.0f + 0.5f * static_cast<float>(m)) * static_cast<float>(1u << (e - 1));
        f[w * 8 + n] = ((code & 8u) ? -value : value) * scale;
      }
    float lo[8], hi[8];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      lo[n] = f[n];
      hi[n] = f[8 + n];
    }
    out[2 * i] = pack8(lo);
    out[2 * i + 1] = pack8(hi);
  }
}

__global__ void __launch_bounds__(kThreads) debug_encode_kernel(const float* in, size_t count, uint8_t* out,
                                                                int format) {
  const size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (i >= count) return;
  if (format == 0) {
    out[i] = static_cast<uint8_t>(encode_e4m3(in[i]));
  } else {
    const float f[8] = {in[i], 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    out[i] = static_cast<uint8_t>(encode_e2m1x8(f) & 0xfu);
  }
}

size_t group_count(size_t rows, size_t rows_per_scale) {
  if (rows == 0) return 0;
  return rows_per_scale == 0 ? 1 : (rows + rows_per_scale - 1) / rows_per_scale;
}

// shared shape checks of the NVFP4 entry points; *done marks a finished no-op
int check_matrix(const void* in, size_t rows, size_t cols, bool* done) {
  using namespace host;
  *done = false;
  if (cols % Q3X_B200_NVFP4_BLOCK != 0) return kInvalid;
  if (mul3_overflows(rows, cols, sizeof(uint16_t))) return kInvalid;
  if (rows == 0 || cols == 0) {
    *done = true;
    return kOk;
  }
  if (in == nullptr) return kInvalid;
  return kOk;
}

void enqueue_amax(const uint16_t* in, size_t rows, size_t cols, size_t rows_per_scale, uint32_t* amax_bits,
                  cudaStream_t s) {
  using namespace host;
  const size_t groups = group_count(rows, rows_per_scale);
  const size_t group_rows = rows_per_scale ? rows_per_scale : rows;
  cudaMemsetAsync(amax_bits, 0, groups * sizeof(uint32_t), s);
  if (aligned16(in) && cols % 8 == 0) {
    const size_t nvec = rows * cols / 8;
    const unsigned grid = grid_for(nvec, kThreads * 8, 8);
    size_t chunk = (nvec + grid - 1) / grid;
    chunk = (chunk + kThreads - 1) / kThreads * kThreads;
    const unsigned ctas = static_cast<unsigned>((nvec + chunk - 1) / chunk);
    group_amax_vec_kernel<<<ctas, kThreads, 0, s>>>(reinterpret_cast<const uint4*>(in), nvec, chunk,
                                                    group_rows * (cols / 8), amax_bits);
  } else {
    const size_t count = rows * cols;
    group_amax_scalar_kernel<<<grid_for(count, kThreads, 8), kThreads, 0, s>>>(in, count, group_rows * cols,
                                                                               amax_bits);
  }
}

void enqueue_scales(const uint32_t* amax_bits, size_t groups, float* global_scales, cudaStream_t s) {
  amax_to_scale_kernel<<<static_cast<unsigned>((groups + 127) / 128), 128, 0, s>>>(amax_bits, groups, global_scales);
}

// global_scales given: quantise with them.  Else amax_bits given: derive each group's scale from its
// amax word inside the quantiser and write it to global_scales_out.
void enqueue_quantize(const uint16_t* in, size_t rows, size_t cols, size_t rows_per_scale, const float* global_scales,
                      const uint32_t* amax_bits, float* global_scales_out, uint8_t* codes, uint8_t* scales,
                      cudaStream_t s) {
  using namespace host;
  if (global_scales == nullptr && !(aligned16(in) && (reinterpret_cast<uintptr_t>(codes) & 3u) == 0)) {
    // the scalar quantiser takes ready-made scales
    enqueue_scales(amax_bits, group_count(rows, rows_per_scale), global_scales_out, s);
    global_scales = global_scales_out;
    amax_bits = nullptr;
  }
  if (aligned16(in) && (reinterpret_cast<uintptr_t>(codes) & 3u) == 0 && cols / 8 <= 0x7fffffffu) {
    const int row_vectors = static_cast<int>(cols / 8);
    const bool wide = aligned16(scales) && (cols / 16) % 16 == 0 && cols / 16 <= kMaxRowScaleBytes;
    auto I = reinterpret_cast<const uint4*>(in);
    auto C = reinterpret_cast<uint32_t*>(codes);
    if (wide)
      nvfp4_quantize_rows_kernel<true><<<wave_grid(nvfp4_quantize_rows_kernel<true>, kRowThreads, rows, 1),
                                         kRowThreads, 0, s>>>(I, rows, row_vectors, rows_per_scale,
                                                                    global_scales, amax_bits, global_scales_out, C,
                                                                    scales);
    else
      nvfp4_quantize_rows_kernel<false><<<wave_grid(nvfp4_quantize_rows_kernel<false>, kRowThreads, rows, 1),
                                          kRowThreads, 0, s>>>(I, rows, row_vectors, rows_per_scale,
                                                                     global_scales, amax_bits, global_scales_out, C,
                                                                     scales);
  } else {
    const size_t blocks = rows * cols / 16;
    nvfp4_quantize_scalar_kernel<<<grid_for(blocks, kThreads, 8), kThreads, 0, s>>>(in, blocks, cols / 16,
                                                                                   rows_per_scale, global_scales,
                                                                                   codes, scales);
  }
}

// Clears the scratch words of a call, the sticky error word (the last one) excepted.  The multi-kernel
// paths clear before their first kernel (their amax words are raised with atomicMax) and again after their
// last one, so that every entry point leaves the scratch zero, which is what the single-kernel forms
// expect to find.
void clear_board(uint32_t* scratch, size_t rows, size_t groups, cudaStream_t s) {
  cudaMemsetAsync(scratch, 0, (fused_scratch_words(rows, groups) - 1) * sizeof(uint32_t), s);
}

// Every operand of an NVFP4 entry point besides the tensor being quantised: the three byte outputs and the
// scratch must not overlap each other nor any of `others` (inputs, weights and bf16 outputs).
struct QuantSpans {
  host::Span codes, scales, globals, scratch;
};
QuantSpans quant_spans(size_t rows, size_t cols, size_t groups, const void* codes, const void* scales,
                       const void* global_scales_out, const void* scratch) {
  using namespace host;
  return QuantSpans{span(codes, rows * cols / 2), span(scales, rows * cols / 16),
                    span(global_scales_out, groups * sizeof(float)),
                    span(scratch, scratch ? fused_scratch_words(rows, groups) * sizeof(uint32_t) : 0)};
}
template <size_t N>
bool quant_spans_collide(const QuantSpans& q, const host::Span (&others)[N]) {
  using namespace host;
  const Span mine[4] = {q.codes, q.scales, q.globals, q.scratch};
  for (int i = 0; i < 4; ++i) {
    if (wraps(mine[i])) return true;
    for (int j = i + 1; j < 4; ++j)
      if (overlap(mine[i], mine[j])) return true;
    for (size_t k = 0; k < N; ++k)
      if (overlap(mine[i], others[k])) return true;
  }
  return false;
}

int check_quant_outputs(const uint16_t* in, size_t rows, size_t cols, const void* codes, const void* scales) {
  using namespace host;
  if (codes == nullptr || scales == nullptr) return kInvalid;
  const Span si = span(in, rows * cols * 2), sc = span(codes, rows * cols / 2), ss = span(scales, rows * cols / 16);
  if (wraps(si) || wraps(sc) || wraps(ss) || overlap(si, sc) || overlap(si, ss) || overlap(sc, ss)) return kInvalid;
  return kOk;
}

}  // namespace
}  // namespace q3x

using namespace q3x;
using namespace q3x::host;

extern "C" size_t q3x_b200_nvfp4_group_count(size_t rows, size_t rows_per_scale) {
  return group_count(rows, rows_per_scale);
}

extern "C" size_t q3x_b200_nvfp4_scratch_words(size_t rows, size_t rows_per_scale) {
  return fused_scratch_words(rows, group_count(rows, rows_per_scale));
}

extern "C" int q3x_b200_group_amax(const uint16_t* in, size_t rows, size_t cols, size_t rows_per_scale,
                                   uint32_t* amax_bits, void* stream) {
  if (mul3_overflows(rows, cols, sizeof(uint16_t))) return kInvalid;
  if (rows == 0 || cols == 0) return kOk;
  if (in == nullptr || amax_bits == nullptr) return kInvalid;
  const Span si = span(in, rows * cols * 2), sa = span(amax_bits, group_count(rows, rows_per_scale) * 4);
  if (wraps(si) || overlap(si, sa)) return kInvalid;
  clear_stale_error();
  enqueue_amax(in, rows, cols, rows_per_scale, amax_bits, as_stream(stream));
  return launch_status();
}

extern "C" int q3x_b200_amax_to_global_scale(const uint32_t* amax_bits, size_t groups, float* global_scales,
                                             void* stream) {
  if (groups == 0) return kOk;
  if (amax_bits == nullptr || global_scales == nullptr || mul_overflows(groups, 4)) return kInvalid;
  if (overlap(span(amax_bits, groups * 4), span(global_scales, groups * 4))) return kInvalid;
  clear_stale_error();
  enqueue_scales(amax_bits, groups, global_scales, as_stream(stream));
  return launch_status();
}

extern "C" int q3x_b200_nvfp4_quantize(const uint16_t* in, size_t rows, size_t cols, size_t rows_per_scale,
                                       const float* global_scales, uint8_t* codes, uint8_t* scales, void* stream) {
  bool done;
  int st = check_matrix(in, rows, cols, &done);
  if (st != kOk || done) return st;
  if (global_scales == nullptr) return kInvalid;
  if ((st = check_quant_outputs(in, rows, cols, codes, scales)) != kOk) return st;
  clear_stale_error();
  enqueue_quantize(in, rows, cols, rows_per_scale, global_scales, nullptr, nullptr, codes, scales, as_stream(stream));
  return launch_status();
}

extern "C" int q3x_b200_nvfp4_quantize_dynamic(const uint16_t* in, size_t rows, size_t cols, size_t rows_per_scale,
                                               uint32_t* scratch, float* global_scales_out, uint8_t* codes,
                                               uint8_t* scales, void* stream) {
  bool done;
  int st = check_matrix(in, rows, cols, &done);
  if (st != kOk || done) return st;
  if (scratch == nullptr || global_scales_out == nullptr) return kInvalid;
  if ((st = check_quant_outputs(in, rows, cols, codes, scales)) != kOk) return st;
  const size_t groups = group_count(rows, rows_per_scale);
  {
    const Span others[] = {span(in, rows * cols * 2)};
    if (quant_spans_collide(quant_spans(rows, cols, groups, codes, scales, global_scales_out, scratch), others))
      return kInvalid;
  }
  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  enqueue_amax(in, rows, cols, rows_per_scale, scratch, s);
  enqueue_quantize(in, rows, cols, rows_per_scale, nullptr, scratch, global_scales_out, codes, scales, s);
  clear_board(scratch, rows, groups, s);
  return launch_status();
}

namespace {

// Which kernels an NVFP4 entry point may run: the single kernel with deferred quantisation
// (fused_nvfp4.cu), or the norm kernel with group amax followed by the quantiser.  Same bytes either way.
enum class Path { kAuto, kSingleKernel, kTwoKernels };

// Shared body of the residual + norm + NVFP4 entry points.  kAuto takes the single kernel where it
// applies and the two kernels otherwise; kSingleKernel refuses instead of falling back.
// `late_scratch`, when given, supplies the scratch after every argument check has passed (and is not
// called at all for a rejected or empty call); `scratch` is ignored then.
using ScratchProvider = uint32_t* (*)(int* status);
int residual_norm_nvfp4(const uint16_t* left, const uint16_t* right, const uint16_t* weight, size_t tokens,
                        size_t hidden, float eps, size_t rows_per_scale, uint16_t* residual_out,
                        uint16_t* normalized_out, uint32_t* scratch, float* global_scales_out, uint8_t* codes,
                        uint8_t* scales, void* stream, Path path, ScratchProvider late_scratch = nullptr) {
  bool done;
  int st = check_residual_norm(left, right, weight, tokens, hidden, eps, residual_out, normalized_out, &done);
  if (st != kOk) return st;
  if (hidden % Q3X_B200_NVFP4_BLOCK != 0) return kInvalid;
  if (done) return kOk;
  if (late_scratch != nullptr) scratch = nullptr;
  if (normalized_out == nullptr || (scratch == nullptr && late_scratch == nullptr) || global_scales_out == nullptr)
    return kInvalid;
  if ((st = check_quant_outputs(normalized_out, tokens, hidden, codes, scales)) != kOk) return st;
  const size_t groups = group_count(tokens, rows_per_scale);
  {
    const size_t bytes = tokens * hidden * 2;
    const Span others[] = {span(left, bytes), span(right, bytes), span(weight, hidden * 2), span(residual_out, bytes),
                           span(normalized_out, bytes)};
    if (quant_spans_collide(quant_spans(tokens, hidden, groups, codes, scales, global_scales_out, scratch), others))
      return kInvalid;
  }
  if (!norm_rows_vector_path(left, right, weight, nullptr, hidden, residual_out, normalized_out, NormMode::kCentered))
    return kNotSupported;
  if (late_scratch != nullptr) {
    int status = kOk;
    scratch = late_scratch(&status);
    if (scratch == nullptr) return status;
  }
  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  if (path != Path::kTwoKernels) {
    if (launch_residual_norm_nvfp4_fused(left, right, weight, tokens, hidden, eps, rows_per_scale, residual_out,
                                         normalized_out, scratch, global_scales_out, codes, scales, s))
      return launch_status();
    if (path == Path::kSingleKernel) return kNotSupported;
  }
  clear_board(scratch, tokens, groups, s);
  launch_norm_rows(NormMode::kCentered, left, right, weight, nullptr, tokens, hidden, eps, 1.0f, residual_out,
                   normalized_out, /*coherent=*/normalized_out == right, scratch,
                   rows_per_scale ? rows_per_scale : tokens, s);
  enqueue_quantize(normalized_out, tokens, hidden, rows_per_scale, nullptr, scratch, global_scales_out, codes, scales,
                   s);
  clear_board(scratch, tokens, groups, s);
  return launch_status();
}

int gated_norm_nvfp4(const uint16_t* in, const uint16_t* weight, const uint16_t* gate, size_t tokens,
                     size_t heads_per_row, size_t dim, float eps, size_t rows_per_scale, uint16_t* out,
                     uint32_t* scratch, float* global_scales_out, uint8_t* codes, uint8_t* scales, void* stream,
                     Path path) {
  if (!valid_epsilon(eps)) return kInvalid;
  if (mul3_overflows(tokens, heads_per_row, dim) || mul_overflows(tokens * heads_per_row * dim, 2)) return kInvalid;
  const size_t cols = heads_per_row * dim;
  if (cols % Q3X_B200_NVFP4_BLOCK != 0) return kInvalid;
  if (tokens == 0 || cols == 0) return kOk;
  if (in == nullptr || weight == nullptr || gate == nullptr || out == nullptr || scratch == nullptr ||
      global_scales_out == nullptr)
    return kInvalid;
  const size_t bytes = tokens * cols * 2;
  const Span si = span(in, bytes), sg = span(gate, bytes), so = span(out, bytes), sw = span(weight, dim * 2);
  if (wraps(si) || wraps(sg) || wraps(so) || partial_overlap(so, si) || partial_overlap(so, sg) || overlap(so, sw))
    return kInvalid;
  int st = check_quant_outputs(out, tokens, cols, codes, scales);
  if (st != kOk) return st;
  const size_t groups = group_count(tokens, rows_per_scale);
  {
    const Span others[] = {si, sg, so, sw};
    if (quant_spans_collide(quant_spans(tokens, cols, groups, codes, scales, global_scales_out, scratch), others))
      return kInvalid;
  }
  if (!norm_rows_vector_path(in, nullptr, weight, gate, dim, nullptr, out, NormMode::kPlainSiluGate) ||
      !(dim == 64 || dim == 128 || dim == 256))
    return kNotSupported;
  const size_t token_group = rows_per_scale ? rows_per_scale : tokens;
  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  if (path != Path::kTwoKernels) {
    if (launch_gated_norm_nvfp4_fused(in, weight, gate, tokens, heads_per_row, dim, eps, rows_per_scale, out, scratch,
                                      global_scales_out, codes, scales, s))
      return launch_status();
    if (path == Path::kSingleKernel) return kNotSupported;
  }
  clear_board(scratch, tokens, groups, s);
  launch_norm_rows(NormMode::kPlainSiluGate, in, nullptr, weight, gate, tokens * heads_per_row, dim, eps, 1.0f,
                   nullptr, out, /*coherent=*/out == in || out == gate, scratch, token_group * heads_per_row, s);
  enqueue_quantize(out, tokens, cols, rows_per_scale, nullptr, scratch, global_scales_out, codes, scales, s);
  clear_board(scratch, tokens, groups, s);
  return launch_status();
}

}  // namespace

extern "C" int q3x_b200_residual_add_rms_norm_nvfp4(const uint16_t* left, const uint16_t* right,
                                                    const uint16_t* weight, size_t tokens, size_t hidden, float eps,
                                                    size_t rows_per_scale, uint16_t* residual_out,
                                                    uint16_t* normalized_out, uint32_t* scratch,
                                                    float* global_scales_out, uint8_t* codes, uint8_t* scales,
                                                    void* stream) {
  return residual_norm_nvfp4(left, right, weight, tokens, hidden, eps, rows_per_scale, residual_out, normalized_out,
                             scratch, global_scales_out, codes, scales, stream, Path::kAuto);
}

extern "C" int q3x_b200_residual_add_rms_norm_nvfp4_single_pass(const uint16_t* left, const uint16_t* right,
                                                                const uint16_t* weight, size_t tokens, size_t hidden,
                                                                float eps, size_t rows_per_scale,
                                                                uint16_t* residual_out, uint16_t* normalized_out,
                                                                uint32_t* scratch, float* global_scales_out,
                                                                uint8_t* codes, uint8_t* scales, void* stream) {
  return residual_norm_nvfp4(left, right, weight, tokens, hidden, eps, rows_per_scale, residual_out, normalized_out,
                             scratch, global_scales_out, codes, scales, stream, Path::kSingleKernel);
}

namespace {

// Shared body of the pointwise + NVFP4 entry points: out = op(first, second) over [tokens, width], then
// its codes and scales.  `swiglu` selects silu(first) * second, else first * sigmoid(second).
int pointwise_nvfp4(bool swiglu, const uint16_t* first, const uint16_t* second, size_t tokens, size_t width,
                    size_t rows_per_scale, uint16_t* out, uint32_t* scratch, float* global_scales_out, uint8_t* codes,
                    uint8_t* scales, void* stream) {
  if (mul3_overflows(tokens, width, sizeof(uint16_t))) return kInvalid;
  if (width % Q3X_B200_NVFP4_BLOCK != 0) return kInvalid;
  if (tokens == 0 || width == 0) return kOk;
  if (first == nullptr || second == nullptr || out == nullptr || scratch == nullptr || global_scales_out == nullptr)
    return kInvalid;
  const size_t bytes = tokens * width * sizeof(uint16_t);
  const Span sa = span(first, bytes), sb = span(second, bytes), so = span(out, bytes);
  // out may be exactly one of the inputs (the reference's in-place forms); any partial overlap is refused
  if (wraps(sa) || wraps(sb) || wraps(so) || partial_overlap(so, sa) || partial_overlap(so, sb)) return kInvalid;
  int st = check_quant_outputs(out, tokens, width, codes, scales);
  if (st != kOk) return st;
  const size_t groups = group_count(tokens, rows_per_scale);
  {
    const Span others[] = {sa, sb, so};
    if (quant_spans_collide(quant_spans(tokens, width, groups, codes, scales, global_scales_out, scratch), others))
      return kInvalid;
  }
  cudaStream_t s = as_stream(stream);
  clear_stale_error();
  const bool fused = swiglu ? launch_silu_mul_nvfp4_fused(first, second, tokens, width, rows_per_scale, out, scratch,
                                                          global_scales_out, codes, scales, s)
                            : launch_sigmoid_gate_nvfp4_fused(first, second, tokens, width, rows_per_scale, out,
                                                              scratch, global_scales_out, codes, scales, s);
  if (fused) return launch_status();
  // separate kernels: the pointwise operator, the group amax of its output, the quantiser
  st = swiglu ? q3x_b200_silu_mul(first, second, tokens * width, out, stream)
              : q3x_b200_sigmoid_gate(first, second, tokens * width, out, stream);
  if (st != kOk) return st;
  clear_board(scratch, tokens, groups, s);
  enqueue_amax(out, tokens, width, rows_per_scale, scratch, s);
  enqueue_quantize(out, tokens, width, rows_per_scale, nullptr, scratch, global_scales_out, codes, scales, s);
  clear_board(scratch, tokens, groups, s);
  return launch_status();
}

}  // namespace

extern "C" int q3x_b200_silu_mul_nvfp4(const uint16_t* gate, const uint16_t* up, size_t tokens, size_t intermediate,
                                       size_t rows_per_scale, uint16_t* out, uint32_t* scratch,
                                       float* global_scales_out, uint8_t* codes, uint8_t* scales, void* stream) {
  return pointwise_nvfp4(true, gate, up, tokens, intermediate, rows_per_scale, out, scratch, global_scales_out, codes,
                         scales, stream);
}

extern "C" int q3x_b200_sigmoid_gate_nvfp4(const uint16_t* value, const uint16_t* gate, size_t tokens, size_t width,
                                           size_t rows_per_scale, uint16_t* out, uint32_t* scratch,
                                           float* global_scales_out, uint8_t* codes, uint8_t* scales, void* stream) {
  return pointwise_nvfp4(false, value, gate, tokens, width, rows_per_scale, out, scratch, global_scales_out, codes,
                         scales, stream);
}

extern "C" int q3x_b200_rms_norm_silu_gate_nvfp4(const uint16_t* in, const uint16_t* weight, const uint16_t* gate,
                                                 size_t tokens, size_t heads_per_row, size_t dim, float eps,
                                                 size_t rows_per_scale, uint16_t* out, uint32_t* scratch,
                                                 float* global_scales_out, uint8_t* codes, uint8_t* scales,
                                                 void* stream) {
  return gated_norm_nvfp4(in, weight, gate, tokens, heads_per_row, dim, eps, rows_per_scale, out, scratch,
                          global_scales_out, codes, scales, stream, Path::kAuto);
}

extern "C" int q3x_b200_rms_norm_silu_gate_nvfp4_single_pass(const uint16_t* in, const uint16_t* weight,
                                                             const uint16_t* gate, size_t tokens,
                                                             size_t heads_per_row, size_t dim, float eps,
                                                             size_t rows_per_scale, uint16_t* out, uint32_t* scratch,
                                                             float* global_scales_out, uint8_t* codes,
                                                             uint8_t* scales, void* stream) {
  return gated_norm_nvfp4(in, weight, gate, tokens, heads_per_row, dim, eps, rows_per_scale, out, scratch,
                          global_scales_out, codes, scales, stream, Path::kSingleKernel);
}

// ---------------------------------------------------------------------------------------------
// Residual add + RMSNorm + NVFP4 for callers that cannot allocate device memory.
//
// The regular entry point takes its scratch words from the caller.  Some callers have no way to
// provide them: code running inside a stream callback, a plugin that is
// handed input and output tensors by its host and nothing else, a real-time loop whose allocator
// is closed after start-up.  For them the scratch lives in the library itself, in the device array
// below; every GPU that loads the library carries these 64 KB until the process exits.
//
// The array's name is only a host-side handle for the symbol, not a device address, so the device
// address is looked up with cudaGetSymbolAddress, once per device and with that device current, and
// it is that pointer the kernels receive.
constexpr size_t kStaticScratchMaxTokens = Q3X_B200_STATIC_SCRATCH_MAX_TOKENS;
constexpr size_t kStaticScratchWords = kStaticScratchMaxTokens + 2;  // fused_scratch_words(max, groups <= max / 2)
static __device__ __align__(256) uint32_t g_static_scratch[kStaticScratchWords];

namespace {

// Device address of g_static_scratch on the current device, or nullptr with *status set.
uint32_t* static_scratch_address(int* status) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static uint32_t* address[kMaxDevices] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *status = static_cast<int>(err != cudaSuccess ? err : cudaErrorInvalidDevice);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (address[dev] == nullptr) {
    void* p = nullptr;
    err = cudaGetSymbolAddress(&p, g_static_scratch);
    if (err != cudaSuccess || p == nullptr) {
      *status = static_cast<int>(err != cudaSuccess ? err : cudaErrorInvalidSymbol);
      return nullptr;
    }
    address[dev] = static_cast<uint32_t*>(p);
  }
  *status = kOk;
  return address[dev];
}

}  // namespace

extern "C" size_t q3x_b200_static_scratch_max_tokens(void) { return kStaticScratchMaxTokens; }

extern "C" int q3x_b200_residual_add_rms_norm_nvfp4_static_scratch(
    const uint16_t* left, const uint16_t* right, const uint16_t* weight, size_t tokens, size_t hidden, float eps,
    size_t rows_per_scale, uint16_t* residual_out, uint16_t* normalized_out, float* global_scales_out, uint8_t* codes,
    uint8_t* scales, void* stream) {
  // more rows than the built-in scratch has words for: refuse before touching anything
  if (tokens > kStaticScratchMaxTokens) return kInvalid;
  if (fused_scratch_words(tokens, group_count(tokens, rows_per_scale)) > kStaticScratchWords) return kInvalid;
  // From here on this is the regular two-kernel path; it clears the scratch words it uses itself.  The
  // array's address is only looked up once every argument check has passed, so a rejected or empty call
  // touches no CUDA state.
  return residual_norm_nvfp4(left, right, weight, tokens, hidden, eps, rows_per_scale, residual_out, normalized_out,
                             nullptr, global_scales_out, codes, scales, stream, Path::kTwoKernels,
                             &static_scratch_address);
}

extern "C" size_t q3x_b200_nvfp4_swizzled_scale_bytes(size_t rows, size_t cols) {
  if (rows == 0 || cols == 0) return 0;
  const size_t row_tiles = (rows + 127) / 128, block_tiles = (cols / Q3X_B200_NVFP4_BLOCK + 3) / 4;
  return mul3_overflows(row_tiles, block_tiles, 512) ? 0 : row_tiles * block_tiles * 512;
}

extern "C" int q3x_b200_nvfp4_swizzle_block_scales(const uint8_t* row_major, size_t rows, size_t cols, uint8_t* swizzled,
                                                   void* stream) {
  if (cols % Q3X_B200_NVFP4_BLOCK != 0 || mul3_overflows(rows, cols, 2)) return kInvalid;
  if (rows == 0 || cols == 0) return kOk;
  if (row_major == nullptr || swizzled == nullptr) return kInvalid;
  const size_t out_bytes = q3x_b200_nvfp4_swizzled_scale_bytes(rows, cols);
  if (out_bytes == 0) return kInvalid;
  const size_t row_blocks = cols / Q3X_B200_NVFP4_BLOCK;
  if (overlap(span(row_major, rows * row_blocks), span(swizzled, out_bytes))) return kInvalid;
  clear_stale_error();
  swizzle_scales_kernel<<<grid_for(out_bytes, kThreads, 8), kThreads, 0, as_stream(stream)>>>(
      row_major, rows, row_blocks, (row_blocks + 3) / 4, out_bytes, swizzled);
  return launch_status();
}

extern "C" int q3x_b200_nvfp4_transpose_block_scales(const uint8_t* row_major, size_t rows, size_t cols,
                                                     uint16_t* transposed, void* stream) {
  if (cols % Q3X_B200_NVFP4_BLOCK != 0 || mul3_overflows(rows, cols, 2)) return kInvalid;
  if (rows == 0 || cols == 0) return kOk;
  if (row_major == nullptr || transposed == nullptr) return kInvalid;
  const size_t row_blocks = cols / Q3X_B200_NVFP4_BLOCK;
  if (overlap(span(row_major, rows * row_blocks), span(transposed, rows * row_blocks * 2))) return kInvalid;
  clear_stale_error();
  transpose_scales_kernel<<<grid_for(rows * row_blocks, kThreads, 8), kThreads, 0, as_stream(stream)>>>(
      row_major, rows, row_blocks, transposed);
  return launch_status();
}

extern "C" int q3x_b200_nvfp4_weights_to_bf16(const uint8_t* packed_weights, const uint8_t* block_scales, size_t rows,
                                              size_t cols, uint16_t* out, void* stream) {
  if (cols % Q3X_B200_NVFP4_BLOCK != 0 || mul3_overflows(rows, cols, 2)) return kInvalid;
  if (rows == 0 || cols == 0) return kOk;
  if (packed_weights == nullptr || block_scales == nullptr || out == nullptr) return kInvalid;
  if (!aligned16(packed_weights) || !aligned16(out)) return kNotSupported;
  const size_t blocks = rows * (cols / Q3X_B200_NVFP4_BLOCK);
  const Span so = span(out, rows * cols * 2);
  if (overlap(so, span(packed_weights, rows * cols / 2)) || overlap(so, span(block_scales, blocks))) return kInvalid;
  clear_stale_error();
  widen_weights_kernel<<<grid_for(blocks, kThreads, 8), kThreads, 0, as_stream(stream)>>>(
      reinterpret_cast<const uint2*>(packed_weights), block_scales, blocks, reinterpret_cast<uint4*>(out));
  return launch_status();
}

// Diagnostics: the two narrow conversions on their own, so that tests can sweep them against the
// CPU definition.  format 0 = E4M3 (one byte per value), 1 = E2M1 (one nibble per value, in a byte).
extern "C" int q3x_b200_debug_encode(const float* in, size_t count, int format, uint8_t* out, void* stream) {
  if (count == 0) return kOk;
  if (in == nullptr || out == nullptr || (format != 0 && format != 1)) return kInvalid;
  clear_stale_error();
  debug_encode_kernel<<<static_cast<unsigned>((count + kThreads - 1) / kThreads), kThreads, 0, as_stream(stream)>>>(
      in, count, out, format);
  return launch_status();
}

// Diagnostics: with `plant` non-zero, leaves a stale error in this library's CUDA runtime through a
// host-side argument error (an invalid copy direction; nothing reaches the GPU), the situation the
// entry points must clear before their own launch.  Returns the pending last-error without
// clearing it.
extern "C" int q3x_b200_debug_stale_error(int plant) {
  if (plant) {
    int dummy = 0;
    (void)cudaMemcpyAsync(&dummy, &dummy, sizeof(dummy), static_cast<cudaMemcpyKind>(99), nullptr);
  }
  return static_cast<int>(cudaPeekAtLastError());
}

extern "C" int q3x_b200_abi_version(void) { return Q3X_B200_ABI_VERSION; }

extern "C" const char* q3x_b200_error_string(int status) {
  return cudaGetErrorString(static_cast<cudaError_t>(status));
}
