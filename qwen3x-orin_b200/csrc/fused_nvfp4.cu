// Single-kernel operator + NVFP4: residual add + centred RMSNorm + quantisation, the GDN gated
// RMSNorm * silu(z) + quantisation, and SwiGLU / sigmoid gate + quantisation, each crossing HBM once.
// (One or two rows take a single-CTA form instead, see "a handful of rows" below.)
//
// The NVFP4 global scale of a group of rows is its amax, which is only known once every row of the
// group has been normalised -- a dependency across CTAs.  It is resolved without a second pass over
// HBM by DEFERRING the quantisation of a row by `lag` rows, inside one launch whose CTAs (128
// threads) alternate between two roles:
//   * even CTAs ("phase A", CTA 2k): normalise row k exactly like the stand-alone norm kernel (whole
//     row in registers, one trip per tensor), write the bf16 outputs, raise the group's amax word with
//     one atomic and then count the row into the group's arrival counter (a release reduction);
//   * odd CTAs ("phase B", CTA 2k + 1): quantise row k - lag, which was written `lag` rows earlier and
//     is still in L2 (lag x row bytes is a few tens of MB at most; the launcher refuses longer groups).
//     They need the arrival counter of that row's group to be complete.  lag = group rows + the number
//     of CTAs that can be resident, so every row of that group belongs to a CTA that is at least one
//     full residency older: the counter is normally complete already and the wait is a single load.
//   The two roles sit in different CTAs so that neither holds registers while the other waits on
//   memory: the in-flight loads of phase A are what keeps HBM busy.
// Progress: phase-A CTAs never wait, and the rows a phase-B CTA waits for belong to CTAs with a
// smaller index, which the hardware has started earlier (CTAs of a 1-D grid start in index order).
// Every wait is bounded all the same; a CTA that gives up sets the error word and carries on, so the
// kernel always terminates and a missed dependency is reported, never silent.  The error word is
// STICKY: the library only ever ORs into it, so a caller clears it once, runs any number of calls and
// reads it once.
// No L2 eviction hints: marking the streamed operands evict-first (so that the normalised rows awaiting
// phase B would be what stays cached) measured 2 - 5 % SLOWER than plain accesses; lag x row bytes is
// small against the L2 as it is.
//
// Scratch words (uint32): G group amax words, then G arrival counters (each on an L2 line of its own
// when the scratch is large enough), last word = error flag.  The words must be ZERO when a launch
// starts and the launch leaves them zero again, so no memset node precedes the kernel: the phase-B CTAs
// of a group count themselves into the group's arrival counter after they have read its amax, and the
// one that brings the counter to twice the group's rows -- the last reader -- clears both words.
#include "device_utils.cuh"
#include "host_checks.hpp"
#include "internal.hpp"
#include "norm_math.cuh"
#include "nvfp4_math.cuh"
#include "pointwise_ops.cuh"
#include "q3x_b200.h"

namespace q3x {
namespace {

constexpr int kMaxWarps = 16;                // warps of the largest CTA shape
// Resident CTAs per SM the kernels are compiled for.  The launch is latency-bound (half of the CTAs sit
// on L2 round trips), so occupancy pays: eight CTAs (64 registers) for rows of up to 768 vectors,
// measured 17 % faster than the five the compiler would pick; wider rows need the registers.
constexpr int min_ctas_per_sm(int team, int vpt) { return team == 128 && vpt <= 6 ? 8 : 5 * 128 / team; }
constexpr int kSpinLimit = 1 << 20;          // polls of the arrival counter before giving up (~1 s)
constexpr size_t kMaxLagBytes = 48u << 20;   // normalised bytes that may sit in L2 between the phases
constexpr int kMaxRowScaleBytes = 512;       // block scales of one row (row_vectors / 2)

__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// counts the caller into *p and returns the previous value; orders the caller's earlier loads before the
// addition and the addition before its later stores, at GPU scope
__device__ __forceinline__ uint32_t add_acq_rel(uint32_t* p) {
  uint32_t old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(p) : "memory");
  return old;
}

struct Board {
  uint32_t* amax;     // group g at amax[g * stride]
  uint32_t* count;    // group g at count[g * stride]
  uint32_t* error;    // [1]
  float* global_out;  // [G] the global scales, written by the CTA that quantises a group's first row
  size_t rows, group_rows;
  unsigned lag;
  unsigned stride;    // words between the slots of neighbouring groups (32 = one L2 line each, or 1)
};

struct QuantOut {
  uint32_t* codes;  // [rows, row_vectors] words
  uint8_t* scales;  // [rows, row_vectors / 2] bytes
  bool wide_scale_stores;
};

constexpr uint32_t kNoTicket = 0xffffffffu;

struct TeamShared {
  float sums[kMaxWarps];
  uint32_t tops[kMaxWarps];
  uint32_t group_amax;
  float inv_table[128];  // indexed by E4M3 code 0..127
  __align__(16) uint8_t scale_bytes[kMaxRowScaleBytes];
};

// Phase A epilogue.  The barrier orders every thread's stores of the row before thread 0's arrival
// count, whose release semantics order them (and the amax atomic) before it at GPU scope.
template <int WARPS>
__device__ __forceinline__ void publish_row(const Board& board, TeamShared& ts, size_t row, float thread_top) {
  const uint32_t warp_top = group_max_u32<32>(amax_bits_of(thread_top));
  if ((threadIdx.x & 31) == 0) ts.tops[threadIdx.x >> 5] = warp_top;
  __syncthreads();
  if (threadIdx.x == 0) {
    const size_t slot = row / board.group_rows * board.stride;
    uint32_t m = 0;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) m = max(m, ts.tops[w]);
    if (m != 0) atomicMax(board.amax + slot, m);
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(board.count + slot) : "memory");
  }
}

// Phase B prologue: the amax bits of the group of `row`, once all of the group's rows have arrived.
// One thread polls (a single request per CTA on the counter's L2 line); the barrier then orders its
// acquire before every thread's loads of the row.  Thread 0 also counts itself into the arrival counter
// as a reader (after its load of the amax word); *ticket receives the counter's previous value, which
// retire_group() looks at once the row is quantised -- the round trip of that atomic is hidden behind
// the quantisation.  kNoTicket = the wait gave up (or not thread 0): nothing to retire.
__device__ __forceinline__ uint32_t await_group_amax(const Board& board, TeamShared& ts, size_t group,
                                                     uint32_t* ticket) {
  *ticket = kNoTicket;
  if (threadIdx.x == 0) {
    const size_t first = group * board.group_rows;
    const uint32_t need = static_cast<uint32_t>(min(board.group_rows, board.rows - first));
    const size_t slot = group * board.stride;
    int polls = 0;
    bool complete = true;
    while (ld_acquire(board.count + slot) < need) {
      if (++polls >= kSpinLimit) {
        atomicOr(board.error, 1u);
        complete = false;
        break;
      }
      __nanosleep(200);
    }
    ts.group_amax = ld_relaxed(board.amax + slot);
    if (complete) *ticket = add_acq_rel(board.count + slot);
  }
  __syncthreads();
  return ts.group_amax;
}

// Phase B epilogue (thread 0): the reader that finds the counter at 2 x rows - 1 is the group's last
// one -- every other reader has loaded the amax word before its own addition -- and returns both words
// to zero for the next launch that uses this scratch.
__device__ __forceinline__ void retire_group(const Board& board, size_t group, uint32_t ticket) {
  if (threadIdx.x != 0 || ticket == kNoTicket) return;
  const size_t first = group * board.group_rows;
  const uint32_t need = static_cast<uint32_t>(min(board.group_rows, board.rows - first));
  if (ticket == 2u * need - 1u) {
    const size_t slot = group * board.stride;
    board.amax[slot] = 0u;
    board.count[slot] = 0u;
  }
}

// Quantises one normalised row, held in registers (thread tid owns vectors tid + k * TEAM), under the global
// scale of `amax_bits`.
template <int TEAM, int VPT, bool FAST>
__device__ __forceinline__ void quantize_held(const uint4 (&y)[VPT], int row_vectors, uint32_t amax_bits,
                                              TeamShared& ts, uint32_t* codes_row, uint8_t* scales_row,
                                              bool wide_scale_stores) {
  const int tid = threadIdx.x;
  const float global = global_scale_from_amax_bits(amax_bits);
  const float k = block_scale_factor(global);
  if (tid < 128) ts.inv_table[tid] = block_inverse(static_cast<uint32_t>(tid), global);
  __syncthreads();
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * TEAM;
    const bool valid = FAST || v < row_vectors;  // lane pairs are valid together (row_vectors is even)
    float f[8];
    unpack8(y[i], f);
    float m = amax8_float(f, y[i]);
    m = fmaxf(m, __shfl_xor_sync(kFullMask, m, 1));
    const uint32_t s = block_scale_code(m, k);
    if (valid) {
      st_u32(codes_row + v, quantize8(f, ts.inv_table[s]));
      if ((tid & 1) == 0) {
        if (FAST || wide_scale_stores) ts.scale_bytes[v >> 1] = static_cast<uint8_t>(s);
        else scales_row[v >> 1] = static_cast<uint8_t>(s);
      }
    }
  }
  if (FAST || wide_scale_stores) {  // row_vectors / 2 bytes, a multiple of 16, written as 128-bit stores
    __syncthreads();
    if (tid < row_vectors / 32)
      st_vec(reinterpret_cast<uint4*>(scales_row) + tid, reinterpret_cast<const uint4*>(ts.scale_bytes)[tid]);
  }
}

// The same for a row that waits in L2: the loads are issued first and are in flight while the reciprocal
// table of the global scale is built.
template <int TEAM, int VPT, bool FAST>
__device__ __forceinline__ void quantize_row(const uint4* row_in, int row_vectors, uint32_t amax_bits, TeamShared& ts,
                                             uint32_t* codes_row, uint8_t* scales_row, bool wide_scale_stores) {
  const int tid = threadIdx.x;
  uint4 y[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * TEAM;
    y[i] = FAST || v < row_vectors ? ld_l2(row_in + v) : make_uint4(0, 0, 0, 0);
  }
  quantize_held<TEAM, VPT, FAST>(y, row_vectors, amax_bits, ts, codes_row, scales_row, wide_scale_stores);
}

// Phase B proper: waits for the group of `row`, publishes its global scale (first row only), quantises.
template <int TEAM, int VPT, bool FAST>
__device__ __forceinline__ void quantize_cached_row(const uint4* row_in, int row_vectors, const Board& board,
                                                    TeamShared& ts, size_t row, uint32_t* codes_row,
                                                    uint8_t* scales_row, bool wide_scale_stores) {
  const size_t group = row / board.group_rows;
  uint32_t ticket;
  const uint32_t amax_bits = await_group_amax(board, ts, group, &ticket);
  if (threadIdx.x == 0 && row == group * board.group_rows)
    board.global_out[group] = global_scale_from_amax_bits(amax_bits);
  quantize_row<TEAM, VPT, FAST>(row_in, row_vectors, amax_bits, ts, codes_row, scales_row, wide_scale_stores);
  retire_group(board, group, ticket);
}

// Phase B of either kernel: CTA 2k + 1 quantises row k - lag of `normalized`.
template <int TEAM, int VPT, bool FAST>
__device__ __forceinline__ void phase_b(const uint4* normalized, int row_vectors, const Board& board, TeamShared& ts,
                                        const QuantOut& q) {
  const size_t idx = blockIdx.x >> 1;
  if (idx < board.lag || idx - board.lag >= board.rows) return;
  const size_t row = idx - board.lag;
  quantize_cached_row<TEAM, VPT, FAST>(normalized + row * static_cast<size_t>(row_vectors), row_vectors, board, ts, row,
                           q.codes + row * static_cast<size_t>(row_vectors),
                           q.scales + row * static_cast<size_t>(row_vectors / 2), q.wide_scale_stores);
}

// Phase A of the residual operator on one row: residual add, rounding, centred RMSNorm, both stores.
// Returns the calling thread's share of the row's amax (see amax8_float).  SINGLE: the form for a CTA that
// handles a row or two and nothing else -- the weights are requested together with the row (a fresh CTA
// finds them in L2, not in L1, and would otherwise wait for them after the reduction) and `held` receives
// the thread's normalised vectors (zeros beyond the row).
template <int TEAM, int VPT, bool FAST, bool SINGLE = false>
__device__ __forceinline__ float residual_norm_row(const uint4* left, const uint4* right,
                                                   const uint4* __restrict__ weight, size_t row, int row_vectors,
                                                   float width, float eps, uint4* residual_out, uint4* normalized_out,
                                                   bool coherent, TeamShared& ts, uint4* held = nullptr) {
  const int tid = threadIdx.x;
  const size_t base = row * static_cast<size_t>(row_vectors);
  uint4 x[VPT], r[VPT], w[SINGLE ? VPT : 1];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * TEAM;
    if (FAST) {
      x[i] = ld_stream(left + base + v);
    } else {
      x[i] = make_uint4(0, 0, 0, 0);
      if (v < row_vectors) x[i] = coherent ? ld_vec(left + base + v) : ld_stream(left + base + v);
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * TEAM;
    if (FAST) {
      r[i] = ld_stream(right + base + v);
    } else {
      r[i] = make_uint4(0, 0, 0, 0);
      if (v < row_vectors) r[i] = coherent ? ld_vec(right + base + v) : ld_stream(right + base + v);
    }
  }
  if (SINGLE) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * TEAM;
      w[i] = v < row_vectors ? ld_weight(weight + v) : make_uint4(0, 0, 0, 0);
    }
  }
  float partial = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    float a[8], b[8];
    unpack8(x[i], a);
    unpack8(r[i], b);
    add8(a, b);
    x[i] = pack8(a);
    const int v = tid + i * TEAM;
    if (FAST || v < row_vectors) st_vec(residual_out + base + v, x[i]);
    partial += sum_squares8(x[i]);
  }
  const float total = block_sum<TEAM / 32>(partial, ts.sums);
  const float inv = inverse_rms(total, 1.0f / width, eps);
  float top = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * TEAM;
    if (FAST || v < row_vectors) {
      const uint4 gamma = SINGLE ? w[i] : ld_weight(weight + v);
      const uint4 y = scale8<NormMode::kCentered, true>(x[i], gamma, make_uint4(0, 0, 0, 0), inv, &top);
      st_vec(normalized_out + base + v, y);  // this is what phase B finds in L2
      if (SINGLE) held[i] = y;
    } else if (SINGLE) {
      held[i] = make_uint4(0, 0, 0, 0);
    }
  }
  return top;
}

// ---- residual add + centred RMSNorm + NVFP4 ------------------------------------------------
// `coherent`: an output aliases an input exactly (row i is read and written by the same CTA only).
// FAST: the row fills the CTA exactly (row_vectors == TEAM * VPT), nothing aliases and the scale bytes go
// out as 128-bit stores -- the bounds checks, zero fills and per-load branches of the general form
// (a fifth of its instructions) are compiled out.
template <int TEAM, int VPT, bool FAST>
__global__ void __launch_bounds__(TEAM, min_ctas_per_sm(TEAM, VPT)) residual_norm_nvfp4_kernel(
    const uint4* left, const uint4* right, const uint4* __restrict__ weight, int row_vectors, float width, float eps,
    uint4* residual_out, uint4* normalized_out, bool coherent, Board board, QuantOut q) {
  __shared__ TeamShared ts;
  if (blockIdx.x & 1u) {
    phase_b<TEAM, VPT, FAST>(normalized_out, row_vectors, board, ts, q);
    return;
  }
  const size_t row = blockIdx.x >> 1;
  if (row >= board.rows) return;
  const float top = residual_norm_row<TEAM, VPT, FAST>(left, right, weight, row, row_vectors, width, eps, residual_out,
                                                       normalized_out, coherent, ts);
  publish_row<TEAM / 32>(board, ts, row, top);
}

// Phase A of the gated-norm operator on one token: per-head RMSNorm * weight * silu(z), store.
template <int TEAM, int VPT, bool FAST>
__device__ __forceinline__ float gated_norm_row(const uint4* in, const uint4* gate, const uint4* __restrict__ weight,
                                                size_t row, int row_vectors, float eps, uint4* out, bool coherent,
                                                uint4* held = nullptr) {
  const int tid = threadIdx.x;
  const size_t base = row * static_cast<size_t>(row_vectors);
  const uint4 w = ld_weight(weight + (tid & 15));
  uint4 x[VPT], z[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * TEAM;
    if (FAST) {
      x[i] = ld_stream(in + base + v);
      z[i] = ld_stream(gate + base + v);
    } else {
      x[i] = z[i] = make_uint4(0, 0, 0, 0);
      if (v < row_vectors) {
        x[i] = coherent ? ld_vec(in + base + v) : ld_stream(in + base + v);
        z[i] = coherent ? ld_vec(gate + base + v) : ld_stream(gate + base + v);
      }
    }
  }
  float top = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * TEAM;
    const float sum = group_sum<16>(sum_squares8(x[i]));  // every lane takes part; idle heads sum zeros
    const float inv = inverse_rms(sum, 1.0f / 128.0f, eps);
    if (FAST || v < row_vectors) {
      const uint4 y = scale8<NormMode::kPlainSiluGate, true>(x[i], w, z[i], inv, &top);
      st_vec(out + base + v, y);
      if (held != nullptr) held[i] = y;
    } else if (held != nullptr) {
      held[i] = make_uint4(0, 0, 0, 0);
    }
  }
  return top;
}

// ---- gated RMSNorm * silu(z) over heads of 128 + NVFP4 ----------------------------------------
// A row is one token: heads_per_row heads of 16 vectors; 16 consecutive lanes own one head.
template <int TEAM, int VPT, bool FAST>
__global__ void __launch_bounds__(TEAM, min_ctas_per_sm(TEAM, VPT)) gated_norm_nvfp4_kernel(
    const uint4* in, const uint4* gate, const uint4* __restrict__ weight, int row_vectors, float eps, uint4* out,
    bool coherent, Board board, QuantOut q) {
  __shared__ TeamShared ts;
  if (blockIdx.x & 1u) {
    phase_b<TEAM, VPT, FAST>(out, row_vectors, board, ts, q);
    return;
  }
  const size_t row = blockIdx.x >> 1;
  if (row >= board.rows) return;
  const float top = gated_norm_row<TEAM, VPT, FAST>(in, gate, weight, row, row_vectors, eps, out, coherent);
  publish_row<TEAM / 32>(board, ts, row, top);
}

// ---- a handful of rows (decode) ------------------------------------------------------------------
// Up to kSmallRows rows: one CTA per scale group normalises its rows, keeps the results in registers,
// reduces the group amax inside the CTA and quantises what it holds -- nothing crosses CTAs: no counters,
// no waits, the scratch is not touched at all, and the normalised rows are not read back.
// Measured per call inside a CUDA graph: 4.3 us against 8.2 us for one row; from four rows on the rows'
// serial walk costs more than the cleared scratch, so the limit is two.
// The kernel may be launched to overlap the end of the kernel before it in the stream (programmatic
// dependent launch): it touches no memory before wait_for_prior_kernels().
constexpr size_t kSmallRows = 2;

template <int WARPS>
__device__ __forceinline__ uint32_t cta_amax_bits(TeamShared& ts, float thread_top) {
  const uint32_t warp_top = group_max_u32<32>(amax_bits_of(thread_top));
  if ((threadIdx.x & 31) == 0) ts.tops[threadIdx.x >> 5] = warp_top;
  __syncthreads();
  uint32_t m = 0;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) m = max(m, ts.tops[w]);
  return m;
}

template <int TEAM, int VPT, bool GATED>
__global__ void __launch_bounds__(TEAM) small_norm_nvfp4_kernel(const uint4* a, const uint4* b,
                                                                 const uint4* __restrict__ weight, int row_vectors,
                                                                 float width, float eps, uint4* residual_out,
                                                                 uint4* out, bool coherent, size_t rows,
                                                                 size_t group_rows, float* global_out, QuantOut q) {
  __shared__ TeamShared ts;
  release_next_kernel();
  wait_for_prior_kernels();
  const size_t first = blockIdx.x * group_rows;
  const size_t last = min(rows, first + group_rows);  // at most kSmallRows rows
  uint4 held[kSmallRows][VPT];
  float top = 0.0f;
#pragma unroll
  for (size_t r = 0; r < kSmallRows; ++r) {
    const size_t row = first + r;
    if (row < last) {
      const float t = GATED ? gated_norm_row<TEAM, VPT, false>(a, b, weight, row, row_vectors, eps, out, coherent, held[r])
                            : residual_norm_row<TEAM, VPT, false, true>(a, b, weight, row, row_vectors, width,
                                                                        eps, residual_out, out, coherent, ts, held[r]);
      top = fmaxf(top, t);
      __syncthreads();  // the reduction scratch is reused by the next row
    }
  }
  const uint32_t amax_bits = cta_amax_bits<TEAM / 32>(ts, top);
  if (threadIdx.x == 0) global_out[blockIdx.x] = global_scale_from_amax_bits(amax_bits);
#pragma unroll
  for (size_t r = 0; r < kSmallRows; ++r) {
    const size_t row = first + r;
    if (row < last) {
      quantize_held<TEAM, VPT, false>(held[r], row_vectors, amax_bits, ts, q.codes + row * static_cast<size_t>(row_vectors),
                                      q.scales + row * static_cast<size_t>(row_vectors / 2), q.wide_scale_stores);
      __syncthreads();  // the reciprocal table and the scale bytes are reused by the next row
    }
  }
}

// ---- pointwise operator (SwiGLU, sigmoid gate) + NVFP4 ------------------------------------------
// The operator is pointwise, so the unit of work is not a row but a CHUNK of TEAM * VPT consecutive
// vectors of the flattened [tokens, intermediate] tensor; the launcher only takes this path when a full
// scale group is a whole number of chunks, so a chunk belongs to exactly one group.  Everything else
// (roles, lag, arrival counters) is the scheme above with "row" read as "chunk".  `count` is the number
// of valid vectors of the tensor; only the last chunk can be short.
template <class Op, int TEAM, int VPT, bool FAST>
__global__ void __launch_bounds__(TEAM, min_ctas_per_sm(TEAM, VPT)) pointwise_nvfp4_kernel(
    const uint4* gate, const uint4* up, uint4* out, size_t count, bool coherent, Board board, QuantOut q) {
  __shared__ TeamShared ts;
  constexpr int kChunk = TEAM * VPT;
  const int tid = threadIdx.x;
  const size_t idx = blockIdx.x >> 1;
  if (blockIdx.x & 1u) {
    if (idx < board.lag || idx - board.lag >= board.rows) return;
    const size_t chunk = idx - board.lag;
    const size_t base = chunk * kChunk;
    const int n = FAST ? kChunk : static_cast<int>(min(static_cast<size_t>(kChunk), count - base));
    quantize_cached_row<TEAM, VPT, FAST>(out + base, n, board, ts, chunk, q.codes + base, q.scales + base / 2,
                                         q.wide_scale_stores);
    return;
  }
  if (idx >= board.rows) return;
  const size_t base = idx * kChunk;
  const int n = FAST ? kChunk : static_cast<int>(min(static_cast<size_t>(kChunk), count - base));
  uint4 g[VPT], u[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * TEAM;
    if (FAST) {
      g[i] = ld_stream(gate + base + v);
      u[i] = ld_stream(up + base + v);
    } else {
      g[i] = u[i] = make_uint4(0, 0, 0, 0);
      if (v < n) {
        g[i] = coherent ? ld_vec(gate + base + v) : ld_stream(gate + base + v);
        u[i] = coherent ? ld_vec(up + base + v) : ld_stream(up + base + v);
      }
    }
  }
  float top = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * TEAM;
    float a[8], b[8];
    unpack8(g[i], a);
    unpack8(u[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = Op::apply(a[j], b[j]);
    const uint4 y = pack8(a);
    top = fmaxf(top, amax8_float(a, y));
    if (FAST || v < n) st_vec(out + base + v, y);  // phase B finds it in L2
  }
  publish_row<TEAM / 32>(board, ts, idx, top);
}

// CTA shapes (threads, vectors per thread), tried in this order: the first one that holds a row wins.
// 128 threads with the whole row in registers measured fastest for 5120- and 6144-wide rows; wider
// CTAs with fewer vectors per thread (160 x 4, 256 x 3, 320 x 2) were 2 - 25 % slower.
#define Q3X_FUSED_SHAPES Q3X_SHAPE(128, 1) Q3X_SHAPE(128, 2) Q3X_SHAPE(128, 3) Q3X_SHAPE(128, 4) Q3X_SHAPE(128, 5) \
    Q3X_SHAPE(128, 6) Q3X_SHAPE(128, 7) Q3X_SHAPE(128, 8)

// Lag and grid of one launch; false when the deferred scheme does not apply (a group so long that its
// rows would not stay in L2 until they are quantised).
template <typename K>
bool plan_launch(K kernel, int team, size_t rows, size_t group_rows, size_t row_bytes, unsigned* lag_out,
                 unsigned* grid_out) {
  const size_t resident = host::resident_grid(kernel, team);
  const size_t lag = group_rows + resident;
  if (lag * row_bytes > kMaxLagBytes || 2 * (rows + lag) > 0x7fffffffu) return false;
  *lag_out = static_cast<unsigned>(lag);
  *grid_out = static_cast<unsigned>(2 * (rows + lag));
  return true;
}

// One L2 line per group and per kind of word when the scratch has room for it (it has whenever a group
// spans 64 rows or more): the amax and arrival words of different groups then live in different L2
// slices instead of all on one hot line.
Board make_board(uint32_t* scratch, size_t words, size_t groups, float* global_out, size_t rows, size_t group_rows,
                 unsigned lag) {
  const unsigned stride = 64 * groups + 1 <= words ? 32u : 1u;
  return Board{scratch, scratch + groups * stride, scratch + words - 1, global_out, rows, group_rows, lag, stride};
}

}  // namespace

// [0, groups) amax words, [groups, 2 groups) arrival counters, spare, error word; never fewer than
// rows + 2 so that callers sized for one word per row keep working
size_t fused_scratch_words(size_t rows, size_t groups) { return (rows > 2 * groups ? rows : 2 * groups) + 2; }

// Both launchers return false when the single-kernel path does not apply (shape, alignment, a group
// too long to stay cached); nothing has been enqueued then and the caller takes the multi-kernel path.
bool launch_residual_norm_nvfp4_fused(const uint16_t* left, const uint16_t* right, const uint16_t* weight,
                                      size_t tokens, size_t hidden, float eps, size_t rows_per_scale,
                                      uint16_t* residual_out, uint16_t* normalized_out, uint32_t* scratch,
                                      float* global_scales_out, uint8_t* codes, uint8_t* scales, cudaStream_t s) {
  using namespace host;
  if (hidden % 16 != 0 || hidden > 8192 || tokens == 0) return false;
  if (!aligned16(left) || !aligned16(right) || !aligned16(weight) || !aligned16(residual_out) ||
      !aligned16(normalized_out) || (reinterpret_cast<uintptr_t>(codes) & 3u) != 0)
    return false;
  const int row_vectors = static_cast<int>(hidden / 8);
  const size_t rps = rows_per_scale ? (rows_per_scale < tokens ? rows_per_scale : tokens) : tokens;
  const size_t groups = (tokens + rps - 1) / rps;
  const size_t words = fused_scratch_words(tokens, groups);
  const bool coherent = residual_out == left || residual_out == right || normalized_out == left ||
                        normalized_out == right;
  QuantOut q{reinterpret_cast<uint32_t*>(codes), scales,
             row_vectors % 32 == 0 && aligned16(scales) && (row_vectors / 2) % 16 == 0};
  const float width = static_cast<float>(hidden);
  auto L = reinterpret_cast<const uint4*>(left);
  auto R = reinterpret_cast<const uint4*>(right);
  auto W = reinterpret_cast<const uint4*>(weight);
  auto RO = reinterpret_cast<uint4*>(residual_out);
  auto NO = reinterpret_cast<uint4*>(normalized_out);
  unsigned lag = 0, grid = 0;
  if (tokens <= kSmallRows) {
#define Q3X_SHAPE(TEAM, V)                                                                                      \
  if (row_vectors <= TEAM * V) {                                                                                \
    launch_kernel(small_norm_nvfp4_kernel<TEAM, V, false>, static_cast<unsigned>(groups), TEAM, 0, s, true,     \
                  L, R, W, row_vectors, width, eps, RO, NO, coherent, tokens, rps, global_scales_out, q);       \
    return true;                                                                                                \
  }
    Q3X_FUSED_SHAPES
#undef Q3X_SHAPE
    return false;
  }
#define Q3X_SHAPE(TEAM, V)                                                                                      \
  if (row_vectors <= TEAM * V) {                                                                                \
    if (!plan_launch(residual_norm_nvfp4_kernel<TEAM, V, true>, TEAM, tokens, rps, hidden * 2, &lag, &grid))          \
      return false;                                                                                             \
    const Board board = make_board(scratch, words, groups, global_scales_out, tokens, rps, lag);                \
    if (row_vectors == TEAM * V && !coherent && q.wide_scale_stores)                                            \
      residual_norm_nvfp4_kernel<TEAM, V, true><<<grid, TEAM, 0, s>>>(L, R, W, row_vectors, width, eps, RO, NO, \
                                                                      coherent, board, q);                      \
    else                                                                                                        \
      residual_norm_nvfp4_kernel<TEAM, V, false><<<grid, TEAM, 0, s>>>(L, R, W, row_vectors, width, eps, RO,    \
                                                                       NO, coherent, board, q);                 \
    return true;                                                                                                \
  }
  Q3X_FUSED_SHAPES
#undef Q3X_SHAPE
  return false;
}

bool launch_gated_norm_nvfp4_fused(const uint16_t* in, const uint16_t* weight, const uint16_t* gate, size_t tokens,
                                   size_t heads_per_row, size_t dim, float eps, size_t rows_per_scale, uint16_t* out,
                                   uint32_t* scratch, float* global_scales_out, uint8_t* codes, uint8_t* scales,
                                   cudaStream_t s) {
  using namespace host;
  const size_t cols = heads_per_row * dim;
  if (dim != Q3X_B200_GDN_HEAD_DIM || cols > 8192 || tokens == 0) return false;
  if (!aligned16(in) || !aligned16(gate) || !aligned16(weight) || !aligned16(out) ||
      (reinterpret_cast<uintptr_t>(codes) & 3u) != 0)
    return false;
  const int row_vectors = static_cast<int>(cols / 8);
  const size_t rps = rows_per_scale ? (rows_per_scale < tokens ? rows_per_scale : tokens) : tokens;
  const size_t groups = (tokens + rps - 1) / rps;
  const size_t words = fused_scratch_words(tokens, groups);
  const bool coherent = out == in || out == gate;
  QuantOut q{reinterpret_cast<uint32_t*>(codes), scales,
             row_vectors % 32 == 0 && aligned16(scales) && (row_vectors / 2) % 16 == 0};
  auto X = reinterpret_cast<const uint4*>(in);
  auto Z = reinterpret_cast<const uint4*>(gate);
  auto W = reinterpret_cast<const uint4*>(weight);
  auto O = reinterpret_cast<uint4*>(out);
  unsigned lag = 0, grid = 0;
  if (tokens <= kSmallRows) {
#define Q3X_SHAPE(TEAM, V)                                                                                      \
  if (row_vectors <= TEAM * V) {                                                                                \
    launch_kernel(small_norm_nvfp4_kernel<TEAM, V, true>, static_cast<unsigned>(groups), TEAM, 0, s, true,      \
                  X, Z, W, row_vectors, 128.0f, eps, static_cast<uint4*>(nullptr), O, coherent, tokens, rps,    \
                  global_scales_out, q);                                                                        \
    return true;                                                                                                \
  }
    Q3X_FUSED_SHAPES
#undef Q3X_SHAPE
    return false;
  }
#define Q3X_SHAPE(TEAM, V)                                                                                      \
  if (row_vectors <= TEAM * V) {                                                                                \
    if (!plan_launch(gated_norm_nvfp4_kernel<TEAM, V, true>, TEAM, tokens, rps, cols * 2, &lag, &grid))         \
      return false;                                                                                             \
    const Board board = make_board(scratch, words, groups, global_scales_out, tokens, rps, lag);                \
    if (row_vectors == TEAM * V && !coherent && q.wide_scale_stores)                                            \
      gated_norm_nvfp4_kernel<TEAM, V, true><<<grid, TEAM, 0, s>>>(X, Z, W, row_vectors, eps, O, coherent,      \
                                                                   board, q);                                   \
    else                                                                                                        \
      gated_norm_nvfp4_kernel<TEAM, V, false><<<grid, TEAM, 0, s>>>(X, Z, W, row_vectors, eps, O, coherent,     \
                                                                    board, q);                                  \
    return true;                                                                                                \
  }
  Q3X_FUSED_SHAPES
#undef Q3X_SHAPE
  return false;
}

namespace {

// out = Op(first, second) + NVFP4 over [tokens, width]; chunks of 512 vectors (4096 elements).  False
// when the shape does not fit the chunk scheme (a scale group that is not a whole number of chunks,
// misaligned pointers); the caller then runs the separate kernels.
template <class Op>
bool launch_pointwise_nvfp4(const uint16_t* gate, const uint16_t* up, size_t tokens, size_t intermediate,
                            size_t rows_per_scale, uint16_t* out, uint32_t* scratch, float* global_scales_out,
                            uint8_t* codes, uint8_t* scales, cudaStream_t s) {
  using namespace host;
  constexpr int kTeam = 128, kVpt = 4, kChunk = kTeam * kVpt;
  if (tokens == 0 || intermediate % 16 != 0) return false;
  if (!aligned16(gate) || !aligned16(up) || !aligned16(out) || (reinterpret_cast<uintptr_t>(codes) & 3u) != 0)
    return false;
  const size_t row_vectors = intermediate / 8;
  const size_t rps = rows_per_scale ? (rows_per_scale < tokens ? rows_per_scale : tokens) : tokens;
  const size_t groups = (tokens + rps - 1) / rps;
  const size_t group_vectors = rps * row_vectors;
  if (groups > 1 && group_vectors % kChunk != 0) return false;
  const size_t count = tokens * row_vectors;
  const size_t chunks_per_group = (group_vectors + kChunk - 1) / kChunk;
  const size_t chunks = (count + kChunk - 1) / kChunk;
  const size_t words = fused_scratch_words(tokens, groups);
  const bool coherent = out == gate || out == up;
  const bool full = count % kChunk == 0;
  QuantOut q{reinterpret_cast<uint32_t*>(codes), scales, aligned16(scales) && (count % kChunk) % 32 == 0};
  unsigned lag = 0, grid = 0;
  if (!plan_launch(pointwise_nvfp4_kernel<Op, kTeam, kVpt, true>, kTeam, chunks, chunks_per_group, kChunk * 16, &lag, &grid))
    return false;
  const Board board = make_board(scratch, words, groups, global_scales_out, chunks, chunks_per_group, lag);
  auto G = reinterpret_cast<const uint4*>(gate);
  auto U = reinterpret_cast<const uint4*>(up);
  auto O = reinterpret_cast<uint4*>(out);
  if (full && !coherent && q.wide_scale_stores)
    pointwise_nvfp4_kernel<Op, kTeam, kVpt, true><<<grid, kTeam, 0, s>>>(G, U, O, count, coherent, board, q);
  else
    pointwise_nvfp4_kernel<Op, kTeam, kVpt, false><<<grid, kTeam, 0, s>>>(G, U, O, count, coherent, board, q);
  return true;
}

}  // namespace

bool launch_silu_mul_nvfp4_fused(const uint16_t* gate, const uint16_t* up, size_t tokens, size_t intermediate,
                                 size_t rows_per_scale, uint16_t* out, uint32_t* scratch, float* global_scales_out,
                                 uint8_t* codes, uint8_t* scales, cudaStream_t s) {
  return launch_pointwise_nvfp4<SiluMul>(gate, up, tokens, intermediate, rows_per_scale, out, scratch,
                                         global_scales_out, codes, scales, s);
}

bool launch_sigmoid_gate_nvfp4_fused(const uint16_t* value, const uint16_t* gate, size_t tokens, size_t width,
                                     size_t rows_per_scale, uint16_t* out, uint32_t* scratch,
                                     float* global_scales_out, uint8_t* codes, uint8_t* scales, cudaStream_t s) {
  return launch_pointwise_nvfp4<SigmoidGate>(value, gate, tokens, width, rows_per_scale, out, scratch,
                                             global_scales_out, codes, scales, s);
}

}  // namespace q3x
