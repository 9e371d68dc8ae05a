// Single-pass norm + NVFP4 kernels: residual add + centred RMSNorm + quantisation, and the GDN
// gated RMSNorm * silu(z) + quantisation, each crossing HBM once.
//
// The NVFP4 global scale of a group of rows is its amax, which is only known once every row of the
// group has been normalised -- a grid-wide dependency.  It is resolved without a second pass over
// memory by DEFERRING the quantisation of a row:
//   * a team (one CTA of 128 threads) owns rows team, team + teams, team + 2 teams, ...; all CTAs
//     are co-resident (cooperative launch);
//   * the inputs of a team's NEXT row are copied global -> shared with cp.async while the current
//     row is processed, so HBM latency is off the critical path; every thread stages, rings and
//     later quantises the same vectors (tid + k * 128), so none of these buffers needs a barrier;
//   * iteration i normalises row i ("phase A"): it writes the bf16 outputs, keeps the normalised
//     row in a shared-memory ring and publishes the row's amax as ONE 32-bit word (magnitude bits
//     plus a valid bit) -- no atomics and no fence, the word itself says that it is there;
//   * the same iteration quantises the row of iteration i - (depth - 1) ("phase B") from the ring:
//     the team reads the amax words of that row's whole group (<= a few KB, from L2), and only
//     spins while a word is not valid yet.  depth is chosen so that every row of that group belongs
//     to an iteration at least one behind the current one of its owner, so the words are normally
//     all there.
// Progress: the team with the smallest iteration number only ever needs words of iterations that
// every team has already finished, so the waits cannot deadlock while all CTAs are resident.  Every
// spin is bounded; a team that gives up sets the error word and carries on, so the kernel always
// terminates.
//
// Scratch words (uint32): [0, rows) per-row amax words, last word = error flag.
#include <atomic>
#include <mutex>

#include "device_utils.cuh"
#include "host_checks.hpp"
#include "internal.hpp"
#include "norm_math.cuh"
#include "nvfp4_math.cuh"
#include "q3x_b200.h"

namespace q3x {
namespace {

constexpr int kTeam = 128;           // threads of a CTA; they own one row at a time
constexpr int kMaxDepth = 8;         // ring slots a team may be given
constexpr int kSpinLimit = 1 << 20;  // polls of one word before giving up (~1 s with the sleep)
constexpr uint32_t kValid = 0x80000000u;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* global_src) {
  const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(global_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ uint32_t ld_volatile(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct RowBoard {
  uint32_t* row_amax;  // [rows]: kValid | bf16 magnitude bits of the row's largest finite output
  uint32_t* error;     // [1]
  size_t rows, rows_per_group;
};

struct TeamShared {
  float sums[4];
  uint32_t tops_a[4];
  uint32_t tops_b[4];
  uint32_t pad[4];
  uint8_t scale_bytes[512];  // one row of block scales (row_vectors / 2 <= 512)
};

// Phase A epilogue: the row's amax as one self-validating word.
__device__ __forceinline__ void publish_row(const RowBoard& board, TeamShared& ts, int tid, size_t row,
                                            uint32_t thread_top) {
  const uint32_t warp_top = group_max_u32<32>(thread_top);
  if ((tid & 31) == 0) ts.tops_a[tid >> 5] = warp_top;
  __syncthreads();
  if (tid == 0) {
    const uint32_t m = max(max(ts.tops_a[0], ts.tops_a[1]), max(ts.tops_a[2], ts.tops_a[3]));
    __stcg(board.row_amax + row, m | kValid);
  }
}

// Phase B prologue: the global scale of the group of `row`, once all of the group's words are valid.
__device__ __forceinline__ float await_group_scale(const RowBoard& board, TeamShared& ts, int tid, size_t row) {
  const size_t group = row / board.rows_per_group;
  const size_t first = group * board.rows_per_group;
  const size_t count = min(board.rows_per_group, board.rows - first);
  uint32_t top = 0;
  for (size_t j = tid; j < count; j += kTeam) {
    uint32_t word = ld_volatile(board.row_amax + first + j);
    int polls = 0;
    while ((word & kValid) == 0) {
      if (++polls >= kSpinLimit) {
        atomicExch(board.error, 1u);
        break;
      }
      __nanosleep(100);
      word = ld_volatile(board.row_amax + first + j);
    }
    top = max(top, word & 0xffffu);
  }
  top = group_max_u32<32>(top);
  if ((tid & 31) == 0) ts.tops_b[tid >> 5] = top;
  __syncthreads();
  const uint32_t m = max(max(ts.tops_b[0], ts.tops_b[1]), max(ts.tops_b[2], ts.tops_b[3]));
  return global_scale_from_amax_bits(m);
}

struct QuantOut {
  uint32_t* codes;   // [rows, row_vectors] words
  uint8_t* scales;   // [rows, row_vectors / 2] bytes
  bool wide_scale_stores;
};

// Phase B: quantises one row from the team's ring slot.  Thread tid owns vectors tid + k * 128.
template <int VPT>
__device__ __forceinline__ void quantize_ring_row(const uint4* slot, int row_vectors, float global, TeamShared& ts,
                                                  int tid, uint32_t* codes_row, uint8_t* scales_row,
                                                  bool wide_scale_stores) {
  const float k = block_scale_factor(global);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * kTeam;
    const bool valid = v < row_vectors;  // lane pairs are valid together (row_vectors is even)
    const uint4 y = valid ? slot[v] : make_uint4(0, 0, 0, 0);
    float f[8];
    unpack8(y, f);
    float m = amax8_float(f, y);
    m = fmaxf(m, __shfl_xor_sync(kFullMask, m, 1));
    const uint32_t s = block_scale_code(m, k);
    const float inv = block_inverse(s, global);
    if (valid) {
      codes_row[v] = quantize8(f, inv);
      if ((tid & 1) == 0) {
        if (wide_scale_stores) ts.scale_bytes[v >> 1] = static_cast<uint8_t>(s);
        else scales_row[v >> 1] = static_cast<uint8_t>(s);
      }
    }
  }
  if (wide_scale_stores) {  // row_vectors / 2 bytes, a multiple of 16, written as 128-bit stores
    __syncthreads();
    const int n = row_vectors / 32;
    if (tid < n) reinterpret_cast<uint4*>(scales_row)[tid] = reinterpret_cast<const uint4*>(ts.scale_bytes)[tid];
  }
}

// Shared-memory carve-up: [2 staging rows][depth ring rows][TeamShared]
template <int VPT>
struct Carve {
  static constexpr int kRowVectors = VPT * kTeam;
  __device__ static uint4* stage(unsigned char* smem, int which) {
    return reinterpret_cast<uint4*>(smem) + which * kRowVectors;
  }
  __device__ static uint4* ring(unsigned char* smem, int slot) {
    return reinterpret_cast<uint4*>(smem) + (2 + slot) * kRowVectors;
  }
  __device__ static TeamShared& shared(unsigned char* smem, int depth) {
    return *reinterpret_cast<TeamShared*>(smem + sizeof(uint4) * (2 + depth) * kRowVectors);
  }
};

template <int VPT>
__device__ __forceinline__ void stage_row(unsigned char* smem, const uint4* a, const uint4* b, size_t base,
                                          int row_vectors, int tid) {
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * kTeam;
    if (v < row_vectors) {
      cp_async16(Carve<VPT>::stage(smem, 0) + v, a + base + v);
      cp_async16(Carve<VPT>::stage(smem, 1) + v, b + base + v);
    }
  }
  cp_async_commit();
}

// ---- residual add + centred RMSNorm + NVFP4 ------------------------------------------------
template <int VPT>
__global__ void __launch_bounds__(kTeam) residual_norm_nvfp4_kernel(
    const uint4* left, const uint4* right, const uint4* __restrict__ weight, int row_vectors, float width, float eps,
    uint4* residual_out, uint4* normalized_out, int depth, RowBoard board, QuantOut q) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int tid = threadIdx.x;
  TeamShared& ts = Carve<VPT>::shared(smem, depth);
  const size_t teams = gridDim.x;
  const size_t first = blockIdx.x;
  const size_t lag = static_cast<size_t>(depth - 1);
  const float inv_width = 1.0f / width;
  if (first < board.rows) stage_row<VPT>(smem, left, right, first * static_cast<size_t>(row_vectors), row_vectors, tid);

  for (size_t it = 0;; ++it) {
    const size_t row = first + it * teams;
    const bool has_row = row < board.rows;
    const bool has_old = it >= lag && first + (it - lag) * teams < board.rows;
    if (!has_row && !has_old) {
      if (it >= lag) break;  // nothing left in the ring either
      continue;              // rows are exhausted but the ring still drains
    }
    if (has_row) {
      const size_t base = row * static_cast<size_t>(row_vectors);
      uint4 x[VPT];
      cp_async_wait_all();
      float partial = 0.0f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * kTeam;
        x[i] = make_uint4(0, 0, 0, 0);
        if (v < row_vectors) {
          float a[8], b[8];
          unpack8(Carve<VPT>::stage(smem, 0)[v], a);
          unpack8(Carve<VPT>::stage(smem, 1)[v], b);
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] = a[j] + b[j];
          x[i] = pack8(a);
          st_vec(residual_out + base + v, x[i]);
        }
        partial += sum_squares8(x[i]);
      }
      // this thread has consumed its staged vectors: refill them with the next row's
      if (row + teams < board.rows)
        stage_row<VPT>(smem, left, right, (row + teams) * static_cast<size_t>(row_vectors), row_vectors, tid);
      partial = group_sum<32>(partial);
      if ((tid & 31) == 0) ts.sums[tid >> 5] = partial;
      __syncthreads();
      const float total = ts.sums[0] + ts.sums[1] + ts.sums[2] + ts.sums[3];
      const float inv = inverse_rms(total, inv_width, eps);
      uint4* slot = Carve<VPT>::ring(smem, static_cast<int>(it % depth));
      float top = 0.0f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * kTeam;
        if (v < row_vectors) {
          const uint4 y =
              scale8<NormMode::kCentered, true>(x[i], ld_weight(weight + v), make_uint4(0, 0, 0, 0), inv, &top);
          st_vec(normalized_out + base + v, y);
          slot[v] = y;
        }
      }
      publish_row(board, ts, tid, row, amax_bits_of(top));
    }
    if (has_old) {
      const size_t old_it = it - lag;
      const size_t old_row = first + old_it * teams;
      const float global = await_group_scale(board, ts, tid, old_row);
      quantize_ring_row<VPT>(Carve<VPT>::ring(smem, static_cast<int>(old_it % depth)), row_vectors, global, ts, tid,
                             q.codes + old_row * static_cast<size_t>(row_vectors),
                             q.scales + old_row * static_cast<size_t>(row_vectors / 2), q.wide_scale_stores);
    }
  }
}

// ---- gated RMSNorm * silu(z) + NVFP4: one row = one token = heads_per_row heads of 128 -------
template <int VPT>
__global__ void __launch_bounds__(kTeam) gated_norm_nvfp4_kernel(
    const uint4* in, const uint4* gate, const uint4* __restrict__ weight, int row_vectors, float eps, uint4* out,
    int depth, RowBoard board, QuantOut q) {
  constexpr int kLanes = Q3X_B200_GDN_HEAD_DIM / 8;  // 16 lanes own one head
  extern __shared__ __align__(16) unsigned char smem[];
  const int tid = threadIdx.x;
  TeamShared& ts = Carve<VPT>::shared(smem, depth);
  const size_t teams = gridDim.x;
  const size_t first = blockIdx.x;
  const size_t lag = static_cast<size_t>(depth - 1);
  const uint4 w = ld_weight(weight + (tid % kLanes));
  if (first < board.rows) stage_row<VPT>(smem, in, gate, first * static_cast<size_t>(row_vectors), row_vectors, tid);

  for (size_t it = 0;; ++it) {
    const size_t row = first + it * teams;
    const bool has_row = row < board.rows;
    const bool has_old = it >= lag && first + (it - lag) * teams < board.rows;
    if (!has_row && !has_old) {
      if (it >= lag) break;
      continue;
    }
    if (has_row) {
      const size_t base = row * static_cast<size_t>(row_vectors);
      uint4 x[VPT], z[VPT];
      cp_async_wait_all();
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * kTeam;
        x[i] = z[i] = make_uint4(0, 0, 0, 0);
        if (v < row_vectors) {
          x[i] = Carve<VPT>::stage(smem, 0)[v];
          z[i] = Carve<VPT>::stage(smem, 1)[v];
        }
      }
      if (row + teams < board.rows)
        stage_row<VPT>(smem, in, gate, (row + teams) * static_cast<size_t>(row_vectors), row_vectors, tid);
      uint4* slot = Carve<VPT>::ring(smem, static_cast<int>(it % depth));
      float top = 0.0f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * kTeam;  // head = v / 16: the 16 lanes of a head sit in one warp
        const float sum = group_sum<kLanes>(sum_squares8(x[i]));
        const float inv = inverse_rms(sum, 1.0f / static_cast<float>(Q3X_B200_GDN_HEAD_DIM), eps);
        if (v < row_vectors) {
          const uint4 y = scale8<NormMode::kPlainSiluGate, true>(x[i], w, z[i], inv, &top);
          st_vec(out + base + v, y);
          slot[v] = y;
        }
      }
      publish_row(board, ts, tid, row, amax_bits_of(top));
    }
    if (has_old) {
      const size_t old_it = it - lag;
      const size_t old_row = first + old_it * teams;
      const float global = await_group_scale(board, ts, tid, old_row);
      quantize_ring_row<VPT>(Carve<VPT>::ring(smem, static_cast<int>(old_it % depth)), row_vectors, global, ts, tid,
                             q.codes + old_row * static_cast<size_t>(row_vectors),
                             q.scales + old_row * static_cast<size_t>(row_vectors / 2), q.wide_scale_stores);
    }
  }
}

// One CTA per group: global scale = f(max of the group's row words).
__global__ void __launch_bounds__(kTeam) finish_scales_kernel(const uint32_t* row_amax, size_t rows,
                                                              size_t rows_per_group, float* global_scales) {
  __shared__ uint32_t tops[4];
  const size_t first = static_cast<size_t>(blockIdx.x) * rows_per_group;
  const size_t count = min(rows_per_group, rows - first);
  uint32_t top = 0;
  for (size_t j = threadIdx.x; j < count; j += kTeam) top = max(top, row_amax[first + j] & 0xffffu);
  top = group_max_u32<32>(top);
  if ((threadIdx.x & 31) == 0) tops[threadIdx.x >> 5] = top;
  __syncthreads();
  if (threadIdx.x == 0)
    global_scales[blockIdx.x] = global_scale_from_amax_bits(max(max(tops[0], tops[1]), max(tops[2], tops[3])));
}

size_t smem_bytes(int vpt, int depth) {
  return sizeof(uint4) * static_cast<size_t>(2 + depth) * vpt * kTeam + sizeof(TeamShared);
}

// Resident CTAs of `kernel` with `smem` bytes on the current device (0 = cannot be configured).
// Cached per (device, kernel family, vectors per thread, depth): a pure function of them.
template <typename K>
int resident_ctas(K kernel, size_t smem, int family, int vpt, int depth) {
  constexpr int kMaxDevices = 64;
  static std::atomic<int> cache[kMaxDevices][2][9][kMaxDepth + 1];
  static std::once_flag once;
  std::call_once(once, [] {
    for (auto& d : cache)
      for (auto& f : d)
        for (auto& v : f)
          for (auto& e : v) e.store(-1);
  });
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  const bool cacheable = dev >= 0 && dev < kMaxDevices;
  if (cacheable) {
    const int hit = cache[dev][family][vpt][depth].load();
    if (hit >= 0) return hit;
  }
  int sms = 0, per_sm = 0, total = 0, limit = 0;
  if (cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess &&
      smem <= static_cast<size_t>(limit) &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, limit) == cudaSuccess &&
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess &&
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kTeam, smem) == cudaSuccess)
    total = sms * per_sm;
  if (cacheable) cache[dev][family][vpt][depth].store(total);
  return total;
}

// Picks the ring depth and grid: depth = 2 + ceil(group rows / teams) so that every row of the group
// being quantised belongs to an iteration its owner has left behind; more ring slots cost shared
// memory and so teams, hence the small search.  Returns false when no configuration fits.
template <typename K>
bool plan_launch(K kernel, int family, int vpt, size_t rows, size_t rows_per_group, int* depth_out,
                 unsigned* grid_out, size_t* smem_out) {
  for (int depth = 3; depth <= kMaxDepth; ++depth) {
    const size_t smem = smem_bytes(vpt, depth);
    const int cap = resident_ctas(kernel, smem, family, vpt, depth);
    if (cap <= 0) return false;
    const size_t grid = rows < static_cast<size_t>(cap) ? rows : static_cast<size_t>(cap);
    const size_t group_rows = rows_per_group < rows ? rows_per_group : rows;
    const size_t sweeps = (group_rows + grid - 1) / grid;  // iterations a group can reach past one of its rows
    if (static_cast<size_t>(depth) >= 2 + sweeps) {
      *depth_out = depth;
      *grid_out = static_cast<unsigned>(grid);
      *smem_out = smem;
      return true;
    }
  }
  return false;
}

template <typename K, typename... Args>
bool launch_cooperative(K kernel, unsigned grid, size_t smem, cudaStream_t s, Args... args) {
  void* params[] = {static_cast<void*>(&args)...};
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3(grid), dim3(kTeam), params, smem,
                                     s) == cudaSuccess;
}

}  // namespace

// [0, rows) row words or [0, groups) group amax words, whichever path runs, + error word + spare
size_t fused_scratch_words(size_t rows, size_t groups) { return (rows > 2 * groups ? rows : 2 * groups) + 2; }

// Both launchers return false when the fused path does not apply (shape, alignment, a group too long
// for the ring, or the cooperative launch is refused); nothing has been enqueued then and the
// caller takes the multi-kernel path.
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
  const int vpt = (row_vectors + kTeam - 1) / kTeam;
  const size_t rps = rows_per_scale ? rows_per_scale : tokens;
  const size_t groups = (tokens + rps - 1) / rps;
  const size_t words = fused_scratch_words(tokens, groups);
  RowBoard board{scratch, scratch + words - 1, tokens, rps};
  QuantOut q{reinterpret_cast<uint32_t*>(codes), scales,
             row_vectors % 32 == 0 && aligned16(scales) && (row_vectors / 2) % 16 == 0};
  const float width = static_cast<float>(hidden);
  auto L = reinterpret_cast<const uint4*>(left);
  auto R = reinterpret_cast<const uint4*>(right);
  auto W = reinterpret_cast<const uint4*>(weight);
  auto RO = reinterpret_cast<uint4*>(residual_out);
  auto NO = reinterpret_cast<uint4*>(normalized_out);
  bool ok = false;
  int depth = 0;
  unsigned grid = 0;
  size_t smem = 0;
#define Q3X_TRY(V)                                                                                             \
  case V:                                                                                                      \
    if (plan_launch(residual_norm_nvfp4_kernel<V>, 0, V, tokens, rps, &depth, &grid, &smem)) {                 \
      cudaMemsetAsync(scratch, 0, words * sizeof(uint32_t), s);                                                \
      ok = launch_cooperative(residual_norm_nvfp4_kernel<V>, grid, smem, s, L, R, W, row_vectors, width, eps,  \
                              RO, NO, depth, board, q);                                                        \
    }                                                                                                          \
    break;
  switch (vpt) { Q3X_TRY(1) Q3X_TRY(2) Q3X_TRY(3) Q3X_TRY(4) Q3X_TRY(5) Q3X_TRY(6) Q3X_TRY(7) Q3X_TRY(8) }
#undef Q3X_TRY
  if (!ok) {
    (void)cudaGetLastError();
    return false;
  }
  finish_scales_kernel<<<static_cast<unsigned>(groups), kTeam, 0, s>>>(scratch, tokens, rps, global_scales_out);
  return true;
}

bool launch_gated_norm_nvfp4_fused(const uint16_t* in, const uint16_t* weight, const uint16_t* gate, size_t tokens,
                                   size_t heads_per_row, size_t dim, float eps, size_t rows_per_scale, uint16_t* out,
                                   uint32_t* scratch, float* global_scales_out, uint8_t* codes, uint8_t* scales,
                                   cudaStream_t s) {
  using namespace host;
  const size_t cols = heads_per_row * dim;
  if (dim != Q3X_B200_GDN_HEAD_DIM || cols > 8192 || tokens == 0) return false;
  // in-place forms would let a staged copy of the next row race with this row's stores
  if (out == in || out == gate) return false;
  if (!aligned16(in) || !aligned16(gate) || !aligned16(weight) || !aligned16(out) ||
      (reinterpret_cast<uintptr_t>(codes) & 3u) != 0)
    return false;
  const int row_vectors = static_cast<int>(cols / 8);
  const int vpt = (row_vectors + kTeam - 1) / kTeam;
  const size_t rps = rows_per_scale ? rows_per_scale : tokens;
  const size_t groups = (tokens + rps - 1) / rps;
  const size_t words = fused_scratch_words(tokens, groups);
  RowBoard board{scratch, scratch + words - 1, tokens, rps};
  QuantOut q{reinterpret_cast<uint32_t*>(codes), scales,
             row_vectors % 32 == 0 && aligned16(scales) && (row_vectors / 2) % 16 == 0};
  auto X = reinterpret_cast<const uint4*>(in);
  auto Z = reinterpret_cast<const uint4*>(gate);
  auto W = reinterpret_cast<const uint4*>(weight);
  auto O = reinterpret_cast<uint4*>(out);
  bool ok = false;
  int depth = 0;
  unsigned grid = 0;
  size_t smem = 0;
#define Q3X_TRY(V)                                                                                          \
  case V:                                                                                                   \
    if (plan_launch(gated_norm_nvfp4_kernel<V>, 1, V, tokens, rps, &depth, &grid, &smem)) {                 \
      cudaMemsetAsync(scratch, 0, words * sizeof(uint32_t), s);                                             \
      ok = launch_cooperative(gated_norm_nvfp4_kernel<V>, grid, smem, s, X, Z, W, row_vectors, eps, O,      \
                              depth, board, q);                                                             \
    }                                                                                                       \
    break;
  switch (vpt) { Q3X_TRY(1) Q3X_TRY(2) Q3X_TRY(3) Q3X_TRY(4) Q3X_TRY(5) Q3X_TRY(6) Q3X_TRY(7) Q3X_TRY(8) }
#undef Q3X_TRY
  if (!ok) {
    (void)cudaGetLastError();
    return false;
  }
  finish_scales_kernel<<<static_cast<unsigned>(groups), kTeam, 0, s>>>(scratch, tokens, rps, global_scales_out);
  return true;
}

}  // namespace q3x
