// Single-pass norm + NVFP4 kernels: residual add + centred RMSNorm + quantisation, and the GDN
// gated RMSNorm * silu(z) + quantisation, each crossing HBM once.
//
// The NVFP4 global scale of a group of rows is its amax, which is only known once every row of the
// group has been normalised -- a grid-wide dependency.  It is resolved without a second pass over
// memory by DEFERRING the quantisation of a row:
//   * a team of 128 threads owns rows team, team + teams, team + 2 teams, ... (all CTAs co-resident,
//     cooperative launch);
//   * iteration i of a team normalises its row i ("phase A"): it writes the bf16 outputs, keeps the
//     normalised row in a shared-memory ring (each thread keeps exactly the vectors it will later
//     quantise, so the ring needs no synchronisation), raises the group's amax with one atomic and
//     then counts the row as finished for its group;
//   * the same iteration quantises the row of iteration i - 2 ("phase B") from the ring.  Because a
//     group is no longer than one sweep of all teams, every row of that group belongs to iteration
//     i - 2 or i - 1 of some team, so by then the group is normally complete; the team checks the
//     group's finished-row counter (acquire load) and only spins if another team lags.
// Progress: the team with the smallest iteration number never waits on anything unfinished, so the
// wait cannot deadlock while all CTAs are resident.  Every spin is bounded; a team that gives up
// sets the error word of the scratch area and carries on with the amax it can see, so the kernel
// always terminates.
//
// Scratch words (uint32): [0,G) group amax bits, [G,2G) finished rows per group, [2G] error flag.
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

constexpr int kTeam = 128;           // threads that own one row
constexpr int kTeamsPerCta = 2;
constexpr int kCtaThreads = kTeam * kTeamsPerCta;
constexpr int kDepth = 3;            // ring slots per team: rows of iterations i, i-1, i-2
constexpr int kSpinLimit = 1 << 21;  // polls of a counter before giving up (~1 s)

__device__ __forceinline__ void team_sync(int team) {
  asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(kTeam) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct GroupBoard {
  uint32_t* amax;      // [groups]
  uint32_t* finished;  // [groups]
  uint32_t* error;     // [1]
  size_t rows, rows_per_group;
  __device__ __forceinline__ size_t group_of(size_t row) const { return row / rows_per_group; }
  __device__ __forceinline__ uint32_t rows_in(size_t group) const {
    const size_t first = group * rows_per_group;
    return static_cast<uint32_t>(min(rows_per_group, rows - first));
  }
};

// Per-team shared memory besides the ring.
struct TeamShared {
  float sums[4];
  uint32_t tops[4];
  float global_scale;
  uint32_t pad[3];
  uint8_t scale_bytes[512];  // one row of block scales (row_vectors / 2 <= 512)
};

// Publishes a finished row: raises the group amax, then (after a fence) counts the row.
__device__ __forceinline__ void publish_row(const GroupBoard& board, TeamShared& ts, int team, int tid, size_t row,
                                            uint32_t thread_top) {
  const uint32_t warp_top = group_max_u32<32>(thread_top);
  if ((tid & 31) == 0) ts.tops[tid >> 5] = warp_top;
  team_sync(team);
  if (tid == 0) {
    const uint32_t m = max(max(ts.tops[0], ts.tops[1]), max(ts.tops[2], ts.tops[3]));
    const size_t g = board.group_of(row);
    if (m != 0) atomicMax(board.amax + g, m);
    __threadfence();
    atomicAdd(board.finished + g, 1u);
  }
}

// Waits (bounded) until the group of `row` is complete and returns its global scale to the team.
__device__ __forceinline__ float await_group_scale(const GroupBoard& board, TeamShared& ts, int team, int tid,
                                                   size_t row) {
  if (tid == 0) {
    const size_t g = board.group_of(row);
    const uint32_t expected = board.rows_in(g);
    int polls = 0;
    while (ld_acquire(board.finished + g) < expected) {
      if (++polls >= kSpinLimit) {
        atomicExch(board.error, 1u);
        break;
      }
      __nanosleep(64);
    }
    ts.global_scale = global_scale_from_amax_bits(ld_acquire(board.amax + g));
  }
  team_sync(team);
  return ts.global_scale;
}

// Phase B: quantises one row from the team's ring slot.  Thread tid owns vectors tid + k * 128.
template <int VPT>
__device__ __forceinline__ void quantize_ring_row(const uint4* slot, int row_vectors, float global, TeamShared& ts,
                                                  int team, int tid, uint32_t* codes_row, uint8_t* scales_row,
                                                  bool wide_scale_stores) {
  const float k = block_scale_factor(global);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * kTeam;
    const bool valid = v < row_vectors;  // lane pairs are valid together (row_vectors is even)
    const uint4 y = valid ? slot[v] : make_uint4(0, 0, 0, 0);
    uint32_t m = amax8(y);
    m = max(m, __shfl_xor_sync(kFullMask, m, 1));
    const uint32_t s = block_scale_code(m, k);
    const float inv = block_inverse(s, global);
    if (valid) {
      codes_row[v] = quantize8(y, inv);
      if ((tid & 1) == 0) {
        if (wide_scale_stores) ts.scale_bytes[v >> 1] = static_cast<uint8_t>(s);
        else scales_row[v >> 1] = static_cast<uint8_t>(s);
      }
    }
  }
  if (wide_scale_stores) {  // row_vectors / 2 bytes, a multiple of 16, written as 128-bit stores
    team_sync(team);
    const int n = row_vectors / 32;
    if (tid < n) reinterpret_cast<uint4*>(scales_row)[tid] = reinterpret_cast<const uint4*>(ts.scale_bytes)[tid];
  }
}

struct QuantOut {
  uint32_t* codes;   // [rows, row_vectors] words
  uint8_t* scales;   // [rows, row_vectors / 2] bytes
  bool wide_scale_stores;
};

// ---- residual add + centred RMSNorm + NVFP4 ------------------------------------------------
template <int VPT>
__global__ void __launch_bounds__(kCtaThreads) residual_norm_nvfp4_kernel(
    const uint4* left, const uint4* right, const uint4* __restrict__ weight, int row_vectors, float width, float eps,
    uint4* residual_out, uint4* normalized_out, bool coherent, GroupBoard board, QuantOut q) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int team = threadIdx.x / kTeam, tid = threadIdx.x % kTeam;
  uint4* ring = reinterpret_cast<uint4*>(smem) + static_cast<size_t>(team) * kDepth * VPT * kTeam;
  TeamShared& ts = reinterpret_cast<TeamShared*>(smem + sizeof(uint4) * kTeamsPerCta * kDepth * VPT * kTeam)[team];
  const size_t teams = static_cast<size_t>(gridDim.x) * kTeamsPerCta;
  const size_t first = static_cast<size_t>(blockIdx.x) * kTeamsPerCta + team;

  for (size_t it = 0;; ++it) {
    const size_t row = first + it * teams;
    const bool has_row = row < board.rows;
    const bool has_old = it >= kDepth - 1 && first + (it - (kDepth - 1)) * teams < board.rows;
    if (!has_row && !has_old) {
      if (it >= kDepth - 1) break;  // nothing left in the ring either
      continue;                     // rows are exhausted but the ring still drains
    }

    if (has_row) {
      const size_t base = row * static_cast<size_t>(row_vectors);
      uint4 x[VPT], r[VPT];
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * kTeam;
        x[i] = r[i] = make_uint4(0, 0, 0, 0);
        if (v < row_vectors) {
          x[i] = ld_stream(left + base + v);
          r[i] = coherent ? ld_vec(right + base + v) : ld_stream(right + base + v);
        }
      }
      float partial = 0.0f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        float a[8], b[8];
        unpack8(x[i], a);
        unpack8(r[i], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = a[j] + b[j];
        x[i] = pack8(a);
        const int v = tid + i * kTeam;
        if (v < row_vectors) st_vec(residual_out + base + v, x[i]);
        partial += sum_squares8(x[i]);
      }
      partial = group_sum<32>(partial);
      if ((tid & 31) == 0) ts.sums[tid >> 5] = partial;
      team_sync(team);
      const float total = ts.sums[0] + ts.sums[1] + ts.sums[2] + ts.sums[3];
      const float inv = inverse_rms(total, width, eps);
      uint4* slot = ring + (it % kDepth) * VPT * kTeam;
      uint32_t top = 0;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * kTeam;
        if (v < row_vectors) {
          const uint4 y = scale8<NormMode::kCentered>(x[i], ld_weight(weight + v), make_uint4(0, 0, 0, 0), inv);
          st_vec(normalized_out + base + v, y);
          slot[v] = y;
          top = max(top, amax8(y));
        }
      }
      publish_row(board, ts, team, tid, row, top);
    }
    if (has_old) {
      const size_t old_it = it - (kDepth - 1);
      const size_t old_row = first + old_it * teams;
      const float global = await_group_scale(board, ts, team, tid, old_row);
      quantize_ring_row<VPT>(ring + (old_it % kDepth) * VPT * kTeam, row_vectors, global, ts, team, tid,
                             q.codes + old_row * static_cast<size_t>(row_vectors),
                             q.scales + old_row * static_cast<size_t>(row_vectors / 2), q.wide_scale_stores);
    }
  }
}

// ---- gated RMSNorm * silu(z) + NVFP4: one row = one token = heads_per_row heads of 128 -------
template <int VPT>
__global__ void __launch_bounds__(kCtaThreads) gated_norm_nvfp4_kernel(
    const uint4* in, const uint4* gate, const uint4* __restrict__ weight, int row_vectors, float eps, uint4* out,
    bool coherent, GroupBoard board, QuantOut q) {
  constexpr int kLanes = Q3X_B200_GDN_HEAD_DIM / 8;  // 16 lanes own one head
  extern __shared__ __align__(16) unsigned char smem[];
  const int team = threadIdx.x / kTeam, tid = threadIdx.x % kTeam;
  uint4* ring = reinterpret_cast<uint4*>(smem) + static_cast<size_t>(team) * kDepth * VPT * kTeam;
  TeamShared& ts = reinterpret_cast<TeamShared*>(smem + sizeof(uint4) * kTeamsPerCta * kDepth * VPT * kTeam)[team];
  const size_t teams = static_cast<size_t>(gridDim.x) * kTeamsPerCta;
  const size_t first = static_cast<size_t>(blockIdx.x) * kTeamsPerCta + team;
  const uint4 w = ld_weight(weight + (tid % kLanes));

  for (size_t it = 0;; ++it) {
    const size_t row = first + it * teams;
    const bool has_row = row < board.rows;
    const bool has_old = it >= kDepth - 1 && first + (it - (kDepth - 1)) * teams < board.rows;
    if (!has_row && !has_old) {
      if (it >= kDepth - 1) break;  // nothing left in the ring either
      continue;                     // rows are exhausted but the ring still drains
    }

    if (has_row) {
      const size_t base = row * static_cast<size_t>(row_vectors);
      uint4 x[VPT], z[VPT];
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * kTeam;
        x[i] = z[i] = make_uint4(0, 0, 0, 0);
        if (v < row_vectors) {
          x[i] = coherent ? ld_vec(in + base + v) : ld_stream(in + base + v);
          z[i] = coherent ? ld_vec(gate + base + v) : ld_stream(gate + base + v);
        }
      }
      uint4* slot = ring + (it % kDepth) * VPT * kTeam;
      uint32_t top = 0;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = tid + i * kTeam;  // head = v / 16: the 16 lanes of a head sit in one warp
        const float sum = group_sum<kLanes>(sum_squares8(x[i]));
        const float inv = inverse_rms(sum, static_cast<float>(Q3X_B200_GDN_HEAD_DIM), eps);
        if (v < row_vectors) {
          const uint4 y = scale8<NormMode::kPlainSiluGate>(x[i], w, z[i], inv);
          st_vec(out + base + v, y);
          slot[v] = y;
          top = max(top, amax8(y));
        }
      }
      publish_row(board, ts, team, tid, row, top);
    }
    if (has_old) {
      const size_t old_it = it - (kDepth - 1);
      const size_t old_row = first + old_it * teams;
      const float global = await_group_scale(board, ts, team, tid, old_row);
      quantize_ring_row<VPT>(ring + (old_it % kDepth) * VPT * kTeam, row_vectors, global, ts, team, tid,
                             q.codes + old_row * static_cast<size_t>(row_vectors),
                             q.scales + old_row * static_cast<size_t>(row_vectors / 2), q.wide_scale_stores);
    }
  }
}

__global__ void finish_scales_kernel(const uint32_t* amax_bits, size_t groups, float* global_scales) {
  const size_t g = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (g < groups) global_scales[g] = global_scale_from_amax_bits(amax_bits[g]);
}

size_t smem_bytes(int vpt) {
  return sizeof(uint4) * kTeamsPerCta * kDepth * vpt * kTeam + sizeof(TeamShared) * kTeamsPerCta;
}

// Resident CTAs of `kernel` on the current device (0 when the kernel cannot be configured).  The
// answer is cached per (device, kernel family, vectors per thread): it is a pure function of them.
template <typename K>
int resident_ctas(K kernel, size_t smem, int family, int vpt) {
  constexpr int kMaxDevices = 64;
  static std::atomic<int> cache[kMaxDevices][2][9];
  static std::atomic<bool> ready{false};
  static std::once_flag once;
  std::call_once(once, [] {
    for (auto& d : cache)
      for (auto& f : d)
        for (auto& v : f) v.store(-1);
    ready.store(true);
  });
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  const bool cacheable = dev >= 0 && dev < kMaxDevices;
  if (cacheable) {
    const int hit = cache[dev][family][vpt].load();
    if (hit >= 0) return hit;
  }
  int sms = 0, per_sm = 0, total = 0;
  if ((smem <= 48 * 1024 ||
       cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) ==
           cudaSuccess) &&
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess &&
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kCtaThreads, smem) == cudaSuccess)
    total = sms * per_sm;
  if (cacheable) cache[dev][family][vpt].store(total);
  return total;
}

template <typename K, typename... Args>
bool launch_cooperative(K kernel, unsigned grid, size_t smem, cudaStream_t s, Args... args) {
  void* params[] = {static_cast<void*>(&args)...};
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3(grid), dim3(kCtaThreads), params,
                                     smem, s) == cudaSuccess;
}

}  // namespace

size_t fused_scratch_words(size_t groups) { return 2 * groups + 2; }

// Both launchers return false when the fused path does not apply (shape, alignment, group longer
// than one sweep of the teams, or the cooperative launch is refused); nothing has been enqueued
// then and the caller takes the multi-kernel path.
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
  const size_t smem = smem_bytes(vpt);
  const size_t rps = rows_per_scale ? rows_per_scale : tokens;
  const size_t groups = (tokens + rps - 1) / rps;
  GroupBoard board{scratch, scratch + groups, scratch + 2 * groups, tokens, rps};
  QuantOut q{reinterpret_cast<uint32_t*>(codes), scales,
             row_vectors % 32 == 0 && aligned16(scales) && (row_vectors / 2) % 16 == 0};
  const bool coherent = normalized_out == right;
  const float width = static_cast<float>(hidden);
  auto L = reinterpret_cast<const uint4*>(left);
  auto R = reinterpret_cast<const uint4*>(right);
  auto W = reinterpret_cast<const uint4*>(weight);
  auto RO = reinterpret_cast<uint4*>(residual_out);
  auto NO = reinterpret_cast<uint4*>(normalized_out);
  bool ok = false;
#define Q3X_TRY(V)                                                                                        \
  case V: {                                                                                               \
    const int cap = resident_ctas(residual_norm_nvfp4_kernel<V>, smem, 0, V);                                   \
    const size_t want = (tokens + kTeamsPerCta - 1) / kTeamsPerCta;                                       \
    const unsigned grid = static_cast<unsigned>(want < static_cast<size_t>(cap) ? want : cap);            \
    if (cap > 0 && rps <= static_cast<size_t>(grid) * kTeamsPerCta) {                                      \
      cudaMemsetAsync(scratch, 0, fused_scratch_words(groups) * sizeof(uint32_t), s);                     \
      ok = launch_cooperative(residual_norm_nvfp4_kernel<V>, grid, smem, s, L, R, W, row_vectors, width,  \
                              eps, RO, NO, coherent, board, q);                                           \
    }                                                                                                     \
  } break;
  switch (vpt) { Q3X_TRY(1) Q3X_TRY(2) Q3X_TRY(3) Q3X_TRY(4) Q3X_TRY(5) Q3X_TRY(6) Q3X_TRY(7) Q3X_TRY(8) }
#undef Q3X_TRY
  if (!ok) {
    (void)cudaGetLastError();
    return false;
  }
  finish_scales_kernel<<<static_cast<unsigned>((groups + 127) / 128), 128, 0, s>>>(scratch, groups, global_scales_out);
  return true;
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
  const int vpt = (row_vectors + kTeam - 1) / kTeam;
  const size_t smem = smem_bytes(vpt);
  const size_t rps = rows_per_scale ? rows_per_scale : tokens;
  const size_t groups = (tokens + rps - 1) / rps;
  GroupBoard board{scratch, scratch + groups, scratch + 2 * groups, tokens, rps};
  QuantOut q{reinterpret_cast<uint32_t*>(codes), scales,
             row_vectors % 32 == 0 && aligned16(scales) && (row_vectors / 2) % 16 == 0};
  const bool coherent = out == in || out == gate;
  auto X = reinterpret_cast<const uint4*>(in);
  auto Z = reinterpret_cast<const uint4*>(gate);
  auto W = reinterpret_cast<const uint4*>(weight);
  auto O = reinterpret_cast<uint4*>(out);
  bool ok = false;
#define Q3X_TRY(V)                                                                                        \
  case V: {                                                                                               \
    const int cap = resident_ctas(gated_norm_nvfp4_kernel<V>, smem, 1, V);                                      \
    const size_t want = (tokens + kTeamsPerCta - 1) / kTeamsPerCta;                                       \
    const unsigned grid = static_cast<unsigned>(want < static_cast<size_t>(cap) ? want : cap);            \
    if (cap > 0 && rps <= static_cast<size_t>(grid) * kTeamsPerCta) {                                      \
      cudaMemsetAsync(scratch, 0, fused_scratch_words(groups) * sizeof(uint32_t), s);                     \
      ok = launch_cooperative(gated_norm_nvfp4_kernel<V>, grid, smem, s, X, Z, W, row_vectors, eps, O,    \
                              coherent, board, q);                                                        \
    }                                                                                                     \
  } break;
  switch (vpt) { Q3X_TRY(1) Q3X_TRY(2) Q3X_TRY(3) Q3X_TRY(4) Q3X_TRY(5) Q3X_TRY(6) Q3X_TRY(7) Q3X_TRY(8) }
#undef Q3X_TRY
  if (!ok) {
    (void)cudaGetLastError();
    return false;
  }
  finish_scales_kernel<<<static_cast<unsigned>((groups + 127) / 128), 128, 0, s>>>(scratch, groups, global_scales_out);
  return true;
}

}  // namespace q3x
