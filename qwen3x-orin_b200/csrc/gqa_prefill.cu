// Bulk causal GQA attention of a tile of tokens (24 query heads, 4 KV heads, head dimension 256) against a KV cache
// that already holds the tile's own keys and values, with the attention sigmoid output gate as its epilogue:
//   out[t, h] = bf16( bf16(softmax(q[t,h] . K[0 .. first + t]^T * scale) V[0 .. first + t]) * sigmoid(gate[t, h]) )
// -- gqa_attention_reference_cpu followed by sigmoid_gate_reference_cpu across a bf16 boundary
// (src/runtime/reference/decode_ops.cpp:302-342,445-508), once per token of the tile, which is the contract of
// launch_bulk_causal_gqa_sigmoid_gate_24_4_256_cuda (include/q3x/runtime/decode_ops.h:419-470).
//
// One CTA owns 16 consecutive tokens and one KV head: its 6 warps are the 6 query heads that share that KV head,
// each holding a 16 x 256 query block, so a K / V tile fetched into shared memory is used by 96 query rows.  Tiles
// of 64 keys stream through a two-stage cp.async pipeline; per tile a warp forms S = Q K^T (16 x 64) with
// mma.sync.m16n8k16 (bf16 operands, FP32 accumulation), runs the online softmax on its two rows per lane
// and accumulates O += P V (16 x 256, 128 FP32 registers per lane).  Operands reach the
// MMAs through ldmatrix from shared memory whose 16-byte chunks are XOR-swizzled by the row, so the eight rows of
// an ldmatrix fall into different banks.  The causal mask only touches tiles that reach past the block's first
// token.  The epilogue normalises, rounds, applies the gate, and leaves through shared memory as 128-bit stores.
// (The host reference keeps the probabilities in FP32; here each one meets V as a pair of bf16 operands, see below.)
#include <atomic>
#include <cstdlib>
#include <string>

#include "device_utils.cuh"
#include "host_checks.hpp"
#include "q3x_b200.h"
#include "tcgen05.cuh"

namespace q3x {
namespace {

constexpr int kQHeads = 24, kKvHeads = 4, kDim = 256, kGroup = kQHeads / kKvHeads;
constexpr int kBlockTokens = 16;                 // query tokens per CTA (one MMA row block per warp)
constexpr int kTileKeys = 64;                    // keys per pipeline stage
// Two shapes of CTA.  Narrow: 6 warps = the 6 query heads of a KV group over one 16-token block (a K / V tile serves
// 96 query rows).  Wide: 8 warps = 8 consecutive 16-token blocks of ONE query head (128 query rows per tile): two warps
// on each of the SM's four schedulers instead of two on two and one on two, which is what bounds the narrow shape on
// long tiles; the 6 heads of a group then read the same K / V tiles from L2 in 6 CTAs.
template <bool kWide>
struct Shape {
  static constexpr int kWarps = kWide ? 8 : kGroup;
  static constexpr int kThreads = kWarps * 32;
  static constexpr int kCtaTokens = kWide ? kWarps * kBlockTokens : kBlockTokens;
  static constexpr size_t kQBytes = static_cast<size_t>(kWarps) * kBlockTokens * kDim * 2;  // 48 / 64 KB
};
constexpr int kRowChunks = kDim * 2 / 16;        // 16-byte chunks in one 256-element bf16 row (32)
constexpr int kStages = 2;
constexpr size_t kTileBytes = static_cast<size_t>(kTileKeys) * kDim * 2;            // 32 KB
template <bool kWide>
constexpr size_t shared_bytes() { return Shape<kWide>::kQBytes + 2 * kStages * kTileBytes; }  // 176 / 192 KB

// byte offset of 16-byte chunk `chunk` of row `row` inside a [rows, 256] bf16 tile
__device__ __forceinline__ uint32_t swizzled(int row, int chunk) {
  return static_cast<uint32_t>(row * (kDim * 2) + ((chunk ^ (row & 7)) << 4));
}
__device__ __forceinline__ void cp_async_16(uint32_t smem, const void* global, bool valid) {
  const int bytes = valid ? 16 : 0;  // a missing row is zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem), "l"(global), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Requests one K and one V tile (keys [first_key, first_key + 64) of KV head `kv`) into a stage.
__device__ __forceinline__ void request_tile(const uint16_t* key_cache, const uint16_t* value_cache, int kv,
                                             size_t first_key, size_t keys, uint32_t k_smem, uint32_t v_smem, int threads) {
  for (int i = threadIdx.x; i < kTileKeys * kRowChunks; i += threads) {
    const int row = i / kRowChunks, chunk = i % kRowChunks;
    const size_t key = first_key + row;
    const bool valid = key < keys;
    const size_t element = ((valid ? key : 0) * kKvHeads + kv) * kDim + chunk * 8;
    cp_async_16(k_smem + swizzled(row, chunk), key_cache + element, valid);
    cp_async_16(v_smem + swizzled(row, chunk), value_cache + element, valid);
  }
}

template <bool kWide>
__global__ void __launch_bounds__(Shape<kWide>::kThreads, 1) gqa_prefill_kernel(const uint16_t* __restrict__ query,
                                                                  const uint16_t* __restrict__ key_cache,
                                                                  const uint16_t* __restrict__ value_cache,
                                                                  const uint16_t* __restrict__ gate, size_t first_position,
                                                                  size_t tokens, float scale_log2e,
                                                                  uint16_t* __restrict__ out) {
  extern __shared__ __align__(128) unsigned char shared[];
  const uint32_t smem = static_cast<uint32_t>(__cvta_generic_to_shared(shared));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  constexpr int kThreads = Shape<kWide>::kThreads;
  constexpr size_t kQBytes = Shape<kWide>::kQBytes;
  const int head = kWide ? static_cast<int>(blockIdx.y) : static_cast<int>(blockIdx.y) * kGroup + warp;
  const int kv = head / kGroup;
  // the last blocks of a tile see the most keys: they are scheduled first, so that the short ones fill the tail
  const size_t cta_token0 = static_cast<size_t>(gridDim.x - 1 - blockIdx.x) * Shape<kWide>::kCtaTokens;
  const size_t token0 = kWide ? cta_token0 + static_cast<size_t>(warp) * kBlockTokens : cta_token0;  // this warp's block
  // keys visible to the CTA's last token: the tiles every warp helps to fetch
  const size_t keys = first_position + min(cta_token0 + Shape<kWide>::kCtaTokens, tokens);
  const int tiles = static_cast<int>((keys + kTileKeys - 1) / kTileKeys);
  // ... and to this warp's last token: the tiles it computes on (none for a block wholly past the tile's end)
  const size_t own_keys = token0 < tokens ? first_position + min(token0 + kBlockTokens, tokens) : 0;
  const int own_tiles = static_cast<int>((own_keys + kTileKeys - 1) / kTileKeys);
  const uint32_t q_smem = smem + warp * (kBlockTokens * kDim * 2);
  auto k_stage = [&](int s) { return smem + static_cast<uint32_t>(kQBytes + (2 * s) * kTileBytes); };
  auto v_stage = [&](int s) { return smem + static_cast<uint32_t>(kQBytes + (2 * s + 1) * kTileBytes); };

  // this warp's 16 x 256 query block (rows beyond the tile are zero) rides in the first cp.async group
  for (int i = lane; i < kBlockTokens * kRowChunks; i += 32) {
    const int row = i / kRowChunks, chunk = i % kRowChunks;
    const size_t token = token0 + row;
    const bool valid = token < tokens;
    cp_async_16(q_smem + swizzled(row, chunk), query + ((valid ? token : 0) * kQHeads + head) * kDim + chunk * 8, valid);
  }
  request_tile(key_cache, value_cache, kv, 0, keys, k_stage(0), v_stage(0), kThreads);
  cp_async_commit();

  float o[kDim / 8][4];
#pragma unroll
  for (int n = 0; n < kDim / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
  // positions of this lane's two rows (g and g + 8); a key is visible when key <= position
  const size_t position[2] = {first_position + token0 + g, first_position + token0 + g + 8};

  for (int tile = 0; tile < tiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < tiles)
      request_tile(key_cache, value_cache, kv, static_cast<size_t>(tile + 1) * kTileKeys, keys, k_stage(stage ^ 1),
                   v_stage(stage ^ 1), kThreads);
    cp_async_commit();
    cp_async_wait<1>();  // everything but the newest group: this tile (and the queries) has landed
    __syncthreads();
    if (tile < own_tiles) {  // (warp-uniform) a warp whose block ends before this tile only helps to fetch it

    // ---- S = Q K^T: 16 rows x 64 keys, 8 column blocks of 8 keys
    float s[kTileKeys / 8][4];
#pragma unroll
    for (int n = 0; n < kTileKeys / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
    const uint32_t ks = k_stage(stage), vs = v_stage(stage);
#pragma unroll
    for (int kk = 0; kk < kDim / 16; ++kk) {
      uint32_t a[4];
      // A fragment: matrices (rows 0-7, dims kk*16..+7), (rows 8-15, same dims), (rows 0-7, dims +8), (rows 8-15, dims +8)
      ldmatrix_x4(a, q_smem + swizzled((lane & 7) + ((lane >> 3) & 1) * 8, kk * 2 + (lane >> 4)));
#pragma unroll
      for (int n2 = 0; n2 < kTileKeys / 16; ++n2) {
        uint32_t b[4];
        // B fragments of two key blocks: (keys n2*16..+7, dims lo), (same keys, dims hi), (keys +8, lo), (keys +8, hi)
        ldmatrix_x4(b, ks + swizzled(n2 * 16 + (lane & 7) + (lane >> 4) * 8, kk * 2 + ((lane >> 3) & 1)));
        mma_bf16(s[2 * n2], a, b[0], b[1]);
        mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
      }
    }

    // ---- causal mask (only tiles that reach past the block's first token) and online softmax
    const size_t tile_key0 = static_cast<size_t>(tile) * kTileKeys;
    if (tile_key0 + kTileKeys - 1 > first_position + token0) {
#pragma unroll
      for (int n = 0; n < kTileKeys / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const size_t key = tile_key0 + n * 8 + 2 * t + (e & 1);
          if (key > position[e >> 1]) s[n][e] = -INFINITY;
        }
    }
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < kTileKeys / 8; ++n) {
      tile_max[0] = fmaxf(tile_max[0], fmaxf(s[n][0], s[n][1]));
      tile_max[1] = fmaxf(tile_max[1], fmaxf(s[n][2], s[n][3]));
    }
    float correction[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(kFullMask, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(kFullMask, tile_max[r], 2));
      const float new_max = fmaxf(row_max[r], tile_max[r]);
      // (key 0 is visible to every row, so new_max is finite from the first tile on)
      correction[r] = exp2_approx((row_max[r] - new_max) * scale_log2e);
      row_max[r] = new_max;
      row_sum[r] *= correction[r];
    }
    // the probabilities replace the scores in place (FP32); the sums take them unrounded
#pragma unroll
    for (int n = 0; n < kTileKeys / 8; ++n) {
      s[n][0] = exp2_approx((s[n][0] - row_max[0]) * scale_log2e);
      s[n][1] = exp2_approx((s[n][1] - row_max[0]) * scale_log2e);
      s[n][2] = exp2_approx((s[n][2] - row_max[1]) * scale_log2e);
      s[n][3] = exp2_approx((s[n][3] - row_max[1]) * scale_log2e);
      row_sum[0] += s[n][0] + s[n][1];
      row_sum[1] += s[n][2] + s[n][3];
    }
#pragma unroll
    for (int n = 0; n < kDim / 8; ++n) {
      o[n][0] *= correction[0];
      o[n][1] *= correction[0];
      o[n][2] *= correction[1];
      o[n][3] *= correction[1];
    }

    // ---- O += P V: 16 rows x 256 dims, 4 key steps of 16.  A probability meets V as TWO bf16 operands, its
    // rounding and the rounding of what that left over (together 16 significant bits), so that the product keeps
    // the host reference's FP32 probabilities to rounding level; the second MMA costs a third more tensor work.
#pragma unroll
    for (int kk = 0; kk < kTileKeys / 16; ++kk) {
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // a0: rows g, keys 2t..; a1: rows g + 8; a2 / a3: the same rows, keys + 8
        const float first = s[2 * kk + (j >> 1)][(j & 1) * 2], second = s[2 * kk + (j >> 1)][(j & 1) * 2 + 1];
        hi[j] = pack_bf16x2(first, second);
        lo[j] = pack_bf16x2(first - bf16_lo(hi[j]), second - bf16_hi(hi[j]));
      }
#pragma unroll
      for (int n2 = 0; n2 < kDim / 16; ++n2) {
        uint32_t b[4];
        // transposed loads: (keys kk*16..+7, dims n2*16..+7), (keys +8, same dims), (keys lo, dims +8), (keys hi, dims +8)
        ldmatrix_x4_trans(b, vs + swizzled(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, n2 * 2 + (lane >> 4)));
        mma_bf16(o[2 * n2], hi, b[0], b[1]);
        mma_bf16(o[2 * n2], lo, b[0], b[1]);
        mma_bf16(o[2 * n2 + 1], hi, b[2], b[3]);
        mma_bf16(o[2 * n2 + 1], lo, b[2], b[3]);
      }
    }
    }  // tile < own_tiles
    __syncthreads();  // the stage is requested again two iterations from now
  }
  cp_async_wait<0>();

  // ---- epilogue: normalise, round, gate, round; through this warp's own query block in shared memory
  float inverse[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float total = row_sum[r];
    total += __shfl_xor_sync(kFullMask, total, 1);
    total += __shfl_xor_sync(kFullMask, total, 2);
    inverse[r] = 1.0f / total;
  }
  __syncwarp();
#pragma unroll
  for (int n = 0; n < kDim / 8; ++n) {
    // row g, dims n*8 + 2t, +1  and  row g + 8: chunk n of the row, byte offset 4t inside it
    const uint32_t upper = pack_bf16x2(o[n][0] * inverse[0], o[n][1] * inverse[0]);
    const uint32_t lower = pack_bf16x2(o[n][2] * inverse[1], o[n][3] * inverse[1]);
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(q_smem + swizzled(g, n) + 4 * t), "r"(upper) : "memory");
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(q_smem + swizzled(g + 8, n) + 4 * t), "r"(lower) : "memory");
  }
  __syncwarp();
  for (int i = lane; i < kBlockTokens * kRowChunks; i += 32) {
    const int row = i / kRowChunks, chunk = i % kRowChunks;
    const size_t token = token0 + row;
    if (token >= tokens) continue;
    uint4 value;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(value.x), "=r"(value.y), "=r"(value.z), "=r"(value.w)
                 : "r"(q_smem + swizzled(row, chunk)));
    const size_t element = (token * kQHeads + head) * kDim + chunk * 8;
    if (gate != nullptr) {
      float v[8], z[8];
      unpack8(value, v);
      unpack8(ld_stream(gate + element), z);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = v[e] * stable_sigmoid(z[e]);
      value = pack8(v);
    }
    st_vec(out + element, value);
  }
}

// ================================================================================================================
// The same attention on the fifth-generation tensor cores (tcgen05).  One CTA = 128 consecutive tokens of one query
// head; thread r owns query row r, which is tensor-memory lane r, so the softmax of a row needs no exchange between
// threads.  Per tile of 64 keys: S = Q K^T (M 128, N 64, K 256) into 64 columns of tensor memory; every thread reads
// its row, masks, exponentiates against the row's reference maximum and leaves the probabilities in shared memory
// as TWO bf16 A operands (rounding and remainder, as above); O += P V (M 128, N 256, K 64, twice) accumulates in 256
// columns.  V is used as it lies in the cache ([key][dimension]: an MN-major B operand); K and Q are K-major.  The
// reference maximum only moves when a tile exceeds it by more than 2^16 in the exponent's scale (then O and the row
// sum are rescaled through tensor memory), so the accumulator is normally never touched between products.  S of the
// next tile is issued together with P V of this one.  Every wait on the tensor cores is bounded; a wait that runs out
// raises a sticky error word (q3x_b200_gqa_prefill_tcgen05_error) and the CTA frees its tensor memory and returns.
// ================================================================================================================
namespace tcattn {
using namespace q3x::tcgen05;
constexpr int kRows = 128, kThreads = 128, kKeys = 64;
constexpr size_t kQ = 0;                                   // [128][256] bf16 in four blocks of [128][64]: 64 KB
constexpr size_t kStages = 65536, kKVBytes = 32768, kStageBytes = 2 * kKVBytes;  // K then V: [64][256] in four blocks
constexpr size_t kPHi = kStages + 2 * kStageBytes, kPLo = kPHi + 16384;          // [128][64] bf16 each
constexpr size_t kBarrier = kPLo + 16384, kShared = kBarrier + 64;
static_assert(kShared <= 227 * 1024, "one CTA per SM");
constexpr uint32_t kColumnsS = 0, kColumnsO = 64, kColumnsAllocated = 512;
constexpr float kRescaleThreshold = 16.0f;  // in units of the exponent (log2)

__device__ unsigned int g_error = 0;

__device__ __forceinline__ void request_tile(const uint16_t* key_cache, const uint16_t* value_cache, int kv, size_t first_key,
                                             size_t keys, uint32_t stage) {
  for (int i = threadIdx.x; i < kKeys * kRowChunks; i += kThreads) {
    const int row = i / kRowChunks, piece = i % kRowChunks;
    const size_t key = first_key + row;
    const bool valid = key < keys;
    const size_t element = ((valid ? key : 0) * kKvHeads + kv) * kDim + piece * 8;
    const uint32_t at = static_cast<uint32_t>((piece >> 3) * (kKeys * 128) + row * 128 + (((piece & 7) ^ (row & 7)) << 4));
    cp_async_16(stage + at, key_cache + element, valid);
    cp_async_16(stage + static_cast<uint32_t>(kKVBytes) + at, value_cache + element, valid);
  }
}

__global__ void __launch_bounds__(kThreads, 1) gqa_prefill_tcgen05_kernel(const uint16_t* __restrict__ query,
                                                                          const uint16_t* __restrict__ key_cache,
                                                                          const uint16_t* __restrict__ value_cache,
                                                                          const uint16_t* __restrict__ gate, size_t first_position,
                                                                          size_t tokens, float scale_log2e,
                                                                          uint16_t* __restrict__ out) {
  extern __shared__ __align__(1024) unsigned char shared[];
  const uint32_t smem = static_cast<uint32_t>(__cvta_generic_to_shared(shared));
  const int row = threadIdx.x, warp = threadIdx.x >> 5;
  const int head = blockIdx.y, kv = head / kGroup;
  const size_t token0 = static_cast<size_t>(gridDim.x - 1 - blockIdx.x) * kRows;  // heaviest blocks first
  const size_t keys = first_position + min(token0 + kRows, tokens);               // visible to the CTA's last token
  const int tiles = static_cast<int>((keys + kKeys - 1) / kKeys);
  const size_t position = first_position + token0 + row;                          // a key is visible when key <= position
  const uint32_t barrier = smem + static_cast<uint32_t>(kBarrier);
  volatile uint32_t* base_slot = reinterpret_cast<volatile uint32_t*>(shared + kBarrier + 16);

  // the queries (rows past the tile are zero) and the first K / V tile
  for (int i = threadIdx.x; i < kRows * kRowChunks; i += kThreads) {
    const int r = i / kRowChunks, piece = i % kRowChunks;
    const size_t token = token0 + r;
    const bool valid = token < tokens;
    cp_async_16(smem + static_cast<uint32_t>(kQ + (piece >> 3) * (kRows * 128) + r * 128 + (((piece & 7) ^ (r & 7)) << 4)),
                query + ((valid ? token : 0) * kQHeads + head) * kDim + piece * 8, valid);
  }
  request_tile(key_cache, value_cache, kv, 0, keys, smem + static_cast<uint32_t>(kStages));
  cp_async_commit();
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(barrier) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem + static_cast<uint32_t>(kBarrier + 16)),
                 "r"(kColumnsAllocated)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  cp_async_wait<0>();
  fence_async_proxy();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *base_slot;
  const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
  if (threadIdx.x == 0) {
    product(tmem + kColumnsS, smem + kQ, kRows * 128, smem + static_cast<uint32_t>(kStages), kKeys * 128, kDim,
            instruction_descriptor(kKeys), false);
    commit(barrier);
  }

  float reference = -INFINITY, row_sum = 0.0f;
  uint32_t parity = 0;
  bool healthy = true;
  for (int tile = 0; tile < tiles; ++tile) {
    const uint32_t stage = smem + static_cast<uint32_t>(kStages + (tile & 1) * kStageBytes);
    healthy = __syncthreads_and(wait(barrier, parity)) != 0;  // S of this tile, P V of the previous one
    parity ^= 1;
    if (!healthy) break;
    fence_after_sync();
    // the other stage is free now: the next tile's keys and values
    if (tile + 1 < tiles)
      request_tile(key_cache, value_cache, kv, static_cast<size_t>(tile + 1) * kKeys, keys,
                   smem + static_cast<uint32_t>(kStages + ((tile + 1) & 1) * kStageBytes));
    cp_async_commit();

    // ---- this row's 64 scores
    float s[kKeys];
    {
      uint32_t raw[2][32];
      load32(lane_base + kColumnsS, raw[0]);
      load32(lane_base + kColumnsS + 32, raw[1]);
      wait_loads();
#pragma unroll
      for (int e = 0; e < kKeys; ++e) s[e] = __uint_as_float(raw[e >> 5][e & 31]);
    }
    const size_t tile_key0 = static_cast<size_t>(tile) * kKeys;
    if (tile_key0 + kKeys - 1 > first_position + token0) {  // (CTA-uniform) the tile reaches past the block's first token
#pragma unroll
      for (int e = 0; e < kKeys; ++e)
        if (tile_key0 + e > position) s[e] = -INFINITY;
    }
    float tile_max = -INFINITY;
#pragma unroll
    for (int e = 0; e < kKeys; ++e) tile_max = fmaxf(tile_max, s[e]);
    // ---- the reference maximum moves only when it has to; then O and the sum follow it
    float factor = 1.0f;
    bool moved = false;
    if (reference == -INFINITY) {
      reference = tile_max;  // (key 0 is visible to every row, so this is finite from the first tile on)
    } else if ((tile_max - reference) * scale_log2e > kRescaleThreshold) {
      factor = exp2_approx((reference - tile_max) * scale_log2e);
      reference = tile_max;
      row_sum *= factor;
      moved = true;
    }
    if (tile > 0 && __any_sync(kFullMask, moved)) {
#pragma unroll 1
      for (int group = 0; group < kDim / 32; ++group) {
        uint32_t o[32];
        load32(lane_base + kColumnsO + group * 32, o);
        wait_loads();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * factor);
        store32(lane_base + kColumnsO + group * 32, o);
      }
      wait_stores();
    }
    // ---- probabilities against the reference, as two bf16 operands; the sum takes them unrounded
#pragma unroll
    for (int piece = 0; piece < kKeys / 8; ++piece) {
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float first = exp2_approx((s[piece * 8 + 2 * j] - reference) * scale_log2e);
        const float second = exp2_approx((s[piece * 8 + 2 * j + 1] - reference) * scale_log2e);
        row_sum += first + second;
        hi[j] = pack_bf16x2(first, second);
        lo[j] = pack_bf16x2(first - bf16_lo(hi[j]), second - bf16_hi(hi[j]));
      }
      const uint32_t at = static_cast<uint32_t>(row * 128 + ((piece ^ (row & 7)) << 4));
      *reinterpret_cast<uint4*>(shared + kPHi + at) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<uint4*>(shared + kPLo + at) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
    cp_async_wait<0>();  // the next tile's keys have to be there before its scores are issued
    fence_async_proxy();
    fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_after_sync();
      const uint32_t values = stage + static_cast<uint32_t>(kKVBytes);
      constexpr uint32_t kIdescPV = instruction_descriptor(kDim) | kBOperandMnMajor;
#pragma unroll
      for (int step = 0; step < kKeys / 16; ++step)
        mma(tmem + kColumnsO, operand_descriptor(smem + static_cast<uint32_t>(kPHi) + step * 32),
            operand_descriptor_mn(values + step * 2048, kKeys * 128), kIdescPV, (tile > 0 || step > 0) ? 1u : 0u);
#pragma unroll
      for (int step = 0; step < kKeys / 16; ++step)
        mma(tmem + kColumnsO, operand_descriptor(smem + static_cast<uint32_t>(kPLo) + step * 32),
            operand_descriptor_mn(values + step * 2048, kKeys * 128), kIdescPV, 1u);
      if (tile + 1 < tiles)
        product(tmem + kColumnsS, smem + kQ, kRows * 128, smem + static_cast<uint32_t>(kStages + ((tile + 1) & 1) * kStageBytes),
                kKeys * 128, kDim, instruction_descriptor(kKeys), false);
      commit(barrier);
    }
  }
  if (healthy) {
    healthy = __syncthreads_and(wait(barrier, parity)) != 0;  // the last P V
    fence_after_sync();
  }
  cp_async_wait<0>();
  if (!healthy) {
    if (threadIdx.x == 0) atomicExch(&g_error, 1u);
  } else {
    // ---- epilogue: normalise, round, gate, round; this thread's row, 512 contiguous bytes.  (The tensor-memory loads
    // are warp-collective: every lane executes them, a lane whose row lies past the tile just stores nothing.)
    const bool stores = token0 + row < tokens;
    const float inverse = 1.0f / row_sum;
    const size_t base = ((stores ? token0 + row : 0) * kQHeads + head) * kDim;
#pragma unroll 1
    for (int group = 0; group < kDim / 32; ++group) {
      uint32_t o[32];
      load32(lane_base + kColumnsO + group * 32, o);
      wait_loads();
      if (stores) {
#pragma unroll
        for (int piece = 0; piece < 4; ++piece) {
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(o[piece * 8 + e]) * inverse;
          uint4 value = pack8(v);
          if (gate != nullptr) {
            float z[8];
            unpack8(value, v);
            unpack8(ld_stream(gate + base + group * 32 + piece * 8), z);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = v[e] * stable_sigmoid(z[e]);
            value = pack8(v);
          }
          st_vec(out + base + group * 32 + piece * 8, value);
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kColumnsAllocated) : "memory");
}
}  // namespace tcattn

// Which kernel serves the entry point: 1 = tcgen05 (the default: 1.5 to 2 times the other from a thousand tokens on,
// level with it below), 0 = mma.sync (two CTA shapes).  Process-wide; Q3X_B200_GQA_PREFILL_PATH = "mma" starts on 0.
std::atomic<int>& prefill_path() {
  static std::atomic<int> path{[] {
    const char* text = std::getenv("Q3X_B200_GQA_PREFILL_PATH");
    return text != nullptr && std::string(text) == "mma" ? 0 : 1;
  }()};
  return path;
}

}  // namespace
}  // namespace q3x

using namespace q3x;
using namespace q3x::host;

extern "C" int q3x_b200_gqa_attention_prefill_sigmoid_gate(const uint16_t* query, const uint16_t* key_cache,
                                                           const uint16_t* value_cache, const uint16_t* gate,
                                                           size_t first_position, size_t tokens, float scale,
                                                           uint16_t* out, void* stream) {
  if (tokens == 0) return kOk;
  if (query == nullptr || key_cache == nullptr || value_cache == nullptr || out == nullptr) return kInvalid;
  if (!(std::isfinite(scale) && scale > 0.0f)) return kInvalid;
  if (first_position > (static_cast<size_t>(1) << 40) || tokens > 0x7fffffffu) return kInvalid;
  const size_t keys = first_position + tokens;
  const size_t tile_bytes = tokens * kQHeads * kDim * 2, cache_bytes = keys * kKvHeads * kDim * 2;
  const Span sq = span(query, tile_bytes), sg = span(gate, gate ? tile_bytes : 0), so = span(out, tile_bytes),
             sk = span(key_cache, cache_bytes), sv = span(value_cache, cache_bytes);
  if (wraps(sq) || wraps(so) || wraps(sk) || wraps(sv)) return kInvalid;
  if (overlap(so, sq) || overlap(so, sg) || overlap(so, sk) || overlap(so, sv)) return kInvalid;
  if (!aligned16(query) || !aligned16(key_cache) || !aligned16(value_cache) || !aligned16(out) ||
      (gate != nullptr && !aligned16(gate)))
    return kNotSupported;
  if (tokens / kBlockTokens + 1 > 0x7fffffffu) return kNotSupported;
  clear_stale_error();
  static const cudaError_t attribute = [] {
    cudaError_t e = cudaFuncSetAttribute(gqa_prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(shared_bytes<false>()));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gqa_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(shared_bytes<true>()));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tcattn::gqa_prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(tcattn::kShared));
    return e;
  }();
  if (attribute != cudaSuccess) {
    (void)cudaGetLastError();
    return static_cast<int>(attribute);
  }
  const float scale_log2e = scale * 1.4426950408889634f;
  // the wide shape for long tiles (8192 tokens at the start of a sequence: 3.6 ms against 4.4; 2048 tokens and
  // tiles deep in a long cache measure the same in both shapes); short tiles keep the narrow one
  // (Q3X_B200_GQA_WIDE_FROM moves the boundary, for measurements)
  static const size_t wide_from = [] {
    const char* text = std::getenv("Q3X_B200_GQA_WIDE_FROM");
    return text != nullptr ? static_cast<size_t>(std::strtoull(text, nullptr, 10)) : static_cast<size_t>(4096);
  }();
  if (prefill_path().load(std::memory_order_relaxed) == 1) {
    const unsigned blocks = static_cast<unsigned>((tokens + tcattn::kRows - 1) / tcattn::kRows);
    tcattn::gqa_prefill_tcgen05_kernel<<<dim3(blocks, kQHeads), tcattn::kThreads, tcattn::kShared, as_stream(stream)>>>(
        query, key_cache, value_cache, gate, first_position, tokens, scale_log2e, out);
  } else if (tokens >= wide_from) {
    const unsigned blocks = static_cast<unsigned>((tokens + Shape<true>::kCtaTokens - 1) / Shape<true>::kCtaTokens);
    gqa_prefill_kernel<true><<<dim3(blocks, kQHeads), Shape<true>::kThreads, shared_bytes<true>(), as_stream(stream)>>>(
        query, key_cache, value_cache, gate, first_position, tokens, scale_log2e, out);
  } else {
    const unsigned blocks = static_cast<unsigned>((tokens + kBlockTokens - 1) / kBlockTokens);
    gqa_prefill_kernel<false><<<dim3(blocks, kKvHeads), Shape<false>::kThreads, shared_bytes<false>(), as_stream(stream)>>>(
        query, key_cache, value_cache, gate, first_position, tokens, scale_log2e, out);
  }
  return launch_status();
}

extern "C" int q3x_b200_gqa_prefill_select_path(int path) {
  if (path != 0 && path != 1) return kInvalid;
  prefill_path().store(path, std::memory_order_relaxed);
  return kOk;
}

extern "C" int q3x_b200_gqa_prefill_tcgen05_error(void) {
  unsigned int word = 0;
  if (cudaMemcpyFromSymbol(&word, tcattn::g_error, sizeof(word)) != cudaSuccess) return -1;
  return static_cast<int>(word);
}
