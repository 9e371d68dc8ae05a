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
#include <cstdlib>

#include "device_utils.cuh"
#include "host_checks.hpp"
#include "q3x_b200.h"

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
  if (tokens >= wide_from) {
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
