// Gated-delta-net recurrence over a prefill span in CHUNKS of 64 tokens (the WY form the reference's production
// prefill uses: gdn_prefill_chunk64_native_detail::launch, src/kernels/sm87/gdn_prefill_chunk64_native_sm87.h:98-109;
// token-sequential definition: gated_delta_net_update_reference_cpu, src/runtime/reference/gdn_decode.cpp:186-293).
//
// Per value head, with M the [dk, dv] state, G_t = exp(sum_{s<=t} g_s) inside a chunk and M_0 the state at its start,
// the token recurrence   M_t = alpha_t M_{t-1} + k_t d_t^T,   d_t = beta_t (v_t - (alpha_t M_{t-1})^T k_t),
// o_t = M_t^T q_t   has the closed form
//     A[t][j] = beta_t (G_t / G_j) (k_t . k_j)   (j < t)          (I + A) W = beta G K     (I + A) U = beta V
//     D = U - W M_0                                                (the 64 deltas of the chunk)
//     O = diag(G) Q M_0 + P D,   P[t][j] = (q_t . k_j) G_t / G_j   (j <= t)
//     M_64 = G_64 M_0 + (diag(G_64 / G) K)^T D
// so everything that does not involve M_0 is computed for all chunks in parallel (first kernel: q / k normalisation,
// the two 64 x 64 Gram matrices on the tensor cores, the triangular solves in FP32 registers, one thread per column
// of W and of U), and only a few small products per chunk stay on the sequential path, which exists in two forms:
// with the state of a head, split over two CTAs by value rows, in the accumulators of mma.sync products (the default),
// and with the state in tensor memory and tcgen05 products issued from shared-memory descriptors; either way the
// chunk's operands stream through a two-stage shared-memory pipeline from images the first kernel wrote.  Operands of the tensor-core products are bf16 with FP32 accumulation, the
// reference's own boundaries for this form; the state between chunks stays FP32 and is rounded once, on the way out.
// Against the token-sequential form, which rounds the state to bf16 after every token, results agree to the noise of
// that rounding, not bit for bit (the reference reports the same comparison as a characterisation, tests/
// reference_gdn_prefill_chunk64_reference_engine_e2e_test.cpp:1990-2080).
#include <atomic>
#include <cstdlib>
#include <string>

#include "device_utils.cuh"
#include "host_checks.hpp"
#include "q3x_b200.h"
#include "tcgen05.cuh"

namespace q3x {
namespace {

constexpr int kHead = Q3X_B200_GDN_HEAD_DIM;                 // 128
constexpr int kValueHeads = Q3X_B200_GDN_V_HEADS;            // 48
constexpr int kKeyHeads = Q3X_B200_GDN_QK_HEADS;             // 16
constexpr int kChannels = Q3X_B200_GDN_CHANNELS;             // 10240
constexpr int kKOffset = kKeyHeads * kHead;                  // 2048
constexpr int kVOffset = 2 * kKOffset;                       // 4096
constexpr int kChunk = 64;

// ---- workspace: per chunk, images that the second kernel copies into shared memory as they are -------------------
// (16-byte pieces of a row are permuted by the row's low three bits, so that ldmatrix reads them without conflicts)
// All images have 128-byte rows (64 bf16): a [rows][128] operand is two blocks of [rows][64], the second `rows` x 128
// bytes after the first -- the layout a tensor-core shared-memory descriptor with 128-byte swizzling names directly.
constexpr size_t kQkTile = static_cast<size_t>(kChunk) * kHead * 2;   // q, W: [64 tokens][128 key dims] in two blocks;
                                                                      // k transposed: [128 key dims][64 tokens]
constexpr size_t kWTile = static_cast<size_t>(kHead) * kChunk * 2;    // U transposed: [128 value rows][64 tokens]
constexpr size_t kPTile = static_cast<size_t>(kChunk) * kChunk * 2;   // [64][64] bf16, 128-byte rows
constexpr size_t kDecayTile = 2 * kChunk * sizeof(float);             // G_t and G_64 / G_t
constexpr size_t kChunkBytes = 2 * kKeyHeads * kQkTile + kValueHeads * (2 * kWTile + kPTile + kDecayTile);

struct Workspace {
  unsigned char* base;
  size_t chunks;
  __host__ __device__ unsigned char* q(size_t c, int kh) const { return base + (c * kKeyHeads + kh) * kQkTile; }
  __host__ __device__ unsigned char* k(size_t c, int kh) const {
    return base + chunks * kKeyHeads * kQkTile + (c * kKeyHeads + kh) * kQkTile;
  }
  __host__ __device__ unsigned char* w(size_t c, int h) const {
    return base + 2 * chunks * kKeyHeads * kQkTile + (c * kValueHeads + h) * kWTile;
  }
  __host__ __device__ unsigned char* u(size_t c, int h) const {
    return base + 2 * chunks * kKeyHeads * kQkTile + chunks * kValueHeads * kWTile + (c * kValueHeads + h) * kWTile;
  }
  __host__ __device__ unsigned char* p(size_t c, int h) const {
    return base + 2 * chunks * kKeyHeads * kQkTile + 2 * chunks * kValueHeads * kWTile + (c * kValueHeads + h) * kPTile;
  }
  __host__ __device__ unsigned char* decay(size_t c, int h) const {
    return base + 2 * chunks * kKeyHeads * kQkTile + chunks * kValueHeads * (2 * kWTile + kPTile) +
           (c * kValueHeads + h) * kDecayTile;
  }
};

// byte offset of 16-byte piece `piece` of row `row` in an image with `pitch`-byte rows
__device__ __forceinline__ uint32_t image(int row, int piece, int pitch) {
  return static_cast<uint32_t>(row * pitch + ((piece ^ (row & 7)) << 4));
}
// ... and of piece `piece` (0 .. 15, eight columns each) of row `row` of a [64][128] operand in two blocks
__device__ __forceinline__ uint32_t blocked(int row, int piece) {
  return static_cast<uint32_t>((piece >> 3) * (kChunk * 128)) + image(row, piece & 7, 128);
}

__device__ __forceinline__ void cp_async_16(uint32_t smem, const void* global) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(global) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// the gate expressions of the token-sequential kernel (src/runtime/reference/gdn_decode.cpp:62-73)
__device__ __forceinline__ float softplus_ref(float v) { return v > 20.0f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float sigmoid_ref(float v) {
  if (v >= 0.0f) return __fdiv_rn(1.0f, 1.0f + expf(-v));
  const float e = expf(v);
  return __fdiv_rn(e, 1.0f + e);
}
__device__ __forceinline__ float dot8(const float (&a)[8], const float (&b)[8]) {
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s = fmaf(a[i], b[i], s);
  return s;
}

// ================================================================================================================
// First kernel: one CTA of 128 threads per (chunk, value head).  The three value heads of a key head repeat its q / k
// normalisation and Gram products (a few hundred MMAs) rather than share them: what bounds this kernel is the
// triangular solve, and the solve is bound by shared-memory broadcasts of its coefficients, one per four FMAs of a
// column -- so every thread owns TWO columns (column c of W and column c of U, which see the same coefficients) and
// three such CTAs share an SM.
// ================================================================================================================
constexpr int kPrepThreads = 128;
constexpr int kGroup = kValueHeads / kKeyHeads;  // value heads per key head (3)
constexpr int kLowerPitch = kChunk + 4;          // FP32 coefficient rows: 16-byte aligned, conflict-free when written
struct PrepShared {
  __align__(16) unsigned char k[kQkTile];        // normalised k, bf16, the workspace image
  __align__(16) unsigned char q[kQkTile];        // normalised and scaled q
  __align__(16) uint16_t v[kChunk][kHead];       // the head's value rows as they come
  __align__(16) float lower_t[kChunk][kLowerPitch];  // A transposed: [j][t], zero for t <= j
  float cumulative[kChunk], growth[kChunk], beta[kChunk];  // log G_t, G_t, beta_t
};

// exp of a difference of cumulative log-decays (<= 0): the fast exponential is accurate to 1e-5 relative even at
// arguments of -100, far inside the rounding of the bf16 operands these factors scale
__device__ __forceinline__ float decay_ratio(float later, float earlier) { return __expf(later - earlier); }

__global__ void __launch_bounds__(kPrepThreads, 3) gdn_chunk_prepare_kernel(
    const uint16_t* __restrict__ conv_qkv, size_t tokens, const uint16_t* __restrict__ a,
    const uint16_t* __restrict__ b, const uint16_t* __restrict__ A_log, const uint16_t* __restrict__ dt_bias,
    float l2_eps, Workspace ws) {
  extern __shared__ __align__(128) unsigned char raw[];
  PrepShared& sh = *reinterpret_cast<PrepShared*>(raw);
  const size_t chunk = blockIdx.x;
  const int head = blockIdx.y, key_head = head / kGroup;
  const bool publishes_qk = head % kGroup == 0;  // one of the three CTAs of a key head writes its q / k images
  const size_t token0 = chunk * kChunk;
  const int live = static_cast<int>(min(static_cast<size_t>(kChunk), tokens - token0));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t k_smem = static_cast<uint32_t>(__cvta_generic_to_shared(sh.k));
  const uint32_t q_smem = static_cast<uint32_t>(__cvta_generic_to_shared(sh.q));

  // ---- the head's value rows: asynchronous copies that land while q / k / the Gram products are worked on
  {
    const uint32_t v_smem = static_cast<uint32_t>(__cvta_generic_to_shared(sh.v));
    for (int i = tid; i < kChunk * (kHead / 8); i += kPrepThreads) {
      const int row = i / (kHead / 8), piece = i % (kHead / 8);
      if (row < live)
        cp_async_16(v_smem + static_cast<uint32_t>(i) * 16,
                    conv_qkv + (token0 + row) * kChannels + kVOffset + head * kHead + piece * 8);
      else
        *reinterpret_cast<uint4*>(&sh.v[row][piece * 8]) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
  }
  // ---- q and k: 1 / sqrt(sum + eps) (and 1 / sqrt(128) for q) in FP32, the same expressions as the sequential
  // kernel; 16 lanes per row, one 16-byte piece per lane; rows past the span are zero
  {
    const int piece = tid & 15;
    const float inv_sqrt_dim = __fdiv_rn(1.0f, sqrtf(static_cast<float>(kHead)));
    unsigned char* q_image = ws.q(chunk, key_head);
#pragma unroll
    for (int pass = 0; pass < kChunk / 8; ++pass) {
      const int row = pass * 8 + (tid >> 4);
      const bool valid = row < live;
      const uint16_t* source = conv_qkv + (token0 + (valid ? row : 0)) * kChannels + key_head * kHead;
      float qv[8], kv[8];
      unpack8(valid ? ld_weight(reinterpret_cast<const uint4*>(source) + piece) : make_uint4(0, 0, 0, 0), qv);
      unpack8(valid ? ld_weight(reinterpret_cast<const uint4*>(source + kKOffset) + piece) : make_uint4(0, 0, 0, 0), kv);
      const float q_scale = __fdiv_rn(1.0f, sqrtf(group_sum<16>(dot8(qv, qv)) + l2_eps)) * inv_sqrt_dim;
      const float k_scale = __fdiv_rn(1.0f, sqrtf(group_sum<16>(dot8(kv, kv)) + l2_eps));
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        qv[i] *= q_scale;
        kv[i] *= k_scale;
      }
      const uint4 qp = pack8(qv), kp = pack8(kv);
      const uint32_t at = image(row, piece, kHead * 2);
      *reinterpret_cast<uint4*>(sh.q + at) = qp;
      *reinterpret_cast<uint4*>(sh.k + at) = kp;
      if (publishes_qk) st_vec(q_image + blocked(row, piece), qp);  // (k leaves transposed, from the solve's prologue)
    }
  }
  // ---- the head's gates: warp 0, two tokens per lane, a scan over the log-decays
  if (warp == 0) {
    const float a_decay = -expf(bf16_to_float(A_log[head]));
    const float bias = bf16_to_float(dt_bias[head]);
    float g2[2], beta2[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int row = 2 * lane + e;
      const bool valid = row < live;  // a row past the span neither decays nor updates the state
      g2[e] = valid ? a_decay * softplus_ref(bf16_to_float(a[(token0 + row) * kValueHeads + head]) + bias) : 0.0f;
      beta2[e] = valid ? sigmoid_ref(bf16_to_float(b[(token0 + row) * kValueHeads + head])) : 0.0f;
    }
    float inclusive = g2[0] + g2[1];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, inclusive, d);
      if (lane >= d) inclusive += up;
    }
    const float last = __shfl_sync(0xffffffffu, inclusive, 31);  // log G_64
    float* decay = reinterpret_cast<float*>(ws.decay(chunk, head));
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int row = 2 * lane + e;
      const float c = e == 0 ? inclusive - g2[1] : inclusive;
      sh.cumulative[row] = c;
      sh.growth[row] = expf(c);
      sh.beta[row] = beta2[e];
      decay[row] = expf(c);                  // G_t
      decay[kChunk + row] = expf(last - c);  // G_64 / G_t
    }
  }
  __syncthreads();

  // ---- the two Gram matrices, a 16-row block per warp; straight from the accumulators, A transposed goes to shared
  // memory (FP32) and P to its workspace image (bf16)
  {
    const int g = lane >> 2, t = lane & 3;
    float kk[kChunk / 8][4], qk[kChunk / 8][4];
#pragma unroll
    for (int n = 0; n < kChunk / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) kk[n][e] = qk[n][e] = 0.0f;
#pragma unroll
    for (int step = 0; step < kHead / 16; ++step) {
      uint32_t ak[4], aq[4];
      const uint32_t a_at = image(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, step * 2 + (lane >> 4), kHead * 2);
      ldmatrix_x4(ak, k_smem + a_at);
      ldmatrix_x4(aq, q_smem + a_at);
#pragma unroll
      for (int n2 = 0; n2 < kChunk / 16; ++n2) {
        uint32_t bk[4];
        ldmatrix_x4(bk, k_smem + image(n2 * 16 + (lane & 7) + (lane >> 4) * 8, step * 2 + ((lane >> 3) & 1), kHead * 2));
        mma_bf16(kk[2 * n2], ak, bk[0], bk[1]);
        mma_bf16(kk[2 * n2 + 1], ak, bk[2], bk[3]);
        mma_bf16(qk[2 * n2], aq, bk[0], bk[1]);
        mma_bf16(qk[2 * n2 + 1], aq, bk[2], bk[3]);
      }
    }
    unsigned char* p_image = ws.p(chunk, head);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = warp * 16 + g + half * 8;  // token t of A[t][j] and P[t][j]
      const float own = sh.cumulative[row], scale = sh.beta[row];
#pragma unroll
      for (int n = 0; n < kChunk / 8; ++n) {
        const int j = n * 8 + 2 * t;
        const float2 earlier = *reinterpret_cast<const float2*>(&sh.cumulative[j]);
        const float r0 = decay_ratio(own, earlier.x), r1 = decay_ratio(own, earlier.y);
        sh.lower_t[j][row] = j < row ? scale * kk[n][half * 2] * r0 : 0.0f;
        sh.lower_t[j + 1][row] = j + 1 < row ? scale * kk[n][half * 2 + 1] * r1 : 0.0f;
        const uint32_t pair = pack_bf16x2(j <= row ? qk[n][half * 2] * r0 : 0.0f, j + 1 <= row ? qk[n][half * 2 + 1] * r1 : 0.0f);
        st_u32(p_image + image(row, n, kChunk * 2) + 4 * t, pair);
      }
    }
  }
  cp_async_wait_all();
  __syncthreads();  // A transposed and the value rows are complete

  // ---- (I + A) [W | U] = [beta G K | beta V]: thread c owns column c of W AND column c of U (128 registers) and
  // eliminates row by row; a coefficient, broadcast from shared memory four rows per load, serves both columns
  float xw[kChunk], xu[kChunk];
  {
    const int piece = tid >> 3, within = tid & 7;
#pragma unroll
    for (int t = 0; t < kChunk; ++t)
      xw[t] = bf16_to_float(*reinterpret_cast<const uint16_t*>(sh.k + image(t, piece, kHead * 2) + within * 2));
    if (publishes_qk) {  // this thread's key dimension over the 64 tokens: one 128-byte row of the transposed k image
      unsigned char* k_image = ws.k(chunk, key_head);
#pragma unroll
      for (int p8 = 0; p8 < kChunk / 8; ++p8) {
        float eight[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) eight[e] = xw[p8 * 8 + e];
        st_vec(k_image + image(tid, p8, kChunk * 2), pack8(eight));  // (bf16 values: the packing is exact)
      }
    }
#pragma unroll
    for (int t = 0; t < kChunk; ++t) {
      const float scale = sh.beta[t];
      xw[t] *= scale * sh.growth[t];
      xu[t] = scale * bf16_to_float(sh.v[t][tid]);
    }
  }
#pragma unroll
  for (int j = 0; j < kChunk - 1; ++j) {
    const float2 minus_w = make_float2(-xw[j], -xw[j]), minus_u = make_float2(-xu[j], -xu[j]);
#pragma unroll
    for (int t4 = (j + 1) / 4; t4 < kChunk / 4; ++t4) {
      // rows t <= j of this group carry a zero coefficient
      const float4 c = *reinterpret_cast<const float4*>(&sh.lower_t[j][t4 * 4]);
      const float2 c01 = make_float2(c.x, c.y), c23 = make_float2(c.z, c.w);
      const float2 w01 = fma2(c01, minus_w, make_float2(xw[t4 * 4 + 0], xw[t4 * 4 + 1]));
      const float2 w23 = fma2(c23, minus_w, make_float2(xw[t4 * 4 + 2], xw[t4 * 4 + 3]));
      const float2 u01 = fma2(c01, minus_u, make_float2(xu[t4 * 4 + 0], xu[t4 * 4 + 1]));
      const float2 u23 = fma2(c23, minus_u, make_float2(xu[t4 * 4 + 2], xu[t4 * 4 + 3]));
      xw[t4 * 4 + 0] = w01.x;
      xw[t4 * 4 + 1] = w01.y;
      xw[t4 * 4 + 2] = w23.x;
      xw[t4 * 4 + 3] = w23.y;
      xu[t4 * 4 + 0] = u01.x;
      xu[t4 * 4 + 1] = u01.y;
      xu[t4 * 4 + 2] = u23.x;
      xu[t4 * 4 + 3] = u23.y;
    }
  }
  // column c of U is row c of its transposed image: 128 contiguous bytes, pieces permuted by the row
  unsigned char* u_image = ws.u(chunk, head);
#pragma unroll
  for (int piece = 0; piece < kChunk / 8; ++piece) {
    float eight[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) eight[e] = xu[piece * 8 + e];
    st_vec(u_image + image(tid, piece, kChunk * 2), pack8(eight));
  }
  // W leaves token-major ([token][key dim] in two blocks, the B operand of S W^T with the key dimension contiguous):
  // transposed through the shared memory that held q (every warp is past the Gram products), then 16 bytes a thread
#pragma unroll
  for (int t = 0; t < kChunk; ++t)
    *reinterpret_cast<uint16_t*>(sh.q + blocked(t, tid >> 3) + (tid & 7) * 2) = float_to_bf16(xw[t]);
  __syncthreads();
  unsigned char* w_image = ws.w(chunk, head);
  for (int i = tid; i < static_cast<int>(kQkTile / 16); i += kPrepThreads)
    st_vec(w_image + i * 16, *reinterpret_cast<const uint4*>(sh.q + i * 16));
}

// ================================================================================================================
// Second kernel: the sequential path.  One CTA per (value head, half of its 128 value rows); a warp owns 16 value
// rows of the state, transposed ([value row][key dimension], the layout the state has in memory), as the FP32
// accumulators of its MMAs.  An accumulator tile read as (row, column pair) is exactly the A operand of the next
// product, so the state, the deltas and the outputs never leave registers between the products of a chunk:
//     D^T  = U^T - S^T W^T              (A = S^T as bf16, B = W^T)
//     O^T  = (S^T Q^T) diag(G) + D^T P^T
//     S^T <- G_64 S^T + (D^T diag(G_64 / G)) K
// ================================================================================================================
constexpr int kStateThreads = 128;
constexpr int kRowsPerCta = 64;  // value rows per CTA: 16 per warp
constexpr int kStateSplits = kHead / kRowsPerCta;
constexpr size_t kUSlice = static_cast<size_t>(kRowsPerCta) * kChunk * 2;
constexpr size_t kStageW = 0, kStageQ = kStageW + kWTile, kStageK = kStageQ + kQkTile, kStageP = kStageK + kQkTile,
                 kStageU = kStageP + kPTile, kStageDecay = kStageU + kUSlice, kStageBytes = kStageDecay + kDecayTile;
constexpr size_t kOutStage = 2 * kStageBytes;                                // [64 tokens][64 value rows] bf16
constexpr size_t kStateShared = kOutStage + static_cast<size_t>(kChunk) * kRowsPerCta * 2;
static_assert(kStageBytes % 16 == 0, "stages are copied in 16-byte pieces");

__device__ __forceinline__ void copy_linear(uint32_t smem, const unsigned char* global, size_t bytes) {
  for (size_t at = static_cast<size_t>(threadIdx.x) * 16; at < bytes; at += static_cast<size_t>(kStateThreads) * 16)
    cp_async_16(smem + static_cast<uint32_t>(at), global + at);
}

__device__ __forceinline__ void request_chunk(const Workspace& ws, size_t chunk, int head, int split, uint32_t stage) {
  copy_linear(stage + kStageW, ws.w(chunk, head), kWTile);
  copy_linear(stage + kStageQ, ws.q(chunk, head / (kValueHeads / kKeyHeads)), kQkTile);
  copy_linear(stage + kStageK, ws.k(chunk, head / (kValueHeads / kKeyHeads)), kQkTile);
  copy_linear(stage + kStageP, ws.p(chunk, head), kPTile);
  copy_linear(stage + kStageU, ws.u(chunk, head) + split * kUSlice, kUSlice);
  copy_linear(stage + kStageDecay, ws.decay(chunk, head), kDecayTile);
}

__global__ void __launch_bounds__(kStateThreads, 1) gdn_chunk_state_kernel(Workspace ws, size_t tokens,
                                                                           const uint16_t* state_in, uint16_t* state_out,
                                                                           uint16_t* __restrict__ out) {
  extern __shared__ __align__(128) unsigned char shared[];
  const uint32_t smem = static_cast<uint32_t>(__cvta_generic_to_shared(shared));
  const int head = blockIdx.x, split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int row_local = warp * 16 + g;                  // and row_local + 8
  const int row_global = split * kRowsPerCta + row_local;

  request_chunk(ws, 0, head, split, smem);
  cp_async_commit();

  // S[n][e]: rows row_global (e < 2) / row_global + 8, key dimensions n * 8 + 2t + (e & 1)
  float S[kHead / 8][4];
  {
    const uint16_t* base = state_in + (static_cast<size_t>(head) * kHead + row_global) * kHead;
#pragma unroll
    for (int n = 0; n < kHead / 8; ++n) {
      const uint32_t upper = *reinterpret_cast<const uint32_t*>(base + n * 8 + 2 * t);
      const uint32_t lower = *reinterpret_cast<const uint32_t*>(base + 8 * kHead + n * 8 + 2 * t);
      S[n][0] = bf16_lo(upper);
      S[n][1] = bf16_hi(upper);
      S[n][2] = bf16_lo(lower);
      S[n][3] = bf16_hi(lower);
    }
  }

  for (size_t chunk = 0; chunk < ws.chunks; ++chunk) {
    const uint32_t stage = smem + static_cast<uint32_t>((chunk & 1) * kStageBytes);
    cp_async_wait_all();
    __syncthreads();  // this chunk's operands are in place; everybody is done with the other stage and the out tile
    if (chunk + 1 < ws.chunks) request_chunk(ws, chunk + 1, head, split, smem + static_cast<uint32_t>(((chunk + 1) & 1) * kStageBytes));
    cp_async_commit();

    const float* growth = reinterpret_cast<const float*>(shared + (chunk & 1) * kStageBytes + kStageDecay);  // G_t
    const float* to_end = growth + kChunk;                                                                   // G_64 / G_t

    // ---- the state as a bf16 A operand: eight steps of 16 key dimensions
    uint32_t sa[kHead / 16][4];
#pragma unroll
    for (int step = 0; step < kHead / 16; ++step) {
      sa[step][0] = pack_bf16x2(S[2 * step][0], S[2 * step][1]);
      sa[step][1] = pack_bf16x2(S[2 * step][2], S[2 * step][3]);
      sa[step][2] = pack_bf16x2(S[2 * step + 1][0], S[2 * step + 1][1]);
      sa[step][3] = pack_bf16x2(S[2 * step + 1][2], S[2 * step + 1][3]);
    }
    // ---- predicted part S^T W^T and the inter-chunk output S^T Q^T: 16 value rows x 64 tokens each
    float pred[kChunk / 8][4], o[kChunk / 8][4];
#pragma unroll
    for (int n = 0; n < kChunk / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) pred[n][e] = o[n][e] = 0.0f;
#pragma unroll
    for (int step = 0; step < kHead / 16; ++step) {
#pragma unroll
      for (int n2 = 0; n2 < kChunk / 16; ++n2) {
        uint32_t bw[4], bq[4];
        // W and Q images: rows are tokens (the product's n), pieces are 8 key dimensions (its k), 64 per block
        ldmatrix_x4(bw, stage + kStageW + (step >> 2) * (kChunk * 128) +
                            image(n2 * 16 + (lane & 7) + (lane >> 4) * 8, (step & 3) * 2 + ((lane >> 3) & 1), 128));
        mma_bf16(pred[2 * n2], sa[step], bw[0], bw[1]);
        mma_bf16(pred[2 * n2 + 1], sa[step], bw[2], bw[3]);
        ldmatrix_x4(bq, stage + kStageQ + (step >> 2) * (kChunk * 128) +
                            image(n2 * 16 + (lane & 7) + (lane >> 4) * 8, (step & 3) * 2 + ((lane >> 3) & 1), 128));
        mma_bf16(o[2 * n2], sa[step], bq[0], bq[1]);
        mma_bf16(o[2 * n2 + 1], sa[step], bq[2], bq[3]);
      }
    }
    // ---- D^T = U^T - pred (FP32), as two bf16 A operands over the tokens: plain, and scaled by G_64 / G_t
    uint32_t da[kChunk / 16][4], ds[kChunk / 16][4];
#pragma unroll
    for (int n = 0; n < kChunk / 8; ++n) {
      const uint32_t upper = *reinterpret_cast<const uint32_t*>(shared + (chunk & 1) * kStageBytes + kStageU +
                                                                image(row_local, n, kChunk * 2) + 4 * t);
      const uint32_t lower = *reinterpret_cast<const uint32_t*>(shared + (chunk & 1) * kStageBytes + kStageU +
                                                                image(row_local + 8, n, kChunk * 2) + 4 * t);
      const float d0 = bf16_lo(upper) - pred[n][0], d1 = bf16_hi(upper) - pred[n][1];
      const float d2 = bf16_lo(lower) - pred[n][2], d3 = bf16_hi(lower) - pred[n][3];
      const float2 grow = *reinterpret_cast<const float2*>(growth + n * 8 + 2 * t);
      const float2 end = *reinterpret_cast<const float2*>(to_end + n * 8 + 2 * t);
      // tokens n * 8 + 2t, + 1: k slots (n & 1) * 8 + 2t of step n / 2
      da[n >> 1][(n & 1) * 2 + 0] = pack_bf16x2(d0, d1);
      da[n >> 1][(n & 1) * 2 + 1] = pack_bf16x2(d2, d3);
      ds[n >> 1][(n & 1) * 2 + 0] = pack_bf16x2(d0 * end.x, d1 * end.y);
      ds[n >> 1][(n & 1) * 2 + 1] = pack_bf16x2(d2 * end.x, d3 * end.y);
      // the inter-chunk output of token i carries G_i
      o[n][0] *= grow.x;
      o[n][1] *= grow.y;
      o[n][2] *= grow.x;
      o[n][3] *= grow.y;
    }
    // ---- O^T += D^T P^T  (P image: rows are output tokens (n), pieces are 8 source tokens (k): plain loads)
#pragma unroll
    for (int step = 0; step < kChunk / 16; ++step) {
#pragma unroll
      for (int n2 = 0; n2 < kChunk / 16; ++n2) {
        uint32_t bp[4];
        ldmatrix_x4(bp, stage + kStageP + image(n2 * 16 + (lane & 7) + (lane >> 4) * 8, step * 2 + ((lane >> 3) & 1), kChunk * 2));
        mma_bf16(o[2 * n2], da[step], bp[0], bp[1]);
        mma_bf16(o[2 * n2 + 1], da[step], bp[2], bp[3]);
      }
    }
    // ---- S^T <- G_64 S^T + (D^T diag(G_64 / G)) K  (transposed K image: rows are key dimensions (n), pieces 8 tokens (k))
    {
      const float whole = growth[kChunk - 1];
#pragma unroll
      for (int n = 0; n < kHead / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) S[n][e] *= whole;
    }
#pragma unroll
    for (int step = 0; step < kChunk / 16; ++step) {
#pragma unroll
      for (int n2 = 0; n2 < kHead / 16; ++n2) {
        uint32_t bk[4];
        ldmatrix_x4(bk, stage + kStageK + image(n2 * 16 + (lane & 7) + (lane >> 4) * 8, step * 2 + ((lane >> 3) & 1), kChunk * 2));
        mma_bf16(S[2 * n2], ds[step], bk[0], bk[1]);
        mma_bf16(S[2 * n2 + 1], ds[step], bk[2], bk[3]);
      }
    }
    // ---- the chunk's outputs: transposed through shared memory, then 128-byte rows to out[token][head][rows]
    {
      unsigned char* tile = shared + kOutStage;
#pragma unroll
      for (int n = 0; n < kChunk / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int token = n * 8 + 2 * t + (e & 1), row = row_local + (e >> 1) * 8;
          *reinterpret_cast<uint16_t*>(tile + image(token, row >> 3, kRowsPerCta * 2) + (row & 7) * 2) = float_to_bf16(o[n][e]);
        }
    }
    __syncthreads();
    {
      const unsigned char* tile = shared + kOutStage;
      const size_t token0 = chunk * kChunk;
      for (int i = threadIdx.x; i < kChunk * (kRowsPerCta / 8); i += kStateThreads) {
        const int token = i / (kRowsPerCta / 8), piece = i % (kRowsPerCta / 8);
        if (token0 + token < tokens)
          st_vec(out + ((token0 + token) * kValueHeads + head) * kHead + split * kRowsPerCta + piece * 8,
                 *reinterpret_cast<const uint4*>(tile + image(token, piece, kRowsPerCta * 2)));
      }
    }
  }
  cp_async_wait_all();
  // ---- the state leaves as bf16, rounded once
  {
    uint16_t* base = state_out + (static_cast<size_t>(head) * kHead + row_global) * kHead;
#pragma unroll
    for (int n = 0; n < kHead / 8; ++n) {
      *reinterpret_cast<uint32_t*>(base + n * 8 + 2 * t) = pack_bf16x2(S[n][0], S[n][1]);
      *reinterpret_cast<uint32_t*>(base + 8 * kHead + n * 8 + 2 * t) = pack_bf16x2(S[n][2], S[n][3]);
    }
  }
}

// ================================================================================================================
// The sequential path on the fifth-generation tensor cores (tcgen05): one CTA of 128 threads per value head.  The
// state S^T [128 value rows x 128 key dimensions] lives in tensor memory as FP32 for the whole call, thread r owning
// value row r (tensor-memory lane r).  Per chunk:
//   1. every thread reads its row of S, leaves it in shared memory as the bf16 A operand of this chunk's products and
//      writes G_64 S back (the decayed state the chunk's update accumulates onto);
//   2. one thread issues  pred^T = S W^T  and  o1^T = S Q^T  (M 128, N 64, K 128 each);
//   3. every thread reads its row of pred, forms D^T = U^T - pred^T, and leaves D and its decayed copy in shared memory
//      as bf16 A operands;
//   4. one thread issues  o2^T = D P^T  (N 64, K 64)  and  S^T += (D diag(G_64 / G)) K  (N 128, K 64);
//   5. every thread reads its rows of o1 and o2, o = o1 G_t + o2, and the chunk's outputs leave through shared memory.
// The B operands are the workspace images as they are (rows of 64 bf16, 16-byte pieces permuted by the row = the
// 128-byte swizzle of a shared-memory matrix descriptor), copied into a two-stage ring by cp.async.  Every wait on
// the MMA barrier is bounded; if one runs out the CTA raises the workspace's error word, frees its tensor memory and
// returns.
// ================================================================================================================
namespace tc {
using namespace q3x::tcgen05;
// 128 value rows x kParts: thread (row, part) owns a quarter of its row's columns in every per-row pass, so that a
// scheduler has four warps to overlap (warps w and w + 4k read the same 32 tensor-memory lanes)
constexpr int kParts = 4;
constexpr int kThreads = 128 * kParts;
// tensor-memory columns (FP32): the state, pred (whose columns o2 takes once every thread has read pred), o1
constexpr uint32_t kColumnsS = 0, kColumnsPred = 128, kColumnsO1 = 192, kColumnsO2 = kColumnsPred, kColumnsAllocated = 256;
constexpr size_t kOperandS = 0;                          // [128][128] bf16 in two blocks of [128][64]: 32 KB
constexpr size_t kOperandD = kOperandS + 32768;          // [128][64] bf16: 16 KB (and the output tile afterwards)
constexpr size_t kOperandDecayed = kOperandD + 16384;    // 16 KB
constexpr size_t kStages = kOperandDecayed + 16384;
constexpr size_t kInW = 0, kInQ = kInW + kQkTile, kInK = kInQ + kQkTile, kInP = kInK + kQkTile, kInU = kInP + kPTile,
                 kInDecay = kInU + kWTile, kStageBytes = (kInDecay + kDecayTile + 1023) / 1024 * 1024;
constexpr size_t kBarrier = kStages + 2 * kStageBytes;   // the MMA barrier (8 bytes), the tensor-memory base (4)
constexpr size_t kShared = kBarrier + 64;
static_assert(kShared <= 227 * 1024, "one CTA per SM");

__device__ __forceinline__ void request_chunk(const Workspace& ws, size_t chunk, int head, uint32_t stage) {
  auto copy = [&](size_t at, const unsigned char* from, size_t bytes) {
    for (size_t i = static_cast<size_t>(threadIdx.x) * 16; i < bytes; i += static_cast<size_t>(kThreads) * 16)
      cp_async_16(stage + static_cast<uint32_t>(at + i), from + i);
  };
  copy(kInW, ws.w(chunk, head), kQkTile);
  copy(kInQ, ws.q(chunk, head / (kValueHeads / kKeyHeads)), kQkTile);
  copy(kInK, ws.k(chunk, head / (kValueHeads / kKeyHeads)), kQkTile);
  copy(kInP, ws.p(chunk, head), kPTile);
  copy(kInU, ws.u(chunk, head), kWTile);
  copy(kInDecay, ws.decay(chunk, head), kDecayTile);
}

__global__ void __launch_bounds__(kThreads, 1) gdn_chunk_state_tcgen05_kernel(Workspace ws, size_t tokens,
                                                                              const uint16_t* state_in, uint16_t* state_out,
                                                                              uint16_t* __restrict__ out, uint32_t* error_word) {
  extern __shared__ __align__(1024) unsigned char shared[];
  const uint32_t smem = static_cast<uint32_t>(__cvta_generic_to_shared(shared));
  const int head = blockIdx.x, row = threadIdx.x & 127, part = threadIdx.x >> 7, warp = threadIdx.x >> 5;
  const uint32_t barrier = smem + static_cast<uint32_t>(kBarrier);
  volatile uint32_t* base_slot = reinterpret_cast<volatile uint32_t*>(shared + kBarrier + 16);

  request_chunk(ws, 0, head, smem + static_cast<uint32_t>(kStages));
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
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *base_slot;
  const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);  // this warp's 32 lanes
  constexpr int kStateColumns = kHead / kParts;   // 32 key dimensions of the state per thread
  constexpr int kTokenColumns = kChunk / kParts;  // 16 tokens of pred / o per thread

  // ---- the state enters tensor memory: thread (r, p) brings key dimensions 32p .. 32p + 31 of value row r
  {
    const uint16_t* source = state_in + (static_cast<size_t>(head) * kHead + row) * kHead + part * kStateColumns;
    uint32_t r[32];
#pragma unroll
    for (int piece = 0; piece < 4; ++piece) {
      float f[8];
      unpack8(ld_vec(source + piece * 8), f);
#pragma unroll
      for (int e = 0; e < 8; ++e) r[piece * 8 + e] = __float_as_uint(f[e]);
    }
    store32(lane_base + kColumnsS + part * kStateColumns, r);
    wait_stores();
  }

  uint32_t parity = 0;
  bool healthy = true;
  for (size_t chunk = 0; chunk < ws.chunks; ++chunk) {
    const size_t stage_at = kStages + (chunk & 1) * kStageBytes;
    const uint32_t stage = smem + static_cast<uint32_t>(stage_at);
    const float* growth = reinterpret_cast<const float*>(shared + stage_at + kInDecay);  // G_t
    const float* to_end = growth + kChunk;                                               // G_64 / G_t
    cp_async_wait_all();
    fence_async_proxy();  // the copies were generic-proxy writes; the tensor core reads through the async proxy
    __syncthreads();      // this chunk's operands are in place; everybody is done with the other stage
    if (chunk + 1 < ws.chunks) request_chunk(ws, chunk + 1, head, smem + static_cast<uint32_t>(kStages + ((chunk + 1) & 1) * kStageBytes));
    cp_async_commit();

    // ---- 1. S as the bf16 A operand of this chunk's first products; they are issued before anything else happens
    uint32_t s_part[32];
    load32(lane_base + kColumnsS + part * kStateColumns, s_part);
    wait_loads();
#pragma unroll
    for (int piece = 0; piece < 4; ++piece) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(s_part[piece * 8 + e]);
      *reinterpret_cast<uint4*>(shared + kOperandS + (part >> 1) * 16384 + image(row, (part & 1) * 4 + piece, 128)) = pack8(f);
    }
    fence_async_proxy();
    fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_after_sync();
      product(tmem + kColumnsPred, smem + kOperandS, 16384, stage + kInW, kChunk * 128, kHead, instruction_descriptor(kChunk), false);
      commit(barrier);  // D needs pred only ...
      product(tmem + kColumnsO1, smem + kOperandS, 16384, stage + kInQ, kChunk * 128, kHead, instruction_descriptor(kChunk),
              false);  // ... o1 completes with the second commit of the chunk
    }
    // ---- underneath those products: G_64 S back to tensor memory (the update accumulates onto it)
    {
      const float whole = growth[kChunk - 1];
#pragma unroll
      for (int e = 0; e < 32; ++e) s_part[e] = __float_as_uint(__uint_as_float(s_part[e]) * whole);
      store32(lane_base + kColumnsS + part * kStateColumns, s_part);
      wait_stores();
    }
    healthy = __syncthreads_and(wait(barrier, parity)) != 0;  // pred
    parity ^= 1;
    if (!healthy) break;
    fence_after_sync();
    // ---- 2. D^T = U^T - pred^T and its decayed copy as bf16 A operands: tokens 16p .. 16p + 15 of row r
    {
      uint32_t r[16];
      load16(lane_base + kColumnsPred + part * kTokenColumns, r);
      wait_loads();
#pragma unroll
      for (int piece = 0; piece < 2; ++piece) {
        float u[8], d[8], decayed[8];
        unpack8(*reinterpret_cast<const uint4*>(shared + stage_at + kInU + image(row, part * 2 + piece, 128)), u);
        const float4 e0 = *reinterpret_cast<const float4*>(to_end + part * kTokenColumns + piece * 8);
        const float4 e1 = *reinterpret_cast<const float4*>(to_end + part * kTokenColumns + piece * 8 + 4);
        const float factor[8] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          d[e] = u[e] - __uint_as_float(r[piece * 8 + e]);
          decayed[e] = d[e] * factor[e];
        }
        *reinterpret_cast<uint4*>(shared + kOperandD + image(row, part * 2 + piece, 128)) = pack8(d);
        *reinterpret_cast<uint4*>(shared + kOperandDecayed + image(row, part * 2 + piece, 128)) = pack8(decayed);
      }
    }
    fence_async_proxy();
    fence_before_sync();
    __syncthreads();
    // ---- S^T += (D diag(G_64 / G)) K, o2^T = D P^T
    if (threadIdx.x == 0) {
      fence_after_sync();
      product(tmem + kColumnsS, smem + kOperandDecayed, 0, stage + kInK, 0, kChunk, instruction_descriptor(kHead), true);
      product(tmem + kColumnsO2, smem + kOperandD, 0, stage + kInP, 0, kChunk, instruction_descriptor(kChunk), false);
      commit(barrier);
    }
    healthy = __syncthreads_and(wait(barrier, parity)) != 0;  // everything issued so far: the state, o1 and o2
    parity ^= 1;
    if (!healthy) break;
    fence_after_sync();
    // ---- 3. the chunk's outputs, o = o1 G_t + o2: tokens 16p .. 16p + 15 of value row r; the 32 rows of a warp make
    // one 64-byte segment per token
    {
      uint32_t first[16], second[16];
      load16(lane_base + kColumnsO1 + part * kTokenColumns, first);
      load16(lane_base + kColumnsO2 + part * kTokenColumns, second);
      wait_loads();
      const size_t token0 = chunk * kChunk + part * kTokenColumns;
      uint16_t* target = out + (token0 * kValueHeads + head) * kHead + row;
#pragma unroll
      for (int token = 0; token < kTokenColumns; ++token)
        if (token0 + token < tokens)
          target[static_cast<size_t>(token) * kValueHeads * kHead] = float_to_bf16(
              fmaf(__uint_as_float(first[token]), growth[part * kTokenColumns + token], __uint_as_float(second[token])));
    }
    fence_before_sync();
  }
  cp_async_wait_all();
  if (!healthy) {
    if (threadIdx.x == 0) atomicExch(error_word, 1u);
  } else {
    fence_after_sync();
    // ---- the state leaves as bf16, rounded once
    uint16_t* target = state_out + (static_cast<size_t>(head) * kHead + row) * kHead + part * kStateColumns;
    uint32_t r[32];
    load32(lane_base + kColumnsS + part * kStateColumns, r);
    wait_loads();
#pragma unroll
    for (int piece = 0; piece < 4; ++piece) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[piece * 8 + e]);
      st_vec(target + piece * 8, pack8(f));
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kColumnsAllocated) : "memory");
}
}  // namespace tc

size_t chunks_of(size_t tokens) { return (tokens + kChunk - 1) / kChunk; }
constexpr size_t kErrorSlot = 256;  // after the chunk images: a word a kernel raises when a bounded wait runs out

__global__ void clear_error_kernel(uint32_t* error_word) { *error_word = 0u; }

// Which form of the sequential kernel runs: 0 = mma.sync (two CTAs per head; the faster one today), 1 = tcgen05 (one
// CTA per head, state in tensor memory).  Process-wide; starts from Q3X_B200_GDN_CHUNK_PATH ("tcgen05" selects 1).
std::atomic<int>& chunk_path() {
  static std::atomic<int> path{[] {
    const char* text = std::getenv("Q3X_B200_GDN_CHUNK_PATH");
    return text != nullptr && std::string(text) == "tcgen05" ? 1 : 0;
  }()};
  return path;
}
bool use_tcgen05() { return chunk_path().load(std::memory_order_relaxed) == 1; }

int launch_chunked(const uint16_t* conv_qkv, size_t tokens, const uint16_t* a, const uint16_t* b, const uint16_t* A_log,
                   const uint16_t* dt_bias, const uint16_t* state_in, uint16_t* state_out, float l2_eps, uint16_t* out,
                   void* workspace, size_t workspace_bytes, void* stream) {
  using namespace host;
  if (!valid_epsilon(l2_eps)) return kInvalid;
  if (mul3_overflows(tokens, kChannels, sizeof(uint16_t)) || mul_overflows(chunks_of(tokens), kChunkBytes)) return kInvalid;
  if (tokens == 0) return kOk;
  if (conv_qkv == nullptr || a == nullptr || b == nullptr || A_log == nullptr || dt_bias == nullptr ||
      state_in == nullptr || state_out == nullptr || out == nullptr || workspace == nullptr)
    return kInvalid;
  const size_t need = chunks_of(tokens) * kChunkBytes + kErrorSlot;
  if (workspace_bytes < need) return kInvalid;
  constexpr size_t kStateBytes = static_cast<size_t>(kValueHeads) * kHead * kHead * 2;
  const size_t out_bytes = tokens * kValueHeads * kHead * 2;
  const Span sc = span(conv_qkv, tokens * kChannels * 2), sa = span(a, tokens * kValueHeads * 2),
             sb = span(b, tokens * kValueHeads * 2), sl = span(A_log, kValueHeads * 2),
             sd = span(dt_bias, kValueHeads * 2), si = span(state_in, kStateBytes), so = span(state_out, kStateBytes),
             sy = span(out, out_bytes), sw = span(workspace, need);
  // state_in == state_out exactly is the one alias allowed, as in the token-sequential entry; the workspace and
  // every written range are disjoint from everything else
  if (partial_overlap(si, so)) return kInvalid;
  const Span readers[] = {sc, sa, sb, sl, sd};
  for (const Span& r : readers)
    if (overlap(so, r) || overlap(sy, r) || overlap(sw, r) || wraps(r)) return kInvalid;
  if (overlap(sy, so) || overlap(sy, si) || overlap(sw, so) || overlap(sw, si) || overlap(sw, sy) || wraps(sy) ||
      wraps(so) || wraps(si) || wraps(sw))
    return kInvalid;
  if (!aligned16(conv_qkv) || !aligned16(state_in) || !aligned16(state_out) || !aligned16(out) || !aligned16(workspace))
    return kNotSupported;
  clear_stale_error();
  static const int configured = [] {
    cudaError_t e = cudaFuncSetAttribute(gdn_chunk_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(sizeof(PrepShared)));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gdn_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kStateShared));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tc::gdn_chunk_state_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(tc::kShared));
    return static_cast<int>(e);
  }();
  if (configured != kOk) return configured;
  cudaStream_t s = as_stream(stream);
  const Workspace ws{static_cast<unsigned char*>(workspace), chunks_of(tokens)};
  if (ws.chunks > 0x7fffffffu) return kInvalid;
  gdn_chunk_prepare_kernel<<<dim3(static_cast<unsigned>(ws.chunks), kValueHeads), kPrepThreads, sizeof(PrepShared), s>>>(
      conv_qkv, tokens, a, b, A_log, dt_bias, l2_eps, ws);
  uint32_t* error_word = reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(workspace) + ws.chunks * kChunkBytes);
  if (use_tcgen05()) {
    clear_error_kernel<<<1, 1, 0, s>>>(error_word);
    tc::gdn_chunk_state_tcgen05_kernel<<<kValueHeads, tc::kThreads, tc::kShared, s>>>(ws, tokens, state_in, state_out, out,
                                                                                      error_word);
  } else {
    gdn_chunk_state_kernel<<<dim3(kValueHeads, kStateSplits), kStateThreads, kStateShared, s>>>(ws, tokens, state_in,
                                                                                               state_out, out);
  }
  return launch_status();
}

}  // namespace
}  // namespace q3x

extern "C" int q3x_b200_gated_delta_net_chunked_select_path(int path) {
  if (path != 0 && path != 1) return q3x::host::kInvalid;
  q3x::chunk_path().store(path, std::memory_order_relaxed);
  return q3x::host::kOk;
}

extern "C" size_t q3x_b200_gated_delta_net_chunked_workspace_bytes(size_t tokens) {
  const size_t chunks = q3x::chunks_of(tokens);
  if (chunks == 0 || q3x::host::mul_overflows(chunks, q3x::kChunkBytes)) return 0;
  return chunks * q3x::kChunkBytes + q3x::kErrorSlot;
}

extern "C" int q3x_b200_gated_delta_net_update_chunked(const uint16_t* conv_qkv, size_t tokens, const uint16_t* a,
                                                       const uint16_t* b, const uint16_t* A_log, const uint16_t* dt_bias,
                                                       const uint16_t* state_in, uint16_t* state_out, float l2_eps,
                                                       uint16_t* out, void* workspace, size_t workspace_bytes,
                                                       void* stream) {
  return q3x::launch_chunked(conv_qkv, tokens, a, b, A_log, dt_bias, state_in, state_out, l2_eps, out, workspace,
                             workspace_bytes, stream);
}
