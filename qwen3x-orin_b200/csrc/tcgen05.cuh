// The few tcgen05 (fifth-generation tensor core) building blocks the hand-written kernels here share: shared-memory
// matrix descriptors for 128-byte-swizzled operands, the instruction descriptor of a bf16 x bf16 -> FP32 product with
// M = 128, issue / commit, a BOUNDED wait on the completion barrier, tensor-memory loads and stores of a thread's own
// lane, and the fences between the proxies.  Operand tiles are rows of 64 bf16 (128 bytes) whose 16-byte pieces are
// permuted by the row's low three bits -- the 128-byte swizzle -- in blocks whose base is 1024-byte aligned.
#pragma once
#include <cstdint>

namespace q3x {
namespace tcgen05 {

constexpr uint32_t kWaitLimit = 1u << 20;  // (and 50 ms, whichever comes first)

// K-major operand ([rows][k], k contiguous) of 64-element rows; groups of eight rows 1024 bytes apart
__device__ __forceinline__ uint64_t operand_descriptor(uint32_t shared_address) {
  return static_cast<uint64_t>((shared_address & 0x3ffffu) >> 4) | (static_cast<uint64_t>(1) << 16) |
         (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) | (static_cast<uint64_t>(2) << 61);
}
// bf16 x bf16 -> FP32, M = 128, N = n, both operands K-major
__host__ __device__ constexpr uint32_t instruction_descriptor(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}
__device__ __forceinline__ void mma(uint32_t accumulator, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(accumulator),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[128, n] (+)= A[128, k] B[n, k]^T: 16 elements of k per instruction; 64 per block of either operand
__device__ __forceinline__ void product(uint32_t accumulator, uint32_t a_base, uint32_t a_block_bytes, uint32_t b_base,
                                        uint32_t b_block_bytes, int k, uint32_t idesc, bool accumulate) {
  for (int step = 0; step < k / 16; ++step) {
    const uint32_t block = step >> 2, inside = (step & 3) * 32;
    mma(accumulator, operand_descriptor(a_base + block * a_block_bytes + inside),
        operand_descriptor(b_base + block * b_block_bytes + inside), idesc, (accumulate || step > 0) ? 1u : 0u);
  }
}
__device__ __forceinline__ void commit(uint32_t barrier) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(barrier) : "memory");
}
// A wait on the completion barrier that is bounded in TIME (50 ms on the global timer; a product here completes in
// microseconds): false means it ran out.
__device__ __forceinline__ bool wait(uint32_t barrier, uint32_t parity) {
  uint64_t start;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
  for (uint32_t spin = 0; spin < kWaitLimit; ++spin) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(barrier), "r"(parity)
                 : "memory");
    if (done) return true;
    uint64_t now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - start > 50000000ull) return false;
  }
  return false;
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }


// n consecutive columns of this thread's lane (the loads are waited for by the caller, so that several can be in flight)
__device__ __forceinline__ void load16(uint32_t address, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(address)
               : "memory");
}
__device__ __forceinline__ void load32(uint32_t address, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(address)
               : "memory");
}
__device__ __forceinline__ void store32(uint32_t address, const uint32_t (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(address), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void wait_loads() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void wait_stores() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }


// MN-major operand ([k][rows], the row index contiguous: e.g. a value cache [key][dimension] as the B operand of P V):
// blocks of [k][64 rows]; eight k-lines of a block are 1024 bytes apart, the next 64 rows `block_bytes` further
__device__ __forceinline__ uint64_t operand_descriptor_mn(uint32_t shared_address, uint32_t block_bytes) {
  return static_cast<uint64_t>((shared_address & 0x3ffffu) >> 4) | (static_cast<uint64_t>((block_bytes >> 4) & 0x3fffu) << 16) |
         (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) | (static_cast<uint64_t>(2) << 61);
}
constexpr uint32_t kBOperandMnMajor = 1u << 16;  // or-ed into an instruction descriptor

}  // namespace tcgen05
}  // namespace q3x
