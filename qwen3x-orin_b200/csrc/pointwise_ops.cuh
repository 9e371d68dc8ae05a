// Element functors of the pointwise operators, shared by the plain stream kernels (pointwise.cu) and
// the single-kernel forms that also quantise the result (fused_nvfp4.cu).
#pragma once

#include "device_utils.cuh"

namespace q3x {

// ---- element functors: the arithmetic of src/runtime/reference/decode_ops.cpp:268-342 ----
// kDepth = independent 128-bit loads per operand a thread keeps in flight; kStreamingStore = the output
// goes out with st.global.cs.  Both are per operator because they were measured per operator at 16384
// tokens: SwiGLU runs 272 -> 257 us with depth 2 and streaming stores (depth 1: 298 us, depth 4 or 8 with
// streaming stores: 266 - 269 us), the sigmoid gate is fastest as it is (depth 4, plain stores: 100 us
// against 104 us for depth 2 with streaming stores).
struct ResidualAdd {
  static constexpr int kDepth = 4;
  static constexpr bool kStreamingStore = false;
  static __device__ __forceinline__ float apply(float l, float r) { return l + r; }
};
struct SiluMul {  // first operand = gate, second = up
  static constexpr int kDepth = 2;
  static constexpr bool kStreamingStore = true;
  static __device__ __forceinline__ float apply(float g, float u) { return silu_unscaled(g) * u; }
};
struct SigmoidGate {  // first operand = value, second = gate
  static constexpr int kDepth = 4;
  static constexpr bool kStreamingStore = false;
  static __device__ __forceinline__ float apply(float v, float g) { return v * stable_sigmoid(g); }
};

}  // namespace q3x
