// Host-side argument checks run by every entry point before anything is enqueued, so that a bad
// call fails with cudaErrorInvalidValue and no device work.  The rules are those of the
// reference launchers (src/kernels/reference/decode_ops.cu:142-211): element counts must not
// overflow size_t, byte ranges must not wrap the address space, an output may alias an input only
// exactly, and epsilon must be finite and positive.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <limits>
#include <mutex>

namespace q3x::host {

inline bool mul_overflows(size_t a, size_t b) {
  return b != 0 && a > std::numeric_limits<size_t>::max() / b;
}
inline bool mul3_overflows(size_t a, size_t b, size_t c) {
  return mul_overflows(a, b) || mul_overflows(a * b, c);
}
inline bool valid_epsilon(float eps) { return std::isfinite(eps) && eps > 0.0f; }

struct Span {
  const void* p;
  size_t bytes;
};
inline Span span(const void* p, size_t bytes) { return Span{p, bytes}; }

inline bool wraps(const Span& s) {
  return s.bytes > std::numeric_limits<uintptr_t>::max() - reinterpret_cast<uintptr_t>(s.p);
}
inline bool overlap(const Span& a, const Span& b) {
  if (a.bytes == 0 || b.bytes == 0) return false;
  if (wraps(a) || wraps(b)) return true;
  const uintptr_t x = reinterpret_cast<uintptr_t>(a.p), y = reinterpret_cast<uintptr_t>(b.p);
  return x < y + b.bytes && y < x + a.bytes;
}
// Overlapping without being the very same range.
inline bool partial_overlap(const Span& a, const Span& b) {
  return !(a.p == b.p && a.bytes == b.bytes) && overlap(a, b);
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

// Clears a stale last-error left by unrelated earlier work of this thread, so that the value
// returned after the launches is this call's own.
inline void clear_stale_error() { (void)cudaGetLastError(); }
inline int launch_status() { return static_cast<int>(cudaGetLastError()); }

constexpr int kInvalid = static_cast<int>(cudaErrorInvalidValue);
constexpr int kNotSupported = static_cast<int>(cudaErrorNotSupported);
constexpr int kOk = static_cast<int>(cudaSuccess);

// Kernel launch with an explicit choice of programmatic stream serialisation: with `overlap` the kernel may
// start before the previous kernel of the stream has finished (it must then call wait_for_prior_kernels()
// before it touches global memory); without it this is the ordinary <<< >>> launch.  Works under stream
// capture (the graph gets a programmatic edge).
template <typename... Params, typename... Args>
inline void launch_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          bool overlap, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  static const bool allowed = std::getenv("Q3X_B200_NO_OVERLAP") == nullptr;
  config.numAttrs = overlap && allowed ? 1u : 0u;
  (void)cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// SM count of the current device (cached per device ordinal; 148 on B200).
inline int current_device_sm_count() {
  constexpr int kMaxDevices = 64;
  static std::atomic<int> cache[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// A launch of at most one CTA per SM costs mostly its start-up and the gap to its neighbours in the stream:
// such launches are made with programmatic stream serialisation (see launch_kernel).
inline bool latency_bound_launch(size_t ctas) { return ctas <= static_cast<size_t>(current_device_sm_count()); }

// Grid sizing: enough CTAs to fill the machine a few times over without exceeding what the work
// needs.  The multiplier is the number of resident CTAs per SM we aim for.
inline unsigned grid_for(size_t work_items, unsigned items_per_cta, unsigned ctas_per_sm_target) {
  const size_t needed = (work_items + items_per_cta - 1) / items_per_cta;
  const size_t cap = static_cast<size_t>(current_device_sm_count()) * ctas_per_sm_target;
  const size_t g = needed < cap ? needed : cap;
  return static_cast<unsigned>(g == 0 ? 1 : g);
}

// CTAs of `kernel` (with `threads` threads and `smem` dynamic bytes) that are resident at once on the
// current device: occupancy per SM x SM count.  A grid-stride kernel launched with exactly this many
// CTAs runs as one full wave; a larger grid would leave a partial last wave that idles most SMs.
// The answer is cached per (kernel, device) pair (a few dozen entries; lock-free reads).
template <typename Kernel>
inline unsigned resident_grid(Kernel kernel, int threads, size_t smem = 0) {
  struct Entry {
    const void* key;
    int device;
    unsigned value;
  };
  constexpr int kSlots = 512;
  static Entry table[kSlots] = {};
  static std::atomic<int> used{0};
  const void* key = reinterpret_cast<const void*>(kernel);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
  const int n = used.load(std::memory_order_acquire);
  for (int i = 0; i < n; ++i)
    if (table[i].key == key && table[i].device == dev) return table[i].value;
  int per_sm = 0;
  const int sms = current_device_sm_count();
  unsigned value = static_cast<unsigned>(sms) * 4u;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) == cudaSuccess && per_sm > 0)
    value = static_cast<unsigned>(sms) * static_cast<unsigned>(per_sm);
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const int m = used.load(std::memory_order_relaxed);
  for (int i = 0; i < m; ++i)
    if (table[i].key == key && table[i].device == dev) return table[i].value;
  if (m < kSlots) {
    table[m] = Entry{key, dev, value};
    used.store(m + 1, std::memory_order_release);
  }
  return value;
}

// Grid of a grid-stride kernel: one full wave, or fewer CTAs when the work is smaller than that.
template <typename Kernel>
inline unsigned wave_grid(Kernel kernel, int threads, size_t work_items, size_t items_per_cta, size_t smem = 0) {
  const size_t needed = (work_items + items_per_cta - 1) / items_per_cta;
  const size_t cap = resident_grid(kernel, threads, smem);
  const size_t g = needed < cap ? needed : cap;
  return static_cast<unsigned>(g == 0 ? 1 : g);
}

}  // namespace q3x::host
