// Host-side helpers shared by the C-ABI translation units of libasc_cuda:
// CUDA error capture, the device status word, and TMA descriptor encoding.
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>

#include <atomic>

#include "common.cuh"

namespace aschost {

// Records the failing CUDA call for asc_cuda_last_cuda_error and maps it to ASC_ERR_CUDA.
int32_t record_cuda_error(cudaError_t e, const char* what);
int32_t record_driver_error(int code, const char* what);

#define ASC_CUDA_TRY(expr)                                                  \
  do {                                                                      \
    cudaError_t _e = (expr);                                                \
    if (_e != cudaSuccess) return ::aschost::record_cuda_error(_e, #expr);  \
  } while (0)

// Address of this device's status word (one 32-bit word per device; zero == healthy).
// Kernels with bounded waits write a non-zero AscDevErr code there when a wait runs out.
int32_t device_status_word(uint32_t** out);

// Number of SMs of the current device (cached per device).
int32_t sm_count(int* out);

// Encode a tiled tensor map.  rank <= 5.  dims/box in elements (innermost first),
// strides_bytes holds rank-1 entries (stride of dim 1.., innermost is contiguous).
int32_t encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, uint32_t rank, const void* base,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo);

// Stream-ordered scratch memory for kernels that need a workspace: taken from a memory pool this library owns
// (one per device, created at first use; freed blocks stay in the pool instead of going back to the driver at
// every synchronisation), allocated and released in stream order, so launches on different streams never share
// a workspace.
int32_t scratch_alloc(void** out, size_t bytes, cudaStream_t stream);
int32_t scratch_free(void* ptr, cudaStream_t stream);

// Kernels launched by this library since load.
extern std::atomic<uint64_t> g_launch_count;
inline void count_launch() { g_launch_count.fetch_add(1, std::memory_order_relaxed); }

// One small cached value per device (a "set-up done" flag, an occupancy figure) that several host threads
// may read and write at once.  Zero means "not computed yet"; threads that race compute the same value.
struct PerDevice {
  static constexpr int kMax = 64;
  std::atomic<int> v[kMax];
  int get(int dev) const { return (dev >= 0 && dev < kMax) ? v[dev].load(std::memory_order_acquire) : 0; }
  void set(int dev, int value) {
    if (dev >= 0 && dev < kMax) v[dev].store(value, std::memory_order_release);
  }
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace aschost
