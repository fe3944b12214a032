// Copy of a [rows, row_bytes] window between two device matrices, whatever the element type.
//
// asc2.store(asc2.load(...)) of a tile whose type the elementwise kernels do not compute on (8-bit and 64-bit
// types) is a pure move of bytes (the reference lowers it to DataCopy in and out of on-chip memory,
// python/asc/language/tile/memory_ops.py).  HBM-bound: 2 bytes of traffic per byte copied.
#include "../../include/asc_cuda.h"
#include "host_common.h"

namespace {

constexpr int kThreads = 256;

// 16-byte vectors when both windows allow it, bytes otherwise; CTAs stride over (row, chunk) pairs
template <typename V>
__global__ void __launch_bounds__(kThreads) copy_window_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                               int64_t rows, int64_t row_units, int64_t src_pitch,
                                                               int64_t dst_pitch) {
  const int64_t total = rows * row_units;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t r = i / row_units, u = i - r * row_units;
    reinterpret_cast<V*>(dst + r * dst_pitch)[u] = reinterpret_cast<const V*>(src + r * src_pitch)[u];
  }
}

}  // namespace

extern "C" int32_t asc_cuda_copy_2d(void* dst, const void* src, int64_t rows, int64_t row_bytes, int64_t dst_pitch,
                                    int64_t src_pitch, void* stream) {
  if (rows < 0 || row_bytes < 0 || dst_pitch < row_bytes || src_pitch < row_bytes) return ASC_ERR_INVALID_ARG;
  if (rows == 0 || row_bytes == 0) return ASC_OK;
  if (dst == nullptr || src == nullptr) return ASC_ERR_INVALID_ARG;
  if (rows > (int64_t{1} << 40) / row_bytes) return ASC_ERR_TOO_LARGE;
  int sms = 0;
  int32_t rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;
  const uintptr_t all = reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) |
                        static_cast<uintptr_t>(row_bytes) | static_cast<uintptr_t>(dst_pitch) |
                        static_cast<uintptr_t>(src_pitch);
  const bool vec = (all & 15) == 0;
  const int64_t units = vec ? row_bytes / 16 : row_bytes;
  int64_t ctas = (rows * units + kThreads - 1) / kThreads;
  const int64_t cap = static_cast<int64_t>(sms) * 32;
  if (ctas > cap) ctas = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint8_t* sp = static_cast<const uint8_t*>(src);
  uint8_t* dp = static_cast<uint8_t*>(dst);
  if (vec)
    copy_window_kernel<uint4><<<static_cast<unsigned>(ctas), kThreads, 0, s>>>(sp, dp, rows, units, src_pitch, dst_pitch);
  else
    copy_window_kernel<uint8_t><<<static_cast<unsigned>(ctas), kThreads, 0, s>>>(sp, dp, rows, units, src_pitch, dst_pitch);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}
