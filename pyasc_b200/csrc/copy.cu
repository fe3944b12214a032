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

// ------------------------------------------------------------------------------------------------
// 8-bit integers <-> int32 words.  The elementwise programs compute on 32- and 16-bit types; a kernel that loads an
// int8 / uint8 tensor (a byte mask, quantised data) or stores one (a quantiser) gets its bytes widened into, or
// narrowed out of, an int32 temporary by these passes, so that the programs' inner loops carry no 8-bit cases
// (inlined there, the extra cases cost the fp32 GELU 2 % and the interpreted mish 7 %).
// HBM-bound: 5 bytes of traffic per element.
// ------------------------------------------------------------------------------------------------
namespace {

template <bool kSigned>
__global__ void __launch_bounds__(kThreads) widen_bytes_kernel(const uint8_t* __restrict__ src, int32_t* __restrict__ dst,
                                                               int64_t n, int vec) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  const int64_t i0 = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (vec) {                                           // four bytes in, one 16-byte store out
    for (int64_t q = i0; q < n / 4; q += stride) {
      const uint32_t w = reinterpret_cast<const uint32_t*>(src)[q];
      int4 o;
      int32_t* e = reinterpret_cast<int32_t*>(&o);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t b = (w >> (8 * k)) & 0xffu;
        e[k] = kSigned ? static_cast<int32_t>(static_cast<int8_t>(b)) : static_cast<int32_t>(b);
      }
      reinterpret_cast<int4*>(dst)[q] = o;
    }
    for (int64_t i = (n / 4) * 4 + i0; i < n; i += stride)
      dst[i] = kSigned ? static_cast<int32_t>(static_cast<int8_t>(src[i])) : static_cast<int32_t>(src[i]);
  } else {
    for (int64_t i = i0; i < n; i += stride)
      dst[i] = kSigned ? static_cast<int32_t>(static_cast<int8_t>(src[i])) : static_cast<int32_t>(src[i]);
  }
}

__global__ void __launch_bounds__(kThreads) narrow_words_kernel(const int32_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                                int64_t n, int vec) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  const int64_t i0 = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (vec) {
    for (int64_t q = i0; q < n / 4; q += stride) {
      const int4 w = reinterpret_cast<const int4*>(src)[q];
      reinterpret_cast<uint32_t*>(dst)[q] = (static_cast<uint32_t>(w.x) & 0xffu) | ((static_cast<uint32_t>(w.y) & 0xffu) << 8) |
                                            ((static_cast<uint32_t>(w.z) & 0xffu) << 16) | (static_cast<uint32_t>(w.w) << 24);
    }
    for (int64_t i = (n / 4) * 4 + i0; i < n; i += stride) dst[i] = static_cast<uint8_t>(src[i]);
  } else {
    for (int64_t i = i0; i < n; i += stride) dst[i] = static_cast<uint8_t>(src[i]);
  }
}

}  // namespace

// mode 0: int8 -> int32 (sign-extended), 1: uint8 -> int32 (zero-extended), 2: int32 -> its low byte (int8 and uint8
// alike).  n elements; the 32-bit side must be 4-byte aligned.
extern "C" int32_t asc_cuda_convert_bytes(void* dst, const void* src, int64_t n, int32_t mode, void* stream) {
  if (n < 0 || mode < 0 || mode > 2) return ASC_ERR_INVALID_ARG;
  if (n == 0) return ASC_OK;
  if (dst == nullptr || src == nullptr) return ASC_ERR_INVALID_ARG;
  const void* words = mode == 2 ? src : dst;
  const void* bytes = mode == 2 ? dst : src;
  if (reinterpret_cast<uintptr_t>(words) % 4 != 0) return ASC_ERR_MISALIGNED;
  int sms = 0;
  int32_t rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;
  const int vec = reinterpret_cast<uintptr_t>(words) % 16 == 0 && reinterpret_cast<uintptr_t>(bytes) % 4 == 0;
  int64_t ctas = ((vec ? (n + 3) / 4 : n) + kThreads - 1) / kThreads;
  const int64_t cap = static_cast<int64_t>(sms) * 32;
  if (ctas > cap) ctas = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(ctas);
  if (mode == 0)
    widen_bytes_kernel<true><<<grid, kThreads, 0, s>>>(static_cast<const uint8_t*>(src), static_cast<int32_t*>(dst), n, vec);
  else if (mode == 1)
    widen_bytes_kernel<false><<<grid, kThreads, 0, s>>>(static_cast<const uint8_t*>(src), static_cast<int32_t*>(dst), n, vec);
  else
    narrow_words_kernel<<<grid, kThreads, 0, s>>>(static_cast<const int32_t*>(src), static_cast<uint8_t*>(dst), n, vec);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}
