// Tile reductions (sum / max / min / prod over one axis of a row-major [rows, cols] fp32 window, or over
// all of it) for sm_100a.
//
// The asc2 surface reduces tiles that fit the Ascend's on-chip buffer (asc2.reduce_sum/max/min/prod,
// python/asc/language/tile/reduction_ops.py; lowered by lib/Conversion/LowerToAsc/LowerAscTile.cpp:428-459),
// so a window is small and many of them are reduced per launch.  HBM-bound: 4 bytes read per element, the
// result is negligible.  No scratch memory: along rows a warp (or a CTA, for long rows) owns a row and
// combines with shuffles; along columns a thread owns a column and consecutive threads read consecutive
// addresses; the full reduction of one window runs in a single CTA.
#include <cfloat>

#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "../../include/asc_cuda.h"
#include "host_common.h"

namespace {

enum ReduceKind : int32_t { R_SUM = 0, R_MAX = 1, R_MIN = 2, R_PROD = 3 };

template <int kKind>
__device__ __forceinline__ float identity() {
  return kKind == R_SUM ? 0.f : kKind == R_PROD ? 1.f : kKind == R_MAX ? -INFINITY : INFINITY;
}
template <int kKind>
__device__ __forceinline__ float combine(float a, float b) {
  if (kKind == R_SUM) return __fadd_rn(a, b);
  if (kKind == R_PROD) return __fmul_rn(a, b);
  if (kKind == R_MAX) return ascdev::max_nan(a, b);
  return ascdev::min_nan(a, b);
}
template <int kKind>
__device__ __forceinline__ float warp_combine(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = combine<kKind>(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// axis 1, one warp per row: out[r] = reduce_c x[r, c].  kVec: rows are 16-byte aligned and a multiple of
// four long, so lanes read float4 and keep four loads in flight.
template <int kKind, bool kVec>
__global__ void __launch_bounds__(256) reduce_rows_warp_kernel(const float* __restrict__ x, float* __restrict__ out,
                                                               int64_t rows, int64_t cols, int64_t ld) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * 8;
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); r < rows; r += warps) {
    const float* row = x + r * ld;
    float v = identity<kKind>();
    if constexpr (kVec) {
      const float4* row4 = reinterpret_cast<const float4*>(row);
      const int64_t n4 = cols >> 2;
      float acc[4] = {identity<kKind>(), identity<kKind>(), identity<kKind>(), identity<kKind>()};
      int64_t c = lane;
      for (; c + 96 < n4; c += 128) {
        float4 t[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) t[u] = __ldcs(row4 + c + 32 * u);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          acc[u] = combine<kKind>(acc[u], combine<kKind>(combine<kKind>(t[u].x, t[u].y), combine<kKind>(t[u].z, t[u].w)));
      }
      for (; c < n4; c += 32) {
        const float4 t = __ldcs(row4 + c);
        acc[0] = combine<kKind>(acc[0], combine<kKind>(combine<kKind>(t.x, t.y), combine<kKind>(t.z, t.w)));
      }
      v = combine<kKind>(combine<kKind>(acc[0], acc[1]), combine<kKind>(acc[2], acc[3]));
    } else {
      for (int64_t c = lane; c < cols; c += 32) v = combine<kKind>(v, __ldcs(row + c));
    }
    v = warp_combine<kKind>(v);
    if (lane == 0) out[r] = v;
  }
}

// axis 1, one CTA per row (long rows)
template <int kKind>
__global__ void __launch_bounds__(256) reduce_rows_cta_kernel(const float* __restrict__ x, float* __restrict__ out,
                                                              int64_t rows, int64_t cols, int64_t ld) {
  __shared__ float part[8];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* row = x + r * ld;
    float v = identity<kKind>();
    for (int64_t c = threadIdx.x; c < cols; c += 256) v = combine<kKind>(v, __ldcs(row + c));
    v = warp_combine<kKind>(v);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = part[0];
#pragma unroll
      for (int w = 1; w < 8; ++w) t = combine<kKind>(t, part[w]);
      out[r] = t;
    }
    __syncthreads();
  }
}

// axis 0: out[c] = reduce_r x[r, c]; a CTA owns 32 columns, its 8 warps take every 8th row
template <int kKind>
__global__ void __launch_bounds__(256) reduce_cols_kernel(const float* __restrict__ x, float* __restrict__ out,
                                                          int64_t rows, int64_t cols, int64_t ld) {
  __shared__ float part[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t c0 = static_cast<int64_t>(blockIdx.x) * 32; c0 < cols; c0 += static_cast<int64_t>(gridDim.x) * 32) {
    const int64_t c = c0 + lane;
    float v = identity<kKind>();
    if (c < cols)
      for (int64_t r = warp; r < rows; r += 8) v = combine<kKind>(v, __ldcs(x + r * ld + c));
    part[warp][lane] = v;
    __syncthreads();
    if (warp == 0 && c < cols) {
      float t = part[0][lane];
#pragma unroll
      for (int w = 1; w < 8; ++w) t = combine<kKind>(t, part[w][lane]);
      out[c] = t;
    }
    __syncthreads();
  }
}

// everything: out[0 .. n_fill) = reduce of the whole window (one CTA: windows are on-chip sized)
__device__ __forceinline__ float widen(float v) { return v; }
__device__ __forceinline__ float widen(__half v) { return __half2float(v); }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void narrow(float v, float& out) { out = v; }
__device__ __forceinline__ void narrow(float v, __half& out) { out = __float2half_rn(v); }
__device__ __forceinline__ void narrow(float v, __nv_bfloat16& out) { out = __float2bfloat16_rn(v); }

template <int kKind, typename T>
__global__ void __launch_bounds__(1024) reduce_all_kernel(const T* __restrict__ x, T* __restrict__ out,
                                                          int64_t rows, int64_t cols, int64_t ld, int64_t n_fill) {
  __shared__ float part[32];
  float v = identity<kKind>();
  const int64_t n = rows * cols;
  for (int64_t i = threadIdx.x; i < n; i += 1024) v = combine<kKind>(v, widen(x[(i / cols) * ld + (i % cols)]));
  v = warp_combine<kKind>(v);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = warp_combine<kKind>(part[threadIdx.x]);
    if (threadIdx.x == 0) part[0] = t;
  }
  __syncthreads();
  T result;
  narrow(part[0], result);       // 16-bit tiles: combined in fp32, rounded once
  for (int64_t i = threadIdx.x; i < n_fill; i += 1024) out[i] = result;
}

template <int kKind>
int32_t launch_reduce(const float* x, float* out, int64_t rows, int64_t cols, int64_t ld, int32_t axis, int64_t n_fill,
                      cudaStream_t stream) {
  int sms = 0;
  int32_t rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;
  if (axis == 1) {
    if (cols >= 4096 && rows < static_cast<int64_t>(sms) * 64) {
      int64_t grid = rows < static_cast<int64_t>(sms) * 8 ? rows : static_cast<int64_t>(sms) * 8;
      reduce_rows_cta_kernel<kKind><<<static_cast<unsigned>(grid), 256, 0, stream>>>(x, out, rows, cols, ld);
    } else {
      int64_t grid = (rows + 7) / 8;
      if (grid > static_cast<int64_t>(sms) * 32) grid = static_cast<int64_t>(sms) * 32;
      const bool vec = (cols % 4 == 0) && (ld % 4 == 0) && aschost::aligned16(x);
      if (vec)
        reduce_rows_warp_kernel<kKind, true><<<static_cast<unsigned>(grid), 256, 0, stream>>>(x, out, rows, cols, ld);
      else
        reduce_rows_warp_kernel<kKind, false><<<static_cast<unsigned>(grid), 256, 0, stream>>>(x, out, rows, cols, ld);
    }
  } else if (axis == 0) {
    int64_t grid = (cols + 31) / 32;
    if (grid > static_cast<int64_t>(sms) * 16) grid = static_cast<int64_t>(sms) * 16;
    reduce_cols_kernel<kKind><<<static_cast<unsigned>(grid), 256, 0, stream>>>(x, out, rows, cols, ld);
  } else {
    reduce_all_kernel<kKind, float><<<1, 1024, 0, stream>>>(x, out, rows, cols, ld, n_fill);
  }
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

template <typename T>
int32_t launch_reduce_all_16(const void* x, void* out, int64_t rows, int64_t cols, int64_t ld, int32_t kind, int64_t n_fill,
                             cudaStream_t stream) {
  const T* xi = static_cast<const T*>(x);
  T* oi = static_cast<T*>(out);
  switch (kind) {
    case R_SUM: reduce_all_kernel<R_SUM, T><<<1, 1024, 0, stream>>>(xi, oi, rows, cols, ld, n_fill); break;
    case R_MAX: reduce_all_kernel<R_MAX, T><<<1, 1024, 0, stream>>>(xi, oi, rows, cols, ld, n_fill); break;
    case R_MIN: reduce_all_kernel<R_MIN, T><<<1, 1024, 0, stream>>>(xi, oi, rows, cols, ld, n_fill); break;
    default: reduce_all_kernel<R_PROD, T><<<1, 1024, 0, stream>>>(xi, oi, rows, cols, ld, n_fill); break;
  }
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

}  // namespace

extern "C" int32_t asc_cuda_reduce_all_f16(const void* x, void* out, int64_t rows, int64_t cols, int64_t ld, int32_t kind,
                                           int64_t n_fill, int32_t dtype, void* stream) {
  if (rows < 0 || cols < 0 || ld < cols || kind < 0 || kind > 3 || n_fill < 0 || dtype < 0 || dtype > 1)
    return ASC_ERR_INVALID_ARG;
  if (n_fill == 0) return ASC_OK;
  if (out == nullptr || (x == nullptr && rows * cols > 0)) return ASC_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 1) return ASC_ERR_MISALIGNED;
  if (rows * cols > (int64_t{1} << 24)) return ASC_ERR_TOO_LARGE;  // one CTA reduces the window
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == 1 ? launch_reduce_all_16<__nv_bfloat16>(x, out, rows, cols, ld, kind, n_fill, s)
                    : launch_reduce_all_16<__half>(x, out, rows, cols, ld, kind, n_fill, s);
}

extern "C" int32_t asc_cuda_reduce_f32(const float* x, float* out, int64_t rows, int64_t cols, int64_t ld,
                                       int32_t axis, int32_t kind, int64_t n_fill, void* stream) {
  if (rows < 0 || cols < 0 || ld < cols || kind < 0 || kind > 3 || axis < -1 || axis > 1) return ASC_ERR_INVALID_ARG;
  if (axis == -1 && n_fill < 0) return ASC_ERR_INVALID_ARG;
  const int64_t n_out = axis == 1 ? rows : axis == 0 ? cols : n_fill;
  if (n_out == 0) return ASC_OK;
  if (out == nullptr || (x == nullptr && rows * cols > 0)) return ASC_ERR_INVALID_ARG;
  if (axis == -1 && rows * cols > (int64_t{1} << 24)) return ASC_ERR_TOO_LARGE;  // one CTA reduces the window
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (kind) {
    case R_SUM: return launch_reduce<R_SUM>(x, out, rows, cols, ld, axis, n_fill, s);
    case R_MAX: return launch_reduce<R_MAX>(x, out, rows, cols, ld, axis, n_fill, s);
    case R_MIN: return launch_reduce<R_MIN>(x, out, rows, cols, ld, axis, n_fill, s);
    default: return launch_reduce<R_PROD>(x, out, rows, cols, ld, axis, n_fill, s);
  }
}
