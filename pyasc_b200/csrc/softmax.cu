// Row softmax (fp32, last dimension, max-subtracted) for sm_100a.
//
// HBM-bound: 8 algorithmic bytes per element (one 4-byte read, one 4-byte write).  One CTA owns a
// row at a time; the row lives in registers between the single global read and the single global
// write (128-bit accesses), row maximum and row sum are reduced with warp shuffles and a small
// shared-memory exchange between warps, and the next row's loads are issued before the current
// row's arithmetic so that memory latency overlaps the exp work.  Rows too long for registers are
// staged in shared memory instead (one global read, one global write); rows too long for shared
// memory are re-read from global memory.
#include <cfloat>
#include <cuda_fp16.h>

#include "../../include/asc_cuda.h"
#include "host_common.h"

namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int kWarps, bool kIsMax>
__device__ __forceinline__ float cta_reduce(float v, float* red) {
  v = kIsMax ? warp_max(v) : warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < kWarps; ++w) r = kIsMax ? fmaxf(r, red[w]) : r + red[w];
  return r;
}

// Register-resident rows: cols % 4 == 0, cols <= kThreads * kVec * 4, rows 16-byte aligned.
template <int kThreads, int kVec>
__global__ void __launch_bounds__(kThreads)
    softmax_rows_reg_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t rows, int cols4,
                            int64_t ld4) {
  constexpr int kWarps = kThreads / 32;
  __shared__ float red_max[kWarps];
  __shared__ float red_sum[kWarps];
  const float4* x4 = reinterpret_cast<const float4*>(x);
  float4* o4 = reinterpret_cast<float4*>(out);
  // idle vector slots hold -inf: they never raise the maximum (which starts at -FLT_MAX) and exp(-inf - m) is 0
  // for every finite m, so they add nothing to the sum -- a row that is all -inf then sums to 0 and comes out NaN,
  // as it does in a row without idle slots and in torch.softmax
  const float ninf = __int_as_float(0xff800000u);
  const float4 neg = make_float4(ninf, ninf, ninf, ninf);

  int64_t row = blockIdx.x;
  if (row >= rows) return;
  float4 v[kVec];
#pragma unroll
  for (int u = 0; u < kVec; ++u) {
    const int c = threadIdx.x + u * kThreads;
    v[u] = (c < cols4) ? __ldcs(x4 + row * ld4 + c) : neg;
  }
  for (; row < rows; row += gridDim.x) {
    const int64_t next = row + gridDim.x;
    float4 nv[kVec];
    if (next < rows) {
#pragma unroll
      for (int u = 0; u < kVec; ++u) {
        const int c = threadIdx.x + u * kThreads;
        nv[u] = (c < cols4) ? __ldcs(x4 + next * ld4 + c) : neg;
      }
    }
    float m = -FLT_MAX;
#pragma unroll
    for (int u = 0; u < kVec; ++u) m = fmaxf(m, fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w)));
    m = cta_reduce<kWarps, true>(m, red_max);
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < kVec; ++u) {
      v[u].x = expf(v[u].x - m);
      v[u].y = expf(v[u].y - m);
      v[u].z = expf(v[u].z - m);
      v[u].w = expf(v[u].w - m);
      s += (v[u].x + v[u].y) + (v[u].z + v[u].w);
    }
    s = cta_reduce<kWarps, false>(s, red_sum);
    const float inv = __frcp_rn(s);
#pragma unroll
    for (int u = 0; u < kVec; ++u) {
      const int c = threadIdx.x + u * kThreads;
      if (c < cols4) {
        float4 r = make_float4(v[u].x * inv, v[u].y * inv, v[u].z * inv, v[u].w * inv);
        __stcs(o4 + row * ld4 + c, r);
      }
    }
    if (next < rows) {
#pragma unroll
      for (int u = 0; u < kVec; ++u) v[u] = nv[u];
    }
  }
}

__device__ __forceinline__ float exp2f_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The same for fp16 rows: 16-byte vectors of 8 halves widened to fp32 registers, one rounding at the store.
// cols % 8 == 0, cols <= kThreads * kVec * 8, rows 16-byte aligned.
template <int kThreads, int kVec>
__global__ void __launch_bounds__(kThreads)
    softmax_rows_reg16_kernel(const __half* __restrict__ x, __half* __restrict__ out, int64_t rows, int cols8,
                              int64_t ld8) {
  constexpr int kWarps = kThreads / 32;
  __shared__ float red_max[kWarps];
  __shared__ float red_sum[kWarps];
  const uint4* x8 = reinterpret_cast<const uint4*>(x);
  uint4* o8 = reinterpret_cast<uint4*>(out);
  const uint32_t kLowest = 0xfbfffbffu;   // two fp16 values of -65504
  const uint4 neg = make_uint4(kLowest, kLowest, kLowest, kLowest);

  int64_t row = blockIdx.x;
  if (row >= rows) return;
  uint4 raw[kVec];
#pragma unroll
  for (int u = 0; u < kVec; ++u) {
    const int c = threadIdx.x + u * kThreads;
    raw[u] = (c < cols8) ? __ldcs(x8 + row * ld8 + c) : neg;
  }
  for (; row < rows; row += gridDim.x) {
    const int64_t next = row + gridDim.x;
    uint4 nraw[kVec];
    if (next < rows) {
#pragma unroll
      for (int u = 0; u < kVec; ++u) {
        const int c = threadIdx.x + u * kThreads;
        nraw[u] = (c < cols8) ? __ldcs(x8 + next * ld8 + c) : neg;
      }
    }
    float v[kVec][8];
    float m = -FLT_MAX;
#pragma unroll
    for (int u = 0; u < kVec; ++u) {
      const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[u][2 * i] = f.x;
        v[u][2 * i + 1] = f.y;
        m = fmaxf(m, fmaxf(f.x, f.y));
      }
    }
    m = cta_reduce<kWarps, true>(m, red_max);
    // exp(x - m) = 2^(x * log2(e) - m * log2(e)): one FMA and one ex2.approx per element.  Its relative error of
    // about 2^-22 is far below the 2^-11 of the fp16 result, and with twice the elements per byte of an fp32 row
    // the full-precision expf would make the kernel instruction-bound (measured 4.4 vs 5.7 TB/s at 4096 columns).
    const float kLog2e = 1.4426950408889634f;
    const float neg_m = -m * kLog2e;
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < kVec; ++u) {
      const bool live = threadIdx.x + u * kThreads < cols8;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[u][i] = live ? exp2f_approx(fmaf(v[u][i], kLog2e, neg_m)) : 0.f;   // padding lanes never count
        s += v[u][i];
      }
    }
    s = cta_reduce<kWarps, false>(s, red_sum);
    const float inv = __frcp_rn(s);
#pragma unroll
    for (int u = 0; u < kVec; ++u) {
      const int c = threadIdx.x + u * kThreads;
      if (c < cols8) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __half2 h = __floats2half2_rn(v[u][2 * i] * inv, v[u][2 * i + 1] * inv);
          w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        __stcs(o8 + row * ld8 + c, make_uint4(w[0], w[1], w[2], w[3]));
      }
    }
    if (next < rows) {
#pragma unroll
      for (int u = 0; u < kVec; ++u) raw[u] = nraw[u];
    }
  }
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Any cols / alignment, fp32 or fp16 elements (arithmetic in fp32, one rounding at the store).
// kStage: the row is kept as fp32 in dynamic shared memory between the passes.
template <bool kStage, typename T>
__global__ void __launch_bounds__(256)
    softmax_rows_generic_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t rows, int64_t cols, int64_t ld) {
  extern __shared__ float row_buf[];
  __shared__ float red_a[8];
  __shared__ float red_b[8];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * ld;
    T* orow = out + row * ld;
    float m = -FLT_MAX;
    for (int64_t c = threadIdx.x; c < cols; c += 256) {
      const float t = to_f32(xr[c]);
      if (kStage) row_buf[c] = t;
      m = fmaxf(m, t);
    }
    m = cta_reduce<8, true>(m, red_a);
    float s = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += 256) {
      const float e = expf((kStage ? row_buf[c] : to_f32(xr[c])) - m);
      if (kStage) row_buf[c] = e;
      s += e;
    }
    s = cta_reduce<8, false>(s, red_b);
    const float inv = __frcp_rn(s);
    for (int64_t c = threadIdx.x; c < cols; c += 256) {
      const float e = kStage ? row_buf[c] : expf(to_f32(xr[c]) - m);
      orow[c] = from_f32<T>(e * inv);
    }
    __syncthreads();  // red_a / red_b / row_buf are reused by the next row
  }
}

template <typename T>
int32_t launch_generic(const T* x, T* out, int64_t rows, int64_t cols, int64_t ld, cudaStream_t stream) {
  int sms = 0;
  int32_t rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;
  const size_t row_bytes = static_cast<size_t>(cols) * sizeof(float);
  constexpr size_t kMaxStage = 200 * 1024;
  if (row_bytes <= kMaxStage) {
    static aschost::PerDevice attr_set;
    int dev = 0;
    ASC_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_set.get(dev)) {
      ASC_CUDA_TRY(cudaFuncSetAttribute(softmax_rows_generic_kernel<true, T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kMaxStage)));
      attr_set.set(dev, 1);
    }
    int64_t per = static_cast<int64_t>((220 * 1024) / (row_bytes + 1024));
    if (per < 1) per = 1;
    if (per > 8) per = 8;
    int64_t grid = static_cast<int64_t>(sms) * per;
    if (grid > rows) grid = rows;
    softmax_rows_generic_kernel<true, T><<<static_cast<unsigned>(grid), 256, row_bytes, stream>>>(x, out, rows, cols, ld);
  } else {
    int64_t grid = static_cast<int64_t>(sms) * 8;
    if (grid > rows) grid = rows;
    softmax_rows_generic_kernel<false, T><<<static_cast<unsigned>(grid), 256, 0, stream>>>(x, out, rows, cols, ld);
  }
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

template <int kThreads, int kVec>
int32_t launch_reg(const float* x, float* out, int64_t rows, int64_t cols, int64_t ld, int ctas_per_sm,
                   cudaStream_t stream) {
  int sms = 0;
  int32_t rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;
  if (ctas_per_sm <= 0) {
    // four full waves of resident CTAs: whole waves keep every SM busy to the end, and several of
    // them even out rows that finish at different times (measured: 6.37 vs 6.22 TB/s with two)
    static aschost::PerDevice resident;
    int dev = 0;
    ASC_CUDA_TRY(cudaGetDevice(&dev));
    int occupancy = resident.get(dev);
    if (occupancy == 0) {
      ASC_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occupancy, softmax_rows_reg_kernel<kThreads, kVec>,
                                                                 kThreads, 0));
      if (occupancy < 1) occupancy = 1;
      resident.set(dev, occupancy);
    }
    // ... unless that leaves a CTA fewer than 32 rows: then one wave, whose CTAs each keep a row in flight behind
    // the one they work on (measured at 4096 columns: 2048 rows 13.0 vs 15.6 us, 4096 rows 22.1 vs 24.8, 8192 rows
    // 43.4 vs 43.2, 16384 rows 89.0 vs 82.0)
    ctas_per_sm = rows >= static_cast<int64_t>(32) * sms * occupancy ? 4 * occupancy : occupancy;
  }
  int64_t grid = static_cast<int64_t>(sms) * ctas_per_sm;
  if (grid > rows) grid = rows;
  softmax_rows_reg_kernel<kThreads, kVec><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
      x, out, rows, static_cast<int>(cols / 4), ld / 4);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

template <int kThreads, int kVec>
int32_t launch_reg16(const __half* x, __half* out, int64_t rows, int64_t cols, int64_t ld, cudaStream_t stream) {
  int sms = 0;
  int32_t rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;
  static aschost::PerDevice resident;
  int dev = 0;
  ASC_CUDA_TRY(cudaGetDevice(&dev));
  int occupancy = resident.get(dev);
  if (occupancy == 0) {
    ASC_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occupancy, softmax_rows_reg16_kernel<kThreads, kVec>,
                                                               kThreads, 0));
    if (occupancy < 1) occupancy = 1;
    resident.set(dev, occupancy);
  }
  // four whole waves, or one when a CTA would get fewer than 32 rows, as for fp32 rows
  int64_t grid = static_cast<int64_t>(sms) * (rows >= static_cast<int64_t>(32) * sms * occupancy ? 4 : 1) * occupancy;
  if (grid > rows) grid = rows;
  softmax_rows_reg16_kernel<kThreads, kVec><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
      x, out, rows, static_cast<int>(cols / 8), ld / 8);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

int32_t launch_softmax(const float* x, float* out, int64_t rows, int64_t cols, int64_t ld, int32_t variant,
                       cudaStream_t stream) {
  if (rows < 0 || cols < 0 || ld < cols) return ASC_ERR_INVALID_ARG;
  if (rows == 0 || cols == 0) return ASC_OK;
  if (x == nullptr || out == nullptr) return ASC_ERR_INVALID_ARG;
  const bool vec_ok = (cols % 4 == 0) && (ld % 4 == 0) && aschost::aligned16(x) && aschost::aligned16(out);
  const int per_sm = (variant >> 8) & 0xff;
  const int shape = variant & 0xff;
  if (vec_ok && cols <= 8192 && shape != 0xff) {
    // the smallest register tile that holds the row: idle vector slots cost issue slots and bytes in flight
    // (measured at 5120 columns: 4.5 TB/s in a tile for 8192, against 5.7 at 8192 itself)
    if (cols <= 512) return launch_reg<128, 1>(x, out, rows, cols, ld, per_sm, stream);
    if (cols <= 1024) return launch_reg<128, 2>(x, out, rows, cols, ld, per_sm, stream);
    if (cols <= 1536) return launch_reg<128, 3>(x, out, rows, cols, ld, per_sm, stream);
    if (cols <= 2048) return launch_reg<128, 4>(x, out, rows, cols, ld, per_sm, stream);
    if (cols <= 3072 && shape == 0) return launch_reg<256, 3>(x, out, rows, cols, ld, per_sm, stream);
    if (cols <= 4096) {
      if (shape == 1) return launch_reg<128, 8>(x, out, rows, cols, ld, per_sm, stream);
      if (shape == 3) return launch_reg<256, 4>(x, out, rows, cols, ld, per_sm, stream);
      return launch_reg<512, 2>(x, out, rows, cols, ld, per_sm, stream);
    }
    if (shape == 1) return launch_reg<256, 8>(x, out, rows, cols, ld, per_sm, stream);
    if (cols <= 6144 && shape == 0) return launch_reg<512, 3>(x, out, rows, cols, ld, per_sm, stream);
    return launch_reg<512, 4>(x, out, rows, cols, ld, per_sm, stream);
  }
  return launch_generic<float>(x, out, rows, cols, ld, stream);
}

}  // namespace

extern "C" {

int32_t asc_cuda_softmax_f32(const float* x, float* out, int64_t rows, int64_t cols, int64_t ld, void* stream) {
  return launch_softmax(x, out, rows, cols, ld, 0, static_cast<cudaStream_t>(stream));
}

// fp16 rows (asc2.softmax accepts fp16 tiles, python/asc/language/tile/unary_ops.py:217): fp32 arithmetic, the
// result rounded once; rows of whole 16-byte vectors up to 16384 columns stay in registers.
int32_t asc_cuda_softmax_f16(const void* x, void* out, int64_t rows, int64_t cols, int64_t ld, void* stream) {
  if (rows < 0 || cols < 0 || ld < cols) return ASC_ERR_INVALID_ARG;
  if (rows == 0 || cols == 0) return ASC_OK;
  if (x == nullptr || out == nullptr) return ASC_ERR_INVALID_ARG;
  const __half* xh = static_cast<const __half*>(x);
  __half* oh = static_cast<__half*>(out);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cols % 8 == 0 && ld % 8 == 0 && aschost::aligned16(x) && aschost::aligned16(out) && cols <= 16384) {
    if (cols <= 1024) return launch_reg16<128, 1>(xh, oh, rows, cols, ld, st);
    if (cols <= 2048) return launch_reg16<128, 2>(xh, oh, rows, cols, ld, st);
    if (cols <= 3072) return launch_reg16<128, 3>(xh, oh, rows, cols, ld, st);
    if (cols <= 4096) return launch_reg16<256, 2>(xh, oh, rows, cols, ld, st);
    if (cols <= 6144) return launch_reg16<256, 3>(xh, oh, rows, cols, ld, st);
    if (cols <= 8192) return launch_reg16<256, 4>(xh, oh, rows, cols, ld, st);
    if (cols <= 12288) return launch_reg16<512, 3>(xh, oh, rows, cols, ld, st);
    return launch_reg16<512, 4>(xh, oh, rows, cols, ld, st);
  }
  return launch_generic<__half>(xh, oh, rows, cols, ld, st);
}

// variant: bits 0-7 CTA shape selector for 2048 < cols <= 4096 (0: 512x2, 1: 128x8, 3: 256x4,
// 0xff: force the generic staged kernel); bits 8-15 CTAs per SM (0: default).
int32_t asc_cuda_softmax_f32_variant(const float* x, float* out, int64_t rows, int64_t cols, int64_t ld,
                                     int32_t variant, void* stream) {
  return launch_softmax(x, out, rows, cols, ld, variant, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
