// RMS normalisation over the last dimension: out[r, c] = x[r, c] / sqrt(mean_c(x[r, :]^2) + eps) * gamma[c]
// (asc2.rms_norm, python/asc/language/tile/unary_ops.py:225-237; lowered to the Ascend C RmsNorm routine by
// lib/Conversion/LowerToAsc/LowerAscTile.cpp:190-289).
//
// HBM-bound: 8 bytes per element (one read, one write); gamma is re-read by every row and stays in L2 / L1.
// One CTA owns a row at a time and keeps it in registers between the single read and the single write
// (128-bit accesses; fp16 rows are widened to fp32), the sum of squares is reduced with warp shuffles and a shared-memory exchange.  Rows
// too long for registers, or not 16-byte aligned, are read twice by a plain kernel.
#include <cuda_fp16.h>

#include "../../include/asc_cuda.h"
#include "host_common.h"

namespace {

template <int kWarps>
__device__ __forceinline__ float cta_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < kWarps; ++w) r += red[w];
  __syncthreads();  // red is reused by the next row
  return r;
}

// One 16-byte vector of a row: 4 floats or 8 halves, widened to fp32 registers.
template <typename T>
struct RowVec;
template <>
struct RowVec<float> {
  static constexpr int kElems = 4;
  __device__ static void load(const float* p, float (&v)[4], bool streaming) {
    const float4 t = streaming ? __ldcs(reinterpret_cast<const float4*>(p)) : __ldg(reinterpret_cast<const float4*>(p));
    v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
  }
  __device__ static void store(float* p, const float (&v)[4]) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
  }
  __device__ static float widen(float x) { return x; }
  __device__ static float narrow(float x) { return x; }
};
template <>
struct RowVec<__half> {
  static constexpr int kElems = 8;
  __device__ static void load(const __half* p, float (&v)[8], bool streaming) {
    const uint4 t = streaming ? __ldcs(reinterpret_cast<const uint4*>(p)) : __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
  }
  __device__ static void store(__half* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    __stcs(reinterpret_cast<uint4*>(p), make_uint4(w[0], w[1], w[2], w[3]));
  }
  __device__ static float widen(__half x) { return __half2float(x); }
  __device__ static __half narrow(float x) { return __float2half_rn(x); }
};

// whole 16-byte vectors only: cols a multiple of kElems and at most kT * kVec * kElems, rows and gamma 16-byte
// aligned; kT threads per CTA (short rows take 128 so that no warp idles through the barriers)
template <typename T, int kVec, int kT>
__global__ void __launch_bounds__(kT) rms_rows_reg_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                                           T* __restrict__ out, int64_t rows, int cols_v, int64_t ld,
                                                           float eps, float inv_cols) {
  constexpr int kE = RowVec<T>::kElems;
  __shared__ float red[kT / 32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float v[kVec][kE];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < kVec; ++u) {
      const int c = threadIdx.x + u * kT;
      if (c < cols_v) {
        RowVec<T>::load(x + row * ld + static_cast<int64_t>(c) * kE, v[u], true);
      } else {
#pragma unroll
        for (int e = 0; e < kE; ++e) v[u][e] = 0.f;
      }
      float part = 0.f;
#pragma unroll
      for (int e = 0; e < kE; ++e) part = fmaf(v[u][e], v[u][e], part);
      ss += part;
    }
    const float scale = 1.f / sqrtf(cta_sum<kT / 32>(ss, red) * inv_cols + eps);
#pragma unroll
    for (int u = 0; u < kVec; ++u) {
      const int c = threadIdx.x + u * kT;
      if (c < cols_v) {
        float g[kE];
        RowVec<T>::load(gamma + static_cast<int64_t>(c) * kE, g, false);
#pragma unroll
        for (int e = 0; e < kE; ++e) v[u][e] = v[u][e] * scale * g[e];
        RowVec<T>::store(out + row * ld + static_cast<int64_t>(c) * kE, v[u]);
      }
    }
  }
}

// any cols / alignment: the row is read twice
template <typename T>
__global__ void __launch_bounds__(256) rms_rows_generic_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                                               T* __restrict__ out, int64_t rows, int64_t cols,
                                                               int64_t ld, float eps, float inv_cols) {
  __shared__ float red[8];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * ld;
    float ss = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += 256) {
      const float t = RowVec<T>::widen(xr[c]);
      ss = fmaf(t, t, ss);
    }
    const float scale = 1.f / sqrtf(cta_sum<8>(ss, red) * inv_cols + eps);
    for (int64_t c = threadIdx.x; c < cols; c += 256)
      out[row * ld + c] = RowVec<T>::narrow(RowVec<T>::widen(xr[c]) * scale * RowVec<T>::widen(gamma[c]));
  }
}

template <typename T>
int32_t launch_rms(const T* x, const T* gamma, T* out, int64_t rows, int64_t cols, int64_t ld, float eps,
                   cudaStream_t s) {
  if (rows < 0 || cols < 0 || ld < cols) return ASC_ERR_INVALID_ARG;
  if (rows == 0 || cols == 0) return ASC_OK;
  if (x == nullptr || gamma == nullptr || out == nullptr) return ASC_ERR_INVALID_ARG;
  int sms = 0;
  int32_t rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;
  constexpr int kE = RowVec<T>::kElems;
  int64_t grid = static_cast<int64_t>(sms) * 16;   // whole waves of resident CTAs; CTAs stride over the rows
  if (grid > rows) grid = rows;
  const unsigned g = static_cast<unsigned>(grid);
  const float inv_cols = 1.f / static_cast<float>(cols);
  const bool vec = cols % kE == 0 && ld % kE == 0 && aschost::aligned16(x) && aschost::aligned16(gamma) &&
                   aschost::aligned16(out);
  const int64_t cols_v = cols / kE;
  if (vec && cols_v <= 256 * 8 / (kE / 4)) {     // at most 32 fp32 registers of row per thread
    const int cv = static_cast<int>(cols_v);
    if (cols_v <= 128) {
      int64_t g128 = static_cast<int64_t>(sms) * 32;
      if (g128 > rows) g128 = rows;
      rms_rows_reg_kernel<T, 1, 128><<<static_cast<unsigned>(g128), 128, 0, s>>>(x, gamma, out, rows, cv, ld, eps, inv_cols);
    } else {
      // the smallest register tile that holds the row: idle vector slots cost issue slots and bytes in flight
#define ASC_RMS_CASE(V) \
  case V: rms_rows_reg_kernel<T, V, 256><<<g, 256, 0, s>>>(x, gamma, out, rows, cv, ld, eps, inv_cols); break;
      switch ((cv + 255) / 256) {
        ASC_RMS_CASE(1) ASC_RMS_CASE(2) ASC_RMS_CASE(3) ASC_RMS_CASE(4) ASC_RMS_CASE(5) ASC_RMS_CASE(6) ASC_RMS_CASE(7)
        default: rms_rows_reg_kernel<T, 8, 256><<<g, 256, 0, s>>>(x, gamma, out, rows, cv, ld, eps, inv_cols); break;
      }
#undef ASC_RMS_CASE
    }
  } else {
    rms_rows_generic_kernel<T><<<g, 256, 0, s>>>(x, gamma, out, rows, cols, ld, eps, inv_cols);
  }
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

}  // namespace

extern "C" int32_t asc_cuda_rms_norm_f32(const float* x, const float* gamma, float* out, int64_t rows, int64_t cols,
                                         int64_t ld, float eps, void* stream) {
  return launch_rms<float>(x, gamma, out, rows, cols, ld, eps, static_cast<cudaStream_t>(stream));
}

extern "C" int32_t asc_cuda_rms_norm_f16(const void* x, const void* gamma, void* out, int64_t rows, int64_t cols,
                                         int64_t ld, float eps, void* stream) {
  return launch_rms<__half>(static_cast<const __half*>(x), static_cast<const __half*>(gamma), static_cast<__half*>(out),
                            rows, cols, ld, eps, static_cast<cudaStream_t>(stream));
}
