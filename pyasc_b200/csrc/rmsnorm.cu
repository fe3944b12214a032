// RMS normalisation over the last dimension: out[r, c] = x[r, c] / sqrt(mean_c(x[r, :]^2) + eps) * gamma[c]
// (asc2.rms_norm, python/asc/language/tile/unary_ops.py:225-237; lowered to the Ascend C RmsNorm routine by
// lib/Conversion/LowerToAsc/LowerAscTile.cpp:190-289).
//
// HBM-bound: 8 bytes per element (one read, one write); gamma is re-read by every row and stays in L2 / L1.
// One CTA owns a row at a time and keeps it in registers between the single read and the single write
// (128-bit accesses), the sum of squares is reduced with warp shuffles and a shared-memory exchange.  Rows
// too long for registers, or not 16-byte aligned, are read twice by a plain kernel.
#include "../../include/asc_cuda.h"
#include "host_common.h"

namespace {

__device__ __forceinline__ float cta_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) r += red[w];
  __syncthreads();  // red is reused by the next row
  return r;
}

// cols % 4 == 0, cols <= 256 * kVec * 4, rows and gamma 16-byte aligned
template <int kVec>
__global__ void __launch_bounds__(256) rms_rows_reg_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                           float* __restrict__ out, int64_t rows, int cols4, int64_t ld4,
                                                           float eps, float inv_cols) {
  __shared__ float red[8];
  const float4* x4 = reinterpret_cast<const float4*>(x);
  const float4* g4 = reinterpret_cast<const float4*>(gamma);
  float4* o4 = reinterpret_cast<float4*>(out);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float4 v[kVec];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < kVec; ++u) {
      const int c = threadIdx.x + u * 256;
      v[u] = (c < cols4) ? __ldcs(x4 + row * ld4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      ss += (v[u].x * v[u].x + v[u].y * v[u].y) + (v[u].z * v[u].z + v[u].w * v[u].w);
    }
    const float scale = 1.f / sqrtf(cta_sum(ss, red) * inv_cols + eps);
#pragma unroll
    for (int u = 0; u < kVec; ++u) {
      const int c = threadIdx.x + u * 256;
      if (c < cols4) {
        const float4 g = __ldg(g4 + c);
        __stcs(o4 + row * ld4 + c,
               make_float4(v[u].x * scale * g.x, v[u].y * scale * g.y, v[u].z * scale * g.z, v[u].w * scale * g.w));
      }
    }
  }
}

// any cols / alignment: the row is read twice
__global__ void __launch_bounds__(256) rms_rows_generic_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                               float* __restrict__ out, int64_t rows, int64_t cols,
                                                               int64_t ld, float eps, float inv_cols) {
  __shared__ float red[8];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * ld;
    float ss = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += 256) ss += xr[c] * xr[c];
    const float scale = 1.f / sqrtf(cta_sum(ss, red) * inv_cols + eps);
    for (int64_t c = threadIdx.x; c < cols; c += 256) out[row * ld + c] = xr[c] * scale * gamma[c];
  }
}

template <int kVec>
void launch_reg(const float* x, const float* gamma, float* out, int64_t rows, int64_t cols, int64_t ld, float eps,
                int64_t grid, cudaStream_t stream) {
  rms_rows_reg_kernel<kVec><<<static_cast<unsigned>(grid), 256, 0, stream>>>(x, gamma, out, rows, static_cast<int>(cols / 4),
                                                                             ld / 4, eps, 1.f / static_cast<float>(cols));
}

}  // namespace

extern "C" int32_t asc_cuda_rms_norm_f32(const float* x, const float* gamma, float* out, int64_t rows, int64_t cols,
                                         int64_t ld, float eps, void* stream) {
  if (rows < 0 || cols < 0 || ld < cols) return ASC_ERR_INVALID_ARG;
  if (rows == 0 || cols == 0) return ASC_OK;
  if (x == nullptr || gamma == nullptr || out == nullptr) return ASC_ERR_INVALID_ARG;
  int sms = 0;
  int32_t rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int64_t grid = static_cast<int64_t>(sms) * 16;   // whole waves of resident CTAs; CTAs stride over the rows
  if (grid > rows) grid = rows;
  const bool vec = cols % 4 == 0 && ld % 4 == 0 && aschost::aligned16(x) && aschost::aligned16(gamma) &&
                   aschost::aligned16(out);
  if (vec && cols <= 8192) {
    if (cols <= 1024) launch_reg<1>(x, gamma, out, rows, cols, ld, eps, grid, s);
    else if (cols <= 2048) launch_reg<2>(x, gamma, out, rows, cols, ld, eps, grid, s);
    else if (cols <= 4096) launch_reg<4>(x, gamma, out, rows, cols, ld, eps, grid, s);
    else launch_reg<8>(x, gamma, out, rows, cols, ld, eps, grid, s);
  } else {
    rms_rows_generic_kernel<<<static_cast<unsigned>(grid), 256, 0, s>>>(x, gamma, out, rows, cols, ld, eps,
                                                                        1.f / static_cast<float>(cols));
  }
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}
