// fp32 elementwise kernels (vector add, multiply-add) for sm_100a.
//
// HBM-bound: 12 algorithmic bytes per element for x + y (two 4-byte reads, one 4-byte write).
// Each thread moves 128-bit vectors; a CTA owns a contiguous chunk of kUnroll * 256 vectors per
// step so that every warp-level access is a fully coalesced 512-byte segment, and all loads of a
// step are issued before the first add so that 2 * kUnroll 16-byte loads per thread are in flight.
// Loads and stores carry streaming (evict-first) hints: nothing is ever re-read.
#include "../../include/asc_cuda.h"
#include "host_common.h"

namespace {

constexpr int kThreads = 256;

template <int kUnroll, bool kMulAdd>
__global__ void __launch_bounds__(kThreads)
    eltwise_f32_vec4_kernel(const float4* __restrict__ x, const float4* __restrict__ y,
                            const float4* __restrict__ z, float4* __restrict__ out, int64_t n4, int64_t n) {
  const int64_t chunk = static_cast<int64_t>(kThreads) * kUnroll;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * chunk;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * chunk + threadIdx.x; base < n4; base += stride) {
    float4 a[kUnroll], b[kUnroll], c[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + static_cast<int64_t>(u) * kThreads;
      if (i < n4) {
        a[u] = __ldcs(x + i);
        b[u] = __ldcs(y + i);
        if (kMulAdd) c[u] = __ldcs(z + i);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + static_cast<int64_t>(u) * kThreads;
      if (i < n4) {
        float4 r;
        if (kMulAdd) {
          // separately rounded multiply and add: no FMA contraction, matches NumPy's x * y + z
          r.x = __fadd_rn(__fmul_rn(a[u].x, b[u].x), c[u].x);
          r.y = __fadd_rn(__fmul_rn(a[u].y, b[u].y), c[u].y);
          r.z = __fadd_rn(__fmul_rn(a[u].z, b[u].z), c[u].z);
          r.w = __fadd_rn(__fmul_rn(a[u].w, b[u].w), c[u].w);
        } else {
          r.x = __fadd_rn(a[u].x, b[u].x);
          r.y = __fadd_rn(a[u].y, b[u].y);
          r.z = __fadd_rn(a[u].z, b[u].z);
          r.w = __fadd_rn(a[u].w, b[u].w);
        }
        __stcs(out + i, r);
      }
    }
  }
  // ragged tail (n % 4 elements), handled by the first threads of CTA 0
  if (blockIdx.x == 0) {
    const int64_t i = n4 * 4 + threadIdx.x;
    if (i < n) {
      const float* xs = reinterpret_cast<const float*>(x);
      const float* ys = reinterpret_cast<const float*>(y);
      float* os = reinterpret_cast<float*>(out);
      if (kMulAdd) {
        const float* zs = reinterpret_cast<const float*>(z);
        os[i] = __fadd_rn(__fmul_rn(xs[i], ys[i]), zs[i]);
      } else {
        os[i] = __fadd_rn(xs[i], ys[i]);
      }
    }
  }
}

// Fallback for pointers that are not 16-byte aligned: scalar grid-stride loop.
template <bool kMulAdd>
__global__ void __launch_bounds__(kThreads)
    eltwise_f32_scalar_kernel(const float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ z,
                              float* __restrict__ out, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    if (kMulAdd) {
      out[i] = __fadd_rn(__fmul_rn(x[i], y[i]), z[i]);
    } else {
      out[i] = __fadd_rn(x[i], y[i]);
    }
  }
}

template <int kUnroll, bool kMulAdd>
int32_t launch_vec4(const float* x, const float* y, const float* z, float* out, int64_t n, int64_t max_ctas,
                    cudaStream_t stream) {
  const int64_t n4 = n / 4;
  const int64_t chunk = static_cast<int64_t>(kThreads) * kUnroll;
  int64_t ctas = (n4 + chunk - 1) / chunk;
  if (ctas < 1) ctas = 1;
  if (max_ctas > 0 && ctas > max_ctas) ctas = max_ctas;
  if (ctas > 0x7fffffff) ctas = 0x7fffffff;
  eltwise_f32_vec4_kernel<kUnroll, kMulAdd><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(
      reinterpret_cast<const float4*>(x), reinterpret_cast<const float4*>(y), reinterpret_cast<const float4*>(z),
      reinterpret_cast<float4*>(out), n4, n);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

// variant: bits 0-3 unroll selector (0 -> default), bits 8.. CTAs per SM for a persistent grid
// (0 -> one chunk per CTA).
template <bool kMulAdd>
int32_t launch_eltwise(const float* x, const float* y, const float* z, float* out, int64_t n, int32_t variant,
                       cudaStream_t stream) {
  if (n < 0) return ASC_ERR_INVALID_ARG;
  if (n == 0) return ASC_OK;
  if (x == nullptr || y == nullptr || out == nullptr || (kMulAdd && z == nullptr)) return ASC_ERR_INVALID_ARG;
  const bool aligned = aschost::aligned16(x) && aschost::aligned16(y) && aschost::aligned16(out) &&
                       (!kMulAdd || aschost::aligned16(z));
  int sms = 0;
  int32_t rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;
  if (!aligned) {
    int64_t ctas = (n + kThreads - 1) / kThreads;
    const int64_t cap = static_cast<int64_t>(sms) * 16;
    if (ctas > cap) ctas = cap;
    eltwise_f32_scalar_kernel<kMulAdd><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(x, y, z, out, n);
    aschost::count_launch();
    ASC_CUDA_TRY(cudaGetLastError());
    return ASC_OK;
  }
  const int unroll_sel = variant & 0xf;
  const int per_sm = (variant >> 8) & 0xff;
  const int64_t max_ctas = per_sm > 0 ? static_cast<int64_t>(per_sm) * sms : 0;
  switch (unroll_sel) {
    // default: one 16-byte vector per thread and array, one chunk per CTA (measured fastest on B200:
    // the hardware CTA scheduler balances 2^18 small CTAs better than a persistent grid-stride loop)
    case 0:
    case 1: return launch_vec4<1, kMulAdd>(x, y, z, out, n, max_ctas, stream);
    case 2: return launch_vec4<2, kMulAdd>(x, y, z, out, n, max_ctas, stream);
    case 8: return launch_vec4<8, kMulAdd>(x, y, z, out, n, max_ctas, stream);
    case 4: return launch_vec4<4, kMulAdd>(x, y, z, out, n, max_ctas, stream);
    default: return ASC_ERR_INVALID_ARG;
  }
}

}  // namespace

extern "C" {

int32_t asc_cuda_vadd_f32(const float* x, const float* y, float* out, int64_t n, void* stream) {
  return launch_eltwise<false>(x, y, nullptr, out, n, 0, static_cast<cudaStream_t>(stream));
}

int32_t asc_cuda_vmuladd_f32(const float* x, const float* y, const float* z, float* out, int64_t n, void* stream) {
  return launch_eltwise<true>(x, y, z, out, n, 0, static_cast<cudaStream_t>(stream));
}

int32_t asc_cuda_vadd_f32_variant(const float* x, const float* y, float* out, int64_t n, int32_t variant,
                                  void* stream) {
  return launch_eltwise<false>(x, y, nullptr, out, n, variant, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
