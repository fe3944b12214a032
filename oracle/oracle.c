/*
 * Plain-C restatement of the five hot-path computations.  TEST INFRASTRUCTURE, NOT PRODUCT: it is
 * built into oracle/_build/liboracle.so by oracle/build_oracle.py and loaded only by tests/ and by
 * bench.py's CPU-baseline leg.  It restates, independently of torch, the expressions the reference's
 * asc2 tests use as goldens:
 *   x + y                      python/test/asc2/kernels/test_vadd.py:48
 *   x * y + z                  python/test/asc2/kernels/test_vmuladd.py:51
 *   softmax(x, dim=1)          python/test/asc2/kernels/test_softmax.py:43
 *   a.float() @ b.float()      python/test/asc2/kernels/test_matmul_tiled.py:49
 *   a.int32 @ b.int32          python/test/generalization/adv/test_matmul_quant.py:134
 * and the workload's definitions of the dequantised int8 product and of attention (no reference
 * counterpart).  Compile with -ffp-contract=off so that multiply and add stay separately rounded.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static float half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while (!(man & 0x400u));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static float bf16_to_float(uint16_t h) {
  uint32_t bits = (uint32_t)h << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* float -> IEEE half, round to nearest even */
static uint16_t float_to_half(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t absx = x & 0x7fffffffu;
  if (absx >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x200u : 0));
  if (absx >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* rounds to inf */
  if (absx < 0x33000001u) return (uint16_t)sign;              /* rounds to zero */
  int32_t exp = (int32_t)(absx >> 23) - 127;
  uint32_t man = (absx & 0x7fffffu) | 0x800000u;
  uint32_t shift, half;
  if (exp < -14) {
    shift = (uint32_t)(13 + (-14 - exp));
    half = 0;
  } else {
    shift = 13;
    half = (uint32_t)(exp + 15) << 10;
  }
  uint32_t rem = man & ((1u << shift) - 1u);
  uint32_t halfway = 1u << (shift - 1);
  uint32_t q = man >> shift;
  if (exp >= -14) q &= 0x3ffu;
  uint32_t res = half + q;
  if (rem > halfway || (rem == halfway && (res & 1u))) ++res;
  return (uint16_t)(sign | res);
}

void oracle_vadd_f32(const float* x, const float* y, float* out, int64_t n) {
#pragma omp parallel for
  for (int64_t i = 0; i < n; ++i) out[i] = x[i] + y[i];
}

void oracle_vmuladd_f32(const float* x, const float* y, const float* z, float* out, int64_t n) {
#pragma omp parallel for
  for (int64_t i = 0; i < n; ++i) {
    volatile float p = x[i] * y[i];
    out[i] = p + z[i];
  }
}

void oracle_softmax_f32(const float* x, float* out, int64_t rows, int64_t cols) {
#pragma omp parallel for
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    float* orow = out + r * cols;
    float m = xr[0];
    for (int64_t c = 1; c < cols; ++c) m = xr[c] > m ? xr[c] : m;
    double s = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
      orow[c] = expf(xr[c] - m);
      s += orow[c];
    }
    const float sf = (float)s;
    for (int64_t c = 0; c < cols; ++c) orow[c] = orow[c] / sf;
  }
}

/* C[M,N] (fp32) = A[M,K] @ B[K,N], 16-bit operands given as raw bits; is_bf16 selects the format. */
void oracle_gemm_16(const uint16_t* a, const uint16_t* b, float* c, int64_t M, int64_t N, int64_t K, int is_bf16) {
  float* bf = (float*)malloc(sizeof(float) * (size_t)(K * N));
  for (int64_t i = 0; i < K * N; ++i) bf[i] = is_bf16 ? bf16_to_float(b[i]) : half_to_float(b[i]);
#pragma omp parallel for
  for (int64_t m = 0; m < M; ++m) {
    double* acc = (double*)calloc((size_t)N, sizeof(double));
    for (int64_t k = 0; k < K; ++k) {
      const double av = is_bf16 ? bf16_to_float(a[m * K + k]) : half_to_float(a[m * K + k]);
      const float* brow = bf + k * N;
      for (int64_t n = 0; n < N; ++n) acc[n] += av * (double)brow[n];
    }
    for (int64_t n = 0; n < N; ++n) c[m * N + n] = (float)acc[n];
    free(acc);
  }
  free(bf);
}

void oracle_gemm_i8(const int8_t* a, const int8_t* b, int32_t* c, int64_t M, int64_t N, int64_t K) {
#pragma omp parallel for
  for (int64_t m = 0; m < M; ++m) {
    int32_t* crow = c + m * N;
    for (int64_t n = 0; n < N; ++n) crow[n] = 0;
    for (int64_t k = 0; k < K; ++k) {
      const int32_t av = a[m * K + k];
      const int8_t* brow = b + k * N;
      for (int64_t n = 0; n < N; ++n) crow[n] += av * (int32_t)brow[n];
    }
  }
}

/* out (half bits) = ((float)acc * a_scale[row]) * b_scale[col], each product rounded to fp32 */
void oracle_dequant_f16(const int32_t* acc, const float* a_scale, const float* b_scale, uint16_t* out, int64_t M,
                        int64_t N) {
#pragma omp parallel for
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      volatile float t = (float)acc[m * N + n] * a_scale[m];
      volatile float u = t * b_scale[n];
      out[m * N + n] = float_to_half(u);
    }
}

/* o (fp32) = softmax(scale * q k^T [+ causal mask]) v for BH heads of [S, D] fp16 (raw bits). */
void oracle_attention_f16(const uint16_t* q, const uint16_t* k, const uint16_t* v, float* o, int64_t BH, int64_t S,
                          int64_t D, float scale, int causal) {
#pragma omp parallel for collapse(2)
  for (int64_t h = 0; h < BH; ++h)
    for (int64_t i = 0; i < S; ++i) {
      const uint16_t* qr = q + (h * S + i) * D;
      const int64_t lim = causal ? i + 1 : S;
      double* p = (double*)malloc(sizeof(double) * (size_t)lim);
      double mx = -INFINITY;
      for (int64_t j = 0; j < lim; ++j) {
        const uint16_t* kr = k + (h * S + j) * D;
        double s = 0.0;
        for (int64_t d = 0; d < D; ++d) s += (double)half_to_float(qr[d]) * (double)half_to_float(kr[d]);
        p[j] = s * (double)scale;
        if (p[j] > mx) mx = p[j];
      }
      double sum = 0.0;
      for (int64_t j = 0; j < lim; ++j) {
        p[j] = exp(p[j] - mx);
        sum += p[j];
      }
      float* orow = o + (h * S + i) * D;
      for (int64_t d = 0; d < D; ++d) {
        double acc = 0.0;
        for (int64_t j = 0; j < lim; ++j) acc += p[j] * (double)half_to_float(v[(h * S + j) * D + d]);
        orow[d] = (float)(acc / sum);
      }
      free(p);
    }
}
