/*
 * Tuning and bring-up hooks of libasc_cuda.  Not part of the drop-in boundary: the Python runtime
 * never calls them; they exist so that variants of a kernel can be timed against each other from a
 * script.  No counterpart in the reference.
 */
#ifndef ASC_CUDA_TUNING_H_
#define ASC_CUDA_TUNING_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* variant: bits 0-3 vectors per thread (1, 2, 4, 8; 0 = default), bits 8-15 CTAs per SM for a
 * grid-stride launch (0 = one chunk per CTA). */
int32_t asc_cuda_vadd_f32_variant(const float* x, const float* y, float* out, int64_t n, int32_t variant,
                                  void* stream);

/* variant: bits 0-7 CTA shape for 2048 < cols <= 4096 (0: 512 threads x 2 vectors, 1: 128 x 8,
 * 3: 256 x 4, 0xff: the shared-memory staged kernel), bits 8-15 CTAs per SM (0 = default). */
int32_t asc_cuda_softmax_f32_variant(const float* x, float* out, int64_t rows, int64_t cols, int64_t ld,
                                     int32_t variant, void* stream);

/* GEMM with a cap on the number of CTAs.  in_dtype: 0 fp16, 1 bf16, 2 int8 (int32 output);
 * out_dtype as asc_cuda_gemm_f16 (ignored for int8); max_ctas 0 = one per SM. */
int32_t asc_cuda_gemm_capped(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                             int64_t ldb, int64_t ldc, int32_t in_dtype, int32_t out_dtype, int32_t max_ctas,
                             void* stream);

/* GEMM kernel selection: 0 choose per problem (default), 1 always the single-CTA 128 x 256 kernel,
 * 2 the CTA-pair 256 x 256 kernel whenever M > 128.  Bit 4 (0x10): run small fp16 / bf16 products with an fp32
 * result on the tensor core as well (by default they take the FMA pipe, see asc_cuda_gemm_f16).  Bit 5 (0x20): never
 * split K over several CTAs per tile.  Process-wide. */
int32_t asc_cuda_gemm_set_mode(int32_t mode);

/* bits 0-7: elements each thread evaluates per opcode dispatch in asc_cuda_eltwise_program's aligned path
 * (4, 8 or 16; anything else: chosen by program length); bit 8: run every program in the interpreter, also
 * those with a compile-time specialised kernel; bits 16-23: waves of resident CTAs in the grid (0: four).
 * Process-wide. */
int32_t asc_cuda_eltwise_set_lanes(int32_t lanes);

/* Self-test of the bounded device-side waits: launches one warp that waits on a barrier nobody arrives on, with a
 * limit of 0.5 ms (the kernels' own waits use the same routine with 400 ms).  The wait gives up, writes code
 * 0x500 to the device's status word and the kernel returns normally; *gave_up (device memory, may be NULL)
 * receives 1.  The next asc_cuda_check_device_status on that stream then reports status 5 and clears the word. */
int32_t asc_cuda_selftest_wait_runs_out(uint32_t* gave_up, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* ASC_CUDA_TUNING_H_ */
