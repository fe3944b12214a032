/*
 * libasc_cuda — C ABI of the CUDA (sm_100a / B200) platform behind PyAsc's asc2 surface.
 *
 * This is the boundary the Python runtime binding (asc.lib.runtime) loads with ctypes,
 * exactly as the reference loads its rt_wrapper shared object
 * (python/asc/lib/runtime/state.py:25-75; wrappers in python/asc/lib/runtime/rt_wrapper.cpp:23-244).
 *
 * Conventions (same as the reference wrappers):
 *   - extern "C", plain pointers and sizes, no C++/torch types;
 *   - every function returns an integer status, 0 == OK; the Python side turns any other
 *     value into RuntimeError("Function <name> returned <code>") (state.py:64-66);
 *   - the caller owns every buffer; the library keeps no reference after return;
 *   - kernel entry points are asynchronous on `stream` (a cudaStream_t passed as void*,
 *     NULL == the legacy default stream) and touch device memory only;
 *   - no entry point ever falls back to a CPU implementation.
 *
 * Status codes: 0 OK, 1 invalid argument, 2 misaligned pointer/stride, 3 unsupported shape or
 * dtype, 4 CUDA call failed (asc_cuda_last_cuda_error gives the text), 5 a bounded device-side
 * wait ran out, 6 size beyond a documented maximum, 7 no usable device.
 */
#ifndef ASC_CUDA_H_
#define ASC_CUDA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------
 * Device / stream / memory wrappers.  Same names and argument order as the reference's CANN
 * wrappers so that asc.lib.runtime.interface keeps calling them unchanged.
 * ---------------------------------------------------------------------------------------- */

/* replaces rt_wrapper.cpp:23 — writes "B200" style SoC name (the CUDA device name). */
int32_t GetSocVersionWrapper(char* ver, uint32_t maxLen);
/* replaces rt_wrapper.cpp:32 */
int32_t GetDeviceCountWrapper(int32_t* cnt);
/* replaces rt_wrapper.cpp:66 — moduleType is ignored; infoType: 0 SM count, 1 HBM bytes,
 * 2 L2 bytes, 3 max SM clock kHz, 4 compute capability (major*10+minor). */
int32_t GetDeviceInfoWrapper(uint32_t deviceId, int32_t moduleType, int32_t infoType, int64_t* val);
/* replaces rt_wrapper.cpp:77 — destroys the streams the library created on the device; never
 * resets the GPU itself (the GPU is shared). */
int32_t DeviceResetWrapper(int32_t devId);
/* replaces rt_wrapper.cpp:86 */
int32_t SetDeviceWrapper(int32_t devId);
/* replaces rt_wrapper.cpp:96 */
int32_t StreamCreateWrapper(void** stm, int32_t priority);
/* replaces rt_wrapper.cpp:105 */
int32_t StreamDestroyWrapper(void* stm);
/* replaces rt_wrapper.cpp:156 — `type` and `moduleId` are accepted and ignored. */
int32_t MallocWrapper(void** devPtr, uint64_t size, int32_t type, uint16_t moduleId);
/* replaces rt_wrapper.cpp:172 — kind: 0 H2H, 1 H2D, 2 D2H, 3 D2D (reference enum values,
 * python/asc/lib/runtime/support.py:96-105).  Synchronous. */
int32_t MemcpyWrapper(void* dst, uint64_t destMax, const void* src, uint64_t cnt, int32_t kind);
/* no reference counterpart: asynchronous copy on `stm` (pinned host memory recommended). */
int32_t MemcpyAsyncWrapper(void* dst, uint64_t destMax, const void* src, uint64_t cnt, int32_t kind, void* stm);
/* replaces rt_wrapper.cpp:203 — timeout in milliseconds; non-zero status when it runs out. */
int32_t StreamSynchronizeWithTimeoutWrapper(void* stm, int32_t timeout);
/* replaces rt_wrapper.cpp:215 */
int32_t StreamSynchronizeWrapper(void* stm);
/* replaces rt_wrapper.cpp:224 */
int32_t FreeWrapper(void* devPtr);
/* replaces rt_wrapper.cpp:232 */
int32_t DeviceSynchronizeWrapper(void);
/* no reference counterpart: page-locked host staging buffers for the launcher's H2D/D2H path
 * (the reference stages through pageable memory, python/asc/runtime/memory_handle.py:82-91). */
int32_t HostMallocWrapper(void** hostPtr, uint64_t size);
int32_t HostFreeWrapper(void* hostPtr);
/* no reference counterpart: pin / unpin a caller-owned host range in place. */
int32_t HostRegisterWrapper(void* hostPtr, uint64_t size);
int32_t HostUnregisterWrapper(void* hostPtr);

/* ------------------------------------------------------------------------------------------
 * Timing (stands in for the reference's msprof task timing,
 * python/asc/lib/profiling/profiler.py:59-129): CUDA events on the launching stream.
 * ---------------------------------------------------------------------------------------- */
int32_t asc_cuda_event_create(void** ev);
/* ordering-only event (no timestamps) and a stream-side wait on an event: the launcher uses them to
 * overlap uploads, kernels and downloads of one launch on three streams.  No reference counterpart
 * (the reference launcher copies, launches and copies back strictly in sequence,
 * python/asc/runtime/launcher.py:176-195). */
int32_t asc_cuda_event_create_notiming(void** ev);
int32_t StreamWaitEventWrapper(void* stm, void* ev);
int32_t asc_cuda_event_record(void* ev, void* stream);
int32_t asc_cuda_event_synchronize(void* ev);
int32_t asc_cuda_event_elapsed_ms(void* start, void* stop, float* ms);
int32_t asc_cuda_event_destroy(void* ev);

/* ------------------------------------------------------------------------------------------
 * Diagnostics
 * ---------------------------------------------------------------------------------------- */
/* Human-readable text for a status code. */
int32_t asc_cuda_status_string(int32_t code, char* buf, uint32_t n);
/* Text of the last failing CUDA call on this thread ("" when none). */
int32_t asc_cuda_last_cuda_error(char* buf, uint32_t n);
/* Synchronises `stream`, then reads and clears the current device's status word.  *dev_code is 0
 * when every kernel finished normally; otherwise the code a kernel left when one of its bounded
 * waits ran out, and the function returns 5. */
int32_t asc_cuda_check_device_status(void* stream, uint32_t* dev_code);
/* Number of kernels this library has launched since load (all threads). */
int32_t asc_cuda_launch_count(uint64_t* count);

/* ------------------------------------------------------------------------------------------
 * Kernels.  Each replaces what the reference's launcher starts for the matching asc2 kernel
 * (python/asc/runtime/launcher.py:156-195 -> rt_wrapper.cpp:189 KernelLaunchWrapper) together
 * with the Ascend C routines its lowering calls.
 * ---------------------------------------------------------------------------------------- */

/* out[i] = x[i] + y[i], fp32, i in [0, n).  Bit-exact IEEE add.
 * Replaces the vector-add tile loop of python/test/asc2/kernels/test_vadd.py:16-28
 * (arith.addf -> AddL2Op, lib/Conversion/LowerToAsc/LowerArithBinary.cpp:113). */
int32_t asc_cuda_vadd_f32(const float* x, const float* y, float* out, int64_t n, void* stream);

/* out[i] = x[i] * y[i] + z[i] with separately rounded multiply and add (no FMA contraction),
 * matching NumPy.  Replaces python/test/asc2/kernels/test_vmuladd.py:16-31. */
int32_t asc_cuda_vmuladd_f32(const float* x, const float* y, const float* z, float* out, int64_t n, void* stream);

/* out[i] = f(in_0[i], ..., in_{k-1}[i]) for i in [0, n): any expression of the asc2 elementwise ops
 * over same-shaped operands, evaluated in one pass over memory.  The expression is a postfix program
 * of n_ops (<= 48) opcodes over an 8-deep stack of 32-bit words (fp32 values, or int32 for the
 * integer opcodes); args[j] is the input index of a LOAD or the 32-bit word a CONST pushes.  Opcodes: 0 LOAD, 1 CONST, 2 ADD, 3 SUB, 4 MUL, 5 DIV, 6 MAX, 7 MIN, 8 NEG,
 * 9 ABS, 10 RELU, 11 EXP, 12 EXP2, 13 LOG, 14 LOG2, 15 SQRT, 16 RSQRT, 17 SIN, 18 COS, 19 TAN,
 * 20 SINH, 21 COSH, 22 TANH, 23 ERF, 24 FLOOR, 25 CEIL, 26 EQ, 27 NE, 28 GT, 29 GE, 30 LT, 31 LE
 * (comparisons push 1.0 / 0.0), 32 WHERE (cond, a, b -> cond != 0 ? a : b), 33 ROUND_F16,
 * 34 ROUND_BF16 (round the top of the stack through that type, so that a chain of 16-bit ops rounds
 * like a per-op evaluation); on int32 stack words 35 IADD, 36 ISUB, 37 IMUL, 38 IMAX, 39 IMIN,
 * 40 ISHL, 41 ISHR (arithmetic), 42 IEQ, 43 INE, 44 IGT, 45 IGE, 46 ILT, 47 ILE, 48 INEG, 49 IABS,
 * 50 IRELU, 51 CVT_I2F, 52 CVT_F2I (truncating), 53 WRAP_I16 (sign-extend the low half); with the
 * operands swapped (rhs op lhs) 54 RSUB, 55 RDIV, 56 IRSUB, 57 IRSHL, 58 IRSHR.  A binary opcode
 * with bit 8 set (| 0x100) takes args[j] as its left operand instead of a stack entry.
 * Element types: 0 fp32, 1 fp16, 2 bf16, 3 int32, 4 int16; at most 6 inputs.
 * The program is validated on the host (status 1 for a malformed one, 6 for a stack deeper than 8).
 * Replaces the per-op vector calls the reference lowers such kernels to
 * (python/asc/language/tile/binary_ops.py, unary_ops.py, indexing_ops.py:where;
 * lib/Conversion/LowerToAsc/LowerArithBinary.cpp, LowerMath.cpp), e.g. the kernels of
 * python/test/asc2/kernels/test_leaky_relu.py:16-27 and test_gelu.py:16-34. */
int32_t asc_cuda_eltwise_program(const int32_t* ops, const int32_t* args, int32_t n_ops, const void* const* inputs,
                                 const int32_t* input_types, int32_t n_inputs, void* out, int32_t out_type,
                                 int64_t n, void* stream);

/* The same over a [rows, cols] window in which every operand has its own row pitch: lds holds the pitch
 * (in elements) of each input, then of the output; every pointer addresses its operand's first element of
 * the window.  An input pitch of 0 repeats one row for every row of the window (asc2.broadcast_to of a
 * [1, cols] tile).  lds == NULL means that all pitches equal cols, i.e. one contiguous range.  This is what
 * 2-D tiles that do not span whole rows touch (asc2.load / asc2.store with 2-D offsets,
 * python/asc/language/tile/memory_ops.py; python/test/asc2/operations/test_memory_ops.py:10-59,
 * test_shape_ops.py:17-18).  A window that is not one contiguous range is limited to 2^32 elements. */
int32_t asc_cuda_eltwise_program_2d(const int32_t* ops, const int32_t* args, int32_t n_ops,
                                    const void* const* inputs, const int32_t* input_types, int32_t n_inputs,
                                    void* out, int32_t out_type, int64_t rows, int64_t cols, const int64_t* lds,
                                    void* stream);

/* A program over the rows of a [rows, cols] window (cols <= 8192) in which four more opcodes reduce the top of
 * the stack over the row: ROW_SUM 59, ROW_MAX 60, ROW_MIN 61, ROW_PROD 62 (fp32).  Every element of the row
 * then sees the reduced value as an ordinary operand, so an expression that mixes elementwise arithmetic with
 * reductions of its own intermediate tiles along the last dimension (x - max(x), exp(..) / sum(exp(..)), a
 * variance) is one pass: a row never leaves the SM between its load and its store.  lds as for the 2-D
 * elementwise call (NULL: all pitches equal cols).  row_result != 0: the program's value is uniform along the
 * row and one element per row is stored, at out[r * lds[n_inputs]] (pitch 1 when lds is NULL).
 * An input type with bit 0x200 set marks an input that holds one element per row (a column: element r at
 * inputs[k][r * lds[k]], pitch 1 when lds is NULL), which every element of the row reads.
 * Two more opcodes let a program compute a shared sub-expression once: TEE 63 copies the top of the stack into
 * temporary slot args[j] (0..3) without popping it, TMP 64 pushes that slot; a slot must be written before it is
 * read (status 1 otherwise).  The two upper stack entries live in registers, deeper entries and the temporary
 * slots in shared memory: a program whose (stack depth - 2, at least 1, + slots used) x ceil(cols / 256 to a power
 * of two) KiB exceeds 200 KiB returns status 6, as does cols > 8192.
 * Replaces the chains of vector calls and ReduceOp calls the reference lowers such kernels to
 * (python/asc/language/tile/reduction_ops.py, shape_ops.py:30-75; lib/Conversion/LowerToAsc/LowerAscTile.cpp:
 * 329-378 BroadcastOp, 428-459 ReduceOp; the manual softmax of python/test/asc2/kernels/test_softmax.py:16-27 is
 * the reference's own example of the shape). */
int32_t asc_cuda_row_program(const int32_t* ops, const int32_t* args, int32_t n_ops, const void* const* inputs,
                             const int32_t* input_types, int32_t n_inputs, void* out, int32_t out_type, int64_t rows,
                             int64_t cols, const int64_t* lds, int32_t row_result, void* stream);

/* An elementwise program (no row opcodes) over a [rows, cols] window, reduced along the rows: out[c] = kind over r of
 * program(r, c); kind: 0 sum, 1 max, 2 min, 3 product, combined in fp32 and rounded once to out_type (fp32, fp16 or
 * bf16).  lds: the row pitch of every input (0: a row every window row reads), NULL: all pitches equal cols.  With
 * rows == 0 every out[c] receives the identity of the reduction.  Serves asc2.reduce_*(expression, 0) on tile-sized
 * windows (python/asc/language/tile/reduction_ops.py:33-188; ReduceOp, lib/Conversion/LowerToAsc/LowerAscTile.cpp:428-459):
 * a thread owns a column, so the grid covers the columns only. */
int32_t asc_cuda_col_program(const int32_t* ops, const int32_t* args, int32_t n_ops, const void* const* inputs,
                             const int32_t* input_types, int32_t n_inputs, void* out, int32_t out_type, int64_t rows,
                             int64_t cols, const int64_t* lds, int32_t kind, void* stream);

/* Registers a kernel specialised for one program, so that asc_cuda_eltwise_program[_2d] (kind 0) or
 * asc_cuda_row_program (kind 1000 + columns per thread: 1, 2, 4, ... 32) runs it instead of the interpreter whenever
 * that program is submitted.  `words[k]` = ops[k] | (args[k] << 16 for a LOAD, TEE or TMP) | (1 << 24 for a LOAD of
 * a one-element-per-row input); `fn` is the entry point `int asc_jit_run(const void* program, int64_t n_or_rows,
 * int32_t flag, int32_t sms, void* stream)` of a shared library built from pyasc_b200/csrc/eltwise_program.cuh
 * (pyasc_b200/jit.py generates, builds and caches such libraries at first use of an expression).  Plays the role of the
 * reference's first-use build and cache of device code (python/asc/runtime/jit.py:158-202, cache.py:57-112). */
int32_t asc_cuda_register_program(int32_t kind, const int32_t* words, int32_t n_words, void* fn);

/* Copy of a window of `rows` rows of `row_bytes` bytes between two device matrices with their own row pitches (bytes;
 * each at least row_bytes).  The windows must not overlap.  Serves asc2.store(asc2.load(...)) of tiles of element
 * types the elementwise kernels do not compute on (8-bit and 64-bit types): a pure move, which the reference lowers
 * to DataCopy between global and on-chip memory (python/asc/language/tile/memory_ops.py). */
int32_t asc_cuda_copy_2d(void* dst, const void* src, int64_t rows, int64_t row_bytes, int64_t dst_pitch,
                         int64_t src_pitch, void* stream);

/* 8-bit integers <-> int32 words, n elements.  mode 0: int8 -> int32 (sign-extended), 1: uint8 -> int32
 * (zero-extended), 2: int32 -> its low byte (int8 and uint8 alike).  The 32-bit side must be 4-byte aligned.
 * The elementwise programs compute on 32- and 16-bit types; a kernel that loads or stores an int8 / uint8 tile gets its
 * bytes widened into, or narrowed out of, an int32 temporary by this call.  Replaces the CastOp between integer
 * widths around such a tile (python/asc/language/tile/tile.py:60-78; ConvertCast, lib/Conversion/LowerToAsc/LowerAscTile.cpp:129-160). */
int32_t asc_cuda_convert_bytes(void* dst, const void* src, int64_t n, int32_t mode, void* stream);

/* Reduction of a row-major [rows, cols] fp32 window with row pitch `ld` (elements).  kind: 0 sum, 1 max,
 * 2 min, 3 product.  axis 1: out[r] = reduce over the columns of row r; axis 0: out[c] = reduce over the
 * rows of column c; axis -1: out[0 .. n_fill) all receive the reduction of the whole window (the window is
 * an on-chip sized tile: at most 2^24 elements).  n_fill is ignored for axis 0 / 1.
 * Replaces asc2.reduce_sum / reduce_max / reduce_min / reduce_prod on a loaded tile
 * (python/asc/language/tile/reduction_ops.py; ReduceOp, lib/Conversion/LowerToAsc/LowerAscTile.cpp:428-459),
 * as exercised by python/test/asc2/operations/test_reduce_ops.py:17-104. */
int32_t asc_cuda_reduce_f32(const float* x, float* out, int64_t rows, int64_t cols, int64_t ld, int32_t axis,
                            int32_t kind, int64_t n_fill, void* stream);
/* The whole-window form (axis -1 above) for fp16 (dtype 0) or bf16 (dtype 1) windows: combined in fp32, rounded once,
 * out[0 .. n_fill) all receive the result.  asc2.reduce_*(tile) without dimensions on a 16-bit tile
 * (ReduceAs1dOp, lib/Conversion/LowerToAsc/LowerAscTile.cpp:427-458).  Along one axis 16-bit tiles go through
 * asc_cuda_row_program / asc_cuda_col_program. */
int32_t asc_cuda_reduce_all_f16(const void* x, void* out, int64_t rows, int64_t cols, int64_t ld, int32_t kind,
                                int64_t n_fill, int32_t dtype, void* stream);

/* Row softmax over the last dimension of a contiguous [rows, cols] fp32 matrix with max
 * subtraction.  `ld` is the row pitch in elements (>= cols).  Replaces both asc2 softmax forms:
 * the manual reduce_max/exp/reduce_sum kernel (python/test/asc2/kernels/test_softmax.py:16-27;
 * LowerAscTile.cpp:428-459, LowerMath.cpp:95) and asc2.softmax
 * (python/asc/language/tile/unary_ops.py:215-223 -> SoftMaxOp, LowerAscTile.cpp:155-188). */
int32_t asc_cuda_softmax_f32(const float* x, float* out, int64_t rows, int64_t cols, int64_t ld, void* stream);
/* The same for fp16 rows (asc2.softmax accepts float16 tiles, python/asc/language/tile/unary_ops.py:217;
 * python/test/asc2/operations/test_softmax.py:35-58): fp32 arithmetic, one rounding at the store. */
int32_t asc_cuda_softmax_f16(const void* x, void* out, int64_t rows, int64_t cols, int64_t ld, void* stream);

/* RMS normalisation over the last dimension of a row-major fp32 window [rows, cols] with row pitch ld:
 *   out[r, c] = x[r, c] / sqrt(mean_c(x[r, :]^2) + eps) * gamma[c]
 * Replaces asc2.rms_norm (python/asc/language/tile/unary_ops.py:225-237), which the reference lowers to the
 * Ascend C RmsNorm routine with a generated tiling (lib/Conversion/LowerToAsc/LowerAscTile.cpp:190-289).
 * x and out may alias; gamma holds cols floats.  Empty windows return ASC_OK without a launch. */
int32_t asc_cuda_rms_norm_f32(const float* x, const float* gamma, float* out, int64_t rows, int64_t cols, int64_t ld,
                              float eps, void* stream);
/* The same for fp16 rows and gamma (asc2.rms_norm accepts float16 tiles, unary_ops.py:227): the row is widened to
 * fp32, the sum of squares and the scaling are fp32, one rounding at the store. */
int32_t asc_cuda_rms_norm_f16(const void* x, const void* gamma, void* out, int64_t rows, int64_t cols, int64_t ld,
                              float eps, void* stream);

/* C[M,N] = epilogue(A[M,K] @ B[K,N]), row-major operands, fp32 accumulation on tcgen05 tensor
 * cores.  in_dtype: 0 fp16, 1 bf16.  out_dtype: 0 fp16, 1 bf16, 2 fp32.
 * flags: bit0 ReLU before the cast; bit1 accumulate into C (C += A@B, fp32 out only).
 * lda/ldb/ldc are row pitches in elements.  Requirements: base pointers 16-byte aligned,
 * lda*2 and ldb*2 multiples of 16 bytes.  A product stored as fp32 with M*N*K <= 2^28 runs on the FMA pipe
 * instead (exact products, round-to-nearest sums: within a few units in the last place of an fp32 CPU matmul,
 * which the reference's own matmul tests assert at torch's default fp32 tolerance,
 * python/test/asc2/kernels/test_matmul_mnblock.py:92); the tensor core's accumulator truncates.
 * Replaces asc2.matmul / matmul_acc + the fixpipe store
 * (python/asc/language/tile/binary_ops.py:181-221; MmadOp, LowerAscTile.cpp:291-315,577-603;
 * FixpipeOp, LowerAscTileDataTransfer.cpp:273-325). */
int32_t asc_cuda_gemm_f16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                          int64_t ldb, int64_t ldc, int32_t in_dtype, int32_t out_dtype, int32_t flags,
                          void* stream);

/* asc_cuda_gemm_f16 with a bias row in the epilogue: C = cast(relu?(A @ B + bias[col])), the addition in fp32
 * (round to nearest) on the fp32 accumulator before the ReLU and the one rounding of the store.  bias holds N
 * values, one per output column; bias_dtype: 0 fp16, 1 bf16, 2 fp32 (widened to fp32 before the addition); no
 * alignment rule.  flags: bit0 ReLU; bit1 (accumulate into C) is refused with status 3.  Everything else as
 * asc_cuda_gemm_f16.  Replaces a matmul whose fixpipe result gets a broadcast row added on the vector unit before
 * the store (python/asc/language/tile/binary_ops.py:181-221 followed by add, binary_ops.py:112; the reference runs the
 * addition as a separate vector pass over the product). */
int32_t asc_cuda_gemm_f16_bias(const void* A, const void* B, void* C, const void* bias, int64_t M, int64_t N,
                               int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int32_t in_dtype, int32_t out_dtype,
                               int32_t bias_dtype, int32_t flags, void* stream);

/* asc_cuda_gemm_f16 for callers that cannot allocate device memory while they run: a latency-critical host thread
 * that must never block in the driver's allocator, a service whose device-memory budget was handed out in full at
 * start-up, code under a rule that forbids cudaMalloc after initialisation.  It has no counterpart in the
 * reference.  The kernel is the
 * split-K one (K cut over several CTAs per 128 x 256 tile, partial tiles summed in slice order), and its
 * workspace is not allocated per call but is a fixed array inside the library, 8 MiB + 1 KiB, which every GPU
 * that loads the library holds until the process exits.  This entry point calls no cudaMalloc, cudaFree or other
 * allocating routine.
 *   - Limit: C may cover at most 64 tiles, ceil(M / 128) * ceil(N / 256) <= 64 (e.g. 1024 x 2048); anything larger
 *     returns status 6 (ASC_ERR_TOO_LARGE).  Arguments, alignment rules and flags as for asc_cuda_gemm_f16.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current) and sets a function attribute; make that first call outside any stream capture.
 *   - All calls on a device share the one array: the part that must start at zero (the per-tile counters) is
 *     cleared on the stream at the start of every call, but two calls that overlap on the GPU (different streams,
 *     or graphs replayed concurrently) race on it and give wrong results.  Keep calls on one stream, or order
 *     them with events. */
int32_t asc_cuda_gemm_f16_static_workspace(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                           int64_t lda, int64_t ldb, int64_t ldc, int32_t in_dtype, int32_t out_dtype,
                                           int32_t flags, void* stream);

/* fp32-input matmul with the same epilogue options (CUDA-core FMA; exists so that the fp32 case of
 * python/test/asc2/kernels/test_matmul_fixpipe.py:36-48 runs; not a tuned path). */
int32_t asc_cuda_gemm_f32(const float* A, const float* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                          int64_t ldb, int64_t ldc, int32_t out_dtype, int32_t flags, void* stream);

/* acc[M,N] = A[M,K] @ B[K,N] with signed int8 operands and exact int32 accumulation
 * (tcgen05 kind::i8); optionally deq[M,N] = fp16( (float(acc) * a_scale[row]) * b_scale[col] ).
 * Either output pointer may be NULL (not both).  a_scale/b_scale are required when deq != NULL.
 * Requirements: A, B 16-byte aligned; lda, ldb multiples of 16.
 * The reference has no asc2 int8 matmul; the nearest definition is the golden of
 * python/test/generalization/adv/test_matmul_quant.py:124-138 (int32 = a.int32 @ b.int32). */
int32_t asc_cuda_gemm_i8(const int8_t* A, const int8_t* B, int32_t* acc, void* deq, const float* a_scale,
                         const float* b_scale, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                         int64_t ldc, void* stream);

/* O = softmax(scale * Q K^T [+ causal mask]) V for contiguous [B, H, S, D] tensors, fp32
 * online-softmax accumulation.  dtype: 0 fp16, 1 bf16.  D must be 128 (the only head size of the
 * workload this library targets; anything else returns status 3); S is any positive length (rows past S
 * read as zero and are never written).  Pointers 16-byte aligned.  causal != 0 masks key j > query i.
 * No counterpart in the reference (it has no attention kernel); defined by the torch expression
 * softmax((Q.float() @ K.float().transpose(-1,-2)) * scale + mask, -1) @ V.float(). */
int32_t asc_cuda_attn_fwd_f16(const void* q, const void* k, const void* v, void* o, int32_t B, int32_t H,
                              int32_t S, int32_t D, float scale, int32_t causal, int32_t dtype, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* ASC_CUDA_H_ */
