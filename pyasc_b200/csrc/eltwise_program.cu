// Generic fused elementwise kernel: one pass over memory for any expression over same-shaped tiles.
//
// The asc2 surface lets a kernel combine loads with arithmetic, math functions, comparisons and
// `where` before one store (python/asc/language/tile/{binary,unary,indexing}_ops.py).  The reference
// lowers each op to its own Ascend C vector call; here the whole expression is compiled by the
// launcher into a small postfix program that every thread evaluates per element on a register
// stack, so the tensors are read once and written once whatever the expression is.
//
// Stack words are 32 bits wide: floating-point values are carried as fp32, integers as int32 (with
// their own opcodes).  An op whose asc2 tile type is 16-bit is followed by a ROUND (or WRAP) op so
// that intermediate results round exactly as a per-op evaluation in that type would (the reference's
// CPU goldens evaluate in the tensor dtype).  HBM-bound: (inputs + 1) x element size bytes per element.
#include <mutex>
#include <vector>

#include "../../include/asc_cuda.h"
#include "host_common.h"
#include "eltwise_program.cuh"

namespace {

// ---- programs specialised at first use ----
// The launcher generates, for an expression it meets for the first time, a translation unit that instantiates the
// compile-time executors for exactly that opcode list, builds it into a small shared library and registers the
// library's entry point here under the list's words.  Dispatch looks a submitted program up and, on a hit, runs the
// specialised kernel instead of the interpreter.  kind 0: elementwise; 1000 + kV: a row program with kV columns per
// thread.
using JitFn = int (*)(const void* prog, int64_t n, int32_t flag, int32_t sms, void* stream);
struct JitEntry {
  int kind;
  std::vector<int32_t> words;
  JitFn fn;
};
std::mutex g_jit_mutex;
std::vector<JitEntry> g_jit;

// The word the generated unit's OpList holds for op k (see RowStep): opcode, operand index, per-row flag.
int32_t jit_word(const int32_t* ops, const int32_t* args, const int32_t* input_types, int k, bool row) {
  const int op = ops[k] & 0xff;
  int32_t w = ops[k];
  if (op == OP_LOAD || op == OP_TEE || op == OP_TMP) w |= args[k] << 16;
  if (row && op == OP_LOAD && (input_types[args[k]] & kRowScalarInput) != 0) w |= kRowScalarWord;
  return w;
}

JitFn find_jit(int kind, const int32_t* ops, const int32_t* args, const int32_t* input_types, int n_ops) {
  std::lock_guard<std::mutex> lock(g_jit_mutex);
  for (const JitEntry& e : g_jit) {
    if (e.kind != kind || static_cast<int>(e.words.size()) != n_ops) continue;
    bool same = true;
    for (int k = 0; k < n_ops && same; ++k) same = e.words[k] == jit_word(ops, args, input_types, k, kind != 0);
    if (same) return e.fn;
  }
  return nullptr;
}

std::atomic<int> g_waves{0};            // tuning hook: waves of resident CTAs in the grid of an elementwise launch (0: four)
std::atomic<int> g_lanes{0};            // interpreter: elements per thread and dispatch on the aligned path (4, 8, 16; 0: by program length)
std::atomic<bool> g_use_compiled{true};  // tuning hook can force the interpreter for every program

template <class Exec, int kLanes>
int32_t launch_program(const EltProgram& prog, int64_t n, size_t smem, int sms, cudaStream_t stream) {
  if (smem + 1024 > 48 * 1024) {     // dynamic plus the kernel's few static words: beyond the default limit
    static aschost::PerDevice attr_set;
    int dev = 0;
    ASC_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_set.get(dev)) {
      ASC_CUDA_TRY(cudaFuncSetAttribute(eltwise_program_kernel<Exec, kLanes>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (kStack - 1) * kThreads * 16 * static_cast<int>(sizeof(float))));
      attr_set.set(dev, 1);
    }
  }
  int resident = 0;
  ASC_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, eltwise_program_kernel<Exec, kLanes>, kThreads, smem));
  if (resident < 1) resident = 1;
  const int64_t per_cta = static_cast<int64_t>(kThreads) * kLanes;
  int64_t ctas = (n + per_cta - 1) / per_cta;
  // four waves of resident CTAs, CTAs stride beyond; one wave when the whole launch is at most eight waves of
  // work (measured on GELU: 2^23 elements 14.0 vs 15.0 us, 2^24 25.3 vs 25.9, no difference from 2^25 on)
  const int forced_waves = g_waves.load(std::memory_order_relaxed);
  const int64_t wave = static_cast<int64_t>(sms) * resident;
  const int64_t cap = wave * (forced_waves > 0 ? forced_waves : (ctas <= 8 * wave ? 1 : 4));
  if (ctas > cap) ctas = cap;
  eltwise_program_kernel<Exec, kLanes><<<static_cast<unsigned>(ctas), kThreads, smem, stream>>>(prog, n);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

template <int kLanes>
int32_t launch_interpreter(const EltProgram& prog, int64_t n, int max_depth, int sms, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(max_depth > 1 ? max_depth - 1 : 1) * kThreads * (kLanes < 4 ? 4 : kLanes) * sizeof(float);
  return launch_program<Interpreter, kLanes>(prog, n, smem, sms, stream);
}

// ---- the compiled programs: exactly what the launcher's expression compiler emits for these kernels ----
constexpr int I = OP_IMM;
// where(x >= 0, x, x * alpha): python/test/asc2/kernels/test_leaky_relu.py:16-27 (fp32 / fp16 / bf16 tiles)
using LeakyReluF32 = OpList<LD(0), OP_LE | I, LD(0), LD(0), OP_MUL | I, OP_WHERE>;
using LeakyReluF16 = OpList<LD(0), OP_LE | I, LD(0), LD(0), OP_MUL | I, OP_ROUND_F16, OP_WHERE>;
using LeakyReluBF16 = OpList<LD(0), OP_LE | I, LD(0), LD(0), OP_MUL | I, OP_ROUND_BF16, OP_WHERE>;
// x * (erf(x * k) + 1) * 0.5 and x - x / (exp(x * (x * x * k2 + k1)) + 1): test_gelu.py:16-34 (fp32)
using GeluErf = OpList<LD(0), LD(0), OP_MUL | I, OP_ERF, OP_ADD | I, OP_MUL, OP_MUL | I>;
using GeluTanh = OpList<LD(0), LD(0), OP_MUL, OP_MUL | I, OP_ADD | I, LD(0), OP_MUL, OP_EXP, OP_ADD | I, LD(0), OP_RDIV,
                        LD(0), OP_RSUB>;

int elem_size(int type) { return (type == T_F16 || type == T_BF16 || type == T_I16) ? 2 : 4; }

// 1 / (1 + exp(-x)) and x / (exp(-x) + 1): the usual spellings of sigmoid and SiLU
using Sigmoid = OpList<LD(0), OP_NEG, OP_EXP, OP_ADD | I, OP_DIV | I>;
using Silu = OpList<LD(0), LD(0), OP_NEG, OP_EXP, OP_ADD | I, OP_DIV>;

template <class P>
bool matches(const int32_t* ops, const int32_t* args, int n_ops) {
  if (n_ops != P::n) return false;
  for (int k = 0; k < n_ops; ++k) {
    const int word = P::at(k);
    if ((word & 0xffff) != ops[k]) return false;
    if ((word & 0xff) == OP_LOAD && ((word >> 16) & 0xff) != args[k]) return false;
  }
  return true;
}

// launches the compiled form of the program when there is one (aligned pointers only); *launched tells
template <class P>
int32_t try_compiled(const EltProgram& prog, const int32_t* ops, const int32_t* args, int n_ops, int64_t n, int sms,
                     cudaStream_t stream, bool* launched) {
  if (*launched || !matches<P>(ops, args, n_ops)) return ASC_OK;
  *launched = true;
  // 16 bytes per access and thread want twice the lanes for 16-bit elements
  bool oct = elem_size(prog.out_type) == 2 && reinterpret_cast<uintptr_t>(prog.out) % 16 == 0;
  for (int i = 0; i < prog.n_inputs; ++i)
    oct = oct && elem_size(prog.in_type[i] & 0xff) == 2 && reinterpret_cast<uintptr_t>(prog.in[i]) % 16 == 0;
  if (oct) return launch_program<Compiled<P, true>, 16>(prog, n, 0, sms, stream);
  return launch_program<Compiled<P, false>, 8>(prog, n, 0, sms, stream);
}


template <int kV>
int32_t launch_row_program(const EltProgram& prog, int64_t rows, int max_depth, int n_tmp, int row_result, int sms,
                           cudaStream_t stream) {
  const int tmp_level = max_depth > 2 ? max_depth - 2 : 1;   // the two upper stack entries are registers
  const size_t smem = static_cast<size_t>(tmp_level + n_tmp) * kV * kThreads * sizeof(float);
  if (smem > 200 * 1024) return ASC_ERR_TOO_LARGE;
  if (smem + 1024 > 48 * 1024) {     // dynamic plus the kernel's few static words: beyond the default limit
    static aschost::PerDevice attr_set;
    int dev = 0;
    ASC_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_set.get(dev)) {
      ASC_CUDA_TRY(cudaFuncSetAttribute(row_program_kernel<kV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      attr_set.set(dev, 1);
    }
  }
  int resident = 0;
  ASC_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, row_program_kernel<kV>, kThreads, smem));
  if (resident < 1) resident = 1;
  int64_t ctas = static_cast<int64_t>(sms) * resident * 4;   // four waves of resident CTAs; CTAs stride over the rows
  if (ctas > rows) ctas = rows;
  row_program_kernel<kV><<<static_cast<unsigned>(ctas), kThreads, smem, stream>>>(prog, static_cast<uint32_t>(rows),
                                                                                   row_result, tmp_level);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

// Validates a program on the host (opcodes, operand indices, stack depth) and copies it, with the input
// pointers and types, into the launch argument.  Row reductions are legal only where the caller says so.
int32_t fill_program(const int32_t* ops, const int32_t* args, int n_ops, const void* const* inputs,
                     const int32_t* input_types, int n_inputs, bool row_ops_allowed, EltProgram& prog, int& max_depth,
                     int* n_tmp = nullptr) {
  prog.n_ops = n_ops;
  prog.n_inputs = n_inputs;
  int depth = 0;
  max_depth = 0;
  uint32_t tmp_set = 0;   // slots a TEE has written so far
  for (int k = 0; k < n_ops; ++k) {
    const int op = ops[k] & 0xff;
    const bool imm = (ops[k] & OP_IMM) != 0;
    if (ops[k] < 0 || (ops[k] & ~(0xff | OP_IMM)) != 0 || op >= OP_COUNT) return ASC_ERR_INVALID_ARG;
    if (imm && !is_binary_op(op)) return ASC_ERR_INVALID_ARG;
    if ((is_row_op(op) || op == OP_TEE || op == OP_TMP) && !row_ops_allowed) return ASC_ERR_INVALID_ARG;
    if (op == OP_TEE || op == OP_TMP) {
      if (args[k] < 0 || args[k] >= kMaxTmp) return ASC_ERR_INVALID_ARG;
      if (op == OP_TEE) {
        if (depth < 1) return ASC_ERR_INVALID_ARG;
        tmp_set |= 1u << args[k];
      } else {
        if (((tmp_set >> args[k]) & 1u) == 0) return ASC_ERR_INVALID_ARG;   // read before any write
        ++depth;
      }
    } else if (op == OP_LOAD) {
      if (args[k] < 0 || args[k] >= n_inputs) return ASC_ERR_INVALID_ARG;
      ++depth;
    } else if (op == OP_CONST || op == OP_INDEX) {
      ++depth;
    } else if (is_binary_op(op)) {
      if (depth < (imm ? 1 : 2)) return ASC_ERR_INVALID_ARG;
      if (!imm) --depth;
    } else if (op == OP_WHERE) {
      if (depth < 3) return ASC_ERR_INVALID_ARG;
      depth -= 2;
    } else if (depth < 1) {
      return ASC_ERR_INVALID_ARG;
    }
    if (depth > kStack) return ASC_ERR_TOO_LARGE;
    if (depth > max_depth) max_depth = depth;
    prog.op[k] = ops[k];
    prog.arg[k] = args[k];
  }
  if (depth != 1) return ASC_ERR_INVALID_ARG;
  if (n_tmp != nullptr) {
    *n_tmp = 0;
    for (int t = 0; t < kMaxTmp; ++t)
      if ((tmp_set >> t) & 1u) *n_tmp = t + 1;
  }
  for (int i = 0; i < n_inputs; ++i) {
    const int row_scalar = row_ops_allowed ? (input_types[i] & kRowScalarInput) : 0;
    const int type = input_types[i] & ~row_scalar;
    if (inputs[i] == nullptr || type < 0 || type >= T_COUNT) return ASC_ERR_INVALID_ARG;
    if (reinterpret_cast<uintptr_t>(inputs[i]) % elem_size(type) != 0) return ASC_ERR_MISALIGNED;
    prog.in[i] = inputs[i];
    int loads = 0;
    for (int k = 0; k < n_ops; ++k) loads += (prog.op[k] == OP_LOAD && prog.arg[k] == i) ? 1 : 0;
    prog.in_type[i] = type | row_scalar | (loads > 1 ? kReusedInput : 0);
  }
  return ASC_OK;
}

}  // namespace

extern "C" int32_t asc_cuda_eltwise_program_2d(const int32_t* ops, const int32_t* args, int32_t n_ops,
                                               const void* const* inputs, const int32_t* input_types, int32_t n_inputs,
                                               void* out, int32_t out_type, int64_t rows, int64_t cols,
                                               const int64_t* lds, void* stream) {
  if (rows < 0 || cols < 0 || n_inputs < 0 || n_inputs > kMaxInputs) return ASC_ERR_INVALID_ARG;
  // lds: row pitch of every input, then of the output; NULL: all pitches equal cols (one contiguous range)
  bool strided = false;
  if (lds != nullptr && rows > 1) {
    for (int k = 0; k <= n_inputs; ++k) {
      const bool broadcast = lds[k] == 0 && k < n_inputs;
      if (!broadcast && lds[k] < cols) return ASC_ERR_INVALID_ARG;
      if (lds[k] >= (int64_t{1} << 32)) return ASC_ERR_TOO_LARGE;
      strided = strided || lds[k] != cols;
    }
  }
  if (strided && rows * cols >= (int64_t{1} << 32)) return ASC_ERR_TOO_LARGE;
  const int64_t n = rows * cols;
  if (n < 0 || n_ops <= 0 || n_ops > kMaxOps || n_inputs < 0 || n_inputs > kMaxInputs) return ASC_ERR_INVALID_ARG;
  if (ops == nullptr || args == nullptr || out == nullptr || (n_inputs > 0 && (inputs == nullptr || input_types == nullptr)))
    return ASC_ERR_INVALID_ARG;
  if (out_type < 0 || out_type >= T_COUNT) return ASC_ERR_INVALID_ARG;
  if (n == 0) return ASC_OK;
  EltProgram prog{};
  int max_depth = 0;
  int32_t rc = fill_program(ops, args, n_ops, inputs, input_types, n_inputs, false, prog, max_depth);
  if (rc != ASC_OK) return rc;
  if (reinterpret_cast<uintptr_t>(out) % elem_size(out_type) != 0) return ASC_ERR_MISALIGNED;
  prog.out = out;
  prog.out_type = out_type;
  prog.cols = strided ? static_cast<uint32_t>(cols) : 0u;
  for (int k = 0; k <= n_inputs; ++k) prog.ld[k] = strided ? static_cast<uint32_t>(lds[k]) : 0u;
  int sms = 0;
  rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;
  bool vec = reinterpret_cast<uintptr_t>(out) % (4 * elem_size(out_type)) == 0;
  for (int i = 0; i < n_inputs; ++i) vec = vec && reinterpret_cast<uintptr_t>(inputs[i]) % (4 * elem_size(input_types[i])) == 0;
  if (strided) {
    vec = vec && cols % 4 == 0;   // a quad must not straddle two rows
    for (int k = 0; k <= n_inputs; ++k) vec = vec && lds[k] % 4 == 0;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!vec) return launch_interpreter<1>(prog, n, max_depth, sms, st);
  if (g_use_compiled && !strided) {
    bool launched = false;
    rc = try_compiled<LeakyReluF32>(prog, ops, args, n_ops, n, sms, st, &launched);
    if (rc == ASC_OK) rc = try_compiled<LeakyReluF16>(prog, ops, args, n_ops, n, sms, st, &launched);
    if (rc == ASC_OK) rc = try_compiled<LeakyReluBF16>(prog, ops, args, n_ops, n, sms, st, &launched);
    if (rc == ASC_OK) rc = try_compiled<GeluErf>(prog, ops, args, n_ops, n, sms, st, &launched);
    if (rc == ASC_OK) rc = try_compiled<GeluTanh>(prog, ops, args, n_ops, n, sms, st, &launched);
    if (rc == ASC_OK) rc = try_compiled<Sigmoid>(prog, ops, args, n_ops, n, sms, st, &launched);
    if (rc == ASC_OK) rc = try_compiled<Silu>(prog, ops, args, n_ops, n, sms, st, &launched);
    if (launched || rc != ASC_OK) return rc;
  }
  if (g_use_compiled && n_inputs > 0) {
    if (JitFn fn = find_jit(0, ops, args, input_types, n_ops)) {
      bool oct = !strided && elem_size(prog.out_type) == 2 && reinterpret_cast<uintptr_t>(prog.out) % 16 == 0;
      for (int i = 0; i < prog.n_inputs; ++i)
        oct = oct && elem_size(prog.in_type[i] & 0xff) == 2 && reinterpret_cast<uintptr_t>(prog.in[i]) % 16 == 0;
      const int e = fn(&prog, n, oct ? 1 : 0, sms, st);
      aschost::count_launch();
      if (e != 0) return aschost::record_cuda_error(static_cast<cudaError_t>(e), "launch of a program specialised at first use");
      return ASC_OK;
    }
  }
  // more elements per dispatch amortise the dispatch of long programs (measured: 7 ops 4.2 vs 3.8 TB/s, 13 ops
  // 2.9 vs 2.5 with 16 instead of 8); short ones are memory-bound either way and keep the smaller register set
  const int forced = g_lanes.load(std::memory_order_relaxed);
  const int lanes = forced != 0 ? forced : (n_ops >= 5 ? 16 : 8);
  if (lanes == 4 || n < kThreads * 8) return launch_interpreter<4>(prog, n, max_depth, sms, st);
  if (lanes == 16 && n >= kThreads * 16) return launch_interpreter<16>(prog, n, max_depth, sms, st);
  return launch_interpreter<8>(prog, n, max_depth, sms, st);
}

extern "C" int32_t asc_cuda_eltwise_program(const int32_t* ops, const int32_t* args, int32_t n_ops,
                                            const void* const* inputs, const int32_t* input_types, int32_t n_inputs,
                                            void* out, int32_t out_type, int64_t n, void* stream) {
  return asc_cuda_eltwise_program_2d(ops, args, n_ops, inputs, input_types, n_inputs, out, out_type, 1, n, nullptr,
                                     stream);
}

// tuning hook: bits 0-7 elements per thread and dispatch in the interpreter's aligned path (4, 8 or 16;
// anything else: chosen by program length); bit 8 set: never use a compiled program
extern "C" int32_t asc_cuda_eltwise_set_lanes(int32_t lanes) {
  const int l = lanes & 0xff;
  g_lanes = (l == 4 || l == 8 || l == 16) ? l : 0;
  g_use_compiled = (lanes & 0x100) == 0;
  g_waves = (lanes >> 16) & 0xff;
  return ASC_OK;
}

// A program over the rows of a [rows, cols] window in which ROW_SUM / ROW_MAX / ROW_MIN / ROW_PROD reduce the
// top of the stack over the row.  lds as for the 2-D elementwise call (0: an input row every window row reads);
// row_result != 0: the program's value is uniform along the row and one element per row is stored, at
// out[r * lds[n_inputs]].
extern "C" int32_t asc_cuda_row_program(const int32_t* ops, const int32_t* args, int32_t n_ops,
                                        const void* const* inputs, const int32_t* input_types, int32_t n_inputs,
                                        void* out, int32_t out_type, int64_t rows, int64_t cols, const int64_t* lds,
                                        int32_t row_result, void* stream) {
  if (rows < 0 || cols < 0 || n_inputs < 0 || n_inputs > kMaxInputs || n_ops <= 0 || n_ops > kMaxOps)
    return ASC_ERR_INVALID_ARG;
  if (ops == nullptr || args == nullptr || out == nullptr || (n_inputs > 0 && (inputs == nullptr || input_types == nullptr)))
    return ASC_ERR_INVALID_ARG;
  if (out_type < 0 || out_type >= T_COUNT) return ASC_ERR_INVALID_ARG;
  if (rows >= (int64_t{1} << 32)) return ASC_ERR_TOO_LARGE;
  if (cols > 32 * kThreads) return ASC_ERR_TOO_LARGE;     // a thread holds at most 32 elements of the row
  EltProgram prog{};
  int max_depth = 0;
  int n_tmp = 0;
  int32_t rc = fill_program(ops, args, n_ops, inputs, input_types, n_inputs, true, prog, max_depth, &n_tmp);
  if (rc != ASC_OK) return rc;
  if (reinterpret_cast<uintptr_t>(out) % elem_size(out_type) != 0) return ASC_ERR_MISALIGNED;
  for (int k = 0; k <= n_inputs; ++k) {
    const bool is_out = k == n_inputs;
    int64_t ld = lds != nullptr ? lds[k] : (is_out && row_result ? 1 : cols);
    const int64_t least = is_out ? (row_result ? 1 : cols) : 0;       // an input pitch of 0 is a broadcast row
    const bool row_scalar = !is_out && (input_types[k] & kRowScalarInput) != 0;   // one element per row: any pitch
    if (lds == nullptr && row_scalar) ld = 1;
    if (ld < least || (!is_out && !row_scalar && ld != 0 && ld < cols)) return ASC_ERR_INVALID_ARG;
    if (ld >= (int64_t{1} << 32)) return ASC_ERR_TOO_LARGE;
    prog.ld[k] = static_cast<uint32_t>(ld);
  }
  if (rows == 0 || cols == 0) return ASC_OK;
  prog.out = out;
  prog.out_type = out_type;
  prog.cols = static_cast<uint32_t>(cols);
  int sms = 0;
  rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t per_thread = (cols + kThreads - 1) / kThreads;
  const int rr = row_result != 0 ? 1 : 0;
  if (g_use_compiled) {
    int kv = 1;
    while (kv < per_thread) kv *= 2;
    if (JitFn fn = find_jit(1000 + kv, ops, args, input_types, n_ops)) {
      const int e = fn(&prog, rows, rr, sms, st);
      aschost::count_launch();
      if (e != 0) return aschost::record_cuda_error(static_cast<cudaError_t>(e), "launch of a row program specialised at first use");
      return ASC_OK;
    }
  }
  if (per_thread <= 1) return launch_row_program<1>(prog, rows, max_depth, n_tmp, rr, sms, st);
  if (per_thread <= 2) return launch_row_program<2>(prog, rows, max_depth, n_tmp, rr, sms, st);
  if (per_thread <= 4) return launch_row_program<4>(prog, rows, max_depth, n_tmp, rr, sms, st);
  if (per_thread <= 8) return launch_row_program<8>(prog, rows, max_depth, n_tmp, rr, sms, st);
  if (per_thread <= 16) return launch_row_program<16>(prog, rows, max_depth, n_tmp, rr, sms, st);
  return launch_row_program<32>(prog, rows, max_depth, n_tmp, rr, sms, st);
}

// out[c] = reduce_kind over the rows r of program(r, c) for a [rows, cols] window; kind: 0 sum, 1 max, 2 min,
// 3 product.  lds: row pitch of every input (0: one row that every window row reads); NULL: all pitches equal cols.
namespace {
// ---- executor 5: an elementwise program reduced along the columns of its window ----
// out[c] = reduce over r of program(r, c) for a [rows, cols] window: a thread owns a column and walks its rows,
// evaluating the program per element in the interpreter (consecutive threads read consecutive columns, so every
// access of a warp is one contiguous run) and combining as it goes.  Made for the tile-sized windows of
// asc2.reduce_*(expression, 0); the grid covers the columns, not the rows.
__global__ void __launch_bounds__(kThreads) col_program_kernel(const __grid_constant__ EltProgram prog, uint32_t rows,
                                                               int row_op) {
  extern __shared__ __align__(16) float stack_mem[];
  const uint32_t cols = prog.cols;
  for (uint32_t c = blockIdx.x * kThreads + threadIdx.x; c < cols; c += gridDim.x * kThreads) {
    float acc = row_identity(row_op);
    for (uint32_t r = 0; r < rows; ++r) {
      float v[1];
      Interpreter::eval<1>(prog, static_cast<int64_t>(r) * cols + c, stack_mem, v);
      acc = row_combine(row_op, acc, v[0]);
    }
    store_elem(prog.out, prog.out_type, c, acc);
  }
}
}  // namespace

extern "C" int32_t asc_cuda_col_program(const int32_t* ops, const int32_t* args, int32_t n_ops, const void* const* inputs,
                                        const int32_t* input_types, int32_t n_inputs, void* out, int32_t out_type,
                                        int64_t rows, int64_t cols, const int64_t* lds, int32_t kind, void* stream) {
  if (rows < 0 || cols < 0 || n_inputs < 0 || n_inputs > kMaxInputs || n_ops <= 0 || n_ops > kMaxOps)
    return ASC_ERR_INVALID_ARG;
  if (ops == nullptr || args == nullptr || out == nullptr || (n_inputs > 0 && (inputs == nullptr || input_types == nullptr)))
    return ASC_ERR_INVALID_ARG;
  if (out_type < 0 || out_type >= T_COUNT || kind < 0 || kind > 3) return ASC_ERR_INVALID_ARG;
  if (out_type == T_I32 || out_type == T_I16) return ASC_ERR_UNSUPPORTED;     // the combination runs on fp32 words
  if (rows >= (int64_t{1} << 32) || cols >= (int64_t{1} << 31) || rows * cols >= (int64_t{1} << 32)) return ASC_ERR_TOO_LARGE;
  EltProgram prog{};
  int max_depth = 0;
  int32_t rc = fill_program(ops, args, n_ops, inputs, input_types, n_inputs, false, prog, max_depth);
  if (rc != ASC_OK) return rc;
  if (reinterpret_cast<uintptr_t>(out) % elem_size(out_type) != 0) return ASC_ERR_MISALIGNED;
  for (int k = 0; k < n_inputs; ++k) {
    const int64_t ld = lds != nullptr ? lds[k] : cols;
    if ((ld != 0 && ld < cols) || ld >= (int64_t{1} << 32)) return ASC_ERR_INVALID_ARG;
    prog.ld[k] = static_cast<uint32_t>(ld);
  }
  if (cols == 0) return ASC_OK;
  prog.out = out;
  prog.out_type = out_type;
  prog.cols = static_cast<uint32_t>(cols);
  prog.ld[n_inputs] = static_cast<uint32_t>(cols);
  const int row_op = OP_ROW_SUM + (kind == 0 ? 0 : kind == 1 ? 1 : kind == 2 ? 2 : 3);
  const size_t smem = static_cast<size_t>(max_depth > 1 ? max_depth - 1 : 1) * kThreads * 4 * sizeof(float);
  const int64_t ctas = (cols + kThreads - 1) / kThreads;
  col_program_kernel<<<static_cast<unsigned>(ctas), kThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      prog, static_cast<uint32_t>(rows), row_op);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

// Registers the entry point of a program specialised at first use (see find_jit): `words` are the opcode-list
// words the unit was generated from, `fn` its `asc_jit_run`.  Registering the same list again replaces the entry.
extern "C" int32_t asc_cuda_register_program(int32_t kind, const int32_t* words, int32_t n_words, void* fn) {
  if (words == nullptr || fn == nullptr || n_words <= 0 || n_words > kMaxOps || kind < 0) return ASC_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(g_jit_mutex);
  std::vector<int32_t> w(words, words + n_words);
  for (JitEntry& e : g_jit) {
    if (e.kind == kind && e.words == w) {
      e.fn = reinterpret_cast<JitFn>(fn);
      return ASC_OK;
    }
  }
  g_jit.push_back(JitEntry{kind, std::move(w), reinterpret_cast<JitFn>(fn)});
  return ASC_OK;
}
