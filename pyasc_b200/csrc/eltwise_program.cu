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
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../../include/asc_cuda.h"
#include "host_common.h"

namespace {

enum EltOp : int32_t {
  OP_LOAD = 0,   // push input[arg]
  OP_CONST = 1,  // push the 32-bit word in arg
  OP_ADD = 2, OP_SUB = 3, OP_MUL = 4, OP_DIV = 5, OP_MAX = 6, OP_MIN = 7,
  OP_NEG = 8, OP_ABS = 9, OP_RELU = 10, OP_EXP = 11, OP_EXP2 = 12, OP_LOG = 13, OP_LOG2 = 14, OP_SQRT = 15,
  OP_RSQRT = 16, OP_SIN = 17, OP_COS = 18, OP_TAN = 19, OP_SINH = 20, OP_COSH = 21, OP_TANH = 22, OP_ERF = 23,
  OP_FLOOR = 24, OP_CEIL = 25,
  OP_EQ = 26, OP_NE = 27, OP_GT = 28, OP_GE = 29, OP_LT = 30, OP_LE = 31,  // push 1.0 / 0.0
  OP_WHERE = 32,      // pop b, a, cond -> cond != 0 ? a : b
  OP_ROUND_F16 = 33,  // round the top of the stack through fp16
  OP_ROUND_BF16 = 34,
  // integer forms: the 32-bit stack word holds an int32 (CONST then carries the integer itself)
  OP_IADD = 35, OP_ISUB = 36, OP_IMUL = 37, OP_IMAX = 38, OP_IMIN = 39, OP_ISHL = 40, OP_ISHR = 41,
  OP_IEQ = 42, OP_INE = 43, OP_IGT = 44, OP_IGE = 45, OP_ILT = 46, OP_ILE = 47,  // push 1.0 / 0.0
  OP_INEG = 48, OP_IABS = 49, OP_IRELU = 50,
  OP_CVT_I2F = 51, OP_CVT_F2I = 52,  // int32 <-> fp32 value conversion (round to nearest even / truncate)
  OP_WRAP_I16 = 53,                  // sign-extend the low 16 bits (int16 arithmetic wraps)
  // operands swapped: f(lhs, rhs) = rhs op lhs
  OP_RSUB = 54, OP_RDIV = 55, OP_IRSUB = 56, OP_IRSHL = 57, OP_IRSHR = 58,
  // row programs only: replace the top of the stack by its reduction over the row (fp32 words), so that
  // every element of the row sees the reduced value
  OP_ROW_SUM = 59, OP_ROW_MAX = 60, OP_ROW_MIN = 61, OP_ROW_PROD = 62,
  // row programs only: a value the expression uses more than once is computed once.  TEE copies the top of
  // the stack into temporary slot arg (the stack is unchanged), TMP pushes slot arg.
  OP_TEE = 63, OP_TMP = 64,
  OP_COUNT = 65,
  // flag on a binary opcode: the left operand is the 32-bit word in arg instead of a stack entry, so a
  // scalar operand costs neither a push nor a pop (with the swapped forms either side can be the scalar)
  OP_IMM = 0x100,
};

enum EltType : int32_t { T_F32 = 0, T_F16 = 1, T_BF16 = 2, T_I32 = 3, T_I16 = 4, T_COUNT = 5 };

__host__ __device__ constexpr bool is_row_op(int op) { return op >= OP_ROW_SUM && op <= OP_ROW_PROD; }
constexpr int kMaxTmp = 4;   // temporary slots of a row program

__host__ __device__ constexpr bool is_binary_op(int op) {
  return (op >= OP_ADD && op <= OP_MIN) || (op >= OP_EQ && op <= OP_LE) || (op >= OP_IADD && op <= OP_ILE) ||
         (op >= OP_RSUB && op <= OP_IRSHR);
}

constexpr int kMaxOps = 48;
constexpr int kMaxInputs = 6;
constexpr int kStack = 8;

struct EltProgram {
  int32_t n_ops;
  int32_t n_inputs;
  int32_t op[kMaxOps];
  int32_t arg[kMaxOps];   // input index for OP_LOAD, float bits for OP_CONST
  const void* in[kMaxInputs];
  int32_t in_type[kMaxInputs];
  void* out;
  int32_t out_type;
  // 2-D window: element i of the window is row i / cols, column i % cols; operand k (the inputs, then the
  // output) has a row pitch of ld[k] elements, 0 meaning that every row of the window reads the same row
  // (a broadcast).  cols == 0: the operands are flat arrays (element i is at index i).
  uint32_t cols;
  uint32_t ld[kMaxInputs + 1];
};

__device__ __forceinline__ int64_t element_offset(const EltProgram& prog, int operand, int64_t i) {
  if (prog.cols == 0) return i;
  const uint32_t u = static_cast<uint32_t>(i);
  const uint32_t r = u / prog.cols;
  return static_cast<int64_t>(r) * prog.ld[operand] + (u - r * prog.cols);
}

constexpr int kThreads = 256;
constexpr int kReusedInput = 0x100;  // flag in EltProgram::in_type: the program loads this input more than once
constexpr int kRowScalarInput = 0x200;  // row programs, flag in the caller's input type: one element per row, at row * pitch
constexpr int kQuadStride = kThreads * 4;  // elements between the quads one thread owns inside a CTA tile

// four consecutive elements starting at element index i (i % 4 == 0, base aligned to four elements:
// one 128-bit or 64-bit access)
template <typename T>
__device__ __forceinline__ T load_vec(const T* p, bool reused) {
  // an input the program loads once streams through (evict-first); one it loads again is cached so
  // that the later loads hit in L1
  return reused ? __ldg(p) : __ldcs(p);
}

__device__ __forceinline__ void load_quad(const void* p, int type, bool reused, int64_t i, float* v) {
  if (type == T_F32) {
    const float4 t = load_vec(reinterpret_cast<const float4*>(p) + (i >> 2), reused);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else if (type == T_I32) {
    const int4 t = load_vec(reinterpret_cast<const int4*>(p) + (i >> 2), reused);
    v[0] = __int_as_float(t.x); v[1] = __int_as_float(t.y);
    v[2] = __int_as_float(t.z); v[3] = __int_as_float(t.w);
  } else {
    const uint2 t = load_vec(reinterpret_cast<const uint2*>(p) + (i >> 2), reused);
    if (type == T_I16) {
      v[0] = __int_as_float(static_cast<int>(static_cast<int16_t>(t.x & 0xffffu)));
      v[1] = __int_as_float(static_cast<int>(static_cast<int16_t>(t.x >> 16)));
      v[2] = __int_as_float(static_cast<int>(static_cast<int16_t>(t.y & 0xffffu)));
      v[3] = __int_as_float(static_cast<int>(static_cast<int16_t>(t.y >> 16)));
    } else if (type == T_F16) {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
      v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    } else {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
      v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
  }
}

__device__ __forceinline__ void store_quad(void* p, int type, int64_t i, const float* v) {
  if (type == T_F32) {
    __stcs(reinterpret_cast<float4*>(p) + (i >> 2), make_float4(v[0], v[1], v[2], v[3]));
  } else if (type == T_I32) {
    __stcs(reinterpret_cast<int4*>(p) + (i >> 2),
           make_int4(__float_as_int(v[0]), __float_as_int(v[1]), __float_as_int(v[2]), __float_as_int(v[3])));
  } else {
    uint2 t;
    if (type == T_I16) {
      t.x = (static_cast<uint32_t>(__float_as_int(v[0])) & 0xffffu) | (static_cast<uint32_t>(__float_as_int(v[1])) << 16);
      t.y = (static_cast<uint32_t>(__float_as_int(v[2])) & 0xffffu) | (static_cast<uint32_t>(__float_as_int(v[3])) << 16);
    } else if (type == T_F16) {
      *reinterpret_cast<__half2*>(&t.x) = __floats2half2_rn(v[0], v[1]);
      *reinterpret_cast<__half2*>(&t.y) = __floats2half2_rn(v[2], v[3]);
    } else {
      *reinterpret_cast<__nv_bfloat162*>(&t.x) = __floats2bfloat162_rn(v[0], v[1]);
      *reinterpret_cast<__nv_bfloat162*>(&t.y) = __floats2bfloat162_rn(v[2], v[3]);
    }
    __stcs(reinterpret_cast<uint2*>(p) + (i >> 2), t);
  }
}

// eight consecutive 16-bit elements starting at element index i (i % 8 == 0, base aligned to 16 bytes):
// one 128-bit access.  Used when every operand of a compiled program is a 16-bit type.
__device__ __forceinline__ void load_oct(const void* p, int type, int64_t i, float* v) {
  const uint4 t = __ldcs(reinterpret_cast<const uint4*>(p) + (i >> 3));
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (type == T_I16) {
      v[2 * k] = __int_as_float(static_cast<int>(static_cast<int16_t>(w[k] & 0xffffu)));
      v[2 * k + 1] = __int_as_float(static_cast<int>(static_cast<int16_t>(w[k] >> 16)));
    } else if (type == T_F16) {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
      v[2 * k] = a.x; v[2 * k + 1] = a.y;
    } else {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[k]));
      v[2 * k] = a.x; v[2 * k + 1] = a.y;
    }
  }
}

__device__ __forceinline__ void store_oct(void* p, int type, int64_t i, const float* v) {
  uint32_t w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (type == T_I16) {
      w[k] = (static_cast<uint32_t>(__float_as_int(v[2 * k])) & 0xffffu) | (static_cast<uint32_t>(__float_as_int(v[2 * k + 1])) << 16);
    } else if (type == T_F16) {
      *reinterpret_cast<__half2*>(&w[k]) = __floats2half2_rn(v[2 * k], v[2 * k + 1]);
    } else {
      *reinterpret_cast<__nv_bfloat162*>(&w[k]) = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
    }
  }
  __stcs(reinterpret_cast<uint4*>(p) + (i >> 3), make_uint4(w[0], w[1], w[2], w[3]));
}

// A thread's kV lanes: kV == 1 is the element at i; otherwise kV / 4 quads, the first at i and the
// others kQuadStride elements apart (so that a warp's accesses stay contiguous inside a CTA tile).
template <int kV, bool kLoadedOnce = false>
__device__ __forceinline__ void load_group(const EltProgram& prog, int input, int64_t i, float (&v)[kV]) {
  const void* p = prog.in[input];
  const int typeword = prog.in_type[input];
  const int type = typeword & 0xff;
  if constexpr (kV >= 4) {
    const bool reused = !kLoadedOnce && (typeword & kReusedInput) != 0;
#pragma unroll
    for (int q = 0; q < kV / 4; ++q)
      load_quad(p, type, reused, element_offset(prog, input, i + q * kQuadStride), &v[4 * q]);
  } else {
    i = element_offset(prog, input, i);
    switch (type) {
      case T_F16: v[0] = __half2float(reinterpret_cast<const __half*>(p)[i]); break;
      case T_BF16: v[0] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]); break;
      case T_I32: v[0] = __int_as_float(reinterpret_cast<const int32_t*>(p)[i]); break;
      case T_I16: v[0] = __int_as_float(static_cast<int>(reinterpret_cast<const int16_t*>(p)[i])); break;
      default: v[0] = reinterpret_cast<const float*>(p)[i]; break;
    }
  }
}

template <int kV>
__device__ __forceinline__ void store_group(const EltProgram& prog, int64_t i, const float (&v)[kV]) {
  void* p = prog.out;
  const int type = prog.out_type;
  if constexpr (kV >= 4) {
#pragma unroll
    for (int q = 0; q < kV / 4; ++q) store_quad(p, type, element_offset(prog, prog.n_inputs, i + q * kQuadStride), &v[4 * q]);
  } else {
    i = element_offset(prog, prog.n_inputs, i);
    switch (type) {
      case T_F16: reinterpret_cast<__half*>(p)[i] = __float2half_rn(v[0]); break;
      case T_BF16: reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v[0]); break;
      case T_I32: reinterpret_cast<int32_t*>(p)[i] = __float_as_int(v[0]); break;
      case T_I16: reinterpret_cast<int16_t*>(p)[i] = static_cast<int16_t>(__float_as_int(v[0])); break;
      default: reinterpret_cast<float*>(p)[i] = v[0]; break;
    }
  }
}

// ---- the meaning of every opcode, in one place (both executors below inline these with a constant op) ----
__device__ __forceinline__ float apply_binary(int op, float a, float b) {
  const int x = __float_as_int(a), y = __float_as_int(b);
  const unsigned ux = static_cast<unsigned>(x), uy = static_cast<unsigned>(y);
  switch (op) {
    case OP_ADD: return __fadd_rn(a, b);
    case OP_SUB: return __fsub_rn(a, b);
    case OP_MUL: return __fmul_rn(a, b);
    case OP_DIV: return __fdiv_rn(a, b);
    case OP_MAX: return ascdev::max_nan(a, b);
    case OP_MIN: return ascdev::min_nan(a, b);
    case OP_EQ: return a == b ? 1.f : 0.f;
    case OP_NE: return a != b ? 1.f : 0.f;
    case OP_GT: return a > b ? 1.f : 0.f;
    case OP_GE: return a >= b ? 1.f : 0.f;
    case OP_LT: return a < b ? 1.f : 0.f;
    case OP_LE: return a <= b ? 1.f : 0.f;
    case OP_IADD: return __int_as_float(static_cast<int>(ux + uy));
    case OP_ISUB: return __int_as_float(static_cast<int>(ux - uy));
    case OP_IMUL: return __int_as_float(static_cast<int>(ux * uy));
    case OP_IMAX: return __int_as_float(max(x, y));
    case OP_IMIN: return __int_as_float(min(x, y));
    case OP_ISHL: return __int_as_float(static_cast<int>(ux << (y & 31)));
    case OP_ISHR: return __int_as_float(x >> (y & 31));
    case OP_IEQ: return x == y ? 1.f : 0.f;
    case OP_INE: return x != y ? 1.f : 0.f;
    case OP_IGT: return x > y ? 1.f : 0.f;
    case OP_IGE: return x >= y ? 1.f : 0.f;
    case OP_ILT: return x < y ? 1.f : 0.f;
    case OP_ILE: return x <= y ? 1.f : 0.f;
    case OP_RSUB: return __fsub_rn(b, a);
    case OP_RDIV: return __fdiv_rn(b, a);
    case OP_IRSUB: return __int_as_float(static_cast<int>(uy - ux));
    case OP_IRSHL: return __int_as_float(static_cast<int>(uy << (x & 31)));
    default: return __int_as_float(y >> (x & 31));  // OP_IRSHR
  }
}

__device__ __forceinline__ float apply_unary(int op, float a) {
  const int x = __float_as_int(a);
  switch (op) {
    case OP_NEG: return -a;
    case OP_ABS: return fabsf(a);
    case OP_RELU: return ascdev::max_nan(a, 0.f);
    case OP_EXP: return expf(a);
    case OP_EXP2: return exp2f(a);
    case OP_LOG: return logf(a);
    case OP_LOG2: return log2f(a);
    case OP_SQRT: return sqrtf(a);
    case OP_RSQRT: return rsqrtf(a);
    case OP_SIN: return sinf(a);
    case OP_COS: return cosf(a);
    case OP_TAN: return tanf(a);
    case OP_SINH: return sinhf(a);
    case OP_COSH: return coshf(a);
    case OP_TANH: return tanhf(a);
    case OP_ERF: return erff(a);
    case OP_FLOOR: return floorf(a);
    case OP_CEIL: return ceilf(a);
    case OP_ROUND_F16: return __half2float(__float2half_rn(a));
    case OP_ROUND_BF16: return __bfloat162float(__float2bfloat16_rn(a));
    case OP_INEG: return __int_as_float(static_cast<int>(0u - static_cast<unsigned>(x)));
    case OP_IABS: return __int_as_float(abs(x));
    case OP_IRELU: return __int_as_float(max(x, 0));
    case OP_CVT_I2F: return __int2float_rn(x);
    case OP_CVT_F2I: return __int_as_float(__float2int_rz(a));
    default: return __int_as_float(static_cast<int>(static_cast<int16_t>(x & 0xffff)));  // OP_WRAP_I16
  }
}

// ---- executor 1: the interpreter, for any valid program ----
// The top of the operand stack is a register group; the entries below it live in shared memory, one
// kV-wide slot per thread and stack level (conflict-free 128-bit accesses), indexed by the
// warp-uniform depth.  That keeps the register count low enough for high occupancy, which is what
// hides the latency of the dependent dispatch chain, and it needs no dynamically indexed registers.
template <int kV>
struct StackSlots {
  float* base;  // this thread's first slot of level 0; a level spans kThreads * kV floats
  __device__ __forceinline__ void put(int level, const float (&v)[kV]) const {
    float* p = base + static_cast<size_t>(level) * (kThreads * kV);
    if constexpr (kV >= 4) {
#pragma unroll
      for (int q = 0; q < kV / 4; ++q)
        *reinterpret_cast<float4*>(p + q * kQuadStride) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
      p[0] = v[0];
    }
  }
  __device__ __forceinline__ void get(int level, float (&v)[kV]) const {
    const float* p = base + static_cast<size_t>(level) * (kThreads * kV);
    if constexpr (kV >= 4) {
#pragma unroll
      for (int q = 0; q < kV / 4; ++q) {
        const float4 t = *reinterpret_cast<const float4*>(p + q * kQuadStride);
        v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
      }
    } else {
      v[0] = p[0];
    }
  }
};

struct Interpreter {
  static constexpr int kGroup = 4;  // consecutive elements per thread and memory access in a CTA tile
  // One opcode dispatch (a single jump through the switch table) serves kV lanes.  The host validated
  // opcodes, operand indices and stack depth.
  template <int kV>
  __device__ __forceinline__ static void run(const EltProgram& prog, int64_t i, float* stack_mem) {
    const StackSlots<kV> slots{stack_mem + threadIdx.x * (kV >= 4 ? 4 : 1)};
    float top[kV];
    int depth = 0;  // entries on the stack, the top included
#define ASC_LANES _Pragma("unroll") for (int e = 0; e < kV; ++e)
#define ASC_BIN(CODE)                                                   \
  case CODE: {                                                          \
    float lhs[kV];                                                      \
    if (imm) {                                                          \
      ASC_LANES lhs[e] = __int_as_float(prog.arg[k]);                   \
    } else {                                                            \
      slots.get(depth - 2, lhs);                                        \
      --depth;                                                          \
    }                                                                   \
    ASC_LANES top[e] = apply_binary(CODE, lhs[e], top[e]);              \
  } break;
#define ASC_UN(CODE) \
  case CODE:         \
    ASC_LANES top[e] = apply_unary(CODE, top[e]); \
    break;
#pragma unroll 1
    for (int k = 0; k < prog.n_ops; ++k) {
      const int op = prog.op[k] & 0xff;
      const bool imm = (prog.op[k] & OP_IMM) != 0;
      switch (op) {
        case OP_LOAD:
          if (depth > 0) slots.put(depth - 1, top);
          ++depth;
          load_group<kV>(prog, prog.arg[k], i, top);
          break;
        case OP_CONST:
          if (depth > 0) slots.put(depth - 1, top);
          ++depth;
          ASC_LANES top[e] = __int_as_float(prog.arg[k]);
          break;
        case OP_WHERE: {
          float a[kV], c[kV];
          slots.get(depth - 2, a);
          slots.get(depth - 3, c);
          depth -= 2;
          ASC_LANES top[e] = c[e] != 0.f ? a[e] : top[e];
        } break;
        ASC_BIN(OP_ADD) ASC_BIN(OP_SUB) ASC_BIN(OP_MUL) ASC_BIN(OP_DIV) ASC_BIN(OP_MAX) ASC_BIN(OP_MIN)
        ASC_BIN(OP_EQ) ASC_BIN(OP_NE) ASC_BIN(OP_GT) ASC_BIN(OP_GE) ASC_BIN(OP_LT) ASC_BIN(OP_LE)
        ASC_BIN(OP_IADD) ASC_BIN(OP_ISUB) ASC_BIN(OP_IMUL) ASC_BIN(OP_IMAX) ASC_BIN(OP_IMIN) ASC_BIN(OP_ISHL)
        ASC_BIN(OP_ISHR) ASC_BIN(OP_IEQ) ASC_BIN(OP_INE) ASC_BIN(OP_IGT) ASC_BIN(OP_IGE) ASC_BIN(OP_ILT)
        ASC_BIN(OP_ILE) ASC_BIN(OP_RSUB) ASC_BIN(OP_RDIV) ASC_BIN(OP_IRSUB) ASC_BIN(OP_IRSHL) ASC_BIN(OP_IRSHR)
        ASC_UN(OP_NEG) ASC_UN(OP_ABS) ASC_UN(OP_RELU) ASC_UN(OP_EXP) ASC_UN(OP_EXP2) ASC_UN(OP_LOG) ASC_UN(OP_LOG2)
        ASC_UN(OP_SQRT) ASC_UN(OP_RSQRT) ASC_UN(OP_SIN) ASC_UN(OP_COS) ASC_UN(OP_TAN) ASC_UN(OP_SINH)
        ASC_UN(OP_COSH) ASC_UN(OP_TANH) ASC_UN(OP_ERF) ASC_UN(OP_FLOOR) ASC_UN(OP_CEIL) ASC_UN(OP_ROUND_F16)
        ASC_UN(OP_ROUND_BF16) ASC_UN(OP_INEG) ASC_UN(OP_IABS) ASC_UN(OP_IRELU) ASC_UN(OP_CVT_I2F)
        ASC_UN(OP_CVT_F2I) ASC_UN(OP_WRAP_I16)
        default: break;
      }
    }
#undef ASC_UN
#undef ASC_BIN
#undef ASC_LANES
    store_group<kV>(prog, i, top);
  }
};

// ---- executor 2: the same machine with the opcode sequence known at compile time ----
// For the expressions the asc2 kernel tests and tutorials produce, the op sequence is a template
// argument: every dispatch, stack index and opcode switch folds away and the stack lives in registers,
// so the kernel is as good as one written by hand for that expression.  Immediates and pointers still
// come from the launch's EltProgram.  A LOAD entry carries its input index in bits 16-23; each input is
// read from memory once, up front, and a LOAD becomes a register copy.
template <int... kWords>
struct OpList {
  static constexpr int n = sizeof...(kWords);
  __host__ __device__ static constexpr int at(int k) {
    constexpr int words[] = {kWords...};
    return words[k];
  }
  __host__ __device__ static constexpr int inputs() {  // highest input index a LOAD names, plus one
    constexpr int words[] = {kWords...};
    int m = 0;
    for (int k = 0; k < n; ++k)
      if ((words[k] & 0xff) == OP_LOAD && ((words[k] >> 16) & 0xff) + 1 > m) m = ((words[k] >> 16) & 0xff) + 1;
    return m;
  }
};
__host__ __device__ constexpr int LD(int input) { return OP_LOAD | (input << 16); }

template <class P, int kV, int K, int D, bool kStore>
struct StaticStep {
  __device__ __forceinline__ static void run(const EltProgram& prog, int64_t i, const float (&in)[P::inputs()][kV],
                                             float (&st)[kStack][kV]) {
    if constexpr (K == P::n) {
      static_assert(D == 1, "a program leaves exactly one value");
      if constexpr (kStore) store_group<kV>(prog, i, st[0]);
    } else {
      constexpr int word = P::at(K);
      constexpr int op = word & 0xff;
      constexpr bool imm = (word & OP_IMM) != 0;
      if constexpr (op == OP_LOAD) {
        constexpr int input = (word >> 16) & 0xff;
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D][e] = in[input][e];
        StaticStep<P, kV, K + 1, D + 1, kStore>::run(prog, i, in, st);
      } else if constexpr (op == OP_CONST) {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D][e] = __int_as_float(prog.arg[K]);
        StaticStep<P, kV, K + 1, D + 1, kStore>::run(prog, i, in, st);
      } else if constexpr (is_binary_op(op) && imm) {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D - 1][e] = apply_binary(op, __int_as_float(prog.arg[K]), st[D - 1][e]);
        StaticStep<P, kV, K + 1, D, kStore>::run(prog, i, in, st);
      } else if constexpr (is_binary_op(op)) {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D - 2][e] = apply_binary(op, st[D - 2][e], st[D - 1][e]);
        StaticStep<P, kV, K + 1, D - 1, kStore>::run(prog, i, in, st);
      } else if constexpr (op == OP_WHERE) {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D - 3][e] = st[D - 3][e] != 0.f ? st[D - 2][e] : st[D - 1][e];
        StaticStep<P, kV, K + 1, D - 2, kStore>::run(prog, i, in, st);
      } else {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D - 1][e] = apply_unary(op, st[D - 1][e]);
        StaticStep<P, kV, K + 1, D, kStore>::run(prog, i, in, st);
      }
    }
  }
};

// kOct: every operand is a 16-bit type with 16-byte aligned pointers; inside a CTA tile a thread then owns
// groups of eight consecutive elements (one 128-bit access each) instead of quads.
template <class P, bool kOct = false>
struct Compiled {
  static constexpr int kGroup = kOct ? 8 : 4;
  template <int kV>
  __device__ __forceinline__ static void run(const EltProgram& prog, int64_t i, float*) {
    float in[P::inputs()][kV];  // every input is read from memory exactly once
    float st[kStack][kV];
    if constexpr (kOct && kV >= 8) {
#pragma unroll
      for (int j = 0; j < P::inputs(); ++j) {
#pragma unroll
        for (int o = 0; o < kV / 8; ++o) load_oct(prog.in[j], prog.in_type[j] & 0xff, i + o * (kThreads * 8), &in[j][8 * o]);
      }
      StaticStep<P, kV, 0, 0, false>::run(prog, i, in, st);
#pragma unroll
      for (int o = 0; o < kV / 8; ++o) store_oct(prog.out, prog.out_type, i + o * (kThreads * 8), &st[0][8 * o]);
    } else {
#pragma unroll
      for (int j = 0; j < P::inputs(); ++j) load_group<kV, true>(prog, j, i, in[j]);
      StaticStep<P, kV, 0, 0, true>::run(prog, i, in, st);
    }
  }
};

// kLanes == 1: some pointer is not aligned to four elements, every element goes through the scalar
// path.  Otherwise a CTA walks tiles of kThreads * kLanes elements (kLanes per thread at a time), then
// the remaining quads, then the scalar tail.
template <class Exec, int kLanes>
__global__ void __launch_bounds__(kThreads) eltwise_program_kernel(const __grid_constant__ EltProgram prog, int64_t n) {
  extern __shared__ __align__(16) float stack_mem[];  // interpreter: (max depth - 1) levels x kThreads x kLanes floats
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  int64_t done = 0;
  if constexpr (kLanes >= 4) {
    if constexpr (kLanes > 4) {
      constexpr int64_t kTile = static_cast<int64_t>(kThreads) * kLanes;
      const int64_t tiles = n / kTile;
      for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x)
        Exec::template run<kLanes>(prog, t * kTile + threadIdx.x * Exec::kGroup, stack_mem);
      done = tiles * kTile;
    }
    const int64_t quads = (n - done) >> 2;
    for (int64_t g = tid; g < quads; g += stride) Exec::template run<4>(prog, done + (g << 2), stack_mem);
    done += quads << 2;
  }
  for (int64_t i = done + tid; i < n; i += stride) Exec::template run<1>(prog, i, stack_mem);
}

std::atomic<int> g_lanes{0};            // interpreter: elements per thread and dispatch on the aligned path (4, 8, 16; 0: by program length)
std::atomic<bool> g_use_compiled{true};  // tuning hook can force the interpreter for every program

template <class Exec, int kLanes>
int32_t launch_program(const EltProgram& prog, int64_t n, size_t smem, int sms, cudaStream_t stream) {
  if (smem > 48 * 1024) {
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
  const int64_t cap = static_cast<int64_t>(sms) * resident * 4;  // four waves of resident CTAs; CTAs stride beyond
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


// ---- executor 3: programs with row reductions ----
// One CTA evaluates one row of the window at a time; thread t owns columns t, t + 256, ... (kV of them), so
// the loads and stores of consecutive threads are consecutive.  The top of the stack is in registers, lower
// levels in shared memory ([level][lane][thread]: conflict-free).  A ROW_* opcode reduces the thread's lanes,
// then the CTA (shuffles + one exchange through shared memory), and every lane of the top takes the result:
// the reduced value is from then on an ordinary operand, which is how `x - max(x)`, `x / sum(x)` or a
// variance are one pass over the row.  No scratch memory: a row never leaves the SM between its load and
// its store.
__device__ __forceinline__ float load_elem(const void* p, int type, int64_t i) {
  switch (type) {
    case T_F16: return __half2float(reinterpret_cast<const __half*>(p)[i]);
    case T_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    case T_I32: return __int_as_float(reinterpret_cast<const int32_t*>(p)[i]);
    case T_I16: return __int_as_float(static_cast<int>(reinterpret_cast<const int16_t*>(p)[i]));
    default: return reinterpret_cast<const float*>(p)[i];
  }
}
__device__ __forceinline__ void store_elem(void* p, int type, int64_t i, float v) {
  switch (type) {
    case T_F16: reinterpret_cast<__half*>(p)[i] = __float2half_rn(v); break;
    case T_BF16: reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); break;
    case T_I32: reinterpret_cast<int32_t*>(p)[i] = __float_as_int(v); break;
    case T_I16: reinterpret_cast<int16_t*>(p)[i] = static_cast<int16_t>(__float_as_int(v)); break;
    default: reinterpret_cast<float*>(p)[i] = v; break;
  }
}

__device__ __forceinline__ float row_identity(int op) {
  return op == OP_ROW_SUM ? 0.f : op == OP_ROW_PROD ? 1.f : op == OP_ROW_MAX ? -INFINITY : INFINITY;
}
__device__ __forceinline__ float row_combine(int op, float a, float b) {
  return op == OP_ROW_SUM ? __fadd_rn(a, b) : op == OP_ROW_PROD ? __fmul_rn(a, b) : op == OP_ROW_MAX ? ascdev::max_nan(a, b) : ascdev::min_nan(a, b);
}

__device__ __forceinline__ int16_t word_to_i16(float v) { return static_cast<int16_t>(__float_as_int(v)); }

// The lanes of one thread for one operand: element c = thread + e * 256 of row `base`.  The element type is
// resolved once per operand, and a row that fills every lane skips the bounds checks.
template <int kV>
__device__ __forceinline__ void row_load(const void* p, int type, int64_t base, uint32_t cols, bool full, float (&v)[kV]) {
#define ASC_ROW_LOAD(T, CONV)                                                         \
  {                                                                                   \
    const T* q = reinterpret_cast<const T*>(p) + base + threadIdx.x;                  \
    if (full) {                                                                       \
      _Pragma("unroll") for (int e = 0; e < kV; ++e) v[e] = CONV(q[e * kThreads]);    \
    } else {                                                                          \
      _Pragma("unroll") for (int e = 0; e < kV; ++e)                                  \
        v[e] = threadIdx.x + e * kThreads < cols ? CONV(q[e * kThreads]) : 0.f;       \
    }                                                                                 \
  }
  switch (type) {
    case T_F16: ASC_ROW_LOAD(__half, __half2float) break;
    case T_BF16: ASC_ROW_LOAD(__nv_bfloat16, __bfloat162float) break;
    case T_I32: ASC_ROW_LOAD(int32_t, __int_as_float) break;
    case T_I16: ASC_ROW_LOAD(int16_t, __int_as_float) break;
    default: ASC_ROW_LOAD(float, ) break;
  }
#undef ASC_ROW_LOAD
}

template <int kV>
__device__ __forceinline__ void row_store(void* p, int type, int64_t base, uint32_t cols, bool full, const float (&v)[kV]) {
#define ASC_ROW_STORE(T, CONV)                                                          \
  {                                                                                     \
    T* q = reinterpret_cast<T*>(p) + base + threadIdx.x;                                \
    _Pragma("unroll") for (int e = 0; e < kV; ++e)                                      \
      if (full || threadIdx.x + e * kThreads < cols) q[e * kThreads] = CONV(v[e]);      \
  }
  switch (type) {
    case T_F16: ASC_ROW_STORE(__half, __float2half_rn) break;
    case T_BF16: ASC_ROW_STORE(__nv_bfloat16, __float2bfloat16_rn) break;
    case T_I32: ASC_ROW_STORE(int32_t, __float_as_int) break;
    case T_I16: ASC_ROW_STORE(int16_t, word_to_i16) break;
    default: ASC_ROW_STORE(float, ) break;
  }
#undef ASC_ROW_STORE
}

template <int kV>
__global__ void __launch_bounds__(kThreads) row_program_kernel(const __grid_constant__ EltProgram prog, uint32_t rows,
                                                               int row_result, int tmp_level) {
  extern __shared__ float stack_mem[];
  __shared__ float red[kThreads / 32];
  float* const slots = stack_mem + threadIdx.x;
  const uint32_t cols = prog.cols;
  const bool full = cols == kV * kThreads;
  // The two upper stack entries (`top`, and `nos` below it) are registers; only entries below them live in
  // shared memory: entry d (0 = bottom) of a stack of `depth` entries is at level d for d < depth - 2.  The
  // expression compiler orders operands so that most programs never go deeper than two.
#define ASC_LANES _Pragma("unroll") for (int e = 0; e < kV; ++e)
#define ASC_PUT(LEVEL, SRC) ASC_LANES slots[((LEVEL) * kV + e) * kThreads] = SRC[e];
#define ASC_GET(LEVEL, DST) ASC_LANES DST[e] = slots[((LEVEL) * kV + e) * kThreads];
  // top_u / nos_u: every lane of the entry holds the same value (a constant, a row reduction, or a function of
  // those).  Unary operations and operations with an immediate then run once instead of once per lane, which
  // is what keeps `sum / n` and `rsqrt(var + eps)` (IEEE division, square root) off the per-element path.
#define ASC_PUSH(UNIFORM)                          \
  {                                                \
    if (depth >= 2) { ASC_PUT(depth - 2, nos) }    \
    if (depth >= 1) {                              \
      ASC_LANES nos[e] = top[e];                   \
      nos_u = top_u;                               \
    }                                              \
    top_u = UNIFORM;                               \
    ++depth;                                       \
  }
#define ASC_REFILL()                              \
  if (depth >= 2) {                               \
    ASC_GET(depth - 2, nos)                       \
    nos_u = false;                                \
  }
#define ASC_BIN(CODE)                                               \
  case CODE: {                                                      \
    if (imm) {                                                      \
      const float w = __int_as_float(prog.arg[k]);                  \
      if (top_u) {                                                  \
        const float t = apply_binary(CODE, w, top[0]);              \
        ASC_LANES top[e] = t;                                       \
      } else {                                                      \
        ASC_LANES top[e] = apply_binary(CODE, w, top[e]);           \
      }                                                             \
    } else {                                                        \
      ASC_LANES top[e] = apply_binary(CODE, nos[e], top[e]);        \
      top_u = top_u && nos_u;                                       \
      --depth;                                                      \
      ASC_REFILL()                                                  \
    }                                                               \
  } break;
#define ASC_UN(CODE)                                \
  case CODE:                                        \
    if (top_u) {                                    \
      const float t = apply_unary(CODE, top[0]);    \
      ASC_LANES top[e] = t;                         \
    } else {                                        \
      ASC_LANES top[e] = apply_unary(CODE, top[e]); \
    }                                               \
    break;
#define ASC_ROW(CODE)                                                                              \
  case CODE: {                                                                                     \
    float v = row_identity(CODE);                                                                  \
    if (full) {                                                                                    \
      ASC_LANES v = row_combine(CODE, v, top[e]);                                                  \
    } else {                                                                                       \
      ASC_LANES if (threadIdx.x + e * kThreads < cols) v = row_combine(CODE, v, top[e]);           \
    }                                                                                              \
    _Pragma("unroll") for (int o = 16; o > 0; o >>= 1) v = row_combine(CODE, v, __shfl_xor_sync(0xffffffffu, v, o)); \
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;                                        \
    __syncthreads();                                                                               \
    v = red[0];                                                                                    \
    _Pragma("unroll") for (int w = 1; w < kThreads / 32; ++w) v = row_combine(CODE, v, red[w]);    \
    __syncthreads();                                                                               \
    ASC_LANES top[e] = v;                                                                          \
    top_u = true;                                                                                  \
  } break;
  for (uint32_t r = blockIdx.x; r < rows; r += gridDim.x) {
    float top[kV], nos[kV];
    bool top_u = false, nos_u = false;
    int depth = 0;
#pragma unroll 1
    for (int k = 0; k < prog.n_ops; ++k) {
      const int op = prog.op[k] & 0xff;
      const bool imm = (prog.op[k] & OP_IMM) != 0;
      switch (op) {
        case OP_LOAD: {
          const int input = prog.arg[k];
          if (prog.in_type[input] & kRowScalarInput) {
            ASC_PUSH(true)
            const float v = load_elem(prog.in[input], prog.in_type[input] & 0xff, static_cast<int64_t>(r) * prog.ld[input]);
            ASC_LANES top[e] = v;
          } else {
            ASC_PUSH(false)
            row_load<kV>(prog.in[input], prog.in_type[input] & 0xff, static_cast<int64_t>(r) * prog.ld[input], cols, full, top);
          }
        } break;
        case OP_CONST:
          ASC_PUSH(true)
          ASC_LANES top[e] = __int_as_float(prog.arg[k]);
          break;
        case OP_WHERE: {
          float c[kV];
          ASC_GET(depth - 3, c)
          ASC_LANES top[e] = c[e] != 0.f ? nos[e] : top[e];
          top_u = false;
          depth -= 2;
          ASC_REFILL()
        } break;
        ASC_BIN(OP_ADD) ASC_BIN(OP_SUB) ASC_BIN(OP_MUL) ASC_BIN(OP_DIV) ASC_BIN(OP_MAX) ASC_BIN(OP_MIN)
        ASC_BIN(OP_EQ) ASC_BIN(OP_NE) ASC_BIN(OP_GT) ASC_BIN(OP_GE) ASC_BIN(OP_LT) ASC_BIN(OP_LE)
        ASC_BIN(OP_IADD) ASC_BIN(OP_ISUB) ASC_BIN(OP_IMUL) ASC_BIN(OP_IMAX) ASC_BIN(OP_IMIN) ASC_BIN(OP_ISHL)
        ASC_BIN(OP_ISHR) ASC_BIN(OP_IEQ) ASC_BIN(OP_INE) ASC_BIN(OP_IGT) ASC_BIN(OP_IGE) ASC_BIN(OP_ILT)
        ASC_BIN(OP_ILE) ASC_BIN(OP_RSUB) ASC_BIN(OP_RDIV) ASC_BIN(OP_IRSUB) ASC_BIN(OP_IRSHL) ASC_BIN(OP_IRSHR)
        ASC_UN(OP_NEG) ASC_UN(OP_ABS) ASC_UN(OP_RELU) ASC_UN(OP_EXP) ASC_UN(OP_EXP2) ASC_UN(OP_LOG) ASC_UN(OP_LOG2)
        ASC_UN(OP_SQRT) ASC_UN(OP_RSQRT) ASC_UN(OP_SIN) ASC_UN(OP_COS) ASC_UN(OP_TAN) ASC_UN(OP_SINH)
        ASC_UN(OP_COSH) ASC_UN(OP_TANH) ASC_UN(OP_ERF) ASC_UN(OP_FLOOR) ASC_UN(OP_CEIL) ASC_UN(OP_ROUND_F16)
        ASC_UN(OP_ROUND_BF16) ASC_UN(OP_INEG) ASC_UN(OP_IABS) ASC_UN(OP_IRELU) ASC_UN(OP_CVT_I2F)
        ASC_UN(OP_CVT_F2I) ASC_UN(OP_WRAP_I16)
        ASC_ROW(OP_ROW_SUM) ASC_ROW(OP_ROW_MAX) ASC_ROW(OP_ROW_MIN) ASC_ROW(OP_ROW_PROD)
        case OP_TEE: {   // temporaries lie above the stack levels in shared memory
          ASC_PUT(tmp_level + prog.arg[k], top)
        } break;
        case OP_TMP:
          ASC_PUSH(false)
          ASC_GET(tmp_level + prog.arg[k], top)
          break;
        default: break;
      }
    }
    const int64_t out_base = static_cast<int64_t>(r) * prog.ld[prog.n_inputs];
    if (row_result) {
      // the program ends in a value that is the same for the whole row: one element per row is stored
      if (threadIdx.x == 0) store_elem(prog.out, prog.out_type, out_base, top[0]);
    } else {
      row_store<kV>(prog.out, prog.out_type, out_base, cols, full, top);
    }
  }
#undef ASC_ROW
#undef ASC_UN
#undef ASC_BIN
#undef ASC_REFILL
#undef ASC_PUSH
#undef ASC_GET
#undef ASC_PUT
#undef ASC_LANES
}

template <int kV>
int32_t launch_row_program(const EltProgram& prog, int64_t rows, int max_depth, int n_tmp, int row_result, int sms,
                           cudaStream_t stream) {
  const int tmp_level = max_depth > 2 ? max_depth - 2 : 1;   // the two upper stack entries are registers
  const size_t smem = static_cast<size_t>(tmp_level + n_tmp) * kV * kThreads * sizeof(float);
  if (smem > 200 * 1024) return ASC_ERR_TOO_LARGE;
  if (smem > 48 * 1024) {
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
    } else if (op == OP_CONST) {
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
  if (per_thread <= 1) return launch_row_program<1>(prog, rows, max_depth, n_tmp, rr, sms, st);
  if (per_thread <= 2) return launch_row_program<2>(prog, rows, max_depth, n_tmp, rr, sms, st);
  if (per_thread <= 4) return launch_row_program<4>(prog, rows, max_depth, n_tmp, rr, sms, st);
  if (per_thread <= 8) return launch_row_program<8>(prog, rows, max_depth, n_tmp, rr, sms, st);
  if (per_thread <= 16) return launch_row_program<16>(prog, rows, max_depth, n_tmp, rr, sms, st);
  return launch_row_program<32>(prog, rows, max_depth, n_tmp, rr, sms, st);
}
