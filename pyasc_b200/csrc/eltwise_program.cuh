// Device side of the generic elementwise and row-program kernels: opcodes, the launch argument, typed loads and
// stores, the meaning of every opcode, and the three executors (interpreter, compile-time specialised program,
// row programs).  Included by eltwise_program.cu, which builds the kernels every installation has, and by the
// one-line translation units generated at first use of a new expression, which instantiate the specialised
// executors for that expression's opcode list.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>


#include "common.cuh"

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
  // push the element's row-major index inside the window of the call as an int32 word (asc2.mask(count=...) compares
  // it with the count)
  OP_INDEX = 65,
  OP_COUNT = 66,
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

// Element index of lane e of the thread whose first element is i (the layouts of load_group / load_oct).
template <int kV, bool kOct>
__device__ __forceinline__ int64_t lane_index(int64_t i, int e) {
  if (kV < 4) return i;
  if (kOct && kV >= 8) return i + (e >> 3) * (kThreads * 8) + (e & 7);
  return i + (e >> 2) * kQuadStride + (e & 3);
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
    float top[kV];
    eval<kV>(prog, i, stack_mem, top);
    store_group<kV>(prog, i, top);
  }
  // The program's value for the kV lanes of element index i, without storing it.
  template <int kV>
  __device__ __forceinline__ static void eval(const EltProgram& prog, int64_t i, float* stack_mem, float (&top)[kV]) {
    const StackSlots<kV> slots{stack_mem + threadIdx.x * (kV >= 4 ? 4 : 1)};
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
        case OP_INDEX:
          if (depth > 0) slots.put(depth - 1, top);
          ++depth;
          ASC_LANES top[e] = __int_as_float(static_cast<int>(lane_index<kV, false>(i, e)));
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

template <class P, int kV, int K, int D, bool kStore, bool kOct = false>
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
        StaticStep<P, kV, K + 1, D + 1, kStore, kOct>::run(prog, i, in, st);
      } else if constexpr (op == OP_CONST) {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D][e] = __int_as_float(prog.arg[K]);
        StaticStep<P, kV, K + 1, D + 1, kStore, kOct>::run(prog, i, in, st);
      } else if constexpr (op == OP_INDEX) {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D][e] = __int_as_float(static_cast<int>(lane_index<kV, kOct>(i, e)));
        StaticStep<P, kV, K + 1, D + 1, kStore, kOct>::run(prog, i, in, st);
      } else if constexpr (is_binary_op(op) && imm) {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D - 1][e] = apply_binary(op, __int_as_float(prog.arg[K]), st[D - 1][e]);
        StaticStep<P, kV, K + 1, D, kStore, kOct>::run(prog, i, in, st);
      } else if constexpr (is_binary_op(op)) {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D - 2][e] = apply_binary(op, st[D - 2][e], st[D - 1][e]);
        StaticStep<P, kV, K + 1, D - 1, kStore, kOct>::run(prog, i, in, st);
      } else if constexpr (op == OP_WHERE) {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D - 3][e] = st[D - 3][e] != 0.f ? st[D - 2][e] : st[D - 1][e];
        StaticStep<P, kV, K + 1, D - 2, kStore, kOct>::run(prog, i, in, st);
      } else {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D - 1][e] = apply_unary(op, st[D - 1][e]);
        StaticStep<P, kV, K + 1, D, kStore, kOct>::run(prog, i, in, st);
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
      StaticStep<P, kV, 0, 0, false, true>::run(prog, i, in, st);
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

// ---- executor 3: programs with row reductions ----
// One CTA evaluates one row of the window at a time; thread t owns kV columns of it (row_col: t, t + 256, ... for short
// rows, quads of consecutive columns for long ones), so the loads and stores of consecutive threads are consecutive.  The top of the stack is in registers, lower
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

// Which column of the row lane e of this thread holds.  Rows of up to 512 columns: thread + e * 256.  Longer rows:
// quads of consecutive columns, 4 * thread + (e / 4) * 1024 + e % 4, so that a thread's accesses are 128-bit (64-bit
// for 16-bit elements) wherever the operand's row start is aligned for them; the mapping itself does not depend on
// alignment, so neither does the order in which a row is summed.
template <int kV>
__device__ __forceinline__ uint32_t row_col(int e) {
  if constexpr (kV >= 4) return 4u * threadIdx.x + static_cast<uint32_t>(e >> 2) * (4u * kThreads) + static_cast<uint32_t>(e & 3);
  return threadIdx.x + static_cast<uint32_t>(e) * kThreads;
}

template <typename T>
struct Quad;                       // four consecutive elements as one memory access
template <>
struct Quad<float> { using type = float4; };
template <>
struct Quad<int32_t> { using type = int4; };
template <>
struct Quad<__half> { using type = uint2; };
template <>
struct Quad<__nv_bfloat16> { using type = uint2; };
template <>
struct Quad<int16_t> { using type = uint2; };

// The lanes of one thread for one operand: columns row_col(e) of the row that starts at element `base`.  The element
// type is resolved once per operand, and a row that fills every lane skips the bounds checks.
template <int kV>
__device__ __forceinline__ void row_load(const void* p, int type, int64_t base, uint32_t cols, bool full, float (&v)[kV]) {
#define ASC_ROW_LOAD(T, CONV)                                                                         \
  {                                                                                                   \
    const T* row = reinterpret_cast<const T*>(p) + base;                                              \
    if constexpr (kV >= 4) {                                                                          \
      using Q = typename Quad<T>::type;                                                               \
      const bool vec = (reinterpret_cast<uintptr_t>(row) & (sizeof(Q) - 1)) == 0;                     \
      _Pragma("unroll") for (int g = 0; g < kV / 4; ++g) {                                            \
        const uint32_t c0 = row_col<kV>(4 * g);                                                       \
        if (vec && (full || c0 + 3 < cols)) {                                                         \
          const Q quad = *reinterpret_cast<const Q*>(row + c0);                                       \
          const T* t4 = reinterpret_cast<const T*>(&quad);                                            \
          _Pragma("unroll") for (int i = 0; i < 4; ++i) v[4 * g + i] = CONV(t4[i]);                   \
        } else {                                                                                      \
          _Pragma("unroll") for (int i = 0; i < 4; ++i)                                               \
            v[4 * g + i] = (full || c0 + i < cols) ? CONV(row[c0 + i]) : 0.f;                         \
        }                                                                                             \
      }                                                                                               \
    } else {                                                                                          \
      _Pragma("unroll") for (int e = 0; e < kV; ++e)                                                  \
        v[e] = (full || row_col<kV>(e) < cols) ? CONV(row[row_col<kV>(e)]) : 0.f;                     \
    }                                                                                                 \
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
#define ASC_ROW_STORE(T, CONV)                                                                        \
  {                                                                                                   \
    T* row = reinterpret_cast<T*>(p) + base;                                                          \
    if constexpr (kV >= 4) {                                                                          \
      using Q = typename Quad<T>::type;                                                               \
      const bool vec = (reinterpret_cast<uintptr_t>(row) & (sizeof(Q) - 1)) == 0;                     \
      _Pragma("unroll") for (int g = 0; g < kV / 4; ++g) {                                            \
        const uint32_t c0 = row_col<kV>(4 * g);                                                       \
        if (vec && (full || c0 + 3 < cols)) {                                                         \
          Q quad;                                                                                     \
          T* t4 = reinterpret_cast<T*>(&quad);                                                        \
          _Pragma("unroll") for (int i = 0; i < 4; ++i) t4[i] = CONV(v[4 * g + i]);                   \
          *reinterpret_cast<Q*>(row + c0) = quad;                                                     \
        } else {                                                                                      \
          _Pragma("unroll") for (int i = 0; i < 4; ++i)                                               \
            if (full || c0 + i < cols) row[c0 + i] = CONV(v[4 * g + i]);                              \
        }                                                                                             \
      }                                                                                               \
    } else {                                                                                          \
      _Pragma("unroll") for (int e = 0; e < kV; ++e)                                                  \
        if (full || row_col<kV>(e) < cols) row[row_col<kV>(e)] = CONV(v[e]);                          \
    }                                                                                                 \
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
      ASC_LANES if (row_col<kV>(e) < cols) v = row_combine(CODE, v, top[e]);                     \
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
        case OP_INDEX:
          ASC_PUSH(false)
          ASC_LANES top[e] = __int_as_float(static_cast<int>(r * cols + row_col<kV>(e)));
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
// ---- executor 4: a row program whose opcode list is known at compile time ----
// The row-program machine of row_program_kernel with every dispatch, stack index and uniformity test folded at
// compile time: the stack and the temporaries are registers, values that are the same along the row (constants,
// reductions, one-element-per-row inputs and functions of them) are evaluated once per row, and the arithmetic is
// the interpreter's own (apply_binary / apply_unary, the same reduction order), so results are bit-identical.
// Word layout of the opcode list: bits 0-8 the opcode (with OP_IMM), bits 16-23 the input index of a LOAD or the
// slot of a TEE / TMP, bit 24 on a LOAD: the input holds one element per row.  U / TU: bit d set = stack entry d /
// temporary d is uniform along the row.
constexpr int kRowScalarWord = 1 << 24;

template <class P, int kV, int K, int D, unsigned U, unsigned TU>
struct RowStep {
  __device__ __forceinline__ static void run(const EltProgram& prog, uint32_t r, uint32_t cols, bool full, int row_result,
                                             float (&st)[kStack][kV], float (&tmp)[kMaxTmp][kV], float* red) {
    if constexpr (K == P::n) {
      static_assert(D == 1, "a program leaves exactly one value");
      const int64_t out_base = static_cast<int64_t>(r) * prog.ld[prog.n_inputs];
      if (row_result) {
        if (threadIdx.x == 0) store_elem(prog.out, prog.out_type, out_base, st[0][0]);
      } else {
        row_store<kV>(prog.out, prog.out_type, out_base, cols, full, st[0]);
      }
    } else {
      constexpr int word = P::at(K);
      constexpr int op = word & 0xff;
      constexpr bool imm = (word & OP_IMM) != 0;
      constexpr int sub = (word >> 16) & 0xff;
      constexpr unsigned top_bit = D > 0 ? 1u << (D - 1) : 0u;
      constexpr bool top_u = D > 0 && (U & top_bit) != 0;
      if constexpr (op == OP_LOAD) {
        if constexpr ((word & kRowScalarWord) != 0) {
          const float v = load_elem(prog.in[sub], prog.in_type[sub] & 0xff, static_cast<int64_t>(r) * prog.ld[sub]);
#pragma unroll
          for (int e = 0; e < kV; ++e) st[D][e] = v;
          RowStep<P, kV, K + 1, D + 1, U | (1u << D), TU>::run(prog, r, cols, full, row_result, st, tmp, red);
        } else {
          row_load<kV>(prog.in[sub], prog.in_type[sub] & 0xff, static_cast<int64_t>(r) * prog.ld[sub], cols, full, st[D]);
          RowStep<P, kV, K + 1, D + 1, U & ~(1u << D), TU>::run(prog, r, cols, full, row_result, st, tmp, red);
        }
      } else if constexpr (op == OP_CONST) {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D][e] = __int_as_float(prog.arg[K]);
        RowStep<P, kV, K + 1, D + 1, U | (1u << D), TU>::run(prog, r, cols, full, row_result, st, tmp, red);
      } else if constexpr (op == OP_INDEX) {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D][e] = __int_as_float(static_cast<int>(r * cols + row_col<kV>(e)));
        RowStep<P, kV, K + 1, D + 1, U & ~(1u << D), TU>::run(prog, r, cols, full, row_result, st, tmp, red);
      } else if constexpr (is_binary_op(op) && imm) {
        const float w = __int_as_float(prog.arg[K]);
        if constexpr (top_u) {
          const float t = apply_binary(op, w, st[D - 1][0]);
#pragma unroll
          for (int e = 0; e < kV; ++e) st[D - 1][e] = t;
        } else {
#pragma unroll
          for (int e = 0; e < kV; ++e) st[D - 1][e] = apply_binary(op, w, st[D - 1][e]);
        }
        RowStep<P, kV, K + 1, D, U, TU>::run(prog, r, cols, full, row_result, st, tmp, red);
      } else if constexpr (is_binary_op(op)) {
        constexpr bool both = top_u && (U & (1u << (D - 2))) != 0;
        if constexpr (both) {
          const float t = apply_binary(op, st[D - 2][0], st[D - 1][0]);
#pragma unroll
          for (int e = 0; e < kV; ++e) st[D - 2][e] = t;
        } else {
#pragma unroll
          for (int e = 0; e < kV; ++e) st[D - 2][e] = apply_binary(op, st[D - 2][e], st[D - 1][e]);
        }
        constexpr unsigned u2 = (U & ~((1u << (D - 2)) | (1u << (D - 1)))) | (both ? 1u << (D - 2) : 0u);
        RowStep<P, kV, K + 1, D - 1, u2, TU>::run(prog, r, cols, full, row_result, st, tmp, red);
      } else if constexpr (op == OP_WHERE) {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D - 3][e] = st[D - 3][e] != 0.f ? st[D - 2][e] : st[D - 1][e];
        constexpr unsigned three = (1u << (D - 3)) | (1u << (D - 2)) | (1u << (D - 1));
        constexpr unsigned u2 = (U & ~three) | ((U & three) == three ? 1u << (D - 3) : 0u);
        RowStep<P, kV, K + 1, D - 2, u2, TU>::run(prog, r, cols, full, row_result, st, tmp, red);
      } else if constexpr (is_row_op(op)) {
        float v = row_identity(op);
        if (full) {
#pragma unroll
          for (int e = 0; e < kV; ++e) v = row_combine(op, v, st[D - 1][e]);
        } else {
#pragma unroll
          for (int e = 0; e < kV; ++e)
            if (row_col<kV>(e) < cols) v = row_combine(op, v, st[D - 1][e]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = row_combine(op, v, __shfl_xor_sync(0xffffffffu, v, o));
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
        __syncthreads();
        v = red[0];
#pragma unroll
        for (int w = 1; w < kThreads / 32; ++w) v = row_combine(op, v, red[w]);
        __syncthreads();
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D - 1][e] = v;
        RowStep<P, kV, K + 1, D, U | top_bit, TU>::run(prog, r, cols, full, row_result, st, tmp, red);
      } else if constexpr (op == OP_TEE) {
#pragma unroll
        for (int e = 0; e < kV; ++e) tmp[sub][e] = st[D - 1][e];
        RowStep<P, kV, K + 1, D, U, (TU & ~(1u << sub)) | (top_u ? 1u << sub : 0u)>::run(prog, r, cols, full, row_result, st,
                                                                                        tmp, red);
      } else if constexpr (op == OP_TMP) {
#pragma unroll
        for (int e = 0; e < kV; ++e) st[D][e] = tmp[sub][e];
        RowStep<P, kV, K + 1, D + 1, (U & ~(1u << D)) | ((TU >> sub) & 1u ? 1u << D : 0u), TU>::run(prog, r, cols, full,
                                                                                                  row_result, st, tmp, red);
      } else {
        if constexpr (top_u) {
          const float t = apply_unary(op, st[D - 1][0]);
#pragma unroll
          for (int e = 0; e < kV; ++e) st[D - 1][e] = t;
        } else {
#pragma unroll
          for (int e = 0; e < kV; ++e) st[D - 1][e] = apply_unary(op, st[D - 1][e]);
        }
        RowStep<P, kV, K + 1, D, U, TU>::run(prog, r, cols, full, row_result, st, tmp, red);
      }
    }
  }
};

template <class P, int kV>
__global__ void __launch_bounds__(kThreads) row_compiled_kernel(const __grid_constant__ EltProgram prog, uint32_t rows,
                                                                int row_result) {
  __shared__ float red[kThreads / 32];
  const uint32_t cols = prog.cols;
  const bool full = cols == kV * kThreads;
  for (uint32_t r = blockIdx.x; r < rows; r += gridDim.x) {
    float st[kStack][kV];
    float tmp[kMaxTmp][kV];
    RowStep<P, kV, 0, 0, 0u, 0u>::run(prog, r, cols, full, row_result, st, tmp, red);
  }
}

// ---- launch helpers of the generated translation units (CUDA runtime calls only) ----
// Grid sizing as for the kernels built into the library: four waves of resident CTAs (one for small launches), CTAs
// stride beyond.
template <class P>
inline int jit_launch_eltwise(const EltProgram& prog, int64_t n, int oct, int sms, cudaStream_t stream) {
  auto launch = [&](auto kernel, int lanes) -> int {
    int resident = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, kThreads, 0);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (resident < 1) resident = 1;
    const int64_t per_cta = static_cast<int64_t>(kThreads) * lanes;
    int64_t ctas = (n + per_cta - 1) / per_cta;
    const int64_t wave = static_cast<int64_t>(sms) * resident;
    const int64_t cap = wave * (ctas <= 8 * wave ? 1 : 4);
    if (ctas > cap) ctas = cap;
    kernel<<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(prog, n);
    return static_cast<int>(cudaGetLastError());
  };
  if (oct) return launch(eltwise_program_kernel<Compiled<P, true>, 16>, 16);
  return launch(eltwise_program_kernel<Compiled<P, false>, 8>, 8);
}

template <class P, int kV>
inline int jit_launch_row(const EltProgram& prog, int64_t rows, int row_result, int sms, cudaStream_t stream) {
  int resident = 0;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, row_compiled_kernel<P, kV>, kThreads, 0);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (resident < 1) resident = 1;
  int64_t ctas = static_cast<int64_t>(sms) * resident * 4;
  if (ctas > rows) ctas = rows;
  row_compiled_kernel<P, kV><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(prog, static_cast<uint32_t>(rows), row_result);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace
