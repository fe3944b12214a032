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
  OP_COUNT = 59,
  // flag on a binary opcode: the left operand is the 32-bit word in arg instead of a stack entry, so a
  // scalar operand costs neither a push nor a pop (with the swapped forms either side can be the scalar)
  OP_IMM = 0x100,
};

enum EltType : int32_t { T_F32 = 0, T_F16 = 1, T_BF16 = 2, T_I32 = 3, T_I16 = 4, T_COUNT = 5 };

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
};

constexpr int kThreads = 256;
constexpr int kReusedInput = 0x100;  // flag in EltProgram::in_type: the program loads this input more than once
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

// A thread's kV lanes: kV == 1 is the element at i; otherwise kV / 4 quads, the first at i and the
// others kQuadStride elements apart (so that a warp's accesses stay contiguous inside a CTA tile).
template <int kV>
__device__ __forceinline__ void load_group(const void* p, int typeword, int64_t i, float (&v)[kV]) {
  const int type = typeword & 0xff;
  if constexpr (kV >= 4) {
    const bool reused = (typeword & kReusedInput) != 0;
#pragma unroll
    for (int q = 0; q < kV / 4; ++q) load_quad(p, type, reused, i + q * kQuadStride, &v[4 * q]);
  } else {
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
__device__ __forceinline__ void store_group(void* p, int type, int64_t i, const float (&v)[kV]) {
  if constexpr (kV >= 4) {
#pragma unroll
    for (int q = 0; q < kV / 4; ++q) store_quad(p, type, i + q * kQuadStride, &v[4 * q]);
  } else {
    switch (type) {
      case T_F16: reinterpret_cast<__half*>(p)[i] = __float2half_rn(v[0]); break;
      case T_BF16: reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v[0]); break;
      case T_I32: reinterpret_cast<int32_t*>(p)[i] = __float_as_int(v[0]); break;
      case T_I16: reinterpret_cast<int16_t*>(p)[i] = static_cast<int16_t>(__float_as_int(v[0])); break;
      default: reinterpret_cast<float*>(p)[i] = v[0]; break;
    }
  }
}

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

// Evaluates the program for kV consecutive elements at once: one opcode dispatch (a single jump
// through the switch table) serves kV lanes.  The host validated opcodes, operand indices and depth.
template <int kV>
__device__ __forceinline__ void run_program(const EltProgram& prog, int64_t i, const StackSlots<kV> slots) {
  float top[kV];
  int depth = 0;  // entries on the stack, the top included
#define ASC_LANES _Pragma("unroll") for (int e = 0; e < kV; ++e)
#define ASC_BIN(CODE, EXPR)                                  \
  case CODE: {                                               \
    float lhs[kV];                                           \
    if (imm) {                                               \
      ASC_LANES lhs[e] = __int_as_float(prog.arg[k]);        \
    } else {                                                 \
      slots.get(depth - 2, lhs);                             \
      --depth;                                               \
    }                                                        \
    ASC_LANES {                                              \
      const float a = lhs[e], b = top[e];                    \
      const int x = __float_as_int(a), y = __float_as_int(b); \
      (void)a; (void)b; (void)x; (void)y;                    \
      top[e] = (EXPR);                                       \
    }                                                        \
  } break;
#define ASC_UN(CODE, EXPR)                \
  case CODE:                              \
    ASC_LANES {                           \
      const float a = top[e];             \
      const int x = __float_as_int(a);    \
      (void)x;                            \
      top[e] = (EXPR);                    \
    }                                     \
    break;
#pragma unroll 1
  for (int k = 0; k < prog.n_ops; ++k) {
    const int op = prog.op[k] & 0xff;
    const bool imm = (prog.op[k] & OP_IMM) != 0;
    switch (op) {
      case OP_LOAD:
        if (depth > 0) slots.put(depth - 1, top);
        ++depth;
        load_group<kV>(prog.in[prog.arg[k]], prog.in_type[prog.arg[k]], i, top);
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
      ASC_BIN(OP_ADD, __fadd_rn(a, b))
      ASC_BIN(OP_SUB, __fsub_rn(a, b))
      ASC_BIN(OP_MUL, __fmul_rn(a, b))
      ASC_BIN(OP_DIV, __fdiv_rn(a, b))
      ASC_BIN(OP_MAX, fmaxf(a, b))
      ASC_BIN(OP_MIN, fminf(a, b))
      ASC_BIN(OP_EQ, a == b ? 1.f : 0.f)
      ASC_BIN(OP_NE, a != b ? 1.f : 0.f)
      ASC_BIN(OP_GT, a > b ? 1.f : 0.f)
      ASC_BIN(OP_GE, a >= b ? 1.f : 0.f)
      ASC_BIN(OP_LT, a < b ? 1.f : 0.f)
      ASC_BIN(OP_LE, a <= b ? 1.f : 0.f)
      ASC_BIN(OP_IADD, __int_as_float(static_cast<int>(static_cast<unsigned>(x) + static_cast<unsigned>(y))))
      ASC_BIN(OP_ISUB, __int_as_float(static_cast<int>(static_cast<unsigned>(x) - static_cast<unsigned>(y))))
      ASC_BIN(OP_IMUL, __int_as_float(static_cast<int>(static_cast<unsigned>(x) * static_cast<unsigned>(y))))
      ASC_BIN(OP_IMAX, __int_as_float(max(x, y)))
      ASC_BIN(OP_IMIN, __int_as_float(min(x, y)))
      ASC_BIN(OP_ISHL, __int_as_float(static_cast<int>(static_cast<unsigned>(x) << (y & 31))))
      ASC_BIN(OP_ISHR, __int_as_float(x >> (y & 31)))
      ASC_BIN(OP_IEQ, x == y ? 1.f : 0.f)
      ASC_BIN(OP_INE, x != y ? 1.f : 0.f)
      ASC_BIN(OP_IGT, x > y ? 1.f : 0.f)
      ASC_BIN(OP_IGE, x >= y ? 1.f : 0.f)
      ASC_BIN(OP_ILT, x < y ? 1.f : 0.f)
      ASC_BIN(OP_ILE, x <= y ? 1.f : 0.f)
      ASC_BIN(OP_RSUB, __fsub_rn(b, a))
      ASC_BIN(OP_RDIV, __fdiv_rn(b, a))
      ASC_BIN(OP_IRSUB, __int_as_float(static_cast<int>(static_cast<unsigned>(y) - static_cast<unsigned>(x))))
      ASC_BIN(OP_IRSHL, __int_as_float(static_cast<int>(static_cast<unsigned>(y) << (x & 31))))
      ASC_BIN(OP_IRSHR, __int_as_float(y >> (x & 31)))
      ASC_UN(OP_NEG, -a)
      ASC_UN(OP_ABS, fabsf(a))
      ASC_UN(OP_RELU, fmaxf(a, 0.f))
      ASC_UN(OP_EXP, expf(a))
      ASC_UN(OP_EXP2, exp2f(a))
      ASC_UN(OP_LOG, logf(a))
      ASC_UN(OP_LOG2, log2f(a))
      ASC_UN(OP_SQRT, sqrtf(a))
      ASC_UN(OP_RSQRT, rsqrtf(a))
      ASC_UN(OP_SIN, sinf(a))
      ASC_UN(OP_COS, cosf(a))
      ASC_UN(OP_TAN, tanf(a))
      ASC_UN(OP_SINH, sinhf(a))
      ASC_UN(OP_COSH, coshf(a))
      ASC_UN(OP_TANH, tanhf(a))
      ASC_UN(OP_ERF, erff(a))
      ASC_UN(OP_FLOOR, floorf(a))
      ASC_UN(OP_CEIL, ceilf(a))
      ASC_UN(OP_ROUND_F16, __half2float(__float2half_rn(a)))
      ASC_UN(OP_ROUND_BF16, __bfloat162float(__float2bfloat16_rn(a)))
      ASC_UN(OP_INEG, __int_as_float(static_cast<int>(0u - static_cast<unsigned>(x))))
      ASC_UN(OP_IABS, __int_as_float(abs(x)))
      ASC_UN(OP_IRELU, __int_as_float(max(x, 0)))
      ASC_UN(OP_CVT_I2F, __int2float_rn(x))
      ASC_UN(OP_CVT_F2I, __int_as_float(__float2int_rz(a)))
      ASC_UN(OP_WRAP_I16, __int_as_float(static_cast<int>(static_cast<int16_t>(x & 0xffff))))
      default: break;
    }
  }
#undef ASC_UN
#undef ASC_BIN
#undef ASC_LANES
  store_group<kV>(prog.out, prog.out_type, i, top);
}

// kLanes == 1: some pointer is not aligned to four elements, every element goes through the scalar
// path.  Otherwise a CTA walks tiles of kThreads * kLanes elements (kLanes per thread and dispatch),
// then the remaining quads, then the scalar tail.
template <int kLanes>
__global__ void __launch_bounds__(kThreads) eltwise_program_kernel(const __grid_constant__ EltProgram prog, int64_t n) {
  extern __shared__ __align__(16) float stack_mem[];  // (max depth - 1) levels x kThreads x kLanes floats
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const StackSlots<1> scalar_slots{stack_mem + threadIdx.x};
  int64_t done = 0;
  if constexpr (kLanes >= 4) {
    const StackSlots<4> quad_slots{stack_mem + threadIdx.x * 4};
    if constexpr (kLanes > 4) {
      constexpr int64_t kTile = static_cast<int64_t>(kThreads) * kLanes;
      const StackSlots<kLanes> slots{stack_mem + threadIdx.x * 4};
      const int64_t tiles = n / kTile;
      for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) run_program<kLanes>(prog, t * kTile + threadIdx.x * 4, slots);
      done = tiles * kTile;
    }
    const int64_t quads = (n - done) >> 2;
    for (int64_t g = tid; g < quads; g += stride) run_program<4>(prog, done + (g << 2), quad_slots);
    done += quads << 2;
  }
  for (int64_t i = done + tid; i < n; i += stride) run_program<1>(prog, i, scalar_slots);
}

int g_lanes = 8;  // elements per thread and dispatch on the aligned path (4, 8 or 16)

template <int kLanes>
int32_t launch_program(const EltProgram& prog, int64_t n, int max_depth, int sms, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(max_depth > 1 ? max_depth - 1 : 1) * kThreads * (kLanes < 4 ? 4 : kLanes) * sizeof(float);
  if (smem > 48 * 1024) {
    static bool attr_set[64] = {false};
    int dev = 0;
    ASC_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
      ASC_CUDA_TRY(cudaFuncSetAttribute(eltwise_program_kernel<kLanes>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (kStack - 1) * kThreads * 16 * static_cast<int>(sizeof(float))));
      attr_set[dev] = true;
    }
  }
  int resident = 0;
  ASC_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, eltwise_program_kernel<kLanes>, kThreads, smem));
  if (resident < 1) resident = 1;
  const int64_t per_cta = static_cast<int64_t>(kThreads) * kLanes;
  int64_t ctas = (n + per_cta - 1) / per_cta;
  const int64_t cap = static_cast<int64_t>(sms) * resident * 4;  // four waves of resident CTAs; CTAs stride beyond
  if (ctas > cap) ctas = cap;
  eltwise_program_kernel<kLanes><<<static_cast<unsigned>(ctas), kThreads, smem, stream>>>(prog, n);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

int elem_size(int type) { return (type == T_F16 || type == T_BF16 || type == T_I16) ? 2 : 4; }

}  // namespace

extern "C" int32_t asc_cuda_eltwise_program(const int32_t* ops, const int32_t* args, int32_t n_ops,
                                            const void* const* inputs, const int32_t* input_types, int32_t n_inputs,
                                            void* out, int32_t out_type, int64_t n, void* stream) {
  if (n < 0 || n_ops <= 0 || n_ops > kMaxOps || n_inputs < 0 || n_inputs > kMaxInputs) return ASC_ERR_INVALID_ARG;
  if (ops == nullptr || args == nullptr || out == nullptr || (n_inputs > 0 && (inputs == nullptr || input_types == nullptr)))
    return ASC_ERR_INVALID_ARG;
  if (out_type < 0 || out_type >= T_COUNT) return ASC_ERR_INVALID_ARG;
  if (n == 0) return ASC_OK;
  EltProgram prog{};
  prog.n_ops = n_ops;
  prog.n_inputs = n_inputs;
  // validate the program on the host: opcodes, operand indices and stack depth
  int depth = 0, max_depth = 0;
  for (int k = 0; k < n_ops; ++k) {
    const int op = ops[k] & 0xff;
    const bool imm = (ops[k] & OP_IMM) != 0;
    if (ops[k] < 0 || (ops[k] & ~(0xff | OP_IMM)) != 0 || op >= OP_COUNT) return ASC_ERR_INVALID_ARG;
    if (imm && !is_binary_op(op)) return ASC_ERR_INVALID_ARG;
    if (op == OP_LOAD) {
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
  for (int i = 0; i < n_inputs; ++i) {
    if (inputs[i] == nullptr || input_types[i] < 0 || input_types[i] >= T_COUNT) return ASC_ERR_INVALID_ARG;
    if (reinterpret_cast<uintptr_t>(inputs[i]) % elem_size(input_types[i]) != 0) return ASC_ERR_MISALIGNED;
    prog.in[i] = inputs[i];
    int loads = 0;
    for (int k = 0; k < n_ops; ++k) loads += (prog.op[k] == OP_LOAD && prog.arg[k] == i) ? 1 : 0;
    prog.in_type[i] = input_types[i] | (loads > 1 ? kReusedInput : 0);
  }
  if (reinterpret_cast<uintptr_t>(out) % elem_size(out_type) != 0) return ASC_ERR_MISALIGNED;
  prog.out = out;
  prog.out_type = out_type;
  int sms = 0;
  int32_t rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;
  bool vec = reinterpret_cast<uintptr_t>(out) % (4 * elem_size(out_type)) == 0;
  for (int i = 0; i < n_inputs; ++i) vec = vec && reinterpret_cast<uintptr_t>(inputs[i]) % (4 * elem_size(input_types[i])) == 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!vec) return launch_program<1>(prog, n, max_depth, sms, st);
  if (g_lanes == 4 || n < kThreads * 8) return launch_program<4>(prog, n, max_depth, sms, st);
  if (g_lanes == 16) return launch_program<16>(prog, n, max_depth, sms, st);
  return launch_program<8>(prog, n, max_depth, sms, st);
}

// tuning hook: elements per thread and dispatch on the aligned path (4, 8 or 16; anything else: default)
extern "C" int32_t asc_cuda_eltwise_set_lanes(int32_t lanes) {
  g_lanes = (lanes == 4 || lanes == 16) ? lanes : 8;
  return ASC_OK;
}
