// Tensor-core GEMMs for sm_100a: fp16/bf16 -> fp32 accumulate (tcgen05 kind::f16) and
// int8 -> int32 (tcgen05 kind::i8), row-major A[M,K] and B[K,N], with a fused epilogue
// (ReLU, down-cast, per-row/per-column dequantisation).
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer: streams 128 x 128-byte A tiles (K-major) and 128-byte-wide B column
//               blocks (N contiguous, i.e. MN-major for the MMA) into a 4-stage 128B-swizzled
//               shared-memory ring, one mbarrier per stage.
//   warp 1      MMA issuer: four tcgen05.mma (128 x 256 x 32 bytes of K) per stage into one of
//               two 128-lane x 256-column fp32/int32 accumulators in tensor memory;
//               tcgen05.commit releases the stage and, after the last K block, publishes the
//               accumulator.
//   warps 2-5   epilogue: tcgen05.ld their 32-lane quarter of the accumulator, apply the
//               epilogue and store 16-byte vectors (in the CTA-pair kernel 16-bit outputs pass
//               through shared memory so that stores cover whole 128-byte lines); the other
//               accumulator is being filled meanwhile, so the epilogue of tile i overlaps the
//               main loop of tile i+1.
// B is never transposed in memory: the MN-major shared-memory descriptor lets the tensor core
// read it as stored.  All waits are bounded (see common.cuh).
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "../../include/asc_cuda.h"
#include "host_common.h"

namespace {

using namespace ascdev;

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kKBytes = 128;  // bytes of K per stage and per swizzle span
constexpr int kStages = 4;
constexpr int kGemmThreads = 192;
constexpr int kTmemCols = 512;
#ifndef ASC_GEMM_GROUP_M
#define ASC_GEMM_GROUP_M 16
#endif
#ifndef ASC_GEMM_HINT_NS
#define ASC_GEMM_HINT_NS 1000
#endif
constexpr int kGroupM = ASC_GEMM_GROUP_M;  // tile rasterisation: M blocks per L2 reuse group
constexpr int kWaitHintNs = ASC_GEMM_HINT_NS;  // mbarrier waits sleep in hardware instead of spinning

constexpr uint32_t kSmemA = kBlockM * kKBytes;                // 16 KiB per stage
constexpr uint32_t kSmemB = kBlockN * kKBytes;                // 32 KiB per stage
constexpr uint32_t kStageBytes = kSmemA + kSmemB;             // 48 KiB
constexpr uint32_t kGemmSmem = kStages * kStageBytes + 1024;  // + slack for 1024-byte alignment

// kMode of the kernels: the output form, | EPI_BIAS for the variants that add a bias row in the epilogue (their own
// instantiations: with the bias as a run-time case the plain fp16 GEMM needed 138 registers instead of 98 and ran
// 1.5-3 % slower at 8192^3)
enum EpiMode : int { EPI_F16 = 0, EPI_BF16 = 1, EPI_F32 = 2, EPI_I8 = 3, EPI_BIAS = 8 };

struct GemmParams {
  void* c;              // fp16 / bf16 / fp32 output, or int32 accumulator output for EPI_I8 (nullable there)
  void* deq;            // EPI_I8 only: fp16 dequantised output (nullable)
  const float* a_scale; // EPI_I8 only: per-row scale
  const float* b_scale; // EPI_I8 only: per-column scale
  int64_t M, N, K;      // K in elements
  int64_t ldc;
  const void* bias;     // one value per output column, added before the ReLU (nullable); see bias_type
  int32_t bias_type;    // 0 none, 1 fp32, 2 fp16, 3 bf16
  int32_t relu;
  int32_t accumulate;   // EPI_F32 only: C += A @ B
  int32_t vec_ok;       // 16-byte vector stores allowed (alignment of c/deq and ldc)
  uint32_t* status;
  uint32_t group_m;     // M blocks per rasterisation group (0 = default)
  // split-K kernel only: every 128 x 256 tile is computed by `split_k` CTAs, each over its own range of K
  int32_t split_k;
  uint32_t* arrivals;   // one counter per tile, zero at launch: slices whose partial tile is in the workspace
  uint32_t* partials;   // [tiles][split_k] partial tiles of 128 x 256 32-bit accumulator words
};

struct SharedCtl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

__device__ __forceinline__ void tile_coords(int64_t tile, int64_t num_m, int64_t num_n, int64_t& m_blk,
                                            int64_t& n_blk, int64_t group_m = kGroupM) {
  const int64_t group_sz = group_m * num_n;
  const int64_t g = tile / group_sz;
  const int64_t first_m = g * group_m;
  const int64_t gm = (num_m - first_m) < group_m ? (num_m - first_m) : group_m;
  const int64_t r = tile - g * group_sz;
  m_blk = first_m + r % gm;
  n_blk = r / gm;
}

__device__ __forceinline__ float bias_at(const void* bias, int32_t bias_type, int64_t col) {
  if (bias_type == 1) return __ldg(static_cast<const float*>(bias) + col);
  if (bias_type == 2) return __half2float(__ldg(static_cast<const __half*>(bias) + col));
  return __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(bias) + col));
}

// The floating-point epilogue of one element of output column `col`: the bias row, then the ReLU (a NaN stays a
// NaN, as in torch.relu).
template <int kMode>
__device__ __forceinline__ float epi_finish(const GemmParams& p, float v, int64_t col) {
  if constexpr ((kMode & EPI_BIAS) != 0) {
    if (col < p.N) v = __fadd_rn(v, bias_at(p.bias, p.bias_type, col));
  }
  if (p.relu) v = v < 0.f ? 0.f : v;
  return v;
}

template <int kMode>
__device__ __forceinline__ void epilogue_store_chunk(const GemmParams& p, const uint32_t (&r)[32], int64_t row,
                                                     int64_t col0) {
  // this thread owns 32 consecutive columns [col0, col0+32) of output row `row`
  if (row >= p.M || col0 >= p.N) return;
  const bool full = (col0 + 32 <= p.N) && p.vec_ok;
  if ((kMode & 7) == EPI_F16 || (kMode & 7) == EPI_BF16) {
    uint32_t packed[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float a = epi_finish<kMode>(p, __uint_as_float(r[2 * i]), col0 + 2 * i);
      const float b = epi_finish<kMode>(p, __uint_as_float(r[2 * i + 1]), col0 + 2 * i + 1);
      if ((kMode & 7) == EPI_F16) {
        __half2 h = __floats2half2_rn(a, b);
        packed[i] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        packed[i] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
    uint16_t* dst = reinterpret_cast<uint16_t*>(p.c) + row * p.ldc + col0;
    if (full) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        reinterpret_cast<uint4*>(dst)[i] =
            make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) dst[i] = static_cast<uint16_t>((packed[i >> 1] >> ((i & 1) * 16)) & 0xffffu);
    }
  } else if ((kMode & 7) == EPI_F32) {
    float* dst = reinterpret_cast<float*>(p.c) + row * p.ldc + col0;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
    if (p.accumulate) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) v[i] += dst[i];
    }
    if (p.relu || (kMode & EPI_BIAS) != 0) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = epi_finish<kMode>(p, v[i], col0 + i);
    }
    if (full) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) dst[i] = v[i];
    }
  } else {  // EPI_I8
    if (p.c != nullptr) {
      int32_t* dst = reinterpret_cast<int32_t*>(p.c) + row * p.ldc + col0;
      if (full) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          reinterpret_cast<uint4*>(dst)[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (col0 + i < p.N) dst[i] = static_cast<int32_t>(r[i]);
      }
    }
    if (p.deq != nullptr) {
      const float as = __ldg(p.a_scale + row);
      uint16_t* dst = reinterpret_cast<uint16_t*>(p.deq) + row * p.ldc + col0;
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int64_t c = col0 + 2 * i;
        const float s0 = (c < p.N) ? __ldg(p.b_scale + c) : 0.f;
        const float s1 = (c + 1 < p.N) ? __ldg(p.b_scale + c + 1) : 0.f;
        // left-to-right in fp32: (acc * a_scale[row]) * b_scale[col]
        const float a = __fmul_rn(__fmul_rn(static_cast<float>(static_cast<int32_t>(r[2 * i])), as), s0);
        const float b = __fmul_rn(__fmul_rn(static_cast<float>(static_cast<int32_t>(r[2 * i + 1])), as), s1);
        __half2 h = __floats2half2_rn(a, b);
        packed[i] = *reinterpret_cast<uint32_t*>(&h);
      }
      if (full) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          reinterpret_cast<uint4*>(dst)[i] =
              make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (col0 + i < p.N) dst[i] = static_cast<uint16_t>((packed[i >> 1] >> ((i & 1) * 16)) & 0xffffu);
      }
    }
  }
}

// kElemBytes: 2 (fp16/bf16, kind::f16, UMMA K = 16) or 1 (int8, kind::i8, UMMA K = 32)
template <int kElemBytes, int kMode>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const GemmParams p, const uint32_t idesc) {
  constexpr int kBlockK = kKBytes / kElemBytes;        // elements of K per stage: 64 or 128
  constexpr int kUmmaK = 32 / kElemBytes;              // elements of K per MMA: 16 or 32
  constexpr int kNBlockCols = 128 / kElemBytes;        // columns of B per 128-byte block: 64 or 128
  constexpr int kNBlocks = kBlockN / kNBlockCols;      // 4 or 2
  constexpr uint32_t kBBlockBytes = kBlockK * 128;     // one column block: kBlockK rows of 128 B
  constexpr uint32_t kBKStep = kUmmaK * 128;           // bytes between consecutive MMA K slices of B

  extern __shared__ uint8_t smem_raw[];
  __shared__ SharedCtl ctl;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile uint32_t* abort_flag = &ctl.abort_flag;

  const int64_t num_m = (p.M + kBlockM - 1) / kBlockM;
  const int64_t num_n = (p.N + kBlockN - 1) / kBlockN;
  const int64_t num_tiles = num_m * num_n;
  const int64_t num_kb = (p.K + kBlockK - 1) / kBlockK;

  if (threadIdx.x == 0) {
    ctl.abort_flag = 0;
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&ctl.full[s]), 1);
      mbar_init(smem_u32(&ctl.empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl.tmem_full[a]), 1);
      mbar_init(smem_u32(&ctl.tmem_empty[a]), 4);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl.tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl.tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // one thread runs the whole loop: waits by a single poller are an order of magnitude cheaper
    // than warp-wide ones, and nothing here needs the other lanes
    uint32_t stage = 0, phase = 0;
    bool ok = lane == 0;
    for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int64_t m_blk, n_blk;
      tile_coords(tile, num_m, num_n, m_blk, n_blk, p.group_m ? p.group_m : kGroupM);
      const int32_t m0 = static_cast<int32_t>(m_blk * kBlockM);
      const int32_t n0 = static_cast<int32_t>(n_blk * kBlockN);
      for (int64_t kb = 0; kb < num_kb; ++kb) {
        ok = mbar_wait<kWaitHintNs>(smem_u32(&ctl.empty[stage]), phase ^ 1, abort_flag, p.status, ASC_DEV_TIMEOUT_EMPTY);
        if (!ok) break;
        {
          const uint32_t full = smem_u32(&ctl.full[stage]);
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kSmemA;
          const int32_t k0 = static_cast<int32_t>(kb * kBlockK);
          mbar_arrive_expect_tx(full, kStageBytes);
          tma_load_2d(sa, &tmap_a, full, k0, m0);
#pragma unroll
          for (int j = 0; j < kNBlocks; ++j)
            tma_load_2d(sb + j * kBBlockBytes, &tmap_b, full, n0 + j * kNBlockCols, k0);
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    uint32_t stage = 0, phase = 0;
    bool ok = lane == 0;   // single-thread loop, see the producer
    int64_t local = 0;
    for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      const uint32_t acc = static_cast<uint32_t>(local & 1);
      const uint32_t acc_phase = static_cast<uint32_t>((local >> 1) & 1);
      ok = mbar_wait<kWaitHintNs>(smem_u32(&ctl.tmem_empty[acc]), acc_phase ^ 1, abort_flag, p.status,
                     ASC_DEV_TIMEOUT_TMEM_EMPTY);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * kBlockN;
      for (int64_t kb = 0; kb < num_kb; ++kb) {
        ok = mbar_wait<kWaitHintNs>(smem_u32(&ctl.full[stage]), phase, abort_flag, p.status, ASC_DEV_TIMEOUT_FULL);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kSmemA;
          const uint64_t adesc = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sb, kBBlockBytes, 1024);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint64_t ad = adesc + static_cast<uint64_t>((k * 32) >> 4);
            const uint64_t bd = bdesc + static_cast<uint64_t>((k * kBKStep) >> 4);
            const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
            if (kElemBytes == 2) {
              umma_f16_ss(d_tmem, ad, bd, idesc, accumulate);
            } else {
              umma_i8_ss(d_tmem, ad, bd, idesc, accumulate);
            }
          }
          umma_commit(smem_u32(&ctl.empty[stage]));
          if (kb == num_kb - 1) umma_commit(smem_u32(&ctl.tmem_full[acc]));
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const uint32_t quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    bool ok = true;
    int64_t local = 0;
    for (int64_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      int64_t m_blk, n_blk;
      tile_coords(tile, num_m, num_n, m_blk, n_blk, p.group_m ? p.group_m : kGroupM);
      const uint32_t acc = static_cast<uint32_t>(local & 1);
      const uint32_t acc_phase = static_cast<uint32_t>((local >> 1) & 1);
      ok = mbar_wait_warp<kWaitHintNs>(smem_u32(&ctl.tmem_full[acc]), acc_phase, abort_flag, p.status, ASC_DEV_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const int64_t row = m_blk * kBlockM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * kBlockN;
#pragma unroll 1
      for (int c = 0; c < kBlockN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        epilogue_store_chunk<kMode>(p, r, row, n_blk * kBlockN + c * 32);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl.tmem_empty[acc]));
    }
  }

  __syncwarp();
  if (*abort_flag) {
    // a wait ran out somewhere: give copies and MMAs still in flight time to land before
    // shared and tensor memory are released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// 16-bit outputs, a chunk that lies wholly inside C: the warp's 32 rows x 64 columns (128 bytes per row) pass
// through shared memory so that every store instruction writes four whole 128-byte lines instead of 16 bytes
// in each of 32 rows.  16-byte pieces are XOR-swizzled by the row, so both the row-per-thread writes and the
// line-per-8-threads reads are free of bank conflicts.
__device__ __forceinline__ void staged_store_64cols(uint32_t stage_smem, const uint32_t (&packed)[32], uint16_t* c,
                                                     int64_t ldc, int64_t row0, int64_t col0, uint32_t lane) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t addr = stage_smem + lane * 128 + ((j ^ (lane & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(packed[4 * j]), "r"(packed[4 * j + 1]),
                 "r"(packed[4 * j + 2]), "r"(packed[4 * j + 3])
                 : "memory");
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t r = 4 * i + (lane >> 3), piece = lane & 7;
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(stage_smem + r * 128 + ((piece ^ (r & 7)) << 4))
                 : "memory");
    *reinterpret_cast<uint4*>(c + (row0 + r) * ldc + col0 + piece * 8) = v;
  }
  __syncwarp();
}

template <int kMode>
__device__ __forceinline__ void pack16(const GemmParams& p, const uint32_t (&r)[32], uint32_t* packed, int64_t col0) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float a = epi_finish<kMode>(p, __uint_as_float(r[2 * i]), col0 + 2 * i);
    const float b = epi_finish<kMode>(p, __uint_as_float(r[2 * i + 1]), col0 + 2 * i + 1);
    if ((kMode & 7) == EPI_F16) {
      __half2 h = __floats2half2_rn(a, b);
      packed[i] = *reinterpret_cast<uint32_t*>(&h);
    } else {
      __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
      packed[i] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
}

// ----------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2): two CTAs of a cluster compute one 256 x 256 tile.  Each CTA
// stages its own 128 rows of A and its own 128 columns of B, so every SM reads and fills half as
// much shared memory per MMA as in the single-CTA kernel; the even CTA issues the 256 x 256 x 32-byte
// MMAs for both, each CTA keeps its 128 x 256 half of the accumulator in its own tensor memory and
// runs its own epilogue.
// ----------------------------------------------------------------------------------------------
constexpr int kPairStages = 6;
constexpr int kPairHalfN = kBlockN / 2;                          // columns of B staged per CTA
constexpr uint32_t kPairSmemB = kPairHalfN * kKBytes;            // 16 KiB
constexpr uint32_t kPairStageBytes = kSmemA + kPairSmemB;        // 32 KiB per CTA and stage
constexpr uint32_t kPairStageRing = kPairStages * kPairStageBytes;
constexpr uint32_t kEpiStageBytes = 32 * 128;                    // one epilogue warp: 32 rows of 128 output bytes
constexpr uint32_t kPairSmem = kPairStageRing + 4 * kEpiStageBytes + 1024;

struct PairCtl {
  uint64_t full[kPairStages];    // used in the even CTA: both CTAs' loads of a stage have landed
  uint64_t empty[kPairStages];   // per CTA: the MMAs reading this stage have retired
  uint64_t tmem_full[2];         // per CTA: accumulator ready for the epilogue
  uint64_t tmem_empty[2];        // used in the even CTA: both epilogues have drained the accumulator
  uint32_t tmem_base;
  uint32_t abort_flag;
};

template <int kElemBytes, int kMode>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                             const GemmParams p, const uint32_t idesc) {
  constexpr int kBlockK = kKBytes / kElemBytes;
  constexpr int kUmmaK = 32 / kElemBytes;
  constexpr int kNBlockCols = 128 / kElemBytes;            // columns per 128-byte block: 64 or 128
  constexpr int kNBlocks = kPairHalfN / kNBlockCols;       // 2 or 1 column blocks per CTA
  constexpr uint32_t kBBlockBytes = kBlockK * 128;
  constexpr uint32_t kBKStep = kUmmaK * 128;
  constexpr int kPairM = 2 * kBlockM;

  extern __shared__ uint8_t smem_raw[];
  __shared__ PairCtl ctl;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0: issues the MMAs, 1: peer
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile uint32_t* abort_flag = &ctl.abort_flag;

  const int64_t num_m = (p.M + kPairM - 1) / kPairM;
  const int64_t num_n = (p.N + kBlockN - 1) / kBlockN;
  const int64_t num_tiles = num_m * num_n;
  const int64_t num_kb = (p.K + kBlockK - 1) / kBlockK;
  const int64_t pair = blockIdx.x >> 1;
  const int64_t num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    ctl.abort_flag = 0;
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(smem_u32(&ctl.full[s]), 1);    // the even CTA's producer announces both CTAs' bytes
      mbar_init(smem_u32(&ctl.empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl.tmem_full[a]), 1);
      mbar_init(smem_u32(&ctl.tmem_empty[a]), 8);   // 4 epilogue warps in each CTA
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&ctl.tmem_base), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();            // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = ctl.tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    uint32_t stage = 0, phase = 0;
    bool ok = lane == 0;   // single-thread loop
    for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int64_t m_blk, n_blk;
      tile_coords(tile, num_m, num_n, m_blk, n_blk, p.group_m ? p.group_m : kGroupM);
      const int32_t m0 = static_cast<int32_t>(m_blk * kPairM + rank * kBlockM);
      const int32_t n0 = static_cast<int32_t>(n_blk * kBlockN + rank * kPairHalfN);
      for (int64_t kb = 0; kb < num_kb; ++kb) {
        ok = mbar_wait<kWaitHintNs>(smem_u32(&ctl.empty[stage]), phase ^ 1, abort_flag, p.status, ASC_DEV_TIMEOUT_EMPTY);
        if (!ok) break;
        {
          const uint32_t full0 = mapa_shared(smem_u32(&ctl.full[stage]), 0);   // the even CTA's barrier
          const uint32_t sa = smem_base + stage * kPairStageBytes;
          const uint32_t sb = sa + kSmemA;
          const int32_t k0 = static_cast<int32_t>(kb * kBlockK);
          // The even CTA announces the bytes of both CTAs' loads on its own barrier; the peer only
          // issues its copies, whose completion bytes are routed to that barrier by the hardware.
          if (rank == 0) mbar_arrive_expect_tx(smem_u32(&ctl.full[stage]), 2 * kPairStageBytes);
          tma_load_2d_pair(sa, &tmap_a, full0, k0, m0);
#pragma unroll
          for (int j = 0; j < kNBlocks; ++j)
            tma_load_2d_pair(sb + j * kBBlockBytes, &tmap_b, full0, n0 + j * kNBlockCols, k0);
        }
        if (++stage == kPairStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1 && rank == 0) {
    // --------------------------- MMA issuer (even CTA only) ---------------------------
    uint32_t stage = 0, phase = 0;
    bool ok = lane == 0;   // single-thread loop
    int64_t local = 0;
    for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
      const uint32_t acc = static_cast<uint32_t>(local & 1);
      const uint32_t acc_phase = static_cast<uint32_t>((local >> 1) & 1);
      ok = mbar_wait<kWaitHintNs>(smem_u32(&ctl.tmem_empty[acc]), acc_phase ^ 1, abort_flag, p.status,
                     ASC_DEV_TIMEOUT_TMEM_EMPTY);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * kBlockN;
      for (int64_t kb = 0; kb < num_kb; ++kb) {
        ok = mbar_wait<kWaitHintNs>(smem_u32(&ctl.full[stage]), phase, abort_flag, p.status, ASC_DEV_TIMEOUT_FULL);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t sa = smem_base + stage * kPairStageBytes;
          const uint32_t sb = sa + kSmemA;
          const uint64_t adesc = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sb, kBBlockBytes, 1024);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint64_t ad = adesc + static_cast<uint64_t>((k * 32) >> 4);
            const uint64_t bd = bdesc + static_cast<uint64_t>((k * kBKStep) >> 4);
            const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
            if (kElemBytes == 2) {
              umma_f16_ss_pair(d_tmem, ad, bd, idesc, accumulate);
            } else {
              umma_i8_ss_pair(d_tmem, ad, bd, idesc, accumulate);
            }
          }
          umma_commit_pair(smem_u32(&ctl.empty[stage]), 3);                 // frees the stage in both CTAs
          if (kb == num_kb - 1) umma_commit_pair(smem_u32(&ctl.tmem_full[acc]), 3);
        }
        if (++stage == kPairStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp >= 2) {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const uint32_t quarter = warp & 3;
    const uint32_t empty0 = mapa_shared(smem_u32(&ctl.tmem_empty[0]), 0);
    const uint32_t empty1 = mapa_shared(smem_u32(&ctl.tmem_empty[1]), 0);
    bool ok = true;
    int64_t local = 0;
    for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
      int64_t m_blk, n_blk;
      tile_coords(tile, num_m, num_n, m_blk, n_blk, p.group_m ? p.group_m : kGroupM);
      const uint32_t acc = static_cast<uint32_t>(local & 1);
      const uint32_t acc_phase = static_cast<uint32_t>((local >> 1) & 1);
      ok = mbar_wait_warp<kWaitHintNs>(smem_u32(&ctl.tmem_full[acc]), acc_phase, abort_flag, p.status, ASC_DEV_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const int64_t row0 = m_blk * kPairM + rank * kBlockM + quarter * 32;
      const int64_t row = row0 + lane;
      const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * kBlockN;
      if (((kMode & 7) == EPI_F16 || (kMode & 7) == EPI_BF16) && p.vec_ok && row0 + 32 <= p.M &&
          (n_blk + 1) * kBlockN <= p.N) {
        const uint32_t stage_smem = smem_base + kPairStageRing + quarter * kEpiStageBytes;
#pragma unroll 1
        for (int c = 0; c < kBlockN / 64; ++c) {
          uint32_t r0[32], r1[32], packed[32];
          tmem_ld_32x32b_x32(taddr + c * 64, r0);
          tmem_ld_32x32b_x32(taddr + c * 64 + 32, r1);
          tmem_ld_wait();
          pack16<kMode>(p, r0, packed, n_blk * kBlockN + c * 64);
          pack16<kMode>(p, r1, packed + 16, n_blk * kBlockN + c * 64 + 32);
          staged_store_64cols(stage_smem, packed, reinterpret_cast<uint16_t*>(p.c), p.ldc, row0, n_blk * kBlockN + c * 64,
                              lane);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < kBlockN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
          epilogue_store_chunk<kMode>(p, r, row, n_blk * kBlockN + c * 32);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc ? empty1 : empty0);
    }
  }

  __syncwarp();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();            // neither CTA leaves while the other may still signal it or read its memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// ----------------------------------------------------------------------------------------------
// Split-K variant for problems with far fewer 128 x 256 tiles than SMs (a long K over a small C): `split_k`
// CTAs share a tile, each runs the same TMA / tcgen05 main loop over its own contiguous range of K blocks and
// writes its 128 x 256 accumulator to a workspace in global memory.  Once all slices of a tile have arrived
// (a counter per tile; the grid is at most one CTA per SM, so all of them are running), every CTA sums a band of
// rows of the tile over all slices, always in slice order, so the result does not depend on which CTA finished
// first, applies the epilogue and stores the band.  The wait is bounded like every other wait in this library.
// ----------------------------------------------------------------------------------------------
constexpr uint32_t kTileWords = kBlockM * kBlockN;      // 32-bit words of one partial tile (128 KiB)

template <int kMode>
__device__ __forceinline__ void splitk_store_pair(const GemmParams& p, int64_t row, int64_t col, uint32_t w0, uint32_t w1) {
  // two neighbouring columns of one output row; w0 / w1 are fp32 (or, for int8, int32) sums over all slices
  if (row >= p.M || col >= p.N) return;
  const bool two = col + 1 < p.N;
  if ((kMode & 7) == EPI_I8) {
    if (p.c != nullptr) {
      int32_t* dst = reinterpret_cast<int32_t*>(p.c) + row * p.ldc + col;
      dst[0] = static_cast<int32_t>(w0);
      if (two) dst[1] = static_cast<int32_t>(w1);
    }
    if (p.deq != nullptr) {
      const float as = __ldg(p.a_scale + row);
      __half* dst = reinterpret_cast<__half*>(p.deq) + row * p.ldc + col;
      dst[0] = __float2half_rn(__fmul_rn(__fmul_rn(static_cast<float>(static_cast<int32_t>(w0)), as), __ldg(p.b_scale + col)));
      if (two)
        dst[1] = __float2half_rn(__fmul_rn(__fmul_rn(static_cast<float>(static_cast<int32_t>(w1)), as), __ldg(p.b_scale + col + 1)));
    }
    return;
  }
  float a = __uint_as_float(w0), b = __uint_as_float(w1);
  if ((kMode & 7) == EPI_F32) {
    float* dst = reinterpret_cast<float*>(p.c) + row * p.ldc + col;
    if (p.accumulate) {
      a += dst[0];
      if (two) b += dst[1];
    }
    a = epi_finish<kMode>(p, a, col);
    b = epi_finish<kMode>(p, b, col + 1);
    dst[0] = a;
    if (two) dst[1] = b;
    return;
  }
  a = epi_finish<kMode>(p, a, col);
  b = epi_finish<kMode>(p, b, col + 1);
  if ((kMode & 7) == EPI_F16) {
    __half* dst = reinterpret_cast<__half*>(p.c) + row * p.ldc + col;
    dst[0] = __float2half_rn(a);
    if (two) dst[1] = __float2half_rn(b);
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + row * p.ldc + col;
    dst[0] = __float2bfloat16_rn(a);
    if (two) dst[1] = __float2bfloat16_rn(b);
  }
}

// Four neighbouring columns of one output row: one 8- or 16-byte store where the output allows it.
template <int kMode>
__device__ __forceinline__ void splitk_store_quad(const GemmParams& p, int64_t row, int64_t col, const uint4& v) {
  if (row >= p.M || col >= p.N) return;
  if (p.vec_ok && col + 4 <= p.N) {
    if ((kMode & 7) == EPI_F16 || (kMode & 7) == EPI_BF16) {
      float f[4] = {__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)};
#pragma unroll
      for (int i = 0; i < 4; ++i) f[i] = epi_finish<kMode>(p, f[i], col + i);
      uint2 w;
      if ((kMode & 7) == EPI_F16) {
        const __half2 a = __floats2half2_rn(f[0], f[1]), b = __floats2half2_rn(f[2], f[3]);
        w = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
      } else {
        const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
        w = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
      }
      *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.c) + row * p.ldc + col) = w;
      return;
    }
    if ((kMode & 7) == EPI_F32 && !p.accumulate) {
      float4 f = make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
      f = make_float4(epi_finish<kMode>(p, f.x, col), epi_finish<kMode>(p, f.y, col + 1), epi_finish<kMode>(p, f.z, col + 2),
                      epi_finish<kMode>(p, f.w, col + 3));
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.c) + row * p.ldc + col) = f;
      return;
    }
    if ((kMode & 7) == EPI_I8 && p.deq == nullptr) {
      *reinterpret_cast<uint4*>(reinterpret_cast<int32_t*>(p.c) + row * p.ldc + col) = v;
      return;
    }
  }
  splitk_store_pair<kMode>(p, row, col, v.x, v.y);
  splitk_store_pair<kMode>(p, row, col + 2, v.z, v.w);
}

// Sums rows [r_lo, r_lo + n_rows) of one tile over all slices and stores them.  The words of one item are added in
// slice order 0, 1, 2, ... whatever kItems is, so the result does not depend on the load schedule.
template <int kMode, int kItems>
__device__ __forceinline__ void splitk_reduce_band(const GemmParams& p, const uint32_t* first, uint32_t e, int r_lo,
                                                   int n_rows, int64_t m_blk, int64_t n_blk) {
  constexpr int kBatch = 16 / kItems;
  const int total = n_rows * (kBlockN / 4);
  for (int item0 = static_cast<int>(e); item0 < total; item0 += 128 * kItems) {
    const uint4* src[kItems];
    uint4 v[kItems];
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      const int item = item0 + j * 128 < total ? item0 + j * 128 : item0;     // past the end: repeat a valid item
      src[j] = reinterpret_cast<const uint4*>(first) + (item / n_rows) * kBlockM + r_lo + item % n_rows;
      v[j] = __ldcg(src[j]);
    }
    for (int s0 = 1; s0 < p.split_k; s0 += kBatch) {
      uint4 w[kItems][kBatch];
#pragma unroll
      for (int i = 0; i < kBatch; ++i)
#pragma unroll
        for (int j = 0; j < kItems; ++j)
          if (s0 + i < p.split_k) w[j][i] = __ldcg(src[j] + static_cast<int64_t>(s0 + i) * (kTileWords / 4));
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        if (s0 + i < p.split_k) {
#pragma unroll
          for (int j = 0; j < kItems; ++j) {
            if ((kMode & 7) == EPI_I8) {
              v[j].x += w[j][i].x;
              v[j].y += w[j][i].y;
              v[j].z += w[j][i].z;
              v[j].w += w[j][i].w;
            } else {
              v[j].x = __float_as_uint(__fadd_rn(__uint_as_float(v[j].x), __uint_as_float(w[j][i].x)));
              v[j].y = __float_as_uint(__fadd_rn(__uint_as_float(v[j].y), __uint_as_float(w[j][i].y)));
              v[j].z = __float_as_uint(__fadd_rn(__uint_as_float(v[j].z), __uint_as_float(w[j][i].z)));
              v[j].w = __float_as_uint(__fadd_rn(__uint_as_float(v[j].w), __uint_as_float(w[j][i].w)));
            }
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kItems; ++j) {
      const int item = item0 + j * 128;
      if (item < total) {
        const int64_t row = m_blk * kBlockM + r_lo + item % n_rows, c0 = n_blk * kBlockN + (item / n_rows) * 4;
        splitk_store_quad<kMode>(p, row, c0, v[j]);
      }
    }
  }
}

template <int kElemBytes, int kMode>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_tcgen05_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                               const GemmParams p, const uint32_t idesc) {
  constexpr int kBlockK = kKBytes / kElemBytes;
  constexpr int kUmmaK = 32 / kElemBytes;
  constexpr int kNBlockCols = 128 / kElemBytes;
  constexpr int kNBlocks = kBlockN / kNBlockCols;
  constexpr uint32_t kBBlockBytes = kBlockK * 128;
  constexpr uint32_t kBKStep = kUmmaK * 128;

  extern __shared__ uint8_t smem_raw[];
  __shared__ SharedCtl ctl;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile uint32_t* abort_flag = &ctl.abort_flag;

  const int64_t num_n = (p.N + kBlockN - 1) / kBlockN;
  const int64_t num_kb = (p.K + kBlockK - 1) / kBlockK;
  const int64_t tile = blockIdx.x / p.split_k;
  const int64_t slice = blockIdx.x % p.split_k;
  const int64_t m_blk = tile / num_n, n_blk = tile % num_n;
  // K blocks of this slice: the first `num_kb % split_k` slices take one block more
  const int64_t kb_each = num_kb / p.split_k, kb_more = num_kb % p.split_k;
  const int64_t kb_lo = slice * kb_each + (slice < kb_more ? slice : kb_more);
  const int64_t kb_hi = kb_lo + kb_each + (slice < kb_more ? 1 : 0);

  if (threadIdx.x == 0) {
    ctl.abort_flag = 0;
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&ctl.full[s]), 1);
      mbar_init(smem_u32(&ctl.empty[s]), 1);
    }
    mbar_init(smem_u32(&ctl.tmem_full[0]), 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl.tmem_base), kBlockN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl.tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    uint32_t stage = 0, phase = 0;
    bool ok = lane == 0;
    const int32_t m0 = static_cast<int32_t>(m_blk * kBlockM);
    const int32_t n0 = static_cast<int32_t>(n_blk * kBlockN);
    for (int64_t kb = kb_lo; kb < kb_hi && ok; ++kb) {
      ok = mbar_wait<kWaitHintNs>(smem_u32(&ctl.empty[stage]), phase ^ 1, abort_flag, p.status, ASC_DEV_TIMEOUT_EMPTY);
      if (!ok) break;
      const uint32_t full = smem_u32(&ctl.full[stage]);
      const uint32_t sa = smem_base + stage * kStageBytes;
      const uint32_t sb = sa + kSmemA;
      const int32_t k0 = static_cast<int32_t>(kb * kBlockK);
      mbar_arrive_expect_tx(full, kStageBytes);
      tma_load_2d(sa, &tmap_a, full, k0, m0);
#pragma unroll
      for (int j = 0; j < kNBlocks; ++j) tma_load_2d(sb + j * kBBlockBytes, &tmap_b, full, n0 + j * kNBlockCols, k0);
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1;
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    uint32_t stage = 0, phase = 0;
    bool ok = lane == 0;
    for (int64_t kb = kb_lo; kb < kb_hi && ok; ++kb) {
      ok = mbar_wait<kWaitHintNs>(smem_u32(&ctl.full[stage]), phase, abort_flag, p.status, ASC_DEV_TIMEOUT_FULL);
      if (!ok) break;
      tc_fence_after();
      const uint32_t sa = smem_base + stage * kStageBytes;
      const uint32_t sb = sa + kSmemA;
      const uint64_t adesc = make_smem_desc_sw128(sa, 16, 1024);
      const uint64_t bdesc = make_smem_desc_sw128(sb, kBBlockBytes, 1024);
#pragma unroll
      for (int k = 0; k < kBlockK / kUmmaK; ++k) {
        const uint64_t ad = adesc + static_cast<uint64_t>((k * 32) >> 4);
        const uint64_t bd = bdesc + static_cast<uint64_t>((k * kBKStep) >> 4);
        const uint32_t accumulate = (kb > kb_lo || k > 0) ? 1u : 0u;
        if (kElemBytes == 2) {
          umma_f16_ss(tmem_base, ad, bd, idesc, accumulate);
        } else {
          umma_i8_ss(tmem_base, ad, bd, idesc, accumulate);
        }
      }
      umma_commit(smem_u32(&ctl.empty[stage]));
      if (kb == kb_hi - 1) umma_commit(smem_u32(&ctl.tmem_full[0]));
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1;
      }
    }
  } else {
    // ---------------- epilogue warps: publish the partial tile, then reduce a band of rows ----------------
    const uint32_t quarter = warp & 3;
    const uint32_t e = threadIdx.x - 64;                      // 0 .. 127 among the epilogue threads
    uint32_t* mine = p.partials + (tile * p.split_k + slice) * static_cast<int64_t>(kTileWords);
    bool ok = true;
    if (kb_hi > kb_lo) {
      ok = mbar_wait_warp<kWaitHintNs>(smem_u32(&ctl.tmem_full[0]), 0, abort_flag, p.status, ASC_DEV_TIMEOUT_TMEM_FULL);
      if (ok) {
        tc_fence_after();
        // Layout of a partial tile: groups of four columns, and inside a group the 128 rows side by side, 16 bytes
        // each.  A thread owns a row, so a warp's store of one column group is 512 contiguous bytes.
        const uint32_t taddr = tmem_base + ((quarter * 32u) << 16);
        uint4* dst = reinterpret_cast<uint4*>(mine) + (quarter * 32u + lane);
#pragma unroll 1
        for (int c = 0; c < kBlockN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[(c * 8 + i) * kBlockM] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
        }
        tc_fence_before();
      }
    } else {
      // a slice without K blocks (more slices than blocks never happens by construction, kept for safety)
      for (uint32_t i = e; i < kTileWords; i += 128) mine[i] = 0u;     // (all zero in any layout)
    }
    __threadfence();
    named_bar_sync(1, 128);
    if (e == 0) {
      if (ok && !*abort_flag) atomicAdd(p.arrivals + tile, 1u);
      // wait for the other slices of this tile
      const uint64_t t0 = global_timer_ns();
      volatile uint32_t* arrived = p.arrivals + tile;
      while (ok && *arrived < static_cast<uint32_t>(p.split_k)) {
        __nanosleep(100);
        if (*abort_flag || global_timer_ns() - t0 > kWaitLimitNs) {
          *abort_flag = 1;
          atomicCAS(p.status, 0u, static_cast<uint32_t>(ASC_DEV_TIMEOUT_OTHER));
          ok = false;
        }
      }
    }
    named_bar_sync(1, 128);
    __threadfence();
    if (!*abort_flag) {
      const int rows_each = (kBlockM + p.split_k - 1) / p.split_k;
      const int r_lo = static_cast<int>(slice) * rows_each;
      const int r_hi = r_lo + rows_each < kBlockM ? r_lo + rows_each : kBlockM;
      const uint32_t* first = p.partials + tile * p.split_k * static_cast<int64_t>(kTileWords);
      // An item is four columns of one row; consecutive threads take consecutive rows of a column group, whose
      // words lie side by side in every partial tile.  Sixteen loads are in flight per thread: with few slices a
      // thread works on several items at once, with many it fetches one item's slices sixteen at a time.
      const int n_rows = r_hi - r_lo;
      if (p.split_k <= 2) {
        splitk_reduce_band<kMode, 8>(p, first, e, r_lo, n_rows, m_blk, n_blk);
      } else if (p.split_k <= 4) {
        splitk_reduce_band<kMode, 4>(p, first, e, r_lo, n_rows, m_blk, n_blk);
      } else if (p.split_k <= 8) {
        splitk_reduce_band<kMode, 2>(p, first, e, r_lo, n_rows, m_blk, n_blk);
      } else {
        splitk_reduce_band<kMode, 1>(p, first, e, r_lo, n_rows, m_blk, n_blk);
      }
    }
  }

  __syncwarp();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kBlockN);
  }
}

// Matmul on the FMA pipe (32 x 32 tiles) for fp32 operands, and for small fp16 / bf16 products whose result is
// stored as fp32.  A product of two 16-bit values is exact in fp32 and every addition here rounds to nearest;
// each 32-long slice of K is summed on its own and then added to the running total, which keeps the rounding
// error of a sum of some hundred terms near one unit in the last place.  The tensor core's accumulator instead
// truncates when it adds, a bias that grows with K / 16 and reaches tens of units for a sum of same-signed terms.
__device__ __forceinline__ float simt_to_f32(float v) { return v; }
__device__ __forceinline__ float simt_to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float simt_to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(256)
    gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ B, void* __restrict__ C, int64_t M,
                     int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int out_dtype, int relu,
                     int accumulate, const void* __restrict__ bias, int bias_type) {
  __shared__ float as[32][33];
  __shared__ float bs[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * 32, n0 = static_cast<int64_t>(blockIdx.x) * 32;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int64_t k0 = 0; k0 < K; k0 += 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty + 8 * i;
      as[r][tx] = (m0 + r < M && k0 + tx < K) ? simt_to_f32(A[(m0 + r) * lda + k0 + tx]) : 0.f;
      bs[r][tx] = (k0 + r < K && n0 + tx < N) ? simt_to_f32(B[(k0 + r) * ldb + n0 + tx]) : 0.f;
    }
    __syncthreads();
    float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kk = 0; kk < 32; ++kk) {
#pragma unroll
      for (int i = 0; i < 4; ++i) part[i] = fmaf(as[ty + 8 * i][kk], bs[kk][tx], part[i]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] += part[i];
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = m0 + ty + 8 * i, c = n0 + tx;
    if (r < M && c < N) {
      float v = acc[i];
      if (accumulate && out_dtype == 2) v += reinterpret_cast<float*>(C)[r * ldc + c];
      if (bias_type != 0) v = __fadd_rn(v, bias_at(bias, bias_type, c));
      if (relu) v = v < 0.f ? 0.f : v;          // NaN stays NaN, as in torch.relu
      if (out_dtype == 2) {
        reinterpret_cast<float*>(C)[r * ldc + c] = v;
      } else if (out_dtype == 0) {
        reinterpret_cast<__half*>(C)[r * ldc + c] = __float2half_rn(v);
      } else {
        reinterpret_cast<__nv_bfloat16*>(C)[r * ldc + c] = __float2bfloat16_rn(v);
      }
    }
  }
}

template <typename T>
int32_t launch_gemm_simt(const T* A, const T* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                         int64_t ldc, int32_t out_dtype, int32_t flags, cudaStream_t stream, const void* bias = nullptr,
                         int32_t bias_type = 0) {
  const int64_t gx = (N + 31) / 32, gy = (M + 31) / 32;
  if (gy > 65535) return ASC_ERR_TOO_LARGE;
  dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
  gemm_simt_kernel<T><<<grid, 256, 0, stream>>>(A, B, C, M, N, K, lda, ldb, ldc, out_dtype, flags & 1, (flags >> 1) & 1,
                                                bias, bias_type);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

// fp16 / bf16 products stored as fp32 run on the FMA pipe up to this many multiply-adds (2^28: a few tens of
// microseconds); larger ones, and every product stored as 16 bits, run on the tensor core.
constexpr int64_t kSimtMaxMacs = 1ll << 28;

template <int kElemBytes, int kMode>
int32_t launch_gemm(const void* A, const void* B, int64_t lda, int64_t ldb, CUtensorMapDataType dt, uint32_t idesc,
                    GemmParams p, int32_t max_ctas, cudaStream_t stream) {
  constexpr int kBlockK = kKBytes / kElemBytes;
  constexpr int kNBlockCols = 128 / kElemBytes;
  CUtensorMap tmap_a, tmap_b;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(lda) * kElemBytes};
    const uint32_t box[2] = {kBlockK, kBlockM};
    int32_t rc = aschost::encode_tmap(&tmap_a, dt, 2, A, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != ASC_OK) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(p.N), static_cast<uint64_t>(p.K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldb) * kElemBytes};
    const uint32_t box[2] = {kNBlockCols, kBlockK};
    int32_t rc = aschost::encode_tmap(&tmap_b, dt, 2, B, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != ASC_OK) return rc;
  }
  int32_t rc = aschost::device_status_word(&p.status);
  if (rc != ASC_OK) return rc;
  int sms = 0;
  rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;

  auto kernel = gemm_tcgen05_kernel<kElemBytes, kMode>;
  static aschost::PerDevice attr_set;
  int dev = 0;
  ASC_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_set.get(dev)) {
    ASC_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem));
    attr_set.set(dev, 1);
  }
  const int64_t num_tiles = ((p.M + kBlockM - 1) / kBlockM) * ((p.N + kBlockN - 1) / kBlockN);
  int64_t grid = num_tiles < sms ? num_tiles : sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  kernel<<<static_cast<unsigned>(grid), kGemmThreads, kGemmSmem, stream>>>(tmap_a, tmap_b, p, idesc);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

// 0: choose per problem, 1: always the single-CTA kernel, 2: the CTA-pair kernel whenever it applies
static std::atomic<int> g_gemm_mode{0};
static std::atomic<uint32_t> g_group_m{0};
static std::atomic<bool> g_no_split_k{false};   // tuning hook: never split K over several CTAs
static std::atomic<bool> g_tensor_only{false};   // tuning hook: small fp32-output products on the tensor core too

template <int kElemBytes, int kMode>
int32_t launch_gemm_pair(const void* A, const void* B, int64_t lda, int64_t ldb, CUtensorMapDataType dt,
                         uint32_t idesc_pair, GemmParams p, int32_t max_ctas, cudaStream_t stream) {
  constexpr int kBlockK = kKBytes / kElemBytes;
  constexpr int kNBlockCols = 128 / kElemBytes;
  CUtensorMap tmap_a, tmap_b;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(lda) * kElemBytes};
    const uint32_t box[2] = {kBlockK, kBlockM};
    int32_t rc = aschost::encode_tmap(&tmap_a, dt, 2, A, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != ASC_OK) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(p.N), static_cast<uint64_t>(p.K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldb) * kElemBytes};
    const uint32_t box[2] = {kNBlockCols, kBlockK};
    int32_t rc = aschost::encode_tmap(&tmap_b, dt, 2, B, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != ASC_OK) return rc;
  }
  int32_t rc = aschost::device_status_word(&p.status);
  if (rc != ASC_OK) return rc;
  int sms = 0;
  rc = aschost::sm_count(&sms);
  if (rc != ASC_OK) return rc;
  auto kernel = gemm_tcgen05_pair_kernel<kElemBytes, kMode>;
  static aschost::PerDevice attr_set;
  int dev = 0;
  ASC_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_set.get(dev)) {
    ASC_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem));
    attr_set.set(dev, 1);
  }
  const int64_t num_tiles = ((p.M + 2 * kBlockM - 1) / (2 * kBlockM)) * ((p.N + kBlockN - 1) / kBlockN);
  // A persistent grid must be fully resident: ask how many 2-CTA clusters fit at once (SMs that have
  // no partner inside their GPC cannot host one), otherwise the surplus clusters run as a second wave.
  static aschost::PerDevice max_clusters;
  if (max_clusters.get(dev) == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(sms - sms % 2));
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = kPairSmem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    ASC_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
    max_clusters.set(dev, n > 0 ? n : 1);
  }
  int64_t pairs = max_clusters.get(dev) > 0 ? max_clusters.get(dev) : sms / 2;
  if (pairs > sms / 2) pairs = sms / 2;
  if (max_ctas > 0 && pairs > max_ctas / 2) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (pairs > num_tiles) pairs = num_tiles;
  kernel<<<static_cast<unsigned>(2 * pairs), kGemmThreads, kPairSmem, stream>>>(tmap_a, tmap_b, p, idesc_pair);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}
// Workspace of the split-K kernel: a 1 KiB header of per-tile arrival counters, then the partial tiles.
constexpr size_t kSplitHeaderBytes = 1024;
constexpr int kSplitMaxTiles = static_cast<int>(kSplitHeaderBytes / sizeof(uint32_t));
constexpr size_t kPartialTileBytes = static_cast<size_t>(kTileWords) * sizeof(uint32_t);

// How many slices of K each 128 x 256 tile is cut into when `ctas` CTAs may run at once (at least four K blocks per
// slice, at most 64 slices).  1 means: do not split.
inline int split_k_slices(int64_t tiles, int64_t num_kb, int64_t ctas) {
  if (tiles <= 0 || tiles > kSplitMaxTiles || tiles * 2 > ctas || num_kb < 16) return 1;
  // Measured on B200: a K block of the main loop costs about 0.29 us per CTA; publishing the partial tiles, waiting
  // for the other slices and summing them costs about 11 us + 0.1 us per CTA of the grid.  Take the number of
  // slices with the shortest predicted time, and split at all only for a gain of a fifth or more.
  const double whole = 0.29 * static_cast<double>(num_kb);
  double best = whole / 1.2;
  int best_s = 1;
  int64_t s_max = ctas / tiles;
  if (s_max > num_kb / 4) s_max = num_kb / 4;
  if (s_max > 64) s_max = 64;
  for (int64_t s = 2; s <= s_max; ++s) {
    const double t = 0.29 * static_cast<double>((num_kb + s - 1) / s) + 11.0 + 0.1 * static_cast<double>(tiles * s);
    if (t < best) {
      best = t;
      best_s = static_cast<int>(s);
    }
  }
  return best_s;
}

// Launches the split-K kernel.  `workspace` (kSplitHeaderBytes + tiles * split * 128 KiB, 256-byte aligned) is the
// caller's when given; otherwise it is taken from the stream-ordered allocator for the duration of the kernel, so
// that calls on different streams never share it.
template <int kElemBytes, int kMode>
int32_t launch_gemm_splitk(const void* A, const void* B, int64_t lda, int64_t ldb, CUtensorMapDataType dt,
                           uint32_t idesc, GemmParams p, int split, void* workspace, cudaStream_t stream) {
  constexpr int kBlockK = kKBytes / kElemBytes;
  constexpr int kNBlockCols = 128 / kElemBytes;
  CUtensorMap tmap_a, tmap_b;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(lda) * kElemBytes};
    const uint32_t box[2] = {kBlockK, kBlockM};
    int32_t rc = aschost::encode_tmap(&tmap_a, dt, 2, A, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != ASC_OK) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(p.N), static_cast<uint64_t>(p.K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ldb) * kElemBytes};
    const uint32_t box[2] = {kNBlockCols, kBlockK};
    int32_t rc = aschost::encode_tmap(&tmap_b, dt, 2, B, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != ASC_OK) return rc;
  }
  int32_t rc = aschost::device_status_word(&p.status);
  if (rc != ASC_OK) return rc;
  auto kernel = gemm_tcgen05_splitk_kernel<kElemBytes, kMode>;
  static aschost::PerDevice attr_set;
  int dev = 0;
  ASC_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_set.get(dev)) {
    ASC_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem));
    attr_set.set(dev, 1);
  }
  const int64_t tiles = ((p.M + kBlockM - 1) / kBlockM) * ((p.N + kBlockN - 1) / kBlockN);
  if (tiles > kSplitMaxTiles || split < 1) return ASC_ERR_TOO_LARGE;
  const size_t bytes = kSplitHeaderBytes + static_cast<size_t>(tiles) * split * kPartialTileBytes;
  void* ws = workspace;
  if (ws == nullptr && (rc = aschost::scratch_alloc(&ws, bytes, stream)) != ASC_OK) return rc;
  p.split_k = split;
  p.arrivals = static_cast<uint32_t*>(ws);
  p.partials = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(ws) + kSplitHeaderBytes);
  // the counters start at zero for every launch; the partial tiles are overwritten before they are read
  cudaError_t e = cudaMemsetAsync(ws, 0, kSplitHeaderBytes, stream);
  if (e == cudaSuccess) {
    kernel<<<static_cast<unsigned>(tiles * split), kGemmThreads, kGemmSmem, stream>>>(tmap_a, tmap_b, p, idesc);
    aschost::count_launch();
    e = cudaGetLastError();
  }
  if (workspace == nullptr) {
    const int32_t rc2 = aschost::scratch_free(ws, stream);
    if (e == cudaSuccess && rc2 != ASC_OK) return rc2;
  }
  ASC_CUDA_TRY(e);
  return ASC_OK;
}

// Single-CTA kernel for small problems (K split over several CTAs per tile when the tiles alone would leave most
// SMs idle), CTA pairs once there are enough 256 x 256 tiles to fill the GPU.
template <int kElemBytes, int kMode>
int32_t dispatch_gemm(const void* A, const void* B, int64_t lda, int64_t ldb, CUtensorMapDataType dt, uint32_t c_fmt,
                      uint32_t ab_fmt, GemmParams p, int32_t max_ctas, cudaStream_t stream) {
  p.group_m = g_group_m.load(std::memory_order_relaxed);
  const int mode = g_gemm_mode.load(std::memory_order_relaxed);
  const int64_t pair_tiles = ((p.M + 2 * kBlockM - 1) / (2 * kBlockM)) * ((p.N + kBlockN - 1) / kBlockN);
  const bool use_pair = mode == 2 ? p.M > kBlockM : (mode == 0 && pair_tiles >= 64);
  if (use_pair) {
    const uint32_t idesc = make_idesc(c_fmt, ab_fmt, ab_fmt, 0, 1, 2 * kBlockM, kBlockN);
    return launch_gemm_pair<kElemBytes, kMode>(A, B, lda, ldb, dt, idesc, p, max_ctas, stream);
  }
  const uint32_t idesc = make_idesc(c_fmt, ab_fmt, ab_fmt, 0, 1, kBlockM, kBlockN);
  if (mode == 0 && max_ctas == 0 && !g_no_split_k.load(std::memory_order_relaxed)) {
    int sms = 0;
    int32_t rc = aschost::sm_count(&sms);
    if (rc != ASC_OK) return rc;
    const int64_t tiles = ((p.M + kBlockM - 1) / kBlockM) * ((p.N + kBlockN - 1) / kBlockN);
    const int64_t num_kb = (p.K * kElemBytes + kKBytes - 1) / kKBytes;
    const int split = split_k_slices(tiles, num_kb, sms);
    if (split > 1) return launch_gemm_splitk<kElemBytes, kMode>(A, B, lda, ldb, dt, idesc, p, split, nullptr, stream);
  }
  return launch_gemm<kElemBytes, kMode>(A, B, lda, ldb, dt, idesc, p, max_ctas, stream);
}

// Workspace of asc_cuda_gemm_f16_static_workspace: room for the counter header and 64 partial tiles (8 MiB + 1 KiB).
// In host code the array's name only stands for the symbol; its device address comes from cudaGetSymbolAddress,
// looked up once per device with that device current.
constexpr int kStaticMaxPartials = 64;
static __device__ __align__(256) unsigned char g_static_splitk_workspace[kSplitHeaderBytes + kStaticMaxPartials * kPartialTileBytes];
static std::atomic<void*> g_static_workspace_addr[aschost::PerDevice::kMax];

int32_t static_scratch_address(void** out) {
  int dev = 0;
  ASC_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= aschost::PerDevice::kMax) return ASC_ERR_INVALID_ARG;
  void* addr = g_static_workspace_addr[dev].load(std::memory_order_acquire);
  if (addr == nullptr) {
    ASC_CUDA_TRY(cudaGetSymbolAddress(&addr, g_static_splitk_workspace));
    g_static_workspace_addr[dev].store(addr, std::memory_order_release);
  }
  *out = addr;
  return ASC_OK;
}

int32_t check_gemm_args(const void* A, const void* B, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                        int64_t ldc, int elem_bytes) {
  if (A == nullptr || B == nullptr) return ASC_ERR_INVALID_ARG;
  if (M <= 0 || N <= 0 || K <= 0) return ASC_ERR_INVALID_ARG;
  if (lda < K || ldb < N || ldc < N) return ASC_ERR_INVALID_ARG;
  if (M > 0x7fffff00ll || N > 0x7fffff00ll || K > 0x7fffff00ll) return ASC_ERR_TOO_LARGE;
  if (!aschost::aligned16(A) || !aschost::aligned16(B)) return ASC_ERR_MISALIGNED;
  if ((lda * elem_bytes) % 16 != 0 || (ldb * elem_bytes) % 16 != 0) return ASC_ERR_MISALIGNED;
  return ASC_OK;
}

int32_t gemm_f16_entry(const void* A, const void* B, void* C, const void* bias, int32_t bias_type, int64_t M, int64_t N,
                       int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int32_t in_dtype, int32_t out_dtype,
                       int32_t flags, void* stream) {
  if (C == nullptr) return ASC_ERR_INVALID_ARG;
  if (in_dtype < 0 || in_dtype > 1 || out_dtype < 0 || out_dtype > 2 || (flags & ~3) != 0) return ASC_ERR_INVALID_ARG;
  if ((flags & 2) && out_dtype != 2) return ASC_ERR_UNSUPPORTED;
  int32_t rc = check_gemm_args(A, B, M, N, K, lda, ldb, ldc, 2);
  if (rc != ASC_OK) return rc;
  GemmParams p{};
  p.c = C;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.relu = flags & 1;
  p.bias = bias;
  p.bias_type = bias_type;
  p.accumulate = (flags >> 1) & 1;
  const int out_bytes = out_dtype == 2 ? 4 : 2;
  p.vec_ok = aschost::aligned16(C) && ((ldc * out_bytes) % 16 == 0);
  // fp32 accumulator, A K-major, B MN-major (row-major [K, N] read as stored)
  const CUtensorMapDataType dt = in_dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_dtype == 2 && M * N <= kSimtMaxMacs / K && !g_tensor_only.load(std::memory_order_relaxed)) {
    // a small product whose fp32 result the caller keeps: exact products, round-to-nearest sums
    if (in_dtype == 0)
      return launch_gemm_simt<__half>(static_cast<const __half*>(A), static_cast<const __half*>(B), C, M, N, K, lda, ldb,
                                      ldc, out_dtype, flags, s, bias, bias_type);
    return launch_gemm_simt<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(B), C, M,
                                           N, K, lda, ldb, ldc, out_dtype, flags, s, bias, bias_type);
  }
  if (bias_type != 0) {
    switch (out_dtype) {
      case 0: return dispatch_gemm<2, EPI_F16 | EPI_BIAS>(A, B, lda, ldb, dt, 1, in_dtype, p, 0, s);
      case 1: return dispatch_gemm<2, EPI_BF16 | EPI_BIAS>(A, B, lda, ldb, dt, 1, in_dtype, p, 0, s);
      default: return dispatch_gemm<2, EPI_F32 | EPI_BIAS>(A, B, lda, ldb, dt, 1, in_dtype, p, 0, s);
    }
  }
  switch (out_dtype) {
    case 0: return dispatch_gemm<2, EPI_F16>(A, B, lda, ldb, dt, 1, in_dtype, p, 0, s);
    case 1: return dispatch_gemm<2, EPI_BF16>(A, B, lda, ldb, dt, 1, in_dtype, p, 0, s);
    default: return dispatch_gemm<2, EPI_F32>(A, B, lda, ldb, dt, 1, in_dtype, p, 0, s);
  }
}

}  // namespace

extern "C" {

int32_t asc_cuda_gemm_f16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                          int64_t ldb, int64_t ldc, int32_t in_dtype, int32_t out_dtype, int32_t flags,
                          void* stream) {
  return gemm_f16_entry(A, B, C, nullptr, 0, M, N, K, lda, ldb, ldc, in_dtype, out_dtype, flags, stream);
}

int32_t asc_cuda_gemm_f16_bias(const void* A, const void* B, void* C, const void* bias, int64_t M, int64_t N,
                               int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int32_t in_dtype, int32_t out_dtype,
                               int32_t bias_dtype, int32_t flags, void* stream) {
  if (bias == nullptr || bias_dtype < 0 || bias_dtype > 2) return ASC_ERR_INVALID_ARG;
  if (flags & 2) return ASC_ERR_UNSUPPORTED;              // C += A @ B + bias: the caller adds the bias once instead
  // bias_dtype: 0 fp16, 1 bf16, 2 fp32 (the codes of out_dtype)
  return gemm_f16_entry(A, B, C, bias, bias_dtype == 2 ? 1 : bias_dtype == 0 ? 2 : 3, M, N, K, lda, ldb, ldc, in_dtype,
                        out_dtype, flags, stream);
}

// The split-K GEMM for callers that must not allocate: its workspace is the file-scope array below, which every
// GPU that loads this library holds until the process exits.  See include/asc_cuda.h for the contract.
int32_t asc_cuda_gemm_f16_static_workspace(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                           int64_t lda, int64_t ldb, int64_t ldc, int32_t in_dtype, int32_t out_dtype,
                                           int32_t flags, void* stream) {
  if (C == nullptr) return ASC_ERR_INVALID_ARG;
  if (in_dtype < 0 || in_dtype > 1 || out_dtype < 0 || out_dtype > 2 || (flags & ~3) != 0) return ASC_ERR_INVALID_ARG;
  if ((flags & 2) && out_dtype != 2) return ASC_ERR_UNSUPPORTED;
  int32_t rc = check_gemm_args(A, B, M, N, K, lda, ldb, ldc, 2);
  if (rc != ASC_OK) return rc;
  const int64_t tiles = ((M + kBlockM - 1) / kBlockM) * ((N + kBlockN - 1) / kBlockN);
  if (tiles > kStaticMaxPartials) return ASC_ERR_TOO_LARGE;      // C larger than 64 tiles of 128 x 256
  void* scratch = nullptr;
  if ((rc = static_scratch_address(&scratch)) != ASC_OK) return rc;
  int sms = 0;
  if ((rc = aschost::sm_count(&sms)) != ASC_OK) return rc;
  const int64_t num_kb = (K * 2 + kKBytes - 1) / kKBytes;
  int64_t room = kStaticMaxPartials / tiles;                    // slices per tile the array has room for
  if (room > sms / tiles) room = sms / tiles;                   // ... and the GPU has SMs for
  int split = split_k_slices(tiles, num_kb, tiles * (room < 1 ? 1 : room));
  if (tiles * split > sms) return ASC_ERR_TOO_LARGE;            // every CTA of the grid must be running at once
  GemmParams p{};
  p.c = C;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.relu = flags & 1;
  p.accumulate = (flags >> 1) & 1;
  p.vec_ok = aschost::aligned16(C) && ((ldc * (out_dtype == 2 ? 4 : 2)) % 16 == 0);
  const CUtensorMapDataType dt = in_dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint32_t idesc = make_idesc(1, in_dtype, in_dtype, 0, 1, kBlockM, kBlockN);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (out_dtype) {
    case 0: return launch_gemm_splitk<2, EPI_F16>(A, B, lda, ldb, dt, idesc, p, split, scratch, s);
    case 1: return launch_gemm_splitk<2, EPI_BF16>(A, B, lda, ldb, dt, idesc, p, split, scratch, s);
    default: return launch_gemm_splitk<2, EPI_F32>(A, B, lda, ldb, dt, idesc, p, split, scratch, s);
  }
}

int32_t asc_cuda_gemm_f32(const float* A, const float* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                          int64_t ldb, int64_t ldc, int32_t out_dtype, int32_t flags, void* stream) {
  if (A == nullptr || B == nullptr || C == nullptr) return ASC_ERR_INVALID_ARG;
  if (M <= 0 || N <= 0 || K <= 0 || lda < K || ldb < N || ldc < N) return ASC_ERR_INVALID_ARG;
  if (out_dtype < 0 || out_dtype > 2 || (flags & ~3) != 0) return ASC_ERR_INVALID_ARG;
  if ((flags & 2) && out_dtype != 2) return ASC_ERR_UNSUPPORTED;
  return launch_gemm_simt<float>(A, B, C, M, N, K, lda, ldb, ldc, out_dtype, flags, static_cast<cudaStream_t>(stream));
}

int32_t asc_cuda_gemm_i8(const int8_t* A, const int8_t* B, int32_t* acc, void* deq, const float* a_scale,
                         const float* b_scale, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                         int64_t ldc, void* stream) {
  if (acc == nullptr && deq == nullptr) return ASC_ERR_INVALID_ARG;
  if (deq != nullptr && (a_scale == nullptr || b_scale == nullptr)) return ASC_ERR_INVALID_ARG;
  int32_t rc = check_gemm_args(A, B, M, N, K, lda, ldb, ldc, 1);
  if (rc != ASC_OK) return rc;
  GemmParams p{};
  p.c = acc;
  p.deq = deq;
  p.a_scale = a_scale;
  p.b_scale = b_scale;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.vec_ok = (acc == nullptr || (aschost::aligned16(acc) && (ldc * 4) % 16 == 0)) &&
             (deq == nullptr || (aschost::aligned16(deq) && (ldc * 2) % 16 == 0));
  // int32 accumulator, signed 8-bit operands
  return dispatch_gemm<1, EPI_I8>(A, B, lda, ldb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, 1, p, 0,
                                  static_cast<cudaStream_t>(stream));
}

// Tuning hook: the same GEMM with a cap on the number of CTAs (how throughput scales with the SMs used).
// in_dtype: 0 fp16, 1 bf16, 2 int8 (int32 output); out_dtype as asc_cuda_gemm_f16 (ignored for int8).
int32_t asc_cuda_gemm_capped(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                             int64_t ldb, int64_t ldc, int32_t in_dtype, int32_t out_dtype, int32_t max_ctas,
                             void* stream) {
  if (C == nullptr) return ASC_ERR_INVALID_ARG;
  int32_t rc = check_gemm_args(A, B, M, N, K, lda, ldb, ldc, in_dtype == 2 ? 1 : 2);
  if (rc != ASC_OK) return rc;
  GemmParams p{};
  p.c = C;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (in_dtype == 2) {
    p.vec_ok = aschost::aligned16(C) && (ldc * 4) % 16 == 0;
    return dispatch_gemm<1, EPI_I8>(A, B, lda, ldb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, 1, p, max_ctas, s);
  }
  const int out_bytes = out_dtype == 2 ? 4 : 2;
  p.vec_ok = aschost::aligned16(C) && ((ldc * out_bytes) % 16 == 0);
  const CUtensorMapDataType dt = in_dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  switch (out_dtype) {
    case 0: return dispatch_gemm<2, EPI_F16>(A, B, lda, ldb, dt, 1, in_dtype, p, max_ctas, s);
    case 1: return dispatch_gemm<2, EPI_BF16>(A, B, lda, ldb, dt, 1, in_dtype, p, max_ctas, s);
    default: return dispatch_gemm<2, EPI_F32>(A, B, lda, ldb, dt, 1, in_dtype, p, max_ctas, s);
  }
}

// Tuning hook: 0 choose per problem, 1 always single-CTA tiles, 2 CTA pairs whenever M > 128.
int32_t asc_cuda_gemm_set_mode(int32_t mode) {
  // bits 0-3 kernel choice, bit 4 tensor core also for small fp32-output products, bit 5 no split-K, bits 20-27 M
  // blocks per rasterisation group (0 = default)
  if ((mode & 0xf) > 2) return ASC_ERR_INVALID_ARG;
  g_gemm_mode = mode & 0xf;
  g_tensor_only = (mode & 0x10) != 0;
  g_no_split_k = (mode & 0x20) != 0;
  g_group_m = (mode >> 20) & 0xff;
  return ASC_OK;
}

}  // extern "C"
