// Flash-attention forward (fp16 / bf16, head size 128) for sm_100a.
//
// Persistent kernel: one CTA per SM walks a static list of work items.  An item is 256 consecutive query
// rows of one (batch, head): two 128-row query tiles that ping-pong on the tensor core so that the
// softmax of one tile overlaps the MMAs of the other.  The producer and MMA warps run ahead into the next
// item (its Q load and first Q K^T) while the softmax warps still write out the previous one, and with a
// causal mask every unit of the list pairs a heavy query block with a light one of the same head, so all
// units cost the same and a round-robin over the CTAs is balanced.
//   warps 0-3   softmax warpgroup of query tile 0: one thread per query row.  Reads the 128 scores
//   warps 4-7   (same for tile 1)  of its row from tensor memory (tcgen05.ld), keeps the running
//               max / sum in fp32, writes P as 16-bit values back into the same tensor-memory
//               columns (tcgen05.st) and, when the running max moved by more than 2^8, rescales
//               its row of the output accumulator in place.
//   warp 8      TMA producer: Q tiles once, then K and V tiles through two 2-stage rings of
//               128B-swizzled shared memory.
//   warp 9      MMA issuer: S = Q K^T (both operands K-major in shared memory) and
//               O += P V (P read from tensor memory, V read as stored, i.e. MN-major), fp32
//               accumulators in tensor memory: S0 S1 O0 O1 = 4 x 128 columns.
// Scores never leave the SM; HBM traffic is Q, K, V in and O out.  All waits are bounded.
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "../../include/asc_cuda.h"
#include "host_common.h"

namespace {

using namespace ascdev;

constexpr int kHeadDim = 128;
constexpr int kTileQ = 128;   // query rows per tile (= TMEM lanes)
constexpr int kTileKV = 128;  // keys per step
constexpr int kAttnThreads = 384;
constexpr uint32_t kHalfTile = 128 * 128;         // one 64-column half of a 128 x 128 16-bit tile: 16 KiB
constexpr uint32_t kTileBytes = 2 * kHalfTile;    // 32 KiB
constexpr uint32_t kSmemQ = 0;                    // 2 tiles
constexpr uint32_t kSmemK = 2 * kTileBytes;       // 2 stages
constexpr uint32_t kSmemV = 4 * kTileBytes;       // 2 stages
constexpr uint32_t kAttnSmem = 6 * kTileBytes + 1024;
constexpr uint32_t kColS = 0;    // S_t at columns [128 t, 128 t + 128); P_t aliases its first 64 columns
constexpr uint32_t kColO = 256;  // O_t at columns [256 + 128 t, ...)
constexpr float kRescaleThreshold = 8.0f;  // in log2 units
// Register split after launch (setmaxnreg): the 8 softmax warps grow, the other 4 shrink.  setmaxnreg is a
// warpgroup-wide instruction: the four warps of a warpgroup (0-3, 4-7, 8-11) must all execute the same one.
// An increase can only take registers a decrease in the same CTA has released, otherwise it waits forever,
// so the split must fit the launch allocation of 168 registers x 384 threads (what __launch_bounds__(384, 1)
// compiles to; check "Used 168 registers" in the ptxas output after changing the kernel).
constexpr int kLaunchRegs = 168, kSoftmaxRegs = 208, kOtherRegs = 88;
static_assert(8 * kSoftmaxRegs + 4 * kOtherRegs <= 12 * kLaunchRegs, "register split exceeds the launch allocation");

struct AttnParams {
  void* o;
  int32_t BH, S;
  float scale_log2;  // softmax scale * log2(e)
  int32_t causal;
  int32_t pairs;     // 256-row query blocks per head
  int32_t units;     // work units: (head, query block) non-causal; (head, heavy + light query block) causal
  int32_t half;      // causal: units per head = ceil(pairs / 2)
  uint32_t* status;
};

// The items of work unit `u`, in order: sub 0 and, with a causal mask, sub 1.  Returns false when the unit
// has no such item.  Heads are the slow axis so that the CTAs running at any time share K and V through L2.
__device__ __forceinline__ bool unit_item(const AttnParams& p, int u, int sub, int& bh, int& pair) {
  if (!p.causal) {
    bh = u / p.pairs;
    pair = p.pairs - 1 - u % p.pairs;
    return sub == 0;
  }
  bh = u / p.half;
  const int q = u % p.half;
  pair = sub == 0 ? p.pairs - 1 - q : q;      // the heavy block first, then its light partner
  return sub == 0 || (sub == 1 && q != p.pairs - 1 - q);
}

struct AttnCtl {
  uint64_t q_full[2], q_empty[2];
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2], p_full[2], o_full[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if (kBf16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// number of key tiles query tile `qt` (128-row index within the head) has to visit
__device__ __forceinline__ int kv_tiles_for(int qt, int S, int causal) {
  if (qt * kTileQ >= S) return 0;
  const int all = (S + kTileKV - 1) / kTileKV;
  if (!causal) return all;
  return (qt + 1) < all ? (qt + 1) : all;
}

// ----------------------------------------------------------------------------------------------
// Softmax warpgroup of one query tile.
// ----------------------------------------------------------------------------------------------
template <bool kBf16>
__device__ __forceinline__ bool softmax_role(const AttnParams& p, AttnCtl& ctl, uint32_t tmem_base, int t, int bh,
                                             int qt, int n_kv, uint32_t& s_it, uint32_t& o_it) {
  volatile uint32_t* abort_flag = &ctl.abort_flag;
  const uint32_t lane_row = threadIdx.x & 127;  // row inside the tile == TMEM lane
  const uint32_t lane_base = ((threadIdx.x >> 5) & 3) * 32;
  const uint32_t t_s = tmem_base + (lane_base << 16) + kColS + t * 128;
  const uint32_t t_o = tmem_base + (lane_base << 16) + kColO + t * 128;
  const int q_row = qt * kTileQ + static_cast<int>(lane_row);
  const float sl2 = p.scale_log2;

  float m_ref = 0.f;  // reference maximum (raw score units) the exponentials are taken against
  float l = 0.f;      // running sum of exp2((s - m_ref) * sl2)

  for (int j = 0; j < n_kv; ++j) {
    if (!mbar_wait(smem_u32(&ctl.s_full[t]), s_it & 1, abort_flag, p.status, ASC_DEV_TIMEOUT_TMEM_FULL)) return false;
    ++s_it;
    tc_fence_after();
    uint32_t s[4][32];
#pragma unroll
    for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(t_s + c * 32, s[c]);
    tmem_ld_wait();

    const int kv0 = j * kTileKV;
    int limit = p.S - 1;
    if (p.causal && q_row < limit) limit = q_row;
    limit -= kv0;  // columns c <= limit are visible
    if (limit < kTileKV - 1) {
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (c * 32 + i > limit) s[c][i] = 0xff800000u;  // -inf
    }
    float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      mx0 = max3(mx0, __uint_as_float(s[0][i]), __uint_as_float(s[0][i + 1]));
      mx1 = max3(mx1, __uint_as_float(s[1][i]), __uint_as_float(s[1][i + 1]));
      mx2 = max3(mx2, __uint_as_float(s[2][i]), __uint_as_float(s[2][i + 1]));
      mx3 = max3(mx3, __uint_as_float(s[3][i]), __uint_as_float(s[3][i + 1]));
    }
    const float row_max = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));

    // Lazy rescaling: the reference maximum only moves when the row maximum exceeds it by more
    // than 2^8; until then exponentials may grow up to 256, well inside fp16/bf16 and fp32 range.
    float alpha = 1.f;
    bool moved = false;
    if (j == 0) {
      m_ref = row_max;
    } else if ((row_max - m_ref) * sl2 > kRescaleThreshold) {
      alpha = ex2_approx((m_ref - row_max) * sl2);
      m_ref = row_max;
      moved = true;
    }
    if (__any_sync(0xffffffffu, moved)) {
      // O_t *= alpha for this thread's row.  The previous P V has retired: its commit is
      // ordered before the commit that published these scores.
      l *= alpha;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(t_o + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st_32x32b_x32(t_o + c * 32, o);
      }
    }
    const float neg_m = -m_ref * sl2;
    float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        // packed fp32 pairs: one FFMA2 scales two scores, one FADD2 adds two exponentials
        // (measured +2-5 % over scalar FFMA / FADD: the softmax warps are issue-bound)
        const float2 x = __ffma2_rn(make_float2(__uint_as_float(s[c][2 * i]), __uint_as_float(s[c][2 * i + 1])),
                                    make_float2(sl2, sl2), make_float2(neg_m, neg_m));
        const float e0 = ex2_approx(x.x);
        const float e1 = ex2_approx(x.y);
        if (i & 1) {
          const float2 t2 = __fadd2_rn(make_float2(l2, l3), make_float2(e0, e1));
          l2 = t2.x;
          l3 = t2.y;
        } else {
          const float2 t2 = __fadd2_rn(make_float2(l0, l1), make_float2(e0, e1));
          l0 = t2.x;
          l1 = t2.y;
        }
        pk[i] = pack2<kBf16>(e0, e1);
      }
      tmem_st_32x32b_x16(t_s + c * 16, pk);
    }
    l += (l0 + l1) + (l2 + l3);
    tmem_st_wait();
    tc_fence_before();
    mbar_arrive(smem_u32(&ctl.p_full[t]));
  }
  if (n_kv == 0) return true;

  // ------------------------------ epilogue: O / l -> 16-bit -> global ------------------------------
  if (!mbar_wait(smem_u32(&ctl.o_full[t]), o_it & 1, abort_flag, p.status, ASC_DEV_TIMEOUT_TMEM_FULL)) return false;
  ++o_it;
  tc_fence_after();
  const float inv = 1.f / l;
  uint16_t* dst = reinterpret_cast<uint16_t*>(p.o) + (static_cast<int64_t>(bh) * p.S + q_row) * kHeadDim;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t o[32];
    tmem_ld_32x32b_x32(t_o + c * 32, o);
    tmem_ld_wait();
    if (q_row < p.S) {
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i)
        pk[i] = pack2<kBf16>(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        reinterpret_cast<uint4*>(dst + c * 32)[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
    }
  }
  // O_t has been read: the first P V of the next item may overwrite it.  That MMA is issued only after this
  // thread's next p_full arrival, which follows in program order.
  tc_fence_before();
  return true;
}

// ----------------------------------------------------------------------------------------------
// Kernel
// ----------------------------------------------------------------------------------------------
template <bool kBf16>
__global__ void __launch_bounds__(kAttnThreads, 1)
    attn_fwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_v, const AttnParams p, const uint32_t idesc_qk,
                            const uint32_t idesc_pv) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ AttnCtl ctl;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile uint32_t* abort_flag = &ctl.abort_flag;

  if (threadIdx.x == 0) {
    ctl.abort_flag = 0;
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctl.q_full[i]), 1);
      mbar_init(smem_u32(&ctl.q_empty[i]), 1);
      mbar_init(smem_u32(&ctl.k_full[i]), 1);
      mbar_init(smem_u32(&ctl.k_empty[i]), 1);
      mbar_init(smem_u32(&ctl.v_full[i]), 1);
      mbar_init(smem_u32(&ctl.v_empty[i]), 1);
      mbar_init(smem_u32(&ctl.s_full[i]), 1);
      mbar_init(smem_u32(&ctl.p_full[i]), 128);
      mbar_init(smem_u32(&ctl.o_full[i]), 1);
    }
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(&ctl.tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl.tmem_base;

  // Every role walks the same list of items, so the running use counts of the barriers (which give stage and
  // phase) advance identically in all of them.
  if (warp < 8) {
    setmaxnreg_inc<kSoftmaxRegs>();
    const int t = static_cast<int>(warp >> 2);
    uint32_t s_it = 0, o_it = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
      for (int sub = 0; sub < 2 && ok; ++sub) {
        int bh, pair;
        if (!unit_item(p, u, sub, bh, pair)) continue;
        const int qt = 2 * pair + t;
        ok = softmax_role<kBf16>(p, ctl, tmem_base, t, bh, qt, kv_tiles_for(qt, p.S, p.causal), s_it, o_it);
      }
    }
  } else {
    setmaxnreg_dec<kOtherRegs>();
    if (warp == 8) {
      // ------------------------------ TMA producer ------------------------------
      bool ok = true;
      uint32_t q_it[2] = {0, 0}, k_it = 0, v_it = 0;
      for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
        for (int sub = 0; sub < 2 && ok; ++sub) {
          int bh, pair;
          if (!unit_item(p, u, sub, bh, pair)) continue;
          const int qt0 = 2 * pair;
          const int n0 = kv_tiles_for(qt0, p.S, p.causal), n1 = kv_tiles_for(qt0 + 1, p.S, p.causal);
          const int n_max = n0 > n1 ? n0 : n1;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (!ok || (t == 0 ? n0 : n1) == 0) continue;
            // the previous item's Q K^T of this tile have retired
            ok = mbar_wait(smem_u32(&ctl.q_empty[t]), (q_it[t] & 1) ^ 1, abort_flag, p.status, ASC_DEV_TIMEOUT_EMPTY);
            if (!ok) continue;
            ++q_it[t];
            if (lane == 0) {
              const uint32_t bar = smem_u32(&ctl.q_full[t]);
              const uint32_t dst = smem_base + kSmemQ + t * kTileBytes;
              mbar_arrive_expect_tx(bar, kTileBytes);
              tma_load_3d(dst, &tmap_q, bar, 0, (qt0 + t) * kTileQ, bh);
              tma_load_3d(dst + kHalfTile, &tmap_q, bar, 64, (qt0 + t) * kTileQ, bh);
            }
            __syncwarp();
          }
          for (int j = 0; j < n_max && ok; ++j) {
            const uint32_t kst = k_it & 1, kph = (k_it >> 1) & 1;
            ok = mbar_wait(smem_u32(&ctl.k_empty[kst]), kph ^ 1, abort_flag, p.status, ASC_DEV_TIMEOUT_EMPTY);
            if (!ok) break;
            ++k_it;
            if (lane == 0) {
              const uint32_t bar = smem_u32(&ctl.k_full[kst]);
              const uint32_t dst = smem_base + kSmemK + kst * kTileBytes;
              mbar_arrive_expect_tx(bar, kTileBytes);
              tma_load_3d(dst, &tmap_k, bar, 0, j * kTileKV, bh);
              tma_load_3d(dst + kHalfTile, &tmap_k, bar, 64, j * kTileKV, bh);
            }
            const uint32_t vst = v_it & 1, vph = (v_it >> 1) & 1;
            ok = mbar_wait(smem_u32(&ctl.v_empty[vst]), vph ^ 1, abort_flag, p.status, ASC_DEV_TIMEOUT_EMPTY);
            if (!ok) break;
            ++v_it;
            if (lane == 0) {
              const uint32_t bar = smem_u32(&ctl.v_full[vst]);
              const uint32_t dst = smem_base + kSmemV + vst * kTileBytes;
              mbar_arrive_expect_tx(bar, kTileBytes);
              tma_load_3d(dst, &tmap_v, bar, 0, j * kTileKV, bh);
              tma_load_3d(dst + kHalfTile, &tmap_v, bar, 64, j * kTileKV, bh);
            }
            __syncwarp();
          }
        }
      }
    } else if (warp == 9) {
      // ------------------------------- MMA issuer -------------------------------
      // Descriptors are built once: only the start address changes between MMAs, and shared-memory
      // addresses >> 4 fit the 14-bit address field with room to spare, so adding to the low bits cannot carry.
      const uint64_t q_desc0 = make_smem_desc_sw128(smem_base + kSmemQ, 16, 1024);
      const uint64_t k_desc0 = make_smem_desc_sw128(smem_base + kSmemK, 16, 1024);
      const uint64_t v_desc0 = make_smem_desc_sw128(smem_base + kSmemV, kHalfTile, 1024);
      // S_t = Q_t K_j^T : 8 MMAs of 128 x 128 x 16, both operands K-major (two 64-column halves).
      auto issue_qk = [&](int t, uint32_t k_stage) {
        const uint64_t qd = q_desc0 + static_cast<uint64_t>(t) * (kTileBytes >> 4);
        const uint64_t kd = k_desc0 + static_cast<uint64_t>(k_stage) * (kTileBytes >> 4);
        const uint32_t d = tmem_base + kColS + t * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = ((ks >> 2) * kHalfTile + (ks & 3) * 32) >> 4;
          umma_f16_ss(d, qd + off, kd + off, idesc_qk, ks > 0 ? 1u : 0u);
        }
      };
      // O_t (+)= P_t V_j : P from tensor memory (8 columns per 16 keys), V MN-major as stored.
      auto issue_pv = [&](int t, uint32_t v_stage, uint32_t accumulate) {
        const uint64_t vd = v_desc0 + static_cast<uint64_t>(v_stage) * (kTileBytes >> 4);
        const uint32_t d = tmem_base + kColO + t * 128;
        const uint32_t a = tmem_base + kColS + t * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_f16_ts(d, a + ks * 8, vd + ((ks * 2048) >> 4), idesc_pv, (accumulate || ks > 0) ? 1u : 0u);
      };
      bool ok = true;
      uint32_t q_it[2] = {0, 0}, p_it[2] = {0, 0}, k_it = 0, v_it = 0;
      for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
        for (int sub = 0; sub < 2 && ok; ++sub) {
          int bh, pair;
          if (!unit_item(p, u, sub, bh, pair)) continue;
          const int qt0 = 2 * pair;
          const int n0 = kv_tiles_for(qt0, p.S, p.causal), n1 = kv_tiles_for(qt0 + 1, p.S, p.causal);
          const int n_max = n0 > n1 ? n0 : n1;
          if (n_max == 0) continue;
          // first scores of both tiles
          uint32_t kst = k_it & 1, kph = (k_it >> 1) & 1;
          ok = mbar_wait(smem_u32(&ctl.k_full[kst]), kph, abort_flag, p.status, ASC_DEV_TIMEOUT_FULL);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (!ok || (t == 0 ? n0 : n1) == 0) continue;
            ok = mbar_wait(smem_u32(&ctl.q_full[t]), q_it[t] & 1, abort_flag, p.status, ASC_DEV_TIMEOUT_FULL);
            if (!ok) continue;
            ++q_it[t];
            tc_fence_after();
            if (lane == 0) {
              issue_qk(t, kst);
              umma_commit(smem_u32(&ctl.s_full[t]));
              if ((t == 0 ? n0 : n1) == 1) umma_commit(smem_u32(&ctl.q_empty[t]));   // the tile's only Q K^T
            }
            __syncwarp();
          }
          if (ok && lane == 0) umma_commit(smem_u32(&ctl.k_empty[kst]));
          __syncwarp();
          ++k_it;
          for (int j = 0; j < n_max && ok; ++j) {
            const uint32_t vst = v_it & 1, vph = (v_it >> 1) & 1;
            ok = mbar_wait(smem_u32(&ctl.v_full[vst]), vph, abort_flag, p.status, ASC_DEV_TIMEOUT_FULL);
            if (!ok) break;
            kst = k_it & 1;
            kph = (k_it >> 1) & 1;
            if (j + 1 < n_max) {
              ok = mbar_wait(smem_u32(&ctl.k_full[kst]), kph, abort_flag, p.status, ASC_DEV_TIMEOUT_FULL);
              if (!ok) break;
            }
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              const int nt = t == 0 ? n0 : n1;
              if (!ok || j >= nt) continue;
              ok = mbar_wait(smem_u32(&ctl.p_full[t]), p_it[t] & 1, abort_flag, p.status, ASC_DEV_TIMEOUT_OTHER);
              if (!ok) continue;
              ++p_it[t];
              tc_fence_after();
              if (lane == 0) {
                issue_pv(t, vst, j > 0 ? 1u : 0u);
                if (j + 1 < nt) {
                  issue_qk(t, kst);
                  umma_commit(smem_u32(&ctl.s_full[t]));
                  // The tile's last Q K^T of this item: once it retires the producer may load the next item's
                  // Q tile, a whole key step before this item ends, so that the load is off the critical path.
                  if (j + 2 == nt) umma_commit(smem_u32(&ctl.q_empty[t]));
                } else {
                  umma_commit(smem_u32(&ctl.o_full[t]));
                }
              }
              __syncwarp();
            }
            if (ok && lane == 0) {
              umma_commit(smem_u32(&ctl.v_empty[vst]));
              if (j + 1 < n_max) umma_commit(smem_u32(&ctl.k_empty[kst]));
            }
            __syncwarp();
            ++v_it;
            if (j + 1 < n_max) ++k_it;
          }
        }
      }
    }
  }

  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <bool kBf16>
int32_t launch_attn(const void* q, const void* k, const void* v, AttnParams p, cudaStream_t stream) {
  const CUtensorMapDataType dt = kBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const uint64_t dims[3] = {kHeadDim, static_cast<uint64_t>(p.S), static_cast<uint64_t>(p.BH)};
  const uint64_t strides[2] = {kHeadDim * 2, static_cast<uint64_t>(p.S) * kHeadDim * 2};
  const uint32_t box[3] = {64, 128, 1};
  CUtensorMap tq, tk, tv;
  int32_t rc;
  if ((rc = aschost::encode_tmap(&tq, dt, 3, q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) != ASC_OK) return rc;
  if ((rc = aschost::encode_tmap(&tk, dt, 3, k, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) != ASC_OK) return rc;
  if ((rc = aschost::encode_tmap(&tv, dt, 3, v, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) != ASC_OK) return rc;
  if ((rc = aschost::device_status_word(&p.status)) != ASC_OK) return rc;
  auto kernel = attn_fwd_tcgen05_kernel<kBf16>;
  static aschost::PerDevice attr_set;
  int dev = 0;
  ASC_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_set.get(dev)) {
    // the register split inside the kernel must fit what the kernel is launched with, or its first
    // setmaxnreg increase would wait forever: refuse to launch a build where it does not
    cudaFuncAttributes fa{};
    ASC_CUDA_TRY(cudaFuncGetAttributes(&fa, kernel));
    if (12 * fa.numRegs < 8 * kSoftmaxRegs + 4 * kOtherRegs) return ASC_ERR_UNSUPPORTED;
    ASC_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem));
    attr_set.set(dev, 1);
  }
  const uint32_t fmt = kBf16 ? 1u : 0u;
  const uint32_t idesc_qk = make_idesc(1, fmt, fmt, 0, 0, kTileQ, kTileKV);
  const uint32_t idesc_pv = make_idesc(1, fmt, fmt, 0, 1, kTileQ, kHeadDim);
  int sms = 0;
  if ((rc = aschost::sm_count(&sms)) != ASC_OK) return rc;
  p.half = (p.pairs + 1) / 2;
  const int64_t units = static_cast<int64_t>(p.BH) * (p.causal ? p.half : p.pairs);
  if (units > 0x7fffffff) return ASC_ERR_TOO_LARGE;
  p.units = static_cast<int32_t>(units);
  const int64_t grid = units < sms ? units : sms;     // one persistent CTA per SM (shared memory allows one)
  kernel<<<static_cast<unsigned>(grid), kAttnThreads, kAttnSmem, stream>>>(tq, tk, tv, p, idesc_qk, idesc_pv);
  aschost::count_launch();
  ASC_CUDA_TRY(cudaGetLastError());
  return ASC_OK;
}

}  // namespace

extern "C" int32_t asc_cuda_attn_fwd_f16(const void* q, const void* k, const void* v, void* o, int32_t B, int32_t H,
                                         int32_t S, int32_t D, float scale, int32_t causal, int32_t dtype,
                                         void* stream) {
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr) return ASC_ERR_INVALID_ARG;
  if (B <= 0 || H <= 0 || S <= 0 || dtype < 0 || dtype > 1) return ASC_ERR_INVALID_ARG;
  if (D != kHeadDim) return ASC_ERR_UNSUPPORTED;
  if (!aschost::aligned16(q) || !aschost::aligned16(k) || !aschost::aligned16(v) || !aschost::aligned16(o))
    return ASC_ERR_MISALIGNED;
  if (static_cast<int64_t>(B) * H > 0x7fffffffll) return ASC_ERR_TOO_LARGE;
  AttnParams p{};
  p.o = o;
  p.BH = B * H;
  p.S = S;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal != 0;
  p.pairs = (S + 2 * kTileQ - 1) / (2 * kTileQ);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == 1 ? launch_attn<true>(q, k, v, p, s) : launch_attn<false>(q, k, v, p, s);
}
