// Prefill forward for fp16 / bf16 on sm_100a tensor cores.
//
// Replaces the score-materialising composition of FuncSDPAttention::forward
// (reference: src/Function/FuncNNLayer.h:231-266) by one fused kernel that never
// writes the [L,S] score matrix to HBM.
//
// One CTA owns two 128-row query tiles of one (batch, head) and walks the
// key/value sequence in 128-row tiles (1 CTA per SM, all 512 TMEM columns):
//   warp 8   producer : TMA tiled loads (128-byte swizzle, no multicast) of both Q
//                       tiles once and of each K and V tile into a 2-stage ring
//   warp 9   issuer   : one thread issues tcgen05.mma; S_t = Q_t.K^T accumulates in
//                       TMEM columns [t*128, t*128+128), O_t += P_t.V in columns
//                       [256 + t*D, 256 + (t+1)*D).  The two tiles are interleaved
//                       so that the tensor pipe computes for one tile while the
//                       other tile's warpgroup is in its softmax.
//   warps 0-3 / 4-7   : softmax warpgroup of tile 0 / 1.  Thread r owns query row r
//                       (= TMEM lane r): it reads the whole 128-column S row with
//                       tcgen05.ld, so the row max and row sum need no cross-thread
//                       reduction in this layout; exponentials run as packed fp32
//                       pairs (fma.rn.f32x2 + ex2); P is written as packed 16-bit
//                       pairs over the S columns with tcgen05.st; O is rescaled
//                       only when the row max grew by more than 2^8; the same
//                       warpgroup finally writes O and LSE.
// P never leaves TMEM: the second MMA takes its A operand from TMEM.
#include <cuda.h>

#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace ttattn {
namespace {

constexpr int BM = 128;      // rows of one query tile (= TMEM lanes)
constexpr int QT = 2;        // query tiles per CTA
constexpr int BN = 128;      // keys per tile
constexpr int NSTAGE = 2;    // K/V ring depth
constexpr int kThreads = 384;  // 2 softmax warpgroups + 1 warpgroup holding the producer and issuer warps
constexpr int kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
#ifndef TT_POLY_NUM
#define TT_POLY_NUM 0
#endif
#ifndef TT_POLY_DEN
#define TT_POLY_DEN 4
#endif
constexpr int kPolyNum = TT_POLY_NUM, kPolyDen = TT_POLY_DEN;

// Developer aid, compiled out by default: with -DTT_ATTN_PROFILE the first CTA
// writes clock64() stamps of its pipeline phases to the buffer passed as `status`
// (int64 [3][64][8]: softmax warpgroup 0, softmax warpgroup 1, issuer).
#ifdef TT_ATTN_PROFILE
#define TT_STAMP(who, j, slot)                                                                          \
  do {                                                                                                  \
    if (prof && (j) < 64) prof[((who)*64 + (j)) * 8 + (slot)] = clock64();                              \
  } while (0)
#else
#define TT_STAMP(who, j, slot) \
  do {                         \
  } while (0)
#endif

struct __align__(8) SmemCtl {
  uint64_t q_full;
  uint64_t k_full[NSTAGE], k_empty[NSTAGE], v_full[NSTAGE], v_empty[NSTAGE];
  uint64_t s_full[QT], p_full[QT], o_full[QT];
  uint32_t tmem_base;
  int abort_flag;
};

template <int D>
constexpr int tile_bytes() {
  return BM * D * 2;
}
template <int D>
constexpr int smem_bytes() {
  return (QT + 2 * NSTAGE) * tile_bytes<D>() + 1024 /*alignment slack*/ + 256 /*SmemCtl*/;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  } else {
    __half2 t = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  }
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
    fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const FwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
#ifdef TT_ATTN_PROFILE
  const long long t_entry = clock64();
#endif
  // 128-byte-swizzled tiles must start on a 1024-byte boundary.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int TB = tile_bytes<D>();
  uint8_t* sQ = smem;                    // QT tiles
  uint8_t* sK = smem + QT * TB;          // NSTAGE tiles
  uint8_t* sV = sK + NSTAGE * TB;        // NSTAGE tiles
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(sV + NSTAGE * TB);
  volatile int* abort_flag = &ctl->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // Heaviest (latest) causal tiles are launched first.
  const int mp = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = h / (a.Hq / a.Hkv);
  const int row0 = mp * (QT * BM);

  int kv_len = a.Skv;
  if (a.kv_lens) {
    int l = a.kv_lens[b];
    kv_len = l < 0 ? 0 : (l < a.Skv ? l : a.Skv);
  }
  // Number of key tiles each query tile walks (0 for a tile wholly beyond Lq).
  auto tiles_of = [&](int t) {
    int kv_end = kv_len;
    if (a.causal && row0 + t * BM + BM < kv_end) kv_end = row0 + t * BM + BM;
    return (row0 + t * BM < a.Lq) ? (kv_end + BN - 1) / BN : 0;
  };
  const int nt0 = tiles_of(0), nt1 = tiles_of(1);
  const int n_max = nt0 > nt1 ? nt0 : nt1;
  auto nt = [&](int t) { return t == 0 ? nt0 : nt1; };

  constexpr int HALVES = D / 64;  // 64-element (128-byte) column blocks per row
  constexpr int HALF_BYTES = BM * 128;

  if (warp == 8 && lane == 0) {
    ptx::mbar_init(&ctl->q_full, 1);
#pragma unroll
    for (int i = 0; i < NSTAGE; ++i) {
      ptx::mbar_init(&ctl->k_full[i], 1);
      ptx::mbar_init(&ctl->k_empty[i], 1);
      ptx::mbar_init(&ctl->v_full[i], 1);
      ptx::mbar_init(&ctl->v_empty[i], 1);
    }
#pragma unroll
    for (int t = 0; t < QT; ++t) {
      ptx::mbar_init(&ctl->s_full[t], 1);
      ptx::mbar_init(&ctl->p_full[t], BM);
      ptx::mbar_init(&ctl->o_full[t], 1);
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    // The first loads do not depend on anything the other warps set up: start
    // them before the CTA-wide barrier so that their latency overlaps the TMEM
    // allocation.
    if (n_max > 0) {
      ptx::mbar_arrive_expect_tx(&ctl->q_full, QT * TB);
#pragma unroll
      for (int t = 0; t < QT; ++t)
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf)
          ptx::tma_load_4d(sQ + t * TB + hf * HALF_BYTES, &tmQ, &ctl->q_full, hf * 64, row0 + t * BM, h, b);
      ptx::mbar_arrive_expect_tx(&ctl->k_full[0], TB);
#pragma unroll
      for (int hf = 0; hf < HALVES; ++hf)
        ptx::tma_load_4d(sK + hf * HALF_BYTES, &tmK, &ctl->k_full[0], hf * 64, 0, hk, b);
      ptx::mbar_arrive_expect_tx(&ctl->v_full[0], TB);
#pragma unroll
      for (int hf = 0; hf < HALVES; ++hf)
        ptx::tma_load_4d(sV + hf * HALF_BYTES, &tmV, &ctl->v_full[0], hf * 64, 0, hk, b);
    }
  }
  if (warp == 9) {
    ptx::tmem_alloc(&ctl->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
#ifdef TT_ATTN_PROFILE
  long long* prof = (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 &&
                     (warp == 0 || warp == 4 || warp == 9) && a.status)
                        ? reinterpret_cast<long long*>(a.status)
                        : nullptr;
  // per-CTA summary for the CTAs of (head 0, batch 0): [blockIdx.x][8] after the per-iteration area
  long long* psum = (blockIdx.y == 0 && blockIdx.z == 0 && tid == 0 && a.status && blockIdx.x < 32)
                        ? reinterpret_cast<long long*>(a.status) + 3 * 64 * 8 + blockIdx.x * 8
                        : nullptr;
  if (psum) psum[0] = t_entry, psum[1] = clock64(), psum[7] = nt1;
#endif
  // TMEM columns: S_t (fp32, 128) at t*128, P_t (16-bit pairs) overlays S_t[0,64); O_t (fp32, D) at 256 + t*D.

  // Register budget: the softmax warpgroups hold a whole 128-column S row per
  // thread; the producer / issuer warpgroup needs almost nothing.
  if (warp >= 8) {
    ptx::setmaxnreg_dec<72>();
  if (warp == 8) {
    // ------------------------------------------------------------ producer --
    if (lane == 0 && n_max > 0) {
      for (int j = 1; j < n_max; ++j) {  // tile 0 was requested during set-up
        const int st = j % NSTAGE;
        const uint32_t ph = static_cast<uint32_t>((j / NSTAGE) & 1);
        if (!ptx::mbar_wait(&ctl->k_empty[st], ph ^ 1, abort_flag)) break;
        ptx::mbar_arrive_expect_tx(&ctl->k_full[st], TB);
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf)
          ptx::tma_load_4d(sK + st * TB + hf * HALF_BYTES, &tmK, &ctl->k_full[st], hf * 64, j * BN, hk, b);
        if (!ptx::mbar_wait(&ctl->v_empty[st], ph ^ 1, abort_flag)) break;
        ptx::mbar_arrive_expect_tx(&ctl->v_full[st], TB);
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf)
          ptx::tma_load_4d(sV + st * TB + hf * HALF_BYTES, &tmV, &ctl->v_full[st], hf * 64, j * BN, hk, b);
      }
    }
  } else if (warp == 9) {
    // -------------------------------------------------------------- issuer --
    // Order per key tile j:  PV(0,j)  QK(0,j+1)  PV(1,j)  QK(1,j+1): while one
    // warpgroup is in its softmax the tensor pipe works for the other.  MMAs of
    // one thread execute in issue order, so QK(t,j+1) overwriting S_t / P_t
    // cannot pass PV(t,j) that still reads P_t.
    if (lane == 0 && n_max > 0) {
      // A negative scale is folded into the sign of Q so that the softmax
      // always works with a non-negative multiplier.
      const uint32_t neg = a.scale < 0.f ? (1u << 13) : 0u;
      const uint32_t idesc_qk = ptx::make_idesc_f16(BM, BN, BF16 ? 1 : 0, 0, 0) | neg;
      const uint32_t idesc_pv = ptx::make_idesc_f16(BM, D, BF16 ? 1 : 0, 0, 1);
      // Descriptor words are prepared once; inside the loops stepping to the next
      // k-slice or ring stage is a single 32-bit add, so that the issuing thread
      // keeps pace with the tensor pipe (one 128x128x16 MMA per 64 cycles).
      constexpr uint32_t kHi = ptx::smem_desc_hi_sw128(1024);
      const uint32_t qlo = ptx::smem_desc_lo(ptx::smem_u32(sQ), 16);
      const uint32_t klo = ptx::smem_desc_lo(ptx::smem_u32(sK), 16);
      const uint32_t vlo = ptx::smem_desc_lo(ptx::smem_u32(sV), HALF_BYTES);
      bool ok = ptx::mbar_wait(&ctl->q_full, 0, abort_flag);

      auto issue_qk = [&](int t, int j) -> bool {
        const int st = j % NSTAGE;
        if (!ptx::mbar_wait(&ctl->k_full[st], static_cast<uint32_t>((j / NSTAGE) & 1), abort_flag)) return false;
        TT_STAMP(2, j, t * 4 + 3);
        ptx::tc_fence_after();
        const uint32_t a0 = qlo + t * (TB >> 4), b0 = klo + st * (TB >> 4), d = tmem + t * 128;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          // K-major operands: 64-element halves HALF_BYTES apart, 32 bytes per k-step
          const uint32_t off = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;
          ptx::mma_ss2(d, a0 + off, kHi, b0 + off, kHi, idesc_qk, ks > 0 ? 1u : 0u);
        }
        ptx::mma_commit(&ctl->s_full[t]);
        TT_STAMP(2, j, t * 4 + 2);
        return true;
      };
      auto issue_pv = [&](int t, int j) -> bool {
        const int st = j % NSTAGE;
        if (!ptx::mbar_wait(&ctl->v_full[st], static_cast<uint32_t>((j / NSTAGE) & 1), abort_flag)) return false;
        if (!ptx::mbar_wait(&ctl->p_full[t], static_cast<uint32_t>(j & 1), abort_flag)) return false;
        TT_STAMP(2, j, t * 4 + 0);
        ptx::tc_fence_after();
        const uint32_t b0 = vlo + st * (TB >> 4), d = tmem + 256 + t * D, a0 = tmem + t * 128;
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          // V is N(=D)-contiguous: 16 keys per k-step = 2048 bytes; the two
          // 64-wide column blocks of D=128 are HALF_BYTES apart (LBO).
          ptx::mma_ts2(d, a0 + ks * 8, b0 + ks * (2048 >> 4), kHi, idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        }
        TT_STAMP(2, j, t * 4 + 1);
        return true;
      };

#pragma unroll
      for (int t = 0; t < QT && ok; ++t)
        if (nt(t) > 0) ok = issue_qk(t, 0);
      if (ok) ptx::mma_commit(&ctl->k_empty[0]);
      for (int j = 0; j < n_max && ok; ++j) {
        const int last_pv = (j < nt1) ? 1 : 0;
        const int last_qk = (j + 1 < nt1) ? 1 : 0;
#pragma unroll
        for (int t = 0; t < QT && ok; ++t) {
          if (j < nt(t)) {
            ok = issue_pv(t, j);
            if (!ok) break;
            if (j == nt(t) - 1) ptx::mma_commit(&ctl->o_full[t]);
            if (t == last_pv) ptx::mma_commit(&ctl->v_empty[j % NSTAGE]);
          }
          if (j + 1 < nt(t)) {
            ok = issue_qk(t, j + 1);
            if (!ok) break;
            if (t == last_qk) ptx::mma_commit(&ctl->k_empty[(j + 1) % NSTAGE]);
          }
        }
      }
    }
  }
  } else {
    ptx::setmaxnreg_inc<216>();
    // ------------------------------------------------------------- softmax --
    const int t = warp >> 2;                     // query tile of this warpgroup
    const int r_in = tid & (BM - 1);             // row within the tile = TMEM lane
    const int row = row0 + t * BM + r_in;        // global query row
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + t * 128 + lane_addr;
    const uint32_t tO = tmem + 256 + t * D + lane_addr;
    const float c = fabsf(a.scale) * kLog2e;
    const float2 c2 = make_float2(c, c);
    const int n_t = nt(t);
    float m_ref = -INFINITY;  // reference max, in scaled log2 units
    float2 l2 = make_float2(0.f, 0.f);
    bool ok = true;
    uint32_t s[BN];

    for (int j = 0; j < n_t && ok; ++j) {
      TT_STAMP(t, j, 0);
      ok = ptx::mbar_wait(&ctl->s_full[t], static_cast<uint32_t>(j & 1), abort_flag);
      if (!ok) break;
      TT_STAMP(t, j, 1);
      ptx::tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) ptx::tmem_ld32p(tS + cc * 32, s + cc * 32);
      ptx::tmem_wait_ld();
      TT_STAMP(t, j, 2);

      const int col0 = j * BN;
      const bool mask_tile = (col0 + BN > kv_len) || (a.causal && col0 + BN - 1 > row0 + t * BM);
      if (mask_tile) {
        // Highest valid column of this row within the tile.
        int lim = kv_len - 1 - col0;
        if (a.causal && row - col0 < lim) lim = row - col0;
#pragma unroll
        for (int i = 0; i < BN; ++i)
          if (i > lim) s[i] = 0xff800000u;  // -inf
      }
      // eight independent 3-input max chains over the 128 columns
      float mx[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) mx[q] = ptx::max3(__uint_as_float(s[q]), __uint_as_float(s[q + 8]), -INFINITY);
#pragma unroll
      for (int i = 16; i < BN; i += 16)
#pragma unroll
        for (int q = 0; q < 8; ++q) mx[q] = ptx::max3(mx[q], __uint_as_float(s[i + q]), __uint_as_float(s[i + q + 8]));
      const float x_max =
          ptx::max3(ptx::max3(mx[0], mx[1], mx[2]), ptx::max3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7])) * c;
      if (j == 0) {
        m_ref = x_max;
      } else {
        const bool grow = x_max - m_ref > kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = grow ? x_max : m_ref;
          const float alpha = grow ? ptx::ex2(m_ref - m_new) : 1.f;
          uint32_t r[32];
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc) {
            ptx::tmem_ld32(tO + cc * 32, r);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            ptx::tmem_st32(tO + cc * 32, r);
          }
          l2.x *= alpha, l2.y *= alpha;
          m_ref = m_new;
        }
      }
      // P = 2^(c*s - m_ref) in packed fp32 pairs; two halves of 64 columns so that
      // the packed 16-bit P of the first half is stored while the second is computed.
      TT_STAMP(t, j, 3);
      const float2 nm2 = make_float2(-m_ref, -m_ref);
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const int e = hf * 64 + i;
          float2 x = ptx::fma2(make_float2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), c2, nm2);
          // kPolyNum of every kPolyDen pairs take their exponential on the FMA
          // pipe, the rest on the special-function unit, so that both pipes work.
          float2 p;
          if ((i >> 1) % kPolyDen < kPolyNum) {
            p = ptx::ex2_poly2(x);
          } else {
            p = make_float2(ptx::ex2(x.x), ptx::ex2(x.y));
          }
          l2 = ptx::add2(l2, p);
          pk[i >> 1] = pack2<BF16>(p.x, p.y);
        }
        ptx::tmem_st32(tS + hf * 32, pk);
      }
      TT_STAMP(t, j, 4);
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(&ctl->p_full[t]);
      TT_STAMP(t, j, 5);
    }

    // epilogue: O / l -> global, LSE
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    T* orow = reinterpret_cast<T*>(a.o) + b * a.os.b + h * a.os.h + static_cast<int64_t>(row) * a.os.s;
    const float l = l2.x + l2.y;
    if (n_t > 0) {
#ifdef TT_ATTN_PROFILE
      if (psum) psum[2] = clock64();
#endif
      if (ok) ok = ptx::mbar_wait(&ctl->o_full[t], 0, abort_flag);
#ifdef TT_ATTN_PROFILE
      if (psum) psum[3] = clock64();
#endif
      ptx::tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint32_t r[32];
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) {
        ptx::tmem_ld32(tO + cc * 32, r);
        ptx::tmem_wait_ld();
        if (ok && row < a.Lq) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack2<BF16>(__uint_as_float(r[i + 0]) * inv, __uint_as_float(r[i + 1]) * inv);
            w.y = pack2<BF16>(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
            w.z = pack2<BF16>(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
            w.w = pack2<BF16>(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + cc * 32 + i) = w;
          }
        }
      }
      if (ok && row < a.Lq && a.lse)
        a.lse[(static_cast<int64_t>(b) * a.Hq + h) * a.Lq + row] = l > 0.f ? (m_ref + log2f(l)) * kLn2 : -INFINITY;
    } else if (row < a.Lq) {
      // no participating key: O = 0, LSE = -inf
#pragma unroll
      for (int i = 0; i < D; i += 8) *reinterpret_cast<uint4*>(orow + i) = make_uint4(0, 0, 0, 0);
      if (a.lse) a.lse[(static_cast<int64_t>(b) * a.Hq + h) * a.Lq + row] = -INFINITY;
    }
  }

#ifdef TT_ATTN_PROFILE
  if (psum) psum[4] = clock64();
#endif
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
#ifdef TT_ATTN_PROFILE
  if (psum) psum[5] = clock64();
#endif
  if (tid == 0 && ctl->abort_flag && a.status) atomicOr(a.status, kStatusWaitExpired);
}

// ------------------------------------------------------------------ host ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// [B, H, S, D] tensor, box = 64 (D) x 128 (S) x 1 x 1, 128-byte swizzle, zero fill.
bool make_map(CUtensorMap* m, int dtype, const void* ptr, int D, int S, int H, int B, const Str3& st) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(H),
                        static_cast<cuuint64_t>(B)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(st.s) * 2, static_cast<cuuint64_t>(st.h) * 2,
                           static_cast<cuuint64_t>(st.b) * 2};
  cuuint32_t box[4] = {64, 128, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, dtype == TT_ATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int D, bool BF16>
cudaError_t launch_t(const FwdArgs& a, int dtype, cudaStream_t stream) {
  CUtensorMap tq, tk, tv;
  if (!make_map(&tq, dtype, a.q, D, a.Lq, a.Hq, a.B, a.qs) || !make_map(&tk, dtype, a.k, D, a.Skv, a.Hkv, a.B, a.ks) ||
      !make_map(&tv, dtype, a.v, D, a.Skv, a.Hkv, a.B, a.vs))
    return cudaErrorInvalidValue;
  auto kern = fwd_tc_kernel<D, BF16>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<D>());
  if (e != cudaSuccess) return e;
  dim3 grid((a.Lq + QT * BM - 1) / (QT * BM), a.Hq, a.B);
  kern<<<grid, kThreads, smem_bytes<D>(), stream>>>(tq, tk, tv, a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fwd_tc(int dtype, int D, const FwdArgs& a, int /*device*/, cudaStream_t stream) {
  const bool bf = dtype == TT_ATTN_BF16;
  if (D == 128) return bf ? launch_t<128, true>(a, dtype, stream) : launch_t<128, false>(a, dtype, stream);
  if (D == 64) return bf ? launch_t<64, true>(a, dtype, stream) : launch_t<64, false>(a, dtype, stream);
  return cudaErrorInvalidValue;
}

}  // namespace ttattn
