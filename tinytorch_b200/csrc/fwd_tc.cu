// Prefill forward for fp16 / bf16 on sm_100a tensor cores.
//
// Replaces the score-materialising composition of FuncSDPAttention::forward
// (reference: src/Function/FuncNNLayer.h:231-266) by one fused kernel that never
// writes the [L,S] score matrix to HBM.
//
// Persistent kernel, one CTA per SM, all 512 TMEM columns.  A work item is a pair
// of 128-row query tiles of one (batch, head); CTAs draw items from a global
// counter, heads in order and, within a head, the longest (latest causal) pair
// first, so that the CTAs running at any moment share few heads' K/V in L2 and
// the last items to be drawn are the shortest.
//   warp 8   producer : draws items and publishes them to the other warps; TMA
//                       tiled loads (128-byte swizzle, one copy per CTA) of the item's
//                       two Q tiles and of each K and V tile into a 2-stage ring.
//                       It runs ahead: the next item's Q and first K/V tiles are
//                       requested while the current item is still being computed.
//   warp 9   issuer   : one thread issues tcgen05.mma; S_t = Q_t.K^T accumulates in
//                       TMEM columns [t*128, t*128+128), O_t += P_t.V in columns
//                       [256 + t*D, 256 + (t+1)*D).  The two tiles are interleaved
//                       (PV_0 QK_0' PV_1 QK_1') so that the tensor pipe computes for
//                       one tile while the other tile's warpgroup is in its softmax.
//   warps 0-3 / 4-7   : softmax warpgroup of tile 0 / 1.  Thread r owns query row r
//                       (= TMEM lane r): it reads the whole 128-column S row with
//                       tcgen05.ld, so the row max and row sum need no cross-thread
//                       reduction in this layout; exponentials run as packed fp32
//                       pairs (fma.rn.f32x2 + ex2); P is written as packed 16-bit
//                       pairs over the S columns with tcgen05.st; O is rescaled
//                       only when the row max grew by more than 2^8; the same
//                       warpgroup writes O and LSE while the issuer already starts
//                       the next item's first QK.
// P never leaves TMEM: the second MMA takes its A operand from TMEM.
// Every mbarrier wait is bounded; an expired wait sets the status word and makes
// the CTA unwind.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace ttattn {
namespace {

constexpr int BM = 128;      // rows of one query tile (= TMEM lanes)
constexpr int QT = 2;        // query tiles per item
constexpr int BN = 128;      // keys per tile
constexpr int NSTAGE = 2;    // K/V ring depth
constexpr int kThreads = 384;  // 2 softmax warpgroups + 1 warpgroup holding the producer and issuer warps
constexpr int kTmemCols = 512;
constexpr int kItemConsumers = 1 + QT * BM;  // issuer thread + every softmax thread
#ifndef TT_FWD_TAIL_WAVES
#define TT_FWD_TAIL_WAVES 2
#endif
constexpr int kTailWaves = TT_FWD_TAIL_WAVES;  // waves of work items at the end that are ordered longest first across heads

struct __align__(8) SmemCtl {
  uint64_t q_full[QT], q_empty[QT];  // per query tile: tile 0 of the next item is loaded while tile 1 still works
  uint64_t k_full[NSTAGE], k_empty[NSTAGE], v_full[NSTAGE], v_empty[NSTAGE];
  uint64_t s_full[QT], p_full[QT], o_full[QT];
  uint64_t item_full[2], item_empty[2];
  int item[2];
  int item_nt0[2];  // key tiles of query tile 0 of the published item (the issuer's look-ahead needs only this)
  uint32_t tmem_base;
  int abort_flag;
};

template <int D>
constexpr int tile_bytes() {
  return BM * D * 2;
}
constexpr int kStageBytes = BM * 128;  // per warpgroup: one 64-column block of an O tile
template <int D>
constexpr int smem_bytes() {
  return (QT + 2 * NSTAGE) * tile_bytes<D>() + QT * kStageBytes + 1024 /*alignment slack*/ + 256 /*SmemCtl*/;
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

// One work item, decoded identically by every role.
struct Item {
  int b, h, hk, row0, kv_len, nt0, nt1, n_max, shift;
};

// GEN: the general variant of the kernel (a mask and / or a causal triangle that is
// not top-left aligned); the fast variant compiles all of that out.
template <bool GEN>
__device__ __forceinline__ Item decode_item(const FwdArgs& a, int w, int n_pairs) {
  Item it;
  // Heads in order, the longest (latest causal) pair of a head first: the CTAs running at any moment share few
  // heads' K/V in L2.  Only the last items are ordered differently: over the final kTailWaves waves the pairs of
  // the remaining heads are taken longest first ACROSS those heads, so that what is drawn last is short and the
  // CTAs finish together (in head order the last head's longest pair, an eighth of a CTA's whole share of
  // config 2, would be drawn when most CTAs are nearly done).  Those heads' K/V together fit L2.
  const int n_heads = a.B * a.Hq;
  int tail_heads = (kTailWaves * static_cast<int>(gridDim.x) + n_pairs - 1) / n_pairs;
  if (tail_heads > n_heads) tail_heads = n_heads;
  const int w0 = (n_heads - tail_heads) * n_pairs;
  int bh, mp;
  if (w < w0) {
    bh = w / n_pairs;
    mp = n_pairs - 1 - (w - bh * n_pairs);
  } else {
    const int x = w - w0, rank = x / tail_heads;
    bh = n_heads - tail_heads + (x - rank * tail_heads);
    mp = n_pairs - 1 - rank;
  }
  it.b = bh / a.Hq;
  it.h = bh - it.b * a.Hq;
  it.hk = it.h / (a.Hq / a.Hkv);
  it.row0 = mp * (QT * BM);
  int kv_len = a.Skv;
  if (a.kv_lens) {
    int l = a.kv_lens[it.b];
    kv_len = l < 0 ? 0 : (l < a.Skv ? l : a.Skv);
  }
  it.kv_len = kv_len;
  // Number of key tiles each query tile walks (0 for a tile wholly beyond Lq).
  int e0 = kv_len, e1 = kv_len;
  it.shift = GEN ? causal_shift(a.causal, kv_len, a.Lq) : 0;  // key j participates iff j <= i + shift
  if (a.causal) {
    int c0 = it.row0 + BM + it.shift, c1 = it.row0 + 2 * BM + it.shift;
    if (GEN) c0 = c0 > 0 ? c0 : 0, c1 = c1 > 0 ? c1 : 0;
    if (c0 < e0) e0 = c0;
    if (c1 < e1) e1 = c1;
  }
  it.nt0 = (it.row0 < a.Lq) ? (e0 + BN - 1) / BN : 0;
  it.nt1 = (it.row0 + BM < a.Lq) ? (e1 + BN - 1) / BN : 0;
  it.n_max = it.nt0 > it.nt1 ? it.nt0 : it.nt1;
  return it;
}

// s[e] <- c * s[e] + mask(row, col0 + e) * log2(e) for the 128 scores of one
// query row; `off` is the mask's element offset of (row, col0) and n_valid the
// number of keys that exist from col0 on.  16-byte loads when the row segment is
// whole and aligned, element loads otherwise.
template <typename T>
__device__ __forceinline__ void add_mask_row(uint32_t (&s)[BN], const MaskArgs& m, int64_t off, int n_valid, float c) {
  const int esz = m.kind == TT_ATTN_MASK_BOOL ? 1 : (m.kind == TT_ATTN_MASK_ADD_F32 ? 4 : 2);
  const uint8_t* base = reinterpret_cast<const uint8_t*>(m.ptr) + off * esz;
  const bool fast = n_valid >= BN && (reinterpret_cast<uintptr_t>(base) & 15) == 0;
#pragma unroll
  for (int ch = 0; ch < BN / 16; ++ch) {
    float bias[16];
    if (fast) {
      if (m.kind == TT_ATTN_MASK_BOOL) {
        const uint4 v = *reinterpret_cast<const uint4*>(base + ch * 16);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) bias[i] = ((w[i >> 2] >> ((i & 3) * 8)) & 0xffu) ? 0.f : -INFINITY;
      } else if (m.kind == TT_ATTN_MASK_ADD_F32) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 v = *reinterpret_cast<const float4*>(base + ch * 64 + q * 16);
          bias[q * 4 + 0] = v.x * kLog2e, bias[q * 4 + 1] = v.y * kLog2e;
          bias[q * 4 + 2] = v.z * kLog2e, bias[q * 4 + 3] = v.w * kLog2e;
        }
      } else {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const uint4 v = *reinterpret_cast<const uint4*>(base + ch * 32 + q * 16);
          const T* t = reinterpret_cast<const T*>(&v);
#pragma unroll
          for (int i = 0; i < 8; ++i) bias[q * 8 + i] = to_f32<T>(t[i]) * kLog2e;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) bias[i] = (ch * 16 + i < n_valid) ? mask_bias2<T>(m, off + ch * 16 + i) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) s[ch * 16 + i] = __float_as_uint(fmaf(__uint_as_float(s[ch * 16 + i]), c, bias[i]));
  }
}

template <int D, bool BF16, bool GEN>
__global__ void __launch_bounds__(kThreads, 1)
    fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                  const FwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles must start on a 1024-byte boundary.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int TB = tile_bytes<D>();
  uint8_t* sQ = smem;                    // QT tiles
  uint8_t* sK = smem + QT * TB;          // NSTAGE tiles
  uint8_t* sV = sK + NSTAGE * TB;        // NSTAGE tiles
  uint8_t* sO = sV + NSTAGE * TB;        // QT staging blocks for the O stores
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(sO + QT * kStageBytes);
  volatile int* abort_flag = &ctl->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int n_pairs = (a.Lq + QT * BM - 1) / (QT * BM);
  const int n_items = n_pairs * a.Hq * a.B;

  constexpr int HALVES = D / 64;  // 64-element (128-byte) column blocks per row
  constexpr int HALF_BYTES = BM * 128;

  if (warp == 8 && lane == 0) {
#pragma unroll
    for (int t = 0; t < QT; ++t) {
      ptx::mbar_init(&ctl->q_full[t], 1);
      ptx::mbar_init(&ctl->q_empty[t], 1);
    }
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
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&ctl->item_full[i], 1);
      ptx::mbar_init(&ctl->item_empty[i], kItemConsumers);
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::tma_prefetch_desc(&tmQ);
    ptx::tma_prefetch_desc(&tmK);
    ptx::tma_prefetch_desc(&tmV);
    ptx::tma_prefetch_desc(&tmO);
  }
  if (warp == 9) {
    ptx::tmem_alloc(&ctl->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;

  // Register budget: the softmax warpgroups hold a whole 128-column S row per
  // thread; the producer / issuer warpgroup needs little.
  if (warp >= 8) {
    // (D = 128: 224 + 224 + 56 registers per thread over the three warpgroups; D = 64, whose issuing loop
    // carries the look-ahead at item boundaries: 216 + 216 + 72.  Both add up to the 168 x 384 registers
    // the CTA was launched with, so the increase below can always be served.)
    ptx::setmaxnreg_dec<D == 128 ? 56 : 72>();
    if (warp == 8) {
      // ---------------------------------------------------------- producer --
      if (lane == 0) {
        uint32_t g = 0;             // K/V tiles requested so far (ring position)
        uint32_t qc0 = 0, qc1 = 0;  // items whose Q tile 0 / 1 was requested so far
        for (uint32_t i = 0;; ++i) {
          int w = atomicAdd(a.sched, 1);
          if (w >= n_items) w = -1;
          const int slot = i & 1;
          Item it{};
          if (w >= 0) it = decode_item<GEN>(a, w, n_pairs);
          if (!ptx::mbar_wait(&ctl->item_empty[slot], ((i >> 1) & 1) ^ 1, abort_flag)) break;
          ctl->item[slot] = w;
          ctl->item_nt0[slot] = w >= 0 ? it.nt0 : 0;
          ptx::mbar_arrive(&ctl->item_full[slot]);
          if (w < 0) break;
          if (it.n_max == 0) continue;
          bool ok = true;
          // a Q tile is loaded only if it has key tiles to walk; tile 0 goes first and, with the first K tile,
          // ahead of tile 1: the issuer starts tile 0 of this item while tile 1 of the previous one still works
          auto load_q = [&](int t, uint32_t& qc) {
            if ((t == 0 ? it.nt0 : it.nt1) == 0) return true;
            if (!ptx::mbar_wait(&ctl->q_empty[t], (qc & 1) ^ 1, abort_flag)) return false;
            ptx::mbar_arrive_expect_tx(&ctl->q_full[t], TB);
#pragma unroll
            for (int hf = 0; hf < HALVES; ++hf)
              ptx::tma_load_4d(sQ + t * TB + hf * HALF_BYTES, &tmQ, &ctl->q_full[t], hf * 64, it.row0 + t * BM, it.h, it.b);
            ++qc;
            return true;
          };
          if (!(ok = load_q(0, qc0))) break;
          for (int j = 0; j < it.n_max; ++j, ++g) {
            const int st = g % NSTAGE;
            const uint32_t ph = (g / NSTAGE) & 1;
            if (!(ok = ptx::mbar_wait(&ctl->k_empty[st], ph ^ 1, abort_flag))) break;
            ptx::mbar_arrive_expect_tx(&ctl->k_full[st], TB);
#pragma unroll
            for (int hf = 0; hf < HALVES; ++hf)
              ptx::tma_load_4d(sK + st * TB + hf * HALF_BYTES, &tmK, &ctl->k_full[st], hf * 64, j * BN, it.hk, it.b);
            if (j == 0 && !(ok = load_q(1, qc1))) break;
            if (!(ok = ptx::mbar_wait(&ctl->v_empty[st], ph ^ 1, abort_flag))) break;
            ptx::mbar_arrive_expect_tx(&ctl->v_full[st], TB);
#pragma unroll
            for (int hf = 0; hf < HALVES; ++hf)
              ptx::tma_load_4d(sV + st * TB + hf * HALF_BYTES, &tmV, &ctl->v_full[st], hf * 64, j * BN, it.hk, it.b);
          }
          if (!ok) break;
        }
      }
    } else if (warp == 9) {
      // ------------------------------------------------------------ issuer --
      // Order per key tile j:  PV(0,j)  QK(0,j+1)  PV(1,j)  QK(1,j+1).  MMAs of one
      // thread execute in issue order, so QK(t,j+1) overwriting S_t / P_t cannot
      // pass PV(t,j) that still reads P_t, and the first QK of the next item
      // cannot pass the last PV of this one.
      // The whole warp runs the loop (waits included, made uniform by a vote); one elected lane issues.
      {
        const bool leader = ptx::elect_one();
        auto uwait = [&](uint64_t* bar, uint32_t parity) {
          return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity, abort_flag)) != 0;
        };
        // A negative scale is folded into the sign of Q so that the softmax
        // always works with a non-negative multiplier.
        const uint32_t neg = a.scale < 0.f ? (1u << 13) : 0u;
        const uint32_t idesc_qk = ptx::make_idesc_f16(BM, BN, BF16 ? 1 : 0, 0, 0) | neg;
        const uint32_t idesc_pv = ptx::make_idesc_f16(BM, D, BF16 ? 1 : 0, 0, 1);
        // Descriptor words are prepared once; stepping to the next k-slice or ring
        // stage is a single 32-bit add, so that this thread keeps pace with the
        // tensor pipe (one 128x128x16 MMA per 64 cycles).
        constexpr uint32_t kHi = ptx::smem_desc_hi_sw128(1024);
        const uint32_t qlo = ptx::smem_desc_lo(ptx::smem_u32(sQ), 16);
        const uint32_t klo = ptx::smem_desc_lo(ptx::smem_u32(sK), 16);
        const uint32_t vlo = ptx::smem_desc_lo(ptx::smem_u32(sV), HALF_BYTES);

        uint32_t g0 = 0;        // ring position of the item's first key tile
        uint32_t c0 = 0, c1 = 0;  // softmax iterations completed per tile (p_full phases)
        uint32_t qc0 = 0, qc1 = 0;  // items whose Q tile 0 / 1 was used so far (q_full phases)
        bool ok = true;
        bool pre0 = false;      // the first QK of tile 0 of the coming item has been issued already

        auto wait_k = [&](uint32_t g) { return uwait(&ctl->k_full[g % NSTAGE], (g / NSTAGE) & 1); };
        auto issue_qk = [&](int t, uint32_t g) {
          const uint32_t a0 = qlo + t * (TB >> 4), b0 = klo + (g % NSTAGE) * (TB >> 4), d = tmem + t * 128;
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            // K-major operands: 64-element halves HALF_BYTES apart, 32 bytes per k-step
            const uint32_t off = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;
            if (leader) ptx::mma_ss2(d, a0 + off, kHi, b0 + off, kHi, idesc_qk, ks > 0 ? 1u : 0u);
          }
          if (leader) ptx::mma_commit(&ctl->s_full[t]);
        };
        auto issue_pv = [&](int t, uint32_t g, bool first) {
          const uint32_t b0 = vlo + (g % NSTAGE) * (TB >> 4), d = tmem + 256 + t * D, a0 = tmem + t * 128;
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks) {
            // V is N(=D)-contiguous: 16 keys per k-step = 2048 bytes; the two
            // 64-wide column blocks of D=128 are HALF_BYTES apart (LBO).
            if (leader) ptx::mma_ts2(d, a0 + ks * 8, b0 + ks * (2048 >> 4), kHi, idesc_pv, (!first || ks > 0) ? 1u : 0u);
          }
        };

        // first QK of tile t of an item whose first key tile sits at ring position g
        auto first_qk = [&](int t, uint32_t& qc, uint32_t g, int nt_t) {
          if (!uwait(&ctl->q_full[t], qc & 1)) return false;
          ++qc;
          if (!wait_k(g)) return false;
          ptx::tc_fence_after();
          issue_qk(t, g);
          if (leader && nt_t == 1) ptx::mma_commit(&ctl->q_empty[t]);  // the only QK of this tile
          return true;
        };
        // non-blocking probe, the same answer in every lane
        auto utest = [&](uint64_t* bar, uint32_t parity) {
          return __all_sync(0xffffffffu, ptx::mbar_test(bar, parity)) != 0;
        };

        for (uint32_t i = 0; ok; ++i) {
          const int slot = i & 1;
          if (!uwait(&ctl->item_full[slot], (i >> 1) & 1)) break;
          const int w = ctl->item[slot];
          __syncwarp();  // every lane has read the slot before it is handed back
          if (leader) ptx::mbar_arrive(&ctl->item_empty[slot]);
          if (w < 0) break;
          const Item it = decode_item<GEN>(a, w, n_pairs);
          if (it.n_max == 0) continue;
          const int nt0 = it.nt0, nt1 = it.nt1, n_max = it.n_max;
          auto nt = [&](int t) { return t == 0 ? nt0 : nt1; };

          if (nt0 > 0 && !pre0 && !(ok = first_qk(0, qc0, g0, nt0))) break;
          pre0 = false;
          if (nt1 > 0 && !(ok = first_qk(1, qc1, g0, nt1))) break;
          if (leader) ptx::mma_commit(&ctl->k_empty[g0 % NSTAGE]);
          // Tile 0 is done and tile 1 still has key tiles to walk (the causal diagonal): if the next item is
          // known and its Q tile 0 and first K tile have landed, start its tile 0 now, so that warpgroup 0
          // does not sit idle for tile 1's last iteration.  Nothing here blocks.  (S_0 is free: its last P has
          // been consumed in issue order; O_0 is not written before warpgroup 0 delivers the next P, i.e.
          // after its epilogue.)
          auto try_pre0 = [&]() {
            if (pre0 || nt0 == 0) return;
            const int nslot = (i + 1) & 1;
            if (!utest(&ctl->item_full[nslot], ((i + 1) >> 1) & 1)) return;
            const int nt0n = ctl->item_nt0[nslot];
            const uint32_t gn = g0 + n_max;
            if (nt0n <= 0 || !utest(&ctl->q_full[0], qc0 & 1) || !utest(&ctl->k_full[gn % NSTAGE], (gn / NSTAGE) & 1))
              return;
            if (!(ok = first_qk(0, qc0, gn, nt0n))) return;
            pre0 = true;
          };

          for (int j = 0; j < n_max && ok; ++j) {
            const uint32_t g = g0 + j;
            const int last_pv = (j < nt1) ? 1 : 0;
            const int last_qk = (j + 1 < nt1) ? 1 : 0;
#pragma unroll
            for (int t = 0; t < QT; ++t) {
              const bool do_pv = j < nt(t), do_qk = j + 1 < nt(t);
              // all waits first, then the MMAs of this tile back to back; the wait for P comes last: it is
              // the one on the critical path (softmax -> PV -> next QK -> softmax), the tiles are long there
              // (one vote for the three: between them the lanes only poll)
              bool okb = true;
              if (do_pv) okb = ptx::mbar_wait(&ctl->v_full[g % NSTAGE], (g / NSTAGE) & 1, abort_flag);
              if (do_qk && okb) okb = ptx::mbar_wait(&ctl->k_full[(g + 1) % NSTAGE], ((g + 1) / NSTAGE) & 1, abort_flag);
              if (do_pv && okb) okb = ptx::mbar_wait(&ctl->p_full[t], ((t == 0 ? c0 : c1) + j) & 1, abort_flag);
              if (!(ok = __all_sync(0xffffffffu, okb) != 0)) break;
              ptx::tc_fence_after();
              if (do_pv) {
                issue_pv(t, g, j == 0);
                if (leader && j == nt(t) - 1) ptx::mma_commit(&ctl->o_full[t]);
                if (leader && t == last_pv) ptx::mma_commit(&ctl->v_empty[g % NSTAGE]);
              }
              if (do_qk) {
                issue_qk(t, g + 1);
                if (leader && j + 2 == nt(t)) ptx::mma_commit(&ctl->q_empty[t]);  // last QK of this tile: its Q may be replaced
                if (leader && t == last_qk) ptx::mma_commit(&ctl->k_empty[(g + 1) % NSTAGE]);
              }
            }
            if constexpr (D == 64) {
              if (ok && j >= nt0 - 1 && nt1 > nt0) try_pre0();
            }
          }
          g0 += n_max;
          c0 += nt0;
          c1 += nt1;
        }
      }
    }
  } else {
    ptx::setmaxnreg_inc<D == 128 ? 224 : 216>();
    // ------------------------------------------------------------- softmax --
    const int t = warp >> 2;          // query tile of this warpgroup
    const int r_in = tid & (BM - 1);  // row within the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + t * 128 + lane_addr;
    const uint32_t tO = tmem + 256 + t * D + lane_addr;
    // > 0 so that a masked (-inf) score stays -inf when it is scaled
    const float c = fmaxf(fabsf(a.scale) * kLog2e, 1e-30f);
    // with a mask the scores are scaled when the mask is added, and the rest of the loop multiplies by 1
    const float cm = (GEN && a.mask.ptr) ? 1.f : c;
    const float2 c2 = make_float2(cm, cm);
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    uint32_t cnt = 0;  // softmax iterations completed (s_full phase)
    uint32_t ec = 0;   // items with work completed (o_full phase)
    bool ok = true;
    uint32_t s[BN];

    // The warpgroup meets at named barriers in the epilogue, so its threads must
    // leave the loop together: an expired wait is voted on (twice per item) and
    // then every thread of the warpgroup unwinds.
    for (uint32_t i = 0;; ++i) {
      const int slot = i & 1;
      ok = ptx::mbar_wait(&ctl->item_full[slot], (i >> 1) & 1, abort_flag);
      if (ptx::named_barrier_or(1 + t, BM, !ok)) break;
      const int w = ctl->item[slot];
      ptx::mbar_arrive(&ctl->item_empty[slot]);
      if (w < 0) break;
      const Item it = decode_item<GEN>(a, w, n_pairs);
      const int n_t = t == 0 ? it.nt0 : it.nt1;
      const int tile_row0 = it.row0 + t * BM;
      const int row = tile_row0 + r_in;  // global query row of this thread
      const int kv_len = it.kv_len;
      T* orow = reinterpret_cast<T*>(a.o) + it.b * a.os.b + it.h * a.os.h + static_cast<int64_t>(row) * a.os.s;
      float* lse_row = a.lse ? a.lse + (static_cast<int64_t>(it.b) * a.Hq + it.h) * a.Lq + row : nullptr;

      if (n_t == 0) {
        // no participating key (or tile beyond Lq): O = 0, LSE = -inf
        if (row < a.Lq) {
#pragma unroll
          for (int e = 0; e < D; e += 8) *reinterpret_cast<uint4*>(orow + e) = make_uint4(0, 0, 0, 0);
          if (lse_row) *lse_row = -INFINITY;
        }
        continue;
      }

      float m_ref = -INFINITY;  // reference max, in scaled log2 units
      float2 l2 = make_float2(0.f, 0.f);
      for (int j = 0; j < n_t && ok; ++j) {
        ok = ptx::mbar_wait(&ctl->s_full[t], (cnt + j) & 1, abort_flag);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) ptx::tmem_ld32p(tS + cc * 32, s + cc * 32);
        ptx::tmem_wait_ld();

        const int col0 = j * BN;
        if constexpr (GEN) {
          if (a.mask.ptr && row < a.Lq)
            add_mask_row<T>(s, a.mask, it.b * a.mask.sb + it.h * a.mask.sh + row * a.mask.sl + col0, a.Skv - col0, c);
        }
        const bool mask_tile = (col0 + BN > kv_len) || (a.causal && col0 + BN - 1 > tile_row0 + it.shift);
        if (mask_tile) {
          // Highest valid column of this row within the tile.
          int lim = kv_len - 1 - col0;
          if (a.causal && row + it.shift - col0 < lim) lim = row + it.shift - col0;
#pragma unroll
          for (int e = 0; e < BN; ++e)
            if (e > lim) s[e] = 0xff800000u;  // -inf
        }
        // The row maximum is only a reference point for the exponentials, so it is
        // not recomputed for every tile: after the first tile the row keeps its
        // reference as long as the tile's exponentials stay small, which the tile's
        // own row sum shows (all terms are positive: sum <= 2^8 implies every term
        // <= 2^8).  Only when the sum is larger (or not finite) is the maximum of
        // the tile taken, O and the running sum rescaled, and the tile redone.
        bool need_max = (j == 0);
        for (;;) {
          if (need_max) {
            // eight independent 3-input max chains over the 128 columns
            float mx[8];
#pragma unroll
            for (int q = 0; q < 8; ++q)
              mx[q] = ptx::max3(__uint_as_float(s[q]), __uint_as_float(s[q + 8]), -INFINITY);
#pragma unroll
            for (int e = 16; e < BN; e += 16)
#pragma unroll
              for (int q = 0; q < 8; ++q)
                mx[q] = ptx::max3(mx[q], __uint_as_float(s[e + q]), __uint_as_float(s[e + q + 8]));
            const float x_max =
                ptx::max3(ptx::max3(mx[0], mx[1], mx[2]), ptx::max3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7])) * cm;
            if (j == 0) {
              m_ref = x_max;
            } else if (__any_sync(0xffffffffu, x_max > m_ref)) {
              // tcgen05.ld / .st are warp-collective: every lane takes part, lanes
              // whose maximum did not grow with alpha = 1
              const float m_new = fmaxf(m_ref, x_max);
              const float alpha = (GEN && m_new == -INFINITY) ? 1.f : ptx::ex2(m_ref - m_new);
              uint32_t r[32];
#pragma unroll
              for (int cc = 0; cc < D / 32; ++cc) {
                ptx::tmem_ld32(tO + cc * 32, r);
                ptx::tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
                ptx::tmem_st32(tO + cc * 32, r);
              }
              l2.x *= alpha, l2.y *= alpha;
              m_ref = m_new;
            }
          }
          // P = 2^(c*s - m_ref) in packed fp32 pairs; two halves of 64 columns so that
          // the packed 16-bit P of the first half is stored while the second is computed.
          // (general variant) a row that has seen no participating key yet keeps
          // m_ref = -inf; its exponentials are taken against 0 and are all 0
          const float m_use = (GEN && m_ref == -INFINITY) ? 0.f : m_ref;
          const float2 nm2 = make_float2(-m_use, -m_use);
          float2 lt = make_float2(0.f, 0.f);
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            uint32_t pk[32];
#pragma unroll
            for (int e2 = 0; e2 < 64; e2 += 2) {
              const int e = hf * 64 + e2;
              float2 x = ptx::fma2(make_float2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), c2, nm2);
              // (D = 64, where the exponentials and not the MMAs set the pace: one in sixteen on the FMA pipe)
              const float2 p = make_float2(ptx::ex2(x.x), (D == 64 && (e2 & 15) == 0) ? ptx::ex2_fma(x.y) : ptx::ex2(x.y));
              lt = ptx::add2(lt, p);
              pk[e2 >> 1] = pack2<BF16>(p.x, p.y);
            }
            ptx::tmem_st32(tS + hf * 32, pk);
          }
          const float tile_sum = lt.x + lt.y;
          // redo with a fresh maximum if any row of the warp needs it (tcgen05.ld /
          // .st are warp-collective, so the warp decides together)
          // ... and such a row takes the maximum of every tile until it has one
          const bool redo = !need_max && (!(tile_sum <= 256.f) || (GEN && m_ref == -INFINITY));
          if (!__any_sync(0xffffffffu, redo)) {
            l2 = ptx::add2(l2, lt);
            break;
          }
          need_max = true;
        }
        ptx::tmem_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive(&ctl->p_full[t]);
      }
      cnt += n_t;

      // epilogue: O / l -> global, LSE.  The issuer may already be computing the
      // next item's first S_t; its first PV waits for this warpgroup's next P.
      if (ok) ok = ptx::mbar_wait(&ctl->o_full[t], ec & 1, abort_flag);
      ++ec;
      if (ptx::named_barrier_or(1 + t, BM, !ok)) break;
      ptx::tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) ptx::tmem_ld32p(tO + cc * 32, s + cc * 32);
      ptx::tmem_wait_ld();
      const float l = l2.x + l2.y;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      // O leaves through shared memory and TMA stores (coalesced; rows beyond Lq
      // are clipped by the tensor map): one 64-column block at a time, written in
      // the 128-byte-swizzled layout the map expects.
      uint8_t* stage = sO + t * kStageBytes;
#pragma unroll
      for (int hf = 0; hf < HALVES; ++hf) {
        if (r_in == 0) ptx::bulk_wait_read();  // previous store out of this block has been read
        ptx::named_barrier(1 + t, BM);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const int e = hf * 64 + ch * 8;
          uint4 wv;
          wv.x = pack2<BF16>(__uint_as_float(s[e + 0]) * inv, __uint_as_float(s[e + 1]) * inv);
          wv.y = pack2<BF16>(__uint_as_float(s[e + 2]) * inv, __uint_as_float(s[e + 3]) * inv);
          wv.z = pack2<BF16>(__uint_as_float(s[e + 4]) * inv, __uint_as_float(s[e + 5]) * inv);
          wv.w = pack2<BF16>(__uint_as_float(s[e + 6]) * inv, __uint_as_float(s[e + 7]) * inv);
          *reinterpret_cast<uint4*>(stage + r_in * 128 + ((ch ^ (r_in & 7)) << 4)) = wv;
        }
        ptx::fence_proxy_async_smem();
        ptx::named_barrier(1 + t, BM);
        if (r_in == 0 && ok) {
          ptx::tma_store_4d(&tmO, stage, hf * 64, tile_row0, it.h, it.b);
          ptx::bulk_commit();
        }
      }
      if (ok && row < a.Lq && lse_row) *lse_row = l > 0.f ? (m_ref + log2f(l)) * kLn2 : -INFINITY;
    }
    if (r_in == 0) ptx::bulk_wait_all();
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
  if (tid == 0 && ctl->abort_flag && a.status) atomicOr(a.status, kStatusWaitExpired);
}

// ------------------------------------------------------------------ host ----
template <int D, bool BF16, bool GEN>
cudaError_t launch_t(const FwdArgs& a, int dtype, int device, cudaStream_t stream) {
  CUtensorMap tq, tk, tv, to;
  if (!make_map(&tq, dtype, a.q, D, a.Lq, a.Hq, a.B, a.qs) || !make_map(&tk, dtype, a.k, D, a.Skv, a.Hkv, a.B, a.ks) ||
      !make_map(&tv, dtype, a.v, D, a.Skv, a.Hkv, a.B, a.vs) || !make_map(&to, dtype, a.o, D, a.Lq, a.Hq, a.B, a.os))
    return cudaErrorInvalidValue;
  auto kern = fwd_tc_kernel<D, BF16, GEN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<D>());
  if (e != cudaSuccess) return e;
  // the work counter must start at zero for every launch
  e = cudaMemsetAsync(a.sched, 0, sizeof(int), stream);
  if (e != cudaSuccess) return e;
  const long long n_items = static_cast<long long>((a.Lq + QT * BM - 1) / (QT * BM)) * a.Hq * a.B;
  const int sms = sm_count(device);
  const int grid = static_cast<int>(n_items < sms ? n_items : sms);
  kern<<<grid, kThreads, smem_bytes<D>(), stream>>>(tq, tk, tv, to, a);
  return cudaGetLastError();
}

}  // namespace

template <bool GEN>
cudaError_t launch_g(int dtype, int D, const FwdArgs& a, int device, cudaStream_t stream) {
  const bool bf = dtype == TT_ATTN_BF16;
  if (D == 128)
    return bf ? launch_t<128, true, GEN>(a, dtype, device, stream) : launch_t<128, false, GEN>(a, dtype, device, stream);
  if (D == 64)
    return bf ? launch_t<64, true, GEN>(a, dtype, device, stream) : launch_t<64, false, GEN>(a, dtype, device, stream);
  return cudaErrorInvalidValue;
}

cudaError_t launch_fwd_tc(int dtype, int D, const FwdArgs& a, int device, cudaStream_t stream) {
  // the general variant only where it is needed: the fast one carries none of its code
  const bool general = a.mask.ptr != nullptr || a.causal == TT_ATTN_CAUSAL_BOTTOM_RIGHT;
  return general ? launch_g<true>(dtype, D, a, device, stream) : launch_g<false>(dtype, D, a, device, stream);
}

}  // namespace ttattn
