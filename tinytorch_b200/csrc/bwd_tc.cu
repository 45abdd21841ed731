// Attention backward for fp16 / bf16 on sm_100a tensor cores.
//
// Supplies the gradient that FuncSDPAttention::backward leaves unimplemented
// (reference: src/Function/FuncNNLayer.h:267); it equals the reference's chain
// linear -> mul -> add -> softmax -> linear (src/Function/FuncNNLayer.h:20-34,
// src/Function/FuncElemWise.h:77-87,113-123, src/Operation/OpNNLayerCpu.h:78-109):
//   P  = exp(scale * Q K^T - LSE)          dP = dO V^T
//   dS = P o (dP - delta) * scale          delta = rowsum(dO o O)
//   dV = P^T dO      dK = dS^T Q      dQ = dS K
//
// A work item is a 128-row key tile of one (batch, kv head): the CTA walks the query
// tiles that see it (and the query heads of its group), one 128 x 128 (key, query) pair
// per step.  CTAs are persistent, one per SM, and draw items from a counter.  Everything is
// kept TRANSPOSED so that a TMEM lane is a key row:
//   S^T  = K Q^T   (SS MMA, both operands K-major)         -> TMEM region A
//   dP^T = V dO^T  (SS MMA)                                -> TMEM region B
//   four compute warpgroups (thread r of each = key row r; warpgroup w takes
//   queries [32w, 32w+32) of the step) read S^T and dP^T, form P^T and dS^T with
//   the per-query LSE / delta vectors from shared memory, and write them back as
//   packed 16-bit pairs over regions A and B; dS^T also goes to shared memory
//   dV  += P^T dO    (A = P^T from TMEM,  B = dO tile, MN-major)
//   dK  += dS^T Q    (A = dS^T from TMEM, B = Q tile,  MN-major)
//   dQ   = dS K      (A = dS^T tile in shared memory read MN-major, i.e. as dS;
//                     B = K tile read MN-major)             -> its own TMEM columns
//                     when D = 64, else region A
// dV and dK accumulate in TMEM over the whole walk of an item and leave once, through
// staging tiles and TMA stores.  dQ of a (key tile, query tile) pair is added to an fp32
// buffer through swizzled staging tiles and TMA reductions (cp.reduce.async.bulk.tensor
// ... add) and converted to the tensor dtype by a second small kernel.  A producer warp
// draws the items, feeds the tiles with TMA (128-byte swizzle) and fetches the per-query
// vectors; an issuer warp runs the issuing loop with one elected lane issuing the MMAs;
// every wait is bounded.
//
// Two kernels, because the 512 TMEM columns and 227 KB of shared memory divide differently:
// D = 128 (bwd_tc_kernel) has no column to spare, so dQ shares region A with S^T and the
// steps of an item run one after the other; D = 64 (bwd_tc64_kernel) overlaps the two
// element-wise phases of a step with the MMAs of the neighbouring phases and gives the
// read-out of results to a warpgroup of its own.
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace ttattn {
namespace {

constexpr int BM = 128;  // key rows per CTA (= TMEM lanes)
constexpr int BQ = 128;  // query rows per step
constexpr int kCompute = 512;  // four compute warpgroups
constexpr int kTmemCols = 512;
constexpr int kHalfBytes = BM * 128;  // one 64-element column block of a 128-row tile

struct __align__(8) SmemCtl {
  uint64_t item_full[2], item_empty[2];  // work items, from the producer to the issuer and the compute threads
  int item[2];
  uint64_t kv_full, kv_empty;            // K / V of the current item
  uint64_t q_full, q_empty;              // Q / dO of the current step
  uint64_t vec_full[2];                  // per-query vectors of a step (buffer g & 1), written by the producer warp
  uint64_t sp_full, pds_half, pds_full;  // pds_half: the first 16 queries of every warpgroup are done
  uint64_t dq_full, dq_free;
  uint64_t acc_full, acc_free;           // dV / dK of the item: complete / read out of TMEM
  uint32_t tmem_base;
  int abort_flag;
};

// D = 128 (the kernel below; D = 64 has its own further down).  TMEM has no columns left for a dQ accumulator
// beside S^T, dP^T, dV and dK, so dQ reuses region A and the steps of an item run one after the other: one
// Q / dO stage, one dS^T tile, one K / V stage.
struct Cfg128 {
  static constexpr int D = 128;
  static constexpr int TB = BM * D * 2;  // bytes of one tile
  // Warps: 16 compute (four warpgroups, 32 queries of every step each), then the producer warp and the issuer warp
  static constexpr int kProdWarp = 16, kIssWarp = 17, kThreads = 576;
  static constexpr int kItemConsumers = 1 + kCompute;  // issuing lane, compute threads
  static constexpr int kDsBytes = BM * BQ * 2;         // the dS^T tile
  static constexpr int kDqStage = (D / 32) * BQ * 128; // dQ staging: boxes of 128 rows x 32 floats, one per compute warpgroup
  static constexpr int kVecBytes = 2 * 2 * BQ * 4;     // lse / delta vectors, two buffers
  static constexpr int kSmem = 2 * TB + 2 * TB + kDsBytes + kDqStage + kVecBytes + 256;
  static_assert(kSmem <= 232448, "exceeds the shared memory a CTA may request");
};

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

// P of 16 queries for this thread's key row: in place of s (S^T, fp32 bits) and as packed 16-bit pairs in pk.
// lse2: -lse * log2(e) of the 16 queries; q_first: index of the first query; mo: offset of (first query, this
// key) in the mask; n_hidden: how many of the 16 queries, from the first on, do not see this key (causal
// triangle; all 16 for a key beyond kv_len).
template <bool BF16, bool GEN, typename T>
__device__ __forceinline__ void p_chunk(const BwdArgs& a, uint32_t (&s)[16], const float* lse2, float2 c2v,
                                        int n_hidden, int kv_row, int q_first, int64_t mo, uint32_t (&pk)[8]) {
  // exponents c*s - lse2, in packed fp32 pairs
#pragma unroll
  for (int i = 0; i < 16; i += 4) {
    const float4 l4 = *reinterpret_cast<const float4*>(lse2 + i);
    float2 x0 = ptx::fma2(make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), c2v, make_float2(l4.x, l4.y));
    float2 x1 =
        ptx::fma2(make_float2(__uint_as_float(s[i + 2]), __uint_as_float(s[i + 3])), c2v, make_float2(l4.z, l4.w));
    if constexpr (GEN) {
      if (a.mask.ptr && kv_row < a.Skv) {
        // the mask element of (query, this thread's key): adjacent threads read adjacent keys
        const int q = q_first + i;
        const int64_t m = mo + static_cast<int64_t>(i) * a.mask.sl;
        if (q + 0 < a.Lq) x0.x += mask_bias2<T>(a.mask, m);
        if (q + 1 < a.Lq) x0.y += mask_bias2<T>(a.mask, m + a.mask.sl);
        if (q + 2 < a.Lq) x1.x += mask_bias2<T>(a.mask, m + 2 * a.mask.sl);
        if (q + 3 < a.Lq) x1.y += mask_bias2<T>(a.mask, m + 3 * a.mask.sl);
      }
    }
    s[i] = __float_as_uint(x0.x), s[i + 1] = __float_as_uint(x0.y);
    s[i + 2] = __float_as_uint(x1.x), s[i + 3] = __float_as_uint(x1.y);
  }
  // Hidden pairs get P = 0 through the exponent.  (Kept apart from the arithmetic before and after, which then
  // is the same straight-line code for every step; only the diagonal step and a ragged last key tile come here.)
  if (n_hidden > 0) {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < n_hidden) s[i] = 0xff800000u;  // -inf
  }
#pragma unroll
  for (int i = 0; i < 16; i += 4) {
    // (one exponential in eight on the FMA pipe: the compute warps saturate the MUFU units in this phase)
    const float p0 = ptx::ex2(__uint_as_float(s[i])), p1 = ptx::ex2(__uint_as_float(s[i + 1]));
    const float p2 = ptx::ex2(__uint_as_float(s[i + 2]));
    const float p3 = (i & 4) ? ptx::ex2_fma(__uint_as_float(s[i + 3])) : ptx::ex2(__uint_as_float(s[i + 3]));
    s[i] = __float_as_uint(p0), s[i + 1] = __float_as_uint(p1);
    s[i + 2] = __float_as_uint(p2), s[i + 3] = __float_as_uint(p3);
    pk[(i >> 1) + 0] = pack2<BF16>(p0, p1);
    pk[(i >> 1) + 1] = pack2<BF16>(p2, p3);
  }
  // (the FMA-pipe exponential of -inf is a denormal, not 0: a hidden pair must leave nothing behind)
  if (n_hidden > 7) {
    s[7] = 0u;
    pk[3] = pack2<BF16>(__uint_as_float(s[6]), 0.f);
    if (n_hidden > 15) {
      s[15] = 0u;
      pk[7] = pack2<BF16>(__uint_as_float(s[14]), 0.f);
    }
  }
}

// dS = P * (scale * dP - scale * delta) of 16 queries, as packed 16-bit pairs.  p: P (fp32 bits); dp: dP^T
// (fp32 bits); dsc: -delta * scale of the 16 queries.
template <bool BF16>
__device__ __forceinline__ void ds_chunk(const uint32_t (&p)[16], const uint32_t (&dp)[16], const float* dsc,
                                         float2 sc2, uint32_t (&dk)[8]) {
#pragma unroll
  for (int i = 0; i < 16; i += 4) {
    const float4 d4 = *reinterpret_cast<const float4*>(dsc + i);
    const float2 g0 =
        ptx::fma2(make_float2(__uint_as_float(dp[i]), __uint_as_float(dp[i + 1])), sc2, make_float2(d4.x, d4.y));
    const float2 g1 =
        ptx::fma2(make_float2(__uint_as_float(dp[i + 2]), __uint_as_float(dp[i + 3])), sc2, make_float2(d4.z, d4.w));
    const float2 ds0 = ptx::mul2(make_float2(__uint_as_float(p[i]), __uint_as_float(p[i + 1])), g0);
    const float2 ds1 = ptx::mul2(make_float2(__uint_as_float(p[i + 2]), __uint_as_float(p[i + 3])), g1);
    dk[(i >> 1) + 0] = pack2<BF16>(ds0.x, ds0.y);
    dk[(i >> 1) + 1] = pack2<BF16>(ds1.x, ds1.y);
  }
}

// GEN: the general variant (a mask and / or a causal triangle that is not top-left
// aligned); the fast variant compiles all of that out.
template <bool BF16, bool GEN>
__global__ void __launch_bounds__(Cfg128::kThreads, 1)
    bwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                  const __grid_constant__ CUtensorMap tmdQ, const __grid_constant__ CUtensorMap tmdK,
                  const __grid_constant__ CUtensorMap tmdV, const BwdArgs a) {
  using C = Cfg128;
  using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  constexpr int D = C::D, TB = C::TB, HALVES = D / 64;
  // 128-byte-swizzled tiles must start on a 1024-byte boundary; with D = 128 there is
  // no room for alignment slack, so the array itself carries the requirement
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((ptx::smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0 && a.status) atomicOr(a.status, kStatusBadSmemAlign);
    return;
  }
  uint8_t* sK = smem;
  uint8_t* sV = sK + TB;
  uint8_t* sQ = sV + TB;
  uint8_t* sdO = sQ + TB;
  uint8_t* sdS = sdO + TB;             // dS^T: [128 key rows][128 queries], two 64-query blocks, 128-byte swizzle
  uint8_t* sdq = sdS + C::kDsBytes;    // dQ staging: boxes of [128 queries][32 floats], swizzled
  float* svec = reinterpret_cast<float*>(sdq + C::kDqStage);  // [2 buffers][lse2 | delta][128]
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(reinterpret_cast<uint8_t*>(svec) + C::kVecBytes);
  volatile int* abort_flag = &ctl->abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Persistent CTAs draw work items (a key tile of one (batch, kv head)) from a counter, so that the start of
  // an item (K / V load, first products) and the end of the one before (read-out of dV / dK) overlap instead of
  // costing every key tile a CTA launch, a ramp and a drain.  Heads in order, and within a head the key tiles
  // in order: under the causal mask the first key tile is seen by every query tile and walks longest.  Only the
  // last `tail_heads` heads are ordered differently, key tile by key tile ACROSS those heads, so that the items
  // drawn last are the short ones and the CTAs finish together.
  const int group = a.Hq / a.Hkv;
  const int n_kt = (a.Skv + BM - 1) / BM, n_heads = a.Hkv * a.B;
  const int n_items = n_kt * n_heads;
  const int n_q_tiles = (a.Lq + BQ - 1) / BQ;
  struct Item {
    int hk, b, kv0, kv_len, shift, qt_begin, per_head, n_steps;
  };
  auto decode_item = [&](int w) {
    Item it;
    const int w0 = (n_heads - a.tail_heads) * n_kt;
    int bh, nt;
    if (w < w0) {
      bh = w / n_kt;
      nt = w - bh * n_kt;
    } else {
      const int x = w - w0;
      nt = x / a.tail_heads;
      bh = n_heads - a.tail_heads + (x - nt * a.tail_heads);
    }
    it.b = bh / a.Hkv, it.hk = bh - it.b * a.Hkv;
    it.kv0 = nt * BM;
    int kv_len = a.Skv;
    if (a.kv_lens) {
      int l = a.kv_lens[it.b];
      kv_len = l < 0 ? 0 : (l < a.Skv ? l : a.Skv);
    }
    it.kv_len = kv_len;
    it.shift = GEN ? causal_shift(a.causal, kv_len, a.Lq) : 0;  // key j participates iff j <= i + shift
    // BM == BQ: query tiles before the key tile see none of it (general: first tile with a row i >= kv0 - shift)
    it.qt_begin = a.causal ? (GEN ? (it.kv0 - it.shift > 0 ? (it.kv0 - it.shift) / BQ : 0) : nt) : 0;
    it.per_head = (it.kv0 < kv_len && it.qt_begin < n_q_tiles) ? n_q_tiles - it.qt_begin : 0;
    it.n_steps = it.per_head * group;
    return it;
  };

  if (warp == C::kProdWarp && lane == 0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&ctl->item_full[i], 1);
      ptx::mbar_init(&ctl->item_empty[i], C::kItemConsumers);
      ptx::mbar_init(&ctl->vec_full[i], 32);  // the lanes of the producer warp
    }
    ptx::mbar_init(&ctl->kv_full, 1);
    ptx::mbar_init(&ctl->kv_empty, 1);
    ptx::mbar_init(&ctl->q_full, 1);
    ptx::mbar_init(&ctl->q_empty, 1);
    ptx::mbar_init(&ctl->dq_full, 1);
    ptx::mbar_init(&ctl->dq_free, kCompute);
    ptx::mbar_init(&ctl->acc_free, 2 * BM);  // the two warpgroups that read dV / dK out
    ptx::mbar_init(&ctl->sp_full, 1);
    ptx::mbar_init(&ctl->pds_full, kCompute);
    ptx::mbar_init(&ctl->pds_half, kCompute);
    ptx::mbar_init(&ctl->acc_full, 1);
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::tma_prefetch_desc(&tmQ);
    ptx::tma_prefetch_desc(&tmK);
    ptx::tma_prefetch_desc(&tmV);
    ptx::tma_prefetch_desc(&tmdO);
    ptx::tma_prefetch_desc(&tmdQ);
    ptx::tma_prefetch_desc(&tmdK);
    ptx::tma_prefetch_desc(&tmdV);
  }
  if (warp == C::kIssWarp) {
    ptx::tmem_alloc(&ctl->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tA = tmem;             // S^T -> P^T (16-bit pairs in cols [32w, 32w+16) per warpgroup w) -> dQ
  const uint32_t tB = tmem + 128;       // dP^T -> dS^T (16-bit pairs)
  const uint32_t tdV = tmem + 256;      // D columns
  const uint32_t tdK = tmem + 256 + D;  // D columns

  // Every role below walks the same sequence of items and, within an item, of steps; g counts the steps over
  // all items of this CTA (per-step barriers and buffers go by it), k the items (per-item barriers).
  if (warp == C::kProdWarp) {
    // -------------------------------------------------------------- producer --
    // Lane 0 draws the items, publishes those with steps to the other warps and feeds their tiles by TMA; the
    // whole warp fetches the per-query vectors of every step (-lse * log2(e) and -delta * scale).  A key tile
    // that no query sees has no steps: the warp writes its zero gradients here and nobody else hears of it.
    uint32_t gq = 0;  // steps of earlier items
    bool dep_waited = false;
    // per-query vectors of running step g into buffer g & 1
    auto fetch_vec = [&](const Item& it, int n, uint32_t g) {
      if (!dep_waited) {
        // This kernel is launched early behind the delta pre-pass: barriers, TMEM and the first loads need
        // only the inputs; delta is first read here.
        ptx::grid_dep_wait();
        dep_waited = true;
      }
      const int h = it.hk * group + n / it.per_head;
      const int q0 = (it.qt_begin + n % it.per_head) * BQ;
      float lv[4], dl[4];
      const int64_t base = (static_cast<int64_t>(it.b) * a.Hq + h) * a.Lq + q0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int row = j * 32 + lane;
        lv[j] = -INFINITY;  // rows beyond Lq behave like rows without any participating key: P = 0
        dl[j] = 0.f;
        if (q0 + row < a.Lq) {
          lv[j] = a.lse[base + row];
          dl[j] = a.delta[base + row];
        }
      }
      float* nv = svec + (g & 1) * 2 * BQ;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int row = j * 32 + lane;
        nv[row] = lv[j] == -INFINITY ? -INFINITY : -lv[j] * kLog2e;
        nv[BQ + row] = -dl[j] * a.scale;
      }
      ptx::mbar_arrive(&ctl->vec_full[g & 1]);
    };
    // The next item is drawn while the last step of this one is fed (lane 0 holds it in `drawn`), so that the
    // latency of the atomic does not sit between two items.
    int drawn = lane == 0 ? atomicAdd(a.sched, 1) : 0;
    for (uint32_t i = 0;;) {  // i: items published so far
      int w = drawn;
      if (w >= n_items) w = -1;
      w = __shfl_sync(0xffffffffu, w, 0);
      const bool redraw = w >= 0;  // (nothing is drawn behind the end of the list)
      Item it = {};
      if (w >= 0) {
        it = decode_item(w);
        if (it.n_steps == 0) {
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            void* base = t == 0 ? a.dv : a.dk;
            const Str3& st = t == 0 ? a.dvs : a.dks;
            if (!base) continue;
            T* out = reinterpret_cast<T*>(base) + it.b * st.b + it.hk * st.h;
            for (int e = lane; e < BM * (D / 8); e += 32) {
              const int row = it.kv0 + e / (D / 8);
              if (row < a.Skv)
                *reinterpret_cast<uint4*>(out + static_cast<int64_t>(row) * st.s + (e % (D / 8)) * 8) =
                    make_uint4(0, 0, 0, 0);
            }
          }
          if (lane == 0) drawn = atomicAdd(a.sched, 1);
          continue;
        }
      }
      int ok = 1;
      if (lane == 0) {
        const int slot = i & 1;
        ok = ptx::mbar_wait(&ctl->item_empty[slot], ((i >> 1) & 1) ^ 1, abort_flag);
        if (ok) {
          ctl->item[slot] = w;
          ptx::mbar_arrive(&ctl->item_full[slot]);
        }
        // every MMA of the item before has completed
        if (ok && w >= 0) ok = ptx::mbar_wait(&ctl->kv_empty, (i & 1) ^ 1, abort_flag);
        if (ok && w >= 0) {
          ptx::mbar_arrive_expect_tx(&ctl->kv_full, 2 * TB);
#pragma unroll
          for (int hf = 0; hf < HALVES; ++hf) {
            ptx::tma_load_4d(sK + hf * kHalfBytes, &tmK, &ctl->kv_full, hf * 64, it.kv0, it.hk, it.b);
            ptx::tma_load_4d(sV + hf * kHalfBytes, &tmV, &ctl->kv_full, hf * 64, it.kv0, it.hk, it.b);
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok || w < 0) break;
      for (int n = 0; n < it.n_steps; ++n) {
        if (redraw && n + 1 == it.n_steps && lane == 0) drawn = atomicAdd(a.sched, 1);
        const uint32_t g = gq + n;
        const int h = it.hk * group + n / it.per_head;
        const int q0 = (it.qt_begin + n % it.per_head) * BQ;
        // The vectors (two buffers) are fetched a step ahead of the tiles (one stage): the wait passed for the
        // tiles of step g - 1 says that step g - 2, the last to read this buffer, is over.
        const bool vec_first = g > 0;
        if (vec_first) fetch_vec(it, n, g);
        if (lane == 0) {
          // the MMAs that read Q / dO of the step before have completed
          ok = ptx::mbar_wait(&ctl->q_empty, (g & 1) ^ 1, abort_flag);
          if (ok) {
            ptx::mbar_arrive_expect_tx(&ctl->q_full, 2 * TB);
#pragma unroll
            for (int hf = 0; hf < HALVES; ++hf) {
              ptx::tma_load_4d(sQ + hf * kHalfBytes, &tmQ, &ctl->q_full, hf * 64, q0, h, it.b);
              ptx::tma_load_4d(sdO + hf * kHalfBytes, &tmdO, &ctl->q_full, hf * 64, q0, h, it.b);
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        if (!vec_first) fetch_vec(it, n, g);
      }
      if (!ok) break;
      gq += it.n_steps;
      ++i;
    }
  } else if (warp == C::kIssWarp) {
    // ---------------------------------------------------------------- issuer --
    // The whole warp runs the loop (waits made uniform by a vote); one elected lane issues, so that addresses
    // and descriptors stay warp-uniform.
    const bool leader = ptx::elect_one();
    auto uwait = [&](uint64_t* bar, uint32_t parity) {
      return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity, abort_flag)) != 0;
    };
    constexpr uint32_t kHi = ptx::smem_desc_hi_sw128(1024);
    const uint32_t fmt = BF16 ? 1 : 0;
    const uint32_t idesc_s = ptx::make_idesc_f16(BM, BQ, fmt, 0, 0);   // S^T, dP^T: N = queries
    const uint32_t idesc_acc = ptx::make_idesc_f16(BM, D, fmt, 0, 1);  // dV, dK: A from TMEM, B MN-major
    const uint32_t idesc_dq = ptx::make_idesc_f16(BQ, D, fmt, 1, 1);   // dQ: both operands MN-major
    const uint32_t klo = ptx::smem_desc_lo(ptx::smem_u32(sK), 16), vlo = ptx::smem_desc_lo(ptx::smem_u32(sV), 16);
    const uint32_t klo_mn = ptx::smem_desc_lo(ptx::smem_u32(sK), kHalfBytes);
    const uint32_t qlo = ptx::smem_desc_lo(ptx::smem_u32(sQ), 16), dolo = ptx::smem_desc_lo(ptx::smem_u32(sdO), 16);
    const uint32_t qlo_mn = ptx::smem_desc_lo(ptx::smem_u32(sQ), kHalfBytes);
    const uint32_t dolo_mn = ptx::smem_desc_lo(ptx::smem_u32(sdO), kHalfBytes);
    const uint32_t dslo_mn = ptx::smem_desc_lo(ptx::smem_u32(sdS), kHalfBytes);
    uint32_t fi = 0;  // items taken from the queue
    // the next item, or false: none is left or a wait ran out
    auto fetch = [&](Item& it) {
      const int slot = fi & 1;
      if (!uwait(&ctl->item_full[slot], (fi >> 1) & 1)) return false;
      const int w = ctl->item[slot];
      __syncwarp();  // every lane has read the slot
      if (leader) ptx::mbar_arrive(&ctl->item_empty[slot]);
      ++fi;
      if (w < 0) return false;
      it = decode_item(w);
      return true;
    };
    // dP^T = V dO^T of running step g into region B
    auto issue_dp = [&]() {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
        if (leader) ptx::mma_ss2(tB, vlo + off, kHi, dolo + off, kHi, idesc_s, ks > 0 ? 1u : 0u);
      }
    };
    // S^T = K Q^T into region A, and the step's first products are on their way
    auto issue_s = [&]() {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
        if (leader) ptx::mma_ss2(tA, klo + off, kHi, qlo + off, kHi, idesc_s, ks > 0 ? 1u : 0u);
      }
      if (leader) ptx::mma_commit(&ctl->sp_full);
    };
    Item cur = {}, nxt = {};
    uint32_t g = 0, k = 0;
    bool have = fetch(cur);
    bool ok = have && uwait(&ctl->kv_full, 0) && uwait(&ctl->q_full, 0);
    if (ok) {
      ptx::tc_fence_after();
      issue_dp();
      issue_s();
    }
    while (have && ok) {
      bool have_next = false;
      for (int n = 0; n < cur.n_steps && ok; ++n, ++g) {
        const bool last = n + 1 == cur.n_steps;
        // dV and dK contract over the 128 queries, 16 per k-step (2048 bytes of B).  Warpgroup w forms
        // the queries of k-step 2w first and of k-step 2w+1 second, so the even k-steps run while the
        // odd ones are still being computed.
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (!(ok = uwait(half == 0 ? &ctl->pds_half : &ctl->pds_full, g & 1))) break;
          // the first products of an item overwrite the accumulators: the item before has been read out
          if (half == 0 && n == 0 && !(ok = uwait(&ctl->acc_free, (k & 1) ^ 1))) break;
          ptx::tc_fence_after();
#pragma unroll
          for (int ks = half; ks < BQ / 16; ks += 2)
            if (leader) ptx::mma_ts2(tdV, tA + (ks >> 1) * 32 + (ks & 1) * 8, dolo_mn + ks * 128, kHi, idesc_acc,
                         (n > 0 || ks > 0) ? 1u : 0u);
#pragma unroll
          for (int ks = half; ks < BQ / 16; ks += 2)
            if (leader) ptx::mma_ts2(tdK, tB + (ks >> 1) * 32 + (ks & 1) * 8, qlo_mn + ks * 128, kHi, idesc_acc,
                         (n > 0 || ks > 0) ? 1u : 0u);
        }
        if (!ok) break;
        // Q and dO of this step have been read, and with these products the step's vectors: the stage is handed
        // back here, so that its reload runs under the dQ MMAs and the read-out.  After the item's last step dV
        // and dK are complete.
        if (leader) ptx::mma_commit(&ctl->q_empty);
        if (last && leader) ptx::mma_commit(&ctl->acc_full);
#pragma unroll
        for (int ks = 0; ks < BM / 16; ++ks)  // dQ = dS K into region A, contraction over the 128 keys
          if (leader) ptx::mma_ss2(tA, dslo_mn + ks * 128, kHi, klo_mn + ks * 128, kHi, idesc_dq, ks > 0 ? 1u : 0u);
        if (leader) ptx::mma_commit(&ctl->dq_full);
        // every MMA of the item has been issued: its K / V go back
        if (last && leader) ptx::mma_commit(&ctl->kv_empty);
        if (last) have_next = fetch(nxt) && (ok = uwait(&ctl->kv_full, (k + 1) & 1));
        if (!ok || (last && !have_next)) break;
        // dP^T of the next step can go into region B at once: dS^T there has been consumed in issue order.
        // Region A holds this step's dQ until the compute threads have read it: S^T of the next step waits for that.
        if (!(ok = uwait(&ctl->q_full, (g + 1) & 1))) break;
        ptx::tc_fence_after();
        issue_dp();
        if (!(ok = uwait(&ctl->dq_free, g & 1))) break;
        ptx::tc_fence_after();
        issue_s();
      }
      cur = nxt;
      have = have_next;
      ++k;
    }
  } else {
    // --------------------------------------------------------------- compute --
    const int wg = warp >> 2;      // which 32 queries of every step
    const int r = tid & (BM - 1);  // key row within the tile (phase 1) / query row of the step (dQ read-out)
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float c = a.scale * kLog2e;
    const float2 c2v = make_float2(c, c), sc2 = make_float2(a.scale, a.scale);
    bool ok = true;
    // (launched early behind the delta pre-pass: the dQ accumulator it clears is first touched after this wait)
    ptx::grid_dep_wait();
    ptx::grid_dep_launch();  // (the conversion kernel may come up; it waits for this grid)

    uint32_t g0 = 0;  // running step at the start of the item
    for (uint32_t k = 0;; ++k) {
      const int slot = k & 1;
      if (ok) ok = ptx::mbar_wait(&ctl->item_full[slot], (k >> 1) & 1, abort_flag);
      const int w = ok ? ctl->item[slot] : -1;
      ptx::mbar_arrive(&ctl->item_empty[slot]);
      // a warpgroup leaves as one (its named barriers below count all 128 threads) when any of its waits ran out
      if (ptx::named_barrier_or(3 + wg, BM, !ok)) break;
      if (w < 0) break;
      const Item it = decode_item(w);
      const int b = it.b, hk = it.hk, kv0 = it.kv0, kv_len = it.kv_len, shift = it.shift, qt_begin = it.qt_begin,
                per_head = it.per_head, n_steps = it.n_steps;
      const int kv_row = kv0 + r;
      const bool row_valid = kv_row < kv_len;

      // dQ of step n shares region A with S^T, so the four compute warpgroups move it out themselves before the
      // next step's S^T may be issued: thread r owns query row q0 + r, warpgroup w the columns [32w, 32w+32),
      // through a swizzled staging tile and one TMA reduction per warpgroup (coalesced; rows beyond Lq are
      // clipped by the tensor map)
      auto read_out_dq = [&](int n) {
        const uint32_t g = g0 + n;
        const int h = hk * group + n / per_head;
        const int q0 = (qt_begin + n % per_head) * BQ;
        if (ok) ok = ptx::mbar_wait(&ctl->dq_full, g & 1, abort_flag);
        ptx::tc_fence_after();
        uint32_t v[32];
        ptx::tmem_ld32(tA + lane_addr + wg * 32, v);
        ptx::tmem_wait_ld();
        ptx::tc_fence_before();
        ptx::mbar_arrive(&ctl->dq_free);
        uint8_t* stage = sdq + wg * (BQ * 128);
        if (r == 0) ptx::bulk_wait_read();  // the previous reduction has read the staging tile
        ptx::named_barrier(3 + wg, BM);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch)
          *reinterpret_cast<uint4*>(stage + r * 128 + ((ch ^ (r & 7)) << 4)) =
              make_uint4(v[ch * 4 + 0], v[ch * 4 + 1], v[ch * 4 + 2], v[ch * 4 + 3]);
        ptx::fence_proxy_async_smem();
        ptx::named_barrier(3 + wg, BM);
        if (r == 0 && ok) {
          ptx::tma_reduce_add_4d(&tmdQ, stage, wg * 32, q0, h, b);
          ptx::bulk_commit();
        }
      };

      for (int n = 0; n < n_steps; ++n) {
        const uint32_t g = g0 + n;
        const int q0 = (qt_begin + n % per_head) * BQ;
        // per-query vectors of the step, written by the producer warp: [0,128) -lse * log2(e), [128,256) -delta * scale
        const float* vec = svec + (g & 1) * 2 * BQ;
        uint8_t* ds_tile = sdS;
        // all threads reach this point every step, expired waits included
        if (ok) ok = ptx::mbar_wait(&ctl->vec_full[g & 1], (g >> 1) & 1, abort_flag);
        if (ok) ok = ptx::mbar_wait(&ctl->sp_full, g & 1, abort_flag);
        ptx::tc_fence_after();
        const bool diag = a.causal && q0 + shift < kv0 + BM;  // some (query, key) pairs of this step are masked
        const bool masked = diag || kv0 + BM > kv_len;
#pragma unroll
        for (int sc = 0; sc < 2; ++sc) {
          const int col = wg * 32 + sc * 16;  // 16 queries of the step
          uint32_t s[16], dp[16];
          ptx::tmem_ld16(tA + lane_addr + col, s);
          ptx::tmem_ld16(tB + lane_addr + col, dp);
          ptx::tmem_wait_ld();
          uint32_t pk[8], dk[8];
          int64_t mo = 0;
          if constexpr (GEN)
            mo = b * a.mask.sb + (hk * group + n / per_head) * a.mask.sh + static_cast<int64_t>(q0 + col) * a.mask.sl +
                 kv_row;
          int n_hidden = 0;
          if (masked) n_hidden = !row_valid ? 16 : (diag ? kv_row - (q0 + col + shift) : 0);
          p_chunk<BF16, GEN, T>(a, s, vec + col, c2v, n_hidden, kv_row, q0 + col, mo, pk);
          ds_chunk<BF16>(s, dp, vec + BQ + col, sc2, dk);
          // Warpgroup w keeps its 16-bit results in columns [32w, 32w+16) of the
          // region, i.e. over the first 16 columns it loaded itself, never over
          // columns another warpgroup still has to read.
          ptx::tmem_st8(tA + lane_addr + wg * 32 + sc * 8, pk);
          ptx::tmem_st8(tB + lane_addr + wg * 32 + sc * 8, dk);
          if (sc == 0) {
            // P^T / dS^T of this warpgroup's first 16 queries are in TMEM: dV / dK may start on them
            ptx::tmem_wait_st();
            ptx::tc_fence_before();
            ptx::mbar_arrive(&ctl->pds_half);
          }
          // dS^T row r, queries [col, col+16): two 16-byte chunks of the 64-query block col/64
          uint8_t* row = ds_tile + (col >> 6) * kHalfBytes + r * 128;
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            const int chunk = ((col & 63) >> 3) + ch;
            *reinterpret_cast<uint4*>(row + ((chunk ^ (r & 7)) << 4)) =
                make_uint4(dk[ch * 4 + 0], dk[ch * 4 + 1], dk[ch * 4 + 2], dk[ch * 4 + 3]);
          }
        }
        ptx::tmem_wait_st();
        ptx::fence_proxy_async_smem();
        ptx::tc_fence_before();
        ptx::mbar_arrive(&ctl->pds_full);
        read_out_dq(n);
      }
      g0 += n_steps;

      // dV (warpgroup 0) and dK (warpgroup 1) of this key tile, 64 columns at a time through the warpgroup's
      // staging tile and a TMA store (coalesced; rows beyond Skv are clipped by the tensor map); the other
      // warpgroups go on to the next item
      if (wg < 2) {
        const bool wanted = wg == 0 ? a.dv != nullptr : a.dk != nullptr;
        if (ok) ok = ptx::mbar_wait(&ctl->acc_full, k & 1, abort_flag);
        ptx::tc_fence_after();
        const uint32_t src = (wg == 0 ? tdV : tdK) + lane_addr;
        uint8_t* stage = sdq + wg * (BQ * 128);
#pragma unroll 1
        for (int hf = 0; hf < HALVES; ++hf) {
          if (r == 0) ptx::bulk_wait_read();  // the previous store / reduction has read the staging tile
          ptx::named_barrier(3 + wg, BM);
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            uint32_t v[32];
            ptx::tmem_ld32(src + hf * 64 + c2 * 32, v);
            ptx::tmem_wait_ld();
            if (hf == HALVES - 1 && c2 == 1) {
              // the accumulators may be overwritten by the next item's first products
              ptx::tc_fence_before();
              ptx::mbar_arrive(&ctl->acc_free);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 w4;
              w4.x = pack2<BF16>(__uint_as_float(v[j * 8 + 0]), __uint_as_float(v[j * 8 + 1]));
              w4.y = pack2<BF16>(__uint_as_float(v[j * 8 + 2]), __uint_as_float(v[j * 8 + 3]));
              w4.z = pack2<BF16>(__uint_as_float(v[j * 8 + 4]), __uint_as_float(v[j * 8 + 5]));
              w4.w = pack2<BF16>(__uint_as_float(v[j * 8 + 6]), __uint_as_float(v[j * 8 + 7]));
              *reinterpret_cast<uint4*>(stage + r * 128 + (((c2 * 4 + j) ^ (r & 7)) << 4)) = w4;
            }
          }
          ptx::fence_proxy_async_smem();
          ptx::named_barrier(3 + wg, BM);
          if (r == 0 && ok && wanted) {
            ptx::tma_store_4d(wg == 0 ? &tmdV : &tmdK, stage, hf * 64, kv0, hk, b);
            ptx::bulk_commit();
          }
        }
      }
    }
    if (r == 0) ptx::bulk_wait_all();
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == C::kIssWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
  if (tid == 0 && ctl->abort_flag && a.status) atomicOr(a.status, kStatusWaitExpired);
}

// ------------------------------------------------------------------ D = 64 --
// With 64 columns per head there is room (TMEM columns and shared memory) to take the step apart in time.  The
// element-wise work of a step has two phases: P^T from S^T (the exponentials), then dS^T from dP^T and the P
// kept in registers.  The issuer follows them: when P^T is ready it issues dV and at once S^T of the NEXT step
// into region A; when dS^T is ready, dK, then dP^T of the next step into region B, then the step's dQ.  So each
// phase of the compute warps runs while the tensor pipe works on what the other phase produced, instead of the
// pipe and the compute warps waiting for each other in turn.  A fifth warpgroup moves the results out of TMEM
// (each of its warps the dQ of its 32 query rows through a staging box of its own and TMA reductions, and dV /
// dK of an item between its last two dQ); the producer warp also fetches the per-query vectors.  Shared memory:
// two K / V stages (the next item's first products are issued before this item's last dQ has read K), three Q
// stages (in use from S^T, a step ahead, to dK) and two dO stages (from dP^T to dV: half a step), two dS^T tiles.
struct __align__(8) Ctl64 {
  uint64_t item_full[2], item_empty[2];
  uint64_t kv_full[2], kv_empty[2];
  uint64_t q_full[3], q_empty[3];
  uint64_t do_full[2], do_empty[2];
  uint64_t vec_full[2];         // per-query vectors of a step (buffer g & 1), written by the producer warp
  uint64_t vec_free[2];         // ... and read by every compute thread
  uint64_t s_full, dp_full;     // S^T / dP^T of a step are in TMEM
  uint64_t p_done, ds_done;     // P^T / dS^T of a step have been formed
  uint64_t dq_full[2], dq_free[2];
  uint64_t acc_full, acc_free;
  int item[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct Cfg64 {
  static constexpr int D = 64, TB = BM * D * 2, NQ = 3;
  static constexpr int kDsBytes = BM * BQ * 2;  // a dS^T tile: [128 key rows][128 queries], two 64-query blocks
  static constexpr int kBox = 32 * 128;         // a drain warp's staging box: 32 query rows x 32 floats
  static constexpr int oKV = 0, oQ = 4 * TB, odO = oQ + NQ * TB, odS = odO + 2 * TB, oDq = odS + 2 * kDsBytes,
                       oVec = oDq + 4 * kBox, oCtl = oVec + 2 * 2 * BQ * 4;
  static constexpr int kSmem = oCtl + 512;
  static_assert(sizeof(Ctl64) <= 512, "control block");
  static_assert(kSmem <= 232448, "exceeds the shared memory a CTA may request");
  // warps: 16 compute, 4 drain, producer, issuer, 2 idle (register reallocation works on whole warpgroups)
  static constexpr int kProdWarp = 20, kIssWarp = 21, kThreads = 768;
};

template <bool BF16, bool GEN>
__global__ void __launch_bounds__(Cfg64::kThreads, 1)
    bwd_tc64_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const __grid_constant__ CUtensorMap tmdQ, const __grid_constant__ CUtensorMap tmdK,
                    const __grid_constant__ CUtensorMap tmdV, const BwdArgs a) {
  using C = Cfg64;
  using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  constexpr int D = C::D, TB = C::TB, NQ = C::NQ;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((ptx::smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0 && a.status) atomicOr(a.status, kStatusBadSmemAlign);
    return;
  }
  uint8_t* sKV = smem + C::oKV;  // 2 stages of [K tile | V tile]
  uint8_t* sQ = smem + C::oQ;    // NQ stages
  uint8_t* sdO = smem + C::odO;  // 2 stages
  uint8_t* sdS = smem + C::odS;  // 2 x dS^T: [128 key rows][128 queries], two 64-query blocks, 128-byte swizzle
  uint8_t* sdq = smem + C::oDq;  // dQ staging: per drain warp [32 queries][32 floats], swizzled
  float* svec = reinterpret_cast<float*>(smem + C::oVec);  // [2 buffers][lse2 | delta][128]
  Ctl64* ctl = reinterpret_cast<Ctl64*>(smem + C::oCtl);
  volatile int* abort_flag = &ctl->abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Work items (a key tile of one (batch, kv head)) are drawn from a counter: heads in order and, within a
  // head, the key tiles in order (under the causal mask the first key tile is seen by every query tile and walks
  // longest).  Only the last `tail_heads` heads are ordered key tile by key tile ACROSS those heads, so that the
  // items drawn last are the short ones and the CTAs finish together.
  const int group = a.Hq / a.Hkv;
  const int n_kt = (a.Skv + BM - 1) / BM, n_heads = a.Hkv * a.B;
  const int n_items = n_kt * n_heads;
  const int n_q_tiles = (a.Lq + BQ - 1) / BQ;
  struct Item {
    int hk, b, kv0, kv_len, shift, qt_begin, per_head, n_steps;
  };
  auto decode_item = [&](int w) {
    Item it;
    const int w0 = (n_heads - a.tail_heads) * n_kt;
    int bh, nt;
    if (w < w0) {
      bh = w / n_kt;
      nt = w - bh * n_kt;
    } else {
      const int x = w - w0;
      nt = x / a.tail_heads;
      bh = n_heads - a.tail_heads + (x - nt * a.tail_heads);
    }
    it.b = bh / a.Hkv, it.hk = bh - it.b * a.Hkv;
    it.kv0 = nt * BM;
    int kv_len = a.Skv;
    if (a.kv_lens) {
      int l = a.kv_lens[it.b];
      kv_len = l < 0 ? 0 : (l < a.Skv ? l : a.Skv);
    }
    it.kv_len = kv_len;
    it.shift = GEN ? causal_shift(a.causal, kv_len, a.Lq) : 0;  // key j participates iff j <= i + shift
    // BM == BQ: query tiles before the key tile see none of it (general: first tile with a row i >= kv0 - shift)
    it.qt_begin = a.causal ? (GEN ? (it.kv0 - it.shift > 0 ? (it.kv0 - it.shift) / BQ : 0) : nt) : 0;
    it.per_head = (it.kv0 < kv_len && it.qt_begin < n_q_tiles) ? n_q_tiles - it.qt_begin : 0;
    it.n_steps = it.per_head * group;
    return it;
  };

  if (warp == C::kProdWarp && lane == 0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&ctl->item_full[i], 1);
      ptx::mbar_init(&ctl->item_empty[i], 1 + kCompute + BM);  // issuing lane, compute threads, drain threads
      ptx::mbar_init(&ctl->kv_full[i], 1);
      ptx::mbar_init(&ctl->kv_empty[i], 1);
      ptx::mbar_init(&ctl->vec_full[i], 32);  // the lanes of the producer warp
      ptx::mbar_init(&ctl->vec_free[i], kCompute);
      ptx::mbar_init(&ctl->do_full[i], 1);
      ptx::mbar_init(&ctl->do_empty[i], 1);
      ptx::mbar_init(&ctl->dq_full[i], 1);
      ptx::mbar_init(&ctl->dq_free[i], BM);
    }
#pragma unroll
    for (int i = 0; i < NQ; ++i) {
      ptx::mbar_init(&ctl->q_full[i], 1);
      ptx::mbar_init(&ctl->q_empty[i], 1);
    }
    ptx::mbar_init(&ctl->s_full, 1);
    ptx::mbar_init(&ctl->dp_full, 1);
    ptx::mbar_init(&ctl->p_done, kCompute);
    ptx::mbar_init(&ctl->ds_done, kCompute);
    ptx::mbar_init(&ctl->acc_full, 1);
    ptx::mbar_init(&ctl->acc_free, BM);
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::tma_prefetch_desc(&tmQ);
    ptx::tma_prefetch_desc(&tmK);
    ptx::tma_prefetch_desc(&tmV);
    ptx::tma_prefetch_desc(&tmdO);
    ptx::tma_prefetch_desc(&tmdQ);
    ptx::tma_prefetch_desc(&tmdK);
    ptx::tma_prefetch_desc(&tmdV);
  }
  if (warp == C::kIssWarp) {
    ptx::tmem_alloc(&ctl->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tA = tmem;         // S^T -> P^T (16-bit pairs in cols [32w, 32w+16) per warpgroup w)
  const uint32_t tB = tmem + 128;   // dP^T -> dS^T, likewise
  const uint32_t tdV = tmem + 256;  // 64 columns
  const uint32_t tdK = tmem + 320;  // 64 columns
  auto tdQ = [&](uint32_t g) { return tmem + 384 + (g & 1) * D; };  // dQ of running step g

  // Every role walks the same sequence of items and, within an item, of steps; g counts the steps over all
  // items of this CTA (per-step barriers and buffers go by it), k the items (per-item barriers).
  if (warp >= 20) {
    // (96 registers for the 512 compute threads, 48 for the other 256: together the 80 x 768 the CTA was
    // launched with, so the increase can always be served)
    ptx::setmaxnreg_dec<48>();
    if (warp == C::kProdWarp) {
      // ------------------------------------------------------------ producer --
      // Lane 0 draws the items, publishes those with steps to the other warps and feeds their tiles by TMA; the
      // whole warp fetches the per-query vectors of every step (-lse * log2(e) and -delta * scale).  A key tile
      // that no query sees has no steps: the warp writes its zero gradients here and nobody else hears of it
      // (so a run of such items cannot fill the two-slot queue while the issuer looks one item ahead).
      uint32_t gq = 0;  // steps of earlier items
      bool dep_waited = false;
      // The next item is drawn while the last step of this one is fed (lane 0 holds it in `drawn`), so that the
      // latency of the atomic does not sit between two items.
      int drawn = lane == 0 ? atomicAdd(a.sched, 1) : 0;
      for (uint32_t i = 0;;) {  // i: items published so far
        int w = drawn;
        if (w >= n_items) w = -1;
        w = __shfl_sync(0xffffffffu, w, 0);
        bool redraw = w >= 0;  // (nothing is drawn behind the end of the list)
        Item it = {};
        if (w >= 0) {
          it = decode_item(w);
          if (it.n_steps == 0) {
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              void* base = t == 0 ? a.dv : a.dk;
              const Str3& st = t == 0 ? a.dvs : a.dks;
              if (!base) continue;
              T* out = reinterpret_cast<T*>(base) + it.b * st.b + it.hk * st.h;
              for (int e = lane; e < BM * (D / 8); e += 32) {
                const int row = it.kv0 + e / (D / 8);
                if (row < a.Skv)
                  *reinterpret_cast<uint4*>(out + static_cast<int64_t>(row) * st.s + (e % (D / 8)) * 8) =
                      make_uint4(0, 0, 0, 0);
              }
            }
            if (lane == 0) drawn = atomicAdd(a.sched, 1);
            continue;
          }
        }
        int ok = 1;
        if (lane == 0) {
          const int slot = i & 1;
          ok = ptx::mbar_wait(&ctl->item_empty[slot], ((i >> 1) & 1) ^ 1, abort_flag);
          if (ok) {
            ctl->item[slot] = w;
            ptx::mbar_arrive(&ctl->item_full[slot]);
          }
          // the MMAs that read this stage (two items ago) have completed
          if (ok && w >= 0) ok = ptx::mbar_wait(&ctl->kv_empty[slot], ((i >> 1) & 1) ^ 1, abort_flag);
          if (ok && w >= 0) {
            ptx::mbar_arrive_expect_tx(&ctl->kv_full[slot], 2 * TB);
            ptx::tma_load_4d(sKV + slot * 2 * TB, &tmK, &ctl->kv_full[slot], 0, it.kv0, it.hk, it.b);
            ptx::tma_load_4d(sKV + slot * 2 * TB + TB, &tmV, &ctl->kv_full[slot], 0, it.kv0, it.hk, it.b);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok || w < 0) break;
        for (int n = 0; n < it.n_steps; ++n) {
          if (redraw && n + 1 == it.n_steps && lane == 0) drawn = atomicAdd(a.sched, 1);
          const uint32_t g = gq + n;
          const int st = g % NQ;
          const int h = it.hk * group + n / it.per_head;
          const int q0 = (it.qt_begin + n % it.per_head) * BQ;
          if (lane == 0) {
            ok = ptx::mbar_wait(&ctl->q_empty[st], ((g / NQ) & 1) ^ 1, abort_flag);
            if (ok) {
              ptx::mbar_arrive_expect_tx(&ctl->q_full[st], TB);
              ptx::tma_load_4d(sQ + st * TB, &tmQ, &ctl->q_full[st], 0, q0, h, it.b);
              ok = ptx::mbar_wait(&ctl->do_empty[g & 1], ((g >> 1) & 1) ^ 1, abort_flag);
            }
            if (ok) {
              ptx::mbar_arrive_expect_tx(&ctl->do_full[g & 1], TB);
              ptx::tma_load_4d(sdO + (g & 1) * TB, &tmdO, &ctl->do_full[g & 1], 0, q0, h, it.b);
            }
            // The vectors' buffer was last read in step g - 2.  (A barrier per buffer: it cannot complete its next
            // phase before this warp has written the buffer again, so the parity below is never ambiguous, as it
            // would be on a barrier that advances every step while this warp is held up at an item boundary.)
            if (ok && g >= 2) ok = ptx::mbar_wait(&ctl->vec_free[g & 1], ((g >> 1) - 1) & 1, abort_flag);
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
          if (!dep_waited) {
            // This kernel is launched early behind the delta pre-pass: barriers, TMEM and the loads above need
            // only the inputs; delta is first read here.
            ptx::grid_dep_wait();
            dep_waited = true;
          }
          float lv[4], dl[4];
          const int64_t base = (static_cast<int64_t>(it.b) * a.Hq + h) * a.Lq + q0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int row = j * 32 + lane;
            lv[j] = -INFINITY;  // rows beyond Lq behave like rows without any participating key: P = 0
            dl[j] = 0.f;
            if (q0 + row < a.Lq) {
              lv[j] = a.lse[base + row];
              dl[j] = a.delta[base + row];
            }
          }
          float* nv = svec + (g & 1) * 2 * BQ;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int row = j * 32 + lane;
            nv[row] = lv[j] == -INFINITY ? -INFINITY : -lv[j] * kLog2e;
            nv[BQ + row] = -dl[j] * a.scale;
          }
          ptx::mbar_arrive(&ctl->vec_full[g & 1]);
        }
        if (!ok) break;
        gq += it.n_steps;
        ++i;
      }
    } else if (warp == C::kIssWarp) {
      // -------------------------------------------------------------- issuer --
      // The whole warp runs the loop (waits made uniform by a vote); one elected lane issues, so that addresses
      // and descriptors stay warp-uniform.
      const bool leader = ptx::elect_one();
      auto uwait = [&](uint64_t* bar, uint32_t parity) {
        return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity, abort_flag)) != 0;
      };
      constexpr uint32_t kHi = ptx::smem_desc_hi_sw128(1024);
      const uint32_t fmt = BF16 ? 1 : 0;
      const uint32_t idesc_s = ptx::make_idesc_f16(BM, BQ, fmt, 0, 0);   // S^T, dP^T: N = queries
      const uint32_t idesc_acc = ptx::make_idesc_f16(BM, D, fmt, 0, 1);  // dV, dK: A from TMEM, B MN-major
      const uint32_t idesc_dq = ptx::make_idesc_f16(BQ, D, fmt, 1, 1);   // dQ: both operands MN-major
      uint32_t fi = 0;  // items taken from the queue
      // the next item, or false: none is left or a wait ran out
      auto fetch = [&](Item& it) {
        const int slot = fi & 1;
        if (!uwait(&ctl->item_full[slot], (fi >> 1) & 1)) return false;
        const int w = ctl->item[slot];
        __syncwarp();  // every lane has read the slot
        if (leader) ptx::mbar_arrive(&ctl->item_empty[slot]);
        ++fi;
        if (w < 0) return false;
        it = decode_item(w);
        return true;
      };
      // K and V of the k-th item of this CTA are in shared memory
      auto kv_ready = [&](uint32_t k) { return uwait(&ctl->kv_full[k & 1], (k >> 1) & 1); };
      // S^T = K Q^T of running step g, on the tiles of the CTA's k-th item
      auto issue_s = [&](uint32_t g, uint32_t k) {
        if (!uwait(&ctl->q_full[g % NQ], (g / NQ) & 1)) return false;
        ptx::tc_fence_after();
        const uint32_t qlo = ptx::smem_desc_lo(ptx::smem_u32(sQ + (g % NQ) * TB), 16);
        const uint32_t klo = ptx::smem_desc_lo(ptx::smem_u32(sKV + (k & 1) * 2 * TB), 16);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          if (leader) ptx::mma_ss2(tA, klo + ks * 2, kHi, qlo + ks * 2, kHi, idesc_s, ks > 0 ? 1u : 0u);
        if (leader) ptx::mma_commit(&ctl->s_full);
        return true;
      };
      // dP^T = V dO^T of running step g
      auto issue_dp = [&](uint32_t g, uint32_t k) {
        if (!uwait(&ctl->do_full[g & 1], (g >> 1) & 1)) return false;
        ptx::tc_fence_after();
        const uint32_t dolo = ptx::smem_desc_lo(ptx::smem_u32(sdO + (g & 1) * TB), 16);
        const uint32_t vlo = ptx::smem_desc_lo(ptx::smem_u32(sKV + (k & 1) * 2 * TB + TB), 16);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          if (leader) ptx::mma_ss2(tB, vlo + ks * 2, kHi, dolo + ks * 2, kHi, idesc_s, ks > 0 ? 1u : 0u);
        if (leader) ptx::mma_commit(&ctl->dp_full);
        return true;
      };
      Item cur = {}, nxt = {};
      uint32_t g = 0, k = 0;
      bool have = fetch(cur);
      bool ok = have && kv_ready(0) && issue_s(0, 0) && issue_dp(0, 0);
      while (have && ok) {
        bool have_next = false;
        for (int n = 0; n < cur.n_steps && ok; ++n, ++g) {
          const bool last = n + 1 == cur.n_steps;
          const uint32_t qlo_mn = ptx::smem_desc_lo(ptx::smem_u32(sQ + (g % NQ) * TB), kHalfBytes);
          const uint32_t dolo_mn = ptx::smem_desc_lo(ptx::smem_u32(sdO + (g & 1) * TB), kHalfBytes);
          // P^T is ready: dV += P^T dO, contraction over the queries, 16 per k-step (2048 bytes of B)
          if (!(ok = uwait(&ctl->p_done, g & 1))) break;
          // the first products of an item overwrite the accumulators: the item before has been read out
          if (n == 0 && !(ok = uwait(&ctl->acc_free, (k & 1) ^ 1))) break;
          ptx::tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < BQ / 16; ++ks)
            if (leader) ptx::mma_ts2(tdV, tA + (ks >> 1) * 32 + (ks & 1) * 8, dolo_mn + ks * 128, kHi, idesc_acc,
                         (n > 0 || ks > 0) ? 1u : 0u);
          if (leader) ptx::mma_commit(&ctl->do_empty[g & 1]);  // dO of this step has been read (dP^T before, dV now)
          // P^T has been consumed from region A (in issue order): S^T of the next step goes in at once (of the
          // next item after this item's last step: its K / V sit in the other stage)
          if (last) have_next = fetch(nxt) && (ok = kv_ready(k + 1));
          const bool next_step = ok && (!last || have_next);
          const uint32_t kn = last ? k + 1 : k;
          if (!ok || (next_step && !(ok = issue_s(g + 1, kn)))) break;
          // dS^T is ready: dK += dS^T Q; then dP^T of the next step into region B; then dQ = dS K (contraction
          // over the 128 keys; dS is the step's dS^T tile in shared memory read MN-major)
          if (!(ok = uwait(&ctl->ds_done, g & 1))) break;
          ptx::tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < BQ / 16; ++ks)
            if (leader) ptx::mma_ts2(tdK, tB + (ks >> 1) * 32 + (ks & 1) * 8, qlo_mn + ks * 128, kHi, idesc_acc,
                         (n > 0 || ks > 0) ? 1u : 0u);
          if (leader) ptx::mma_commit(&ctl->q_empty[g % NQ]);  // Q of this step has been read (S^T before, dK now)
          if (last && leader) ptx::mma_commit(&ctl->acc_full);  // dV and dK of the item are complete
          if (next_step && !(ok = issue_dp(g + 1, kn))) break;
          if (g >= 2 && !(ok = uwait(&ctl->dq_free[g & 1], ((g >> 1) - 1) & 1))) break;
          const uint32_t dslo_mn = ptx::smem_desc_lo(ptx::smem_u32(sdS + (g & 1) * C::kDsBytes), kHalfBytes);
          const uint32_t klo_mn = ptx::smem_desc_lo(ptx::smem_u32(sKV + (k & 1) * 2 * TB), kHalfBytes);
#pragma unroll
          for (int ks = 0; ks < BM / 16; ++ks)
            if (leader) ptx::mma_ss2(tdQ(g), dslo_mn + ks * 128, kHi, klo_mn + ks * 128, kHi, idesc_dq, ks > 0 ? 1u : 0u);
          if (leader) ptx::mma_commit(&ctl->dq_full[g & 1]);
          // every MMA of the item has been issued: its K / V stage goes back
          if (last && leader) ptx::mma_commit(&ctl->kv_empty[k & 1]);
        }
        cur = nxt;
        have = have_next;
        ++k;
      }
    }
  } else if (warp >= 16) {
    // ----------------------------------------------------------------- drain --
    // Warp j of this warpgroup owns TMEM lanes [32j, 32j+32): dQ of those query rows in every step (32 columns
    // at a time through the warp's swizzled staging box and a TMA reduction: coalesced, rows beyond Lq are
    // clipped by the tensor map), and dV / dK of those key rows (through the same box and TMA stores) between
    // the item's last two dQ.
    ptx::setmaxnreg_dec<48>();
    const int wj = warp & 3;
    const uint32_t lane_addr = static_cast<uint32_t>(wj * 32) << 16;
    uint8_t* box = sdq + wj * C::kBox;
    bool ok = true;
    // (the warp stays together: its waits' outcomes are made uniform)
    auto wwait = [&](uint64_t* bar, uint32_t parity) {
      if (ok) ok = __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity, abort_flag)) != 0;
    };
    ptx::grid_dep_wait();  // the reductions below need the dQ accumulator cleared by the pre-pass
    uint32_t g = 0;
    for (uint32_t k = 0;; ++k) {
      const int slot = k & 1;
      wwait(&ctl->item_full[slot], (k >> 1) & 1);
      const int w = ok ? ctl->item[slot] : -1;
      ptx::mbar_arrive(&ctl->item_empty[slot]);
      if (w < 0) break;
      const Item it = decode_item(w);
      for (int n = 0; n < it.n_steps; ++n, ++g) {
        if (n + 1 == it.n_steps) {
          // dV, then dK: complete once the last step's products are (before its dQ); through the warp's staging
          // box (as [32 key rows][64 elements]) and a TMA store: coalesced, rows beyond Skv clipped
          wwait(&ctl->acc_full, k & 1);
          ptx::tc_fence_after();
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (lane == 0) ptx::bulk_wait_read();  // the previous store / reduction has read the box
            __syncwarp();
#pragma unroll
            for (int cc = 0; cc < D / 32; ++cc) {
              uint32_t v[32];
              ptx::tmem_ld32((t == 0 ? tdV : tdK) + lane_addr + cc * 32, v);
              ptx::tmem_wait_ld();
              if (t == 1 && cc == D / 32 - 1) {
                // the accumulators may be overwritten by the next item's first products
                ptx::tc_fence_before();
                ptx::mbar_arrive(&ctl->acc_free);
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 w4;
                w4.x = pack2<BF16>(__uint_as_float(v[j * 8 + 0]), __uint_as_float(v[j * 8 + 1]));
                w4.y = pack2<BF16>(__uint_as_float(v[j * 8 + 2]), __uint_as_float(v[j * 8 + 3]));
                w4.z = pack2<BF16>(__uint_as_float(v[j * 8 + 4]), __uint_as_float(v[j * 8 + 5]));
                w4.w = pack2<BF16>(__uint_as_float(v[j * 8 + 6]), __uint_as_float(v[j * 8 + 7]));
                *reinterpret_cast<uint4*>(box + lane * 128 + (((cc * 4 + j) ^ (lane & 7)) << 4)) = w4;
              }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && ok && (t == 0 ? a.dv != nullptr : a.dk != nullptr) && it.kv0 + wj * 32 < a.Skv) {
              ptx::tma_store_4d(t == 0 ? &tmdV : &tmdK, box, 0, it.kv0 + wj * 32, it.hk, it.b);
              ptx::bulk_commit();
            }
          }
        }
        const int h = it.hk * group + n / it.per_head;
        const int q0 = (it.qt_begin + n % it.per_head) * BQ + wj * 32;
        wwait(&ctl->dq_full[g & 1], (g >> 1) & 1);
        ptx::tc_fence_after();
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t v[32];
          ptx::tmem_ld32(tdQ(g) + lane_addr + cc * 32, v);
          ptx::tmem_wait_ld();
          if (cc == D / 32 - 1) {
            ptx::tc_fence_before();
            ptx::mbar_arrive(&ctl->dq_free[g & 1]);
          }
          if (lane == 0) ptx::bulk_wait_read();  // the previous reduction has read the box
          __syncwarp();
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(box + lane * 128 + ((ch ^ (lane & 7)) << 4)) =
                make_uint4(v[ch * 4 + 0], v[ch * 4 + 1], v[ch * 4 + 2], v[ch * 4 + 3]);
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && ok && q0 < a.Lq) {
            ptx::tma_reduce_add_4d(&tmdQ, box, cc * 32, q0, h, it.b);
            ptx::bulk_commit();
          }
        }
      }
    }
    if (lane == 0) ptx::bulk_wait_all();
  } else {
    // --------------------------------------------------------------- compute --
    ptx::setmaxnreg_inc<96>();
    const int wg = warp >> 2;      // which 32 queries of every step
    const int r = tid & (BM - 1);  // key row within the tile
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float c = a.scale * kLog2e;
    const float2 c2v = make_float2(c, c), sc2 = make_float2(a.scale, a.scale);
    bool ok = true;
    ptx::grid_dep_launch();  // (the conversion kernel may come up; it waits for this grid)
    uint32_t g = 0;
    for (uint32_t k = 0;; ++k) {
      const int slot = k & 1;
      if (ok) ok = ptx::mbar_wait(&ctl->item_full[slot], (k >> 1) & 1, abort_flag);
      const int w = ok ? ctl->item[slot] : -1;
      ptx::mbar_arrive(&ctl->item_empty[slot]);
      if (w < 0) break;
      const Item it = decode_item(w);
      const int kv_row = it.kv0 + r;
      for (int n = 0; n < it.n_steps; ++n, ++g) {
        const int hq = it.hk * group + n / it.per_head;
        const int q0 = (it.qt_begin + n % it.per_head) * BQ;
        const float* vec = svec + (g & 1) * 2 * BQ;
        // some (query, key) pairs of this step are hidden: the diagonal step, a ragged last key tile
        const bool diag = a.causal && q0 + it.shift < it.kv0 + BM;
        const bool masked = diag || it.kv0 + BM > it.kv_len;
        if (ok) ok = ptx::mbar_wait(&ctl->vec_full[g & 1], (g >> 1) & 1, abort_flag);
        // phase 1: P^T from S^T; P stays in registers for phase 2
        if (ok) ok = ptx::mbar_wait(&ctl->s_full, g & 1, abort_flag);
        ptx::tc_fence_after();
        uint32_t p[2][16];
#pragma unroll
        for (int sc = 0; sc < 2; ++sc) {
          const int col = wg * 32 + sc * 16;  // 16 queries of the step
          ptx::tmem_ld16(tA + lane_addr + col, p[sc]);
          ptx::tmem_wait_ld();
          uint32_t pk[8];
          int64_t mo = 0;
          if constexpr (GEN)
            mo = it.b * a.mask.sb + hq * a.mask.sh + static_cast<int64_t>(q0 + col) * a.mask.sl + kv_row;
          int n_hidden = 0;
          if (masked) n_hidden = kv_row >= it.kv_len ? 16 : (diag ? kv_row - (q0 + col + it.shift) : 0);
          p_chunk<BF16, GEN, T>(a, p[sc], vec + col, c2v, n_hidden, kv_row, q0 + col, mo, pk);
          // Warpgroup w keeps its 16-bit results in columns [32w, 32w+16) of the region, i.e. over the first 16
          // columns it loaded itself, never over columns another warpgroup still has to read.
          ptx::tmem_st8(tA + lane_addr + wg * 32 + sc * 8, pk);
        }
        ptx::tmem_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive(&ctl->p_done);
        // phase 2: dS^T from dP^T and P, to TMEM (for dK) and to shared memory (for dQ)
        uint8_t* ds_tile = sdS + (g & 1) * C::kDsBytes;
        if (ok) ok = ptx::mbar_wait(&ctl->dp_full, g & 1, abort_flag);
        ptx::tc_fence_after();
#pragma unroll
        for (int sc = 0; sc < 2; ++sc) {
          const int col = wg * 32 + sc * 16;
          uint32_t dp[16], dk[8];
          ptx::tmem_ld16(tB + lane_addr + col, dp);
          ptx::tmem_wait_ld();
          ds_chunk<BF16>(p[sc], dp, vec + BQ + col, sc2, dk);
          ptx::tmem_st8(tB + lane_addr + wg * 32 + sc * 8, dk);
          // dS^T row r, queries [col, col+16): two 16-byte chunks of the 64-query block col/64
          uint8_t* row = ds_tile + (col >> 6) * kHalfBytes + r * 128;
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            const int chunk = ((col & 63) >> 3) + ch;
            *reinterpret_cast<uint4*>(row + ((chunk ^ (r & 7)) << 4)) =
                make_uint4(dk[ch * 4 + 0], dk[ch * 4 + 1], dk[ch * 4 + 2], dk[ch * 4 + 3]);
          }
        }
        ptx::mbar_arrive(&ctl->vec_free[g & 1]);
        ptx::tmem_wait_st();
        ptx::fence_proxy_async_smem();
        ptx::tc_fence_before();
        ptx::mbar_arrive(&ctl->ds_done);
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == C::kIssWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
  if (tid == 0 && ctl->abort_flag && a.status) atomicOr(a.status, kStatusWaitExpired);
}

// dq_accum (fp32, dense [B,Hq,Lq,D]) -> dq (tensor dtype, strided)
template <typename T, int D>
__global__ void __launch_bounds__(256) dq_convert_kernel(const BwdArgs a) {
  ptx::grid_dep_wait();  // launched early: the accumulator is complete from here on
  const int64_t total = static_cast<int64_t>(a.B) * a.Hq * a.Lq * (D / 8);
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c8 = static_cast<int>(idx % (D / 8));
    const int64_t rowi = idx / (D / 8);
    const int i = static_cast<int>(rowi % a.Lq);
    const int h = static_cast<int>((rowi / a.Lq) % a.Hq);
    const int b = static_cast<int>(rowi / (static_cast<int64_t>(a.Lq) * a.Hq));
    const float4* src = reinterpret_cast<const float4*>(a.dq_accum + rowi * D + c8 * 8);
    const float4 x = src[0], y = src[1];
    T out[8] = {from_f32<T>(x.x), from_f32<T>(x.y), from_f32<T>(x.z), from_f32<T>(x.w),
                from_f32<T>(y.x), from_f32<T>(y.y), from_f32<T>(y.z), from_f32<T>(y.w)};
    T* dst = reinterpret_cast<T*>(a.dq) + b * a.dqs.b + h * a.dqs.h + static_cast<int64_t>(i) * a.dqs.s + c8 * 8;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(out);
  }
}

template <int D, bool BF16, bool GEN>
cudaError_t launch_t(const BwdArgs& a, int dtype, int device, cudaStream_t stream) {
  using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  CUtensorMap tq, tk, tv, tdo, tdq, tdk, tdv;
  if (!make_map(&tq, dtype, a.q, D, a.Lq, a.Hq, a.B, a.qs) || !make_map(&tk, dtype, a.k, D, a.Skv, a.Hkv, a.B, a.ks) ||
      !make_map(&tv, dtype, a.v, D, a.Skv, a.Hkv, a.B, a.vs) ||
      !make_map(&tdo, dtype, a.d_o, D, a.Lq, a.Hq, a.B, a.dos) ||
      !make_map_f32(&tdq, a.dq_accum, D, a.Lq, a.Hq, a.B, D == 64 ? 32 : 128))
    return cudaErrorInvalidValue;
  // dK / dV leave through TMA stores (boxes of 64 columns x 32 or 128 rows); an absent output gets a map that is never used
  constexpr int kOutRows = D == 64 ? 32 : 128;
  if (!make_map(&tdk, dtype, a.dk ? a.dk : a.k, D, a.Skv, a.Hkv, a.B, a.dk ? a.dks : a.ks, kOutRows) ||
      !make_map(&tdv, dtype, a.dv ? a.dv : a.v, D, a.Skv, a.Hkv, a.B, a.dv ? a.dvs : a.vs, kOutRows))
    return cudaErrorInvalidValue;
  cudaError_t e;  // (dq_accum has been cleared by the delta pre-pass)
  void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, BwdArgs);
  if constexpr (D == 64) kern = bwd_tc64_kernel<BF16, GEN>;
  else kern = bwd_tc_kernel<BF16, GEN>;
  constexpr int kSmemBytes = D == 64 ? Cfg64::kSmem : Cfg128::kSmem;
  constexpr int kBlock = D == 64 ? Cfg64::kThreads : Cfg128::kThreads;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  const int n_kt = (a.Skv + BM - 1) / BM;
  const long long n_items = static_cast<long long>(n_kt) * a.Hkv * a.B;
  if (n_items > 0x7fffffffll) return cudaErrorInvalidValue;
  const int sms = sm_count(device);
  dim3 grid(static_cast<unsigned>(n_items < sms ? n_items : sms));  // persistent: one CTA per SM
  BwdArgs ka = a;
  // two waves' worth of heads at the end of the item order; only worth it where walks differ in length
  ka.tail_heads = 0;
  if (a.causal) {
    const long long heads = static_cast<long long>(a.Hkv) * a.B;
    const long long want = (2ll * sm_count(device) + n_kt - 1) / n_kt;
    ka.tail_heads = static_cast<int>(want < heads ? want : heads);
  }
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kBlock);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cfg.attrs = attr, cfg.numAttrs = 1;  // early launch behind the delta pre-pass
  e = cudaLaunchKernelEx(&cfg, kern, tq, tk, tv, tdo, tdq, tdk, tdv, ka);
  if (e != cudaSuccess || !a.dq) return e;
  const int64_t total = static_cast<int64_t>(a.B) * a.Hq * a.Lq * (D / 8);
  const int blocks = static_cast<int>((total + 255) / 256 < 8 * sm_count(device) ? (total + 255) / 256 : 8 * sm_count(device));
  cudaLaunchConfig_t cv = {};
  cv.gridDim = dim3(blocks);
  cv.blockDim = dim3(256);
  cv.stream = stream;
  cv.attrs = attr, cv.numAttrs = 1;
  return cudaLaunchKernelEx(&cv, dq_convert_kernel<T, D>, a);
}

}  // namespace

template <bool GEN>
cudaError_t launch_g(int dtype, int D, const BwdArgs& a, int device, cudaStream_t stream) {
  const bool bf = dtype == TT_ATTN_BF16;
  if (D == 128)
    return bf ? launch_t<128, true, GEN>(a, dtype, device, stream) : launch_t<128, false, GEN>(a, dtype, device, stream);
  if (D == 64)
    return bf ? launch_t<64, true, GEN>(a, dtype, device, stream) : launch_t<64, false, GEN>(a, dtype, device, stream);
  return cudaErrorInvalidValue;
}

cudaError_t launch_bwd_tc(int dtype, int D, const BwdArgs& a, int device, cudaStream_t stream) {
  BwdArgs pre = a;
  pre.zero_dq_accum = 1;
  // The work counter starts at zero for every launch; cleared ahead of the pre-pass so that the kernel
  // launched early behind the pre-pass already sees it.
  cudaError_t e = cudaMemsetAsync(a.sched, 0, sizeof(int), stream);
  if (e != cudaSuccess) return e;
  e = launch_bwd_delta(dtype, D, pre, stream);
  if (e != cudaSuccess) return e;
  const bool general = a.mask.ptr != nullptr || a.causal == TT_ATTN_CAUSAL_BOTTOM_RIGHT;
  return general ? launch_g<true>(dtype, D, a, device, stream) : launch_g<false>(dtype, D, a, device, stream);
}

}  // namespace ttattn
