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
// One CTA owns a 128-row key tile of one (batch, kv head) and walks the query
// tiles that see it (and the query heads of its group).  Everything is kept
// TRANSPOSED so that a TMEM lane is a key row:
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
// dV and dK accumulate in TMEM over the whole walk and are written once.  dQ of a
// (key tile, query tile) pair is added to an fp32 buffer through swizzled staging
// tiles and TMA reductions (cp.reduce.async.bulk.tensor ... add) and converted to
// the tensor dtype by a second small kernel.  Warp 16 feeds the tiles
// with TMA (128-byte swizzle, one copy per CTA), warp 17 runs the issuing loop with one elected lane issuing the MMAs;
// every wait is bounded.
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace ttattn {
namespace {

constexpr int BM = 128;  // key rows per CTA (= TMEM lanes)
constexpr int BQ = 128;  // query rows per step
constexpr int kThreads = 576;  // four compute warpgroups (32 queries of every step each) + producer warp + issuer warp
constexpr int kCompute = 512;
constexpr int kReaders = 256;  // D = 64: warpgroups 0 and 1 move dQ out of TMEM (D = 128: all four do)
constexpr int kTmemCols = 512;
constexpr int kHalfBytes = BM * 128;  // one 64-element column block of a 128-row tile

struct __align__(8) SmemCtl {
  uint64_t kv_full;
  uint64_t q_full[2], q_empty[2];
  uint64_t sp_full, pds_half, pds_full, acc_full;  // pds_half: the first 16 queries of every warpgroup are done
  uint64_t dq_full[2], dq_free[2];  // per dQ buffer
  uint64_t vec_full[2];             // per-query vectors of a step are in shared memory (written by warpgroup 0)
  uint32_t tmem_base;
  int abort_flag;
};

template <int D>
struct Cfg {
  static constexpr int TB = BM * D * 2;            // bytes of one tile
  // With D = 64 there is room (TMEM columns and shared memory) to overlap the
  // steps: two dQ accumulators, two dS^T tiles, two Q / dO stages, and dQ leaves
  // through a staging tile and TMA reductions.  With D = 128 the steps run one
  // after the other.
  static constexpr bool kPipe = (D == 64);
  static constexpr int NQ = kPipe ? 2 : 1;         // Q / dO ring depth
  static constexpr int NDS = kPipe ? 2 : 1;        // dS^T tiles
  static constexpr int kDsBytes = BM * BQ * 2;     // one dS^T tile
  // dQ staging: boxes of 128 rows x 32 floats, one per warpgroup that drains (two with D = 64, four with D = 128)
  static constexpr int kDqStage = (kPipe ? 2 : 4) * BQ * 128;
  static constexpr int kVecBytes = 2 * 2 * BQ * 4; // lse / delta vectors, double buffered
  static constexpr int kSmem = 2 * TB + 2 * NQ * TB + NDS * kDsBytes + kDqStage + kVecBytes + 256;
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

// GEN: the general variant (a mask and / or a causal triangle that is not top-left
// aligned); the fast variant compiles all of that out.
template <int D, bool BF16, bool GEN>
__global__ void __launch_bounds__(kThreads, 1)
    bwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                  const __grid_constant__ CUtensorMap tmdQ, const BwdArgs a) {
  using C = Cfg<D>;
  using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  constexpr int TB = C::TB, NQ = C::NQ, HALVES = D / 64;
  constexpr bool kPipe = C::kPipe;
  // 128-byte-swizzled tiles must start on a 1024-byte boundary; with D = 128 there is
  // no room for alignment slack, so the array itself carries the requirement
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((ptx::smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0 && a.status) atomicOr(a.status, kStatusBadSmemAlign);
    return;
  }
  uint8_t* sK = smem;
  uint8_t* sV = sK + TB;
  uint8_t* sQ = sV + TB;          // NQ tiles
  uint8_t* sdO = sQ + NQ * TB;    // NQ tiles
  uint8_t* sdS = sdO + NQ * TB;   // NDS x dS^T: [128 key rows][128 queries], two 64-query blocks, 128-byte swizzle
  uint8_t* sdq = sdS + C::NDS * C::kDsBytes;  // dQ staging: per draining warpgroup [128 queries][32 floats], swizzled
  float* svec = reinterpret_cast<float*>(sdq + C::kDqStage);  // [2 buffers][lse2 | delta][128]
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(reinterpret_cast<uint8_t*>(svec) + C::kVecBytes);
  volatile int* abort_flag = &ctl->abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // key tiles near the start see the most query tiles under the causal mask: launch them first
  // CTAs start in the order of the linear block index.  Heads in order, and within a head the key tiles in
  // order: under the causal mask the first key tile is seen by every query tile and walks longest.  Only the
  // last `tail_heads` heads are ordered differently, key tile by key tile ACROSS those heads, so that the CTAs
  // started last are the short ones and the grid ends together (in head order the last head's first key tile,
  // the longest walk there is, would start when most SMs are nearly done).
  const int n_kt = (a.Skv + BM - 1) / BM, n_heads = a.Hkv * a.B;
  int nt, bh;
  {
    const int w = blockIdx.x, w0 = (n_heads - a.tail_heads) * n_kt;
    if (w < w0) {
      bh = w / n_kt;
      nt = w - bh * n_kt;
    } else {
      const int x = w - w0;
      nt = x / a.tail_heads;
      bh = n_heads - a.tail_heads + (x - nt * a.tail_heads);
    }
  }
  const int b = bh / a.Hkv, hk = bh - b * a.Hkv;
  const int group = a.Hq / a.Hkv;
  const int kv0 = nt * BM;
  int kv_len = a.Skv;
  if (a.kv_lens) {
    int l = a.kv_lens[b];
    kv_len = l < 0 ? 0 : (l < a.Skv ? l : a.Skv);
  }
  const int n_q_tiles = (a.Lq + BQ - 1) / BQ;
  const int shift = GEN ? causal_shift(a.causal, kv_len, a.Lq) : 0;  // key j participates iff j <= i + shift
  // BM == BQ: query tiles before the key tile see none of it (general: first tile with a row i >= kv0 - shift)
  const int qt_begin = a.causal ? (GEN ? (kv0 - shift > 0 ? (kv0 - shift) / BQ : 0) : nt) : 0;
  const int per_head = (kv0 < kv_len && qt_begin < n_q_tiles) ? n_q_tiles - qt_begin : 0;
  const int n_steps = per_head * group;

  if (warp == 16 && lane == 0) {
    ptx::mbar_init(&ctl->kv_full, 1);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&ctl->q_full[i], 1);
      ptx::mbar_init(&ctl->q_empty[i], 1);
    }
    ptx::mbar_init(&ctl->sp_full, 1);
    ptx::mbar_init(&ctl->pds_full, kCompute);
    ptx::mbar_init(&ctl->pds_half, kCompute);
    ptx::mbar_init(&ctl->acc_full, 1);
    ptx::mbar_init(&ctl->vec_full[0], BM);
    ptx::mbar_init(&ctl->vec_full[1], BM);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&ctl->dq_full[i], 1);
      ptx::mbar_init(&ctl->dq_free[i], kPipe ? kReaders : kCompute);
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::tma_prefetch_desc(&tmQ);
    ptx::tma_prefetch_desc(&tmK);
    ptx::tma_prefetch_desc(&tmV);
    ptx::tma_prefetch_desc(&tmdO);
    ptx::tma_prefetch_desc(&tmdQ);
  }
  if (warp == 17) {
    ptx::tmem_alloc(&ctl->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tA = tmem;              // S^T -> P^T (16-bit pairs in cols [32w, 32w+16) per warpgroup w) -> dQ (D = 128)
  const uint32_t tB = tmem + 128;        // dP^T -> dS^T (16-bit pairs)
  const uint32_t tdV = tmem + 256;       // D columns
  const uint32_t tdK = tmem + 256 + D;   // D columns
  // dQ of step n: two buffers of D columns when there is room (D = 64), so that the
  // read-out of one step overlaps the MMAs of the next; else region A is reused
  auto tdQ = [&](int n) { return kPipe ? tmem + 384 + (n & 1) * D : tA; };

  if (warp == 16) {
    // -------------------------------------------------------------- producer --
    if (lane == 0 && n_steps > 0) {
      ptx::mbar_arrive_expect_tx(&ctl->kv_full, 2 * TB);
#pragma unroll
      for (int hf = 0; hf < HALVES; ++hf) {
        ptx::tma_load_4d(sK + hf * kHalfBytes, &tmK, &ctl->kv_full, hf * 64, kv0, hk, b);
        ptx::tma_load_4d(sV + hf * kHalfBytes, &tmV, &ctl->kv_full, hf * 64, kv0, hk, b);
      }
      for (int n = 0; n < n_steps; ++n) {
        const int st = n % NQ;
        const uint32_t ph = (n / NQ) & 1;
        const int h = hk * group + n / per_head;
        const int q0 = (qt_begin + n % per_head) * BQ;
        if (!ptx::mbar_wait(&ctl->q_empty[st], ph ^ 1, abort_flag)) break;
        ptx::mbar_arrive_expect_tx(&ctl->q_full[st], 2 * TB);
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) {
          ptx::tma_load_4d(sQ + st * TB + hf * kHalfBytes, &tmQ, &ctl->q_full[st], hf * 64, q0, h, b);
          ptx::tma_load_4d(sdO + st * TB + hf * kHalfBytes, &tmdO, &ctl->q_full[st], hf * 64, q0, h, b);
        }
      }
    }
  } else if (warp == 17) {
    // ---------------------------------------------------------------- issuer --
    // The whole warp runs the loop (waits made uniform by a vote); one elected lane issues, so that addresses
    // and descriptors stay warp-uniform.
    if (n_steps > 0) {
      const bool leader = ptx::elect_one();
      auto uwait = [&](uint64_t* bar, uint32_t parity) {
        return __all_sync(0xffffffffu, ptx::mbar_wait(bar, parity, abort_flag)) != 0;
      };
      constexpr uint32_t kHi = ptx::smem_desc_hi_sw128(1024);
      const uint32_t fmt = BF16 ? 1 : 0;
      const uint32_t idesc_s = ptx::make_idesc_f16(BM, BQ, fmt, 0, 0);   // S^T, dP^T: N = queries
      const uint32_t idesc_acc = ptx::make_idesc_f16(BM, D, fmt, 0, 1);  // dV, dK: A from TMEM, B MN-major
      const uint32_t idesc_dq = ptx::make_idesc_f16(BQ, D, fmt, 1, 1);   // dQ: both operands MN-major
      const uint32_t klo = ptx::smem_desc_lo(ptx::smem_u32(sK), 16);
      const uint32_t vlo = ptx::smem_desc_lo(ptx::smem_u32(sV), 16);
      const uint32_t klo_mn = ptx::smem_desc_lo(ptx::smem_u32(sK), kHalfBytes);
      bool ok = uwait(&ctl->kv_full, 0);
      auto stage_lo = [&](const uint8_t* base, int n, uint32_t lbo) {
        return ptx::smem_desc_lo(ptx::smem_u32(base + (n % NQ) * TB), lbo);
      };
      // S^T = K Q^T and dP^T = V dO^T of step n
      auto issue_s_dp = [&](int n) {
        if (!uwait(&ctl->q_full[n % NQ], (n / NQ) & 1)) return false;
        ptx::tc_fence_after();
        const uint32_t qlo = stage_lo(sQ, n, 16), dolo = stage_lo(sdO, n, 16);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
          if (leader) ptx::mma_ss2(tA, klo + off, kHi, qlo + off, kHi, idesc_s, ks > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
          if (leader) ptx::mma_ss2(tB, vlo + off, kHi, dolo + off, kHi, idesc_s, ks > 0 ? 1u : 0u);
        }
        if (leader) ptx::mma_commit(&ctl->sp_full);
        return true;
      };
      if (ok) ok = issue_s_dp(0);
      for (int n = 0; n < n_steps && ok; ++n) {
        const int st = n % NQ;
        const uint32_t qlo_mn = stage_lo(sQ, n, kHalfBytes), dolo_mn = stage_lo(sdO, n, kHalfBytes);
        const uint32_t dslo_mn = ptx::smem_desc_lo(ptx::smem_u32(sdS + (n % C::NDS) * C::kDsBytes), kHalfBytes);
        // dV and dK contract over the 128 queries, 16 per k-step (2048 bytes of B).  Warpgroup w forms
        // the queries of k-step 2w first and of k-step 2w+1 second, so the even k-steps run while the
        // odd ones are still being computed.
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (!(ok = uwait(half == 0 ? &ctl->pds_half : &ctl->pds_full, n & 1))) break;
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
        if (!kPipe) if (leader) ptx::mma_commit(&ctl->q_empty[st]);  // Q and dO of this step have been read (dV, dK above)
        if (kPipe) {
          // P^T / dS^T of this step have been consumed from TMEM (in issue order):
          // the next step's S^T / dP^T go first, then this step's dQ, which reads
          // dS^T from shared memory
          if (n + 1 < n_steps && !(ok = issue_s_dp(n + 1))) break;
          if (n >= 2 && !(ok = uwait(&ctl->dq_free[n & 1], ((n >> 1) - 1) & 1))) break;
        }
#pragma unroll
        for (int ks = 0; ks < BM / 16; ++ks) {  // contraction over the 128 keys
          if (leader) ptx::mma_ss2(tdQ(n), dslo_mn + ks * 128, kHi, klo_mn + ks * 128, kHi, idesc_dq, ks > 0 ? 1u : 0u);
        }
        if (leader) ptx::mma_commit(&ctl->dq_full[kPipe ? (n & 1) : 0]);
        if (kPipe) if (leader) ptx::mma_commit(&ctl->q_empty[st]);
        if (!kPipe && n + 1 < n_steps) {
          // (the single Q / dO stage was handed back after dK above, so its reload runs under
          // the dQ MMAs and the read-out.)  dP^T of the next step can go into region B at once:
          // dS^T there has been consumed in issue order.  Region A holds this step's dQ until the
          // compute threads have read it: S^T of the next step waits for that.
          if (!(ok = uwait(&ctl->q_full[(n + 1) % NQ], ((n + 1) / NQ) & 1))) break;
          ptx::tc_fence_after();
          const uint32_t qlo = stage_lo(sQ, n + 1, 16), dolo = stage_lo(sdO, n + 1, 16);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
            if (leader) ptx::mma_ss2(tB, vlo + off, kHi, dolo + off, kHi, idesc_s, ks > 0 ? 1u : 0u);
          }
          if (!(ok = uwait(&ctl->dq_free[0], n & 1))) break;
          ptx::tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
            if (leader) ptx::mma_ss2(tA, klo + off, kHi, qlo + off, kHi, idesc_s, ks > 0 ? 1u : 0u);
          }
          if (leader) ptx::mma_commit(&ctl->sp_full);
        }
      }
      if (ok) if (leader) ptx::mma_commit(&ctl->acc_full);
    }
  } else {
    // --------------------------------------------------------------- compute --
    const int wg = warp >> 2;   // which 32 queries of every step
    const int r = tid & (BM - 1);  // key row within the tile (phase 1) / query row of the step (dQ read-out)
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int kv_row = kv0 + r;
    const bool row_valid = kv_row < kv_len;
    const float c = a.scale * kLog2e;
    const float2 c2v = make_float2(c, c), sc2 = make_float2(a.scale, a.scale);
    bool ok = true;
    // This kernel is launched early behind the delta pre-pass: loads, barriers, TMEM and the first S^T / dP^T
    // MMAs need only the inputs; delta and the cleared dQ accumulator are first touched by these threads.
    ptx::grid_dep_wait();
    ptx::grid_dep_launch();  // (the conversion kernel may come up; it waits for this grid)

    // per-query vectors of step n live in svec[(n & 1)]: [0,128) -lse * log2(e), [128,256) -delta * scale;
    // warpgroup 0 fetches them one step ahead.  load_vec only issues the two loads (raw values: nothing
    // may depend on them before the step's barrier, or the whole CTA would wait for their latency);
    // store_vec converts and stores them a step's work later.
    auto load_vec = [&](int n, float& lse, float& delta) {
      const int h = hk * group + n / per_head;
      const int q = (qt_begin + n % per_head) * BQ + r;
      lse = -INFINITY;  // rows beyond Lq behave like rows without any participating key: P = 0
      delta = 0.f;
      if (q < a.Lq) {
        const int64_t idx = (static_cast<int64_t>(b) * a.Hq + h) * a.Lq + q;
        lse = a.lse[idx];
        delta = a.delta[idx];
      }
    };
    auto store_vec = [&](int n, float lse, float delta) {
      float* nv = svec + (n & 1) * 2 * BQ;
      nv[r] = lse == -INFINITY ? -INFINITY : -lse * kLog2e;
      nv[BQ + r] = -delta * a.scale;
    };
    if (n_steps > 0 && wg == 0) {
      float l0, d0;
      load_vec(0, l0, d0);
      store_vec(0, l0, d0);
      ptx::mbar_arrive(&ctl->vec_full[0]);
    }
    // dQ of step n -> global; thread r owns query row q0 + r, warpgroup w the columns
    // [32w, 32w+32) (D = 64: warpgroups 0 and 1; D = 128: all four): through a swizzled
    // staging tile and one TMA reduction per warpgroup (coalesced; rows beyond Lq are
    // clipped by the tensor map)
    auto read_out_dq = [&](int n) {
      const int h = hk * group + n / per_head;
      const int q0 = (qt_begin + n % per_head) * BQ;
      const int buf = kPipe ? (n & 1) : 0;
      if (ok) ok = ptx::mbar_wait(&ctl->dq_full[buf], (kPipe ? (n >> 1) : n) & 1, abort_flag);
      ptx::tc_fence_after();
      uint32_t v[32];
      ptx::tmem_ld32(tdQ(n) + lane_addr + wg * 32, v);
      ptx::tmem_wait_ld();
      ptx::tc_fence_before();
      ptx::mbar_arrive(&ctl->dq_free[buf]);
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
      const int q0 = (qt_begin + n % per_head) * BQ;
      const float* vec = svec + (n & 1) * 2 * BQ;
      uint8_t* ds_tile = sdS + (n % C::NDS) * C::kDsBytes;
      float ln = -INFINITY, dn = 0.f;
      if (wg == 0 && n + 1 < n_steps) load_vec(n + 1, ln, dn);  // prefetch for the next step
      // all threads reach this point every step, expired waits included
      // This step's vectors are in shared memory.  (An mbarrier, not a barrier over the four warpgroups: the two
      // that drain dQ take longer per step, and the others may go on into the next step's exponentials meanwhile.
      // Warpgroup 0 cannot overwrite a buffer that is still read: it writes buffer n & 1 again after the first
      // MMAs of step n + 1 have completed, which every warpgroup's results of step n precede.)
      if (ok) ok = ptx::mbar_wait(&ctl->vec_full[n & 1], (n >> 1) & 1, abort_flag);
      if (ok) ok = ptx::mbar_wait(&ctl->sp_full, n & 1, abort_flag);
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
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(vec + col + i);
          const float4 d4 = *reinterpret_cast<const float4*>(vec + BQ + col + i);
          // P = 2^(c*s - lse2), dS = P * (scale*dP - scale*delta), in packed fp32 pairs
          float2 x0 = ptx::fma2(make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), c2v,
                                make_float2(l4.x, l4.y));
          float2 x1 = ptx::fma2(make_float2(__uint_as_float(s[i + 2]), __uint_as_float(s[i + 3])), c2v,
                                make_float2(l4.z, l4.w));
          if constexpr (GEN) {
            if (a.mask.ptr && kv_row < a.Skv) {
              // the mask element of (query, this thread's key): adjacent threads read adjacent keys
              const int q = q0 + col + i;
              const int64_t mo = b * a.mask.sb + (hk * group + n / per_head) * a.mask.sh + q * a.mask.sl + kv_row;
              if (q + 0 < a.Lq) x0.x += mask_bias2<T>(a.mask, mo);
              if (q + 1 < a.Lq) x0.y += mask_bias2<T>(a.mask, mo + a.mask.sl);
              if (q + 2 < a.Lq) x1.x += mask_bias2<T>(a.mask, mo + 2 * a.mask.sl);
              if (q + 3 < a.Lq) x1.y += mask_bias2<T>(a.mask, mo + 3 * a.mask.sl);
            }
          }
          // (one exponential in eight on the FMA pipe: the 16 compute warps saturate the MUFU units in this phase;
          // one in four is as fast within half a percent, three in eight and more are slower again)
          float2 p0 = make_float2(ptx::ex2(x0.x), ptx::ex2(x0.y)), p1 = make_float2(ptx::ex2(x1.x), (i & 4) ? ptx::ex2_fma(x1.y) : ptx::ex2(x1.y));
          if (masked) {  // uniform over the CTA: only the diagonal step and a ragged last key tile
            const int q = q0 + col + i + shift;
            if (!row_valid || (diag && q + 0 < kv_row)) p0.x = 0.f;
            if (!row_valid || (diag && q + 1 < kv_row)) p0.y = 0.f;
            if (!row_valid || (diag && q + 2 < kv_row)) p1.x = 0.f;
            if (!row_valid || (diag && q + 3 < kv_row)) p1.y = 0.f;
          }
          const float2 g0 = ptx::fma2(make_float2(__uint_as_float(dp[i]), __uint_as_float(dp[i + 1])), sc2,
                                      make_float2(d4.x, d4.y));
          const float2 g1 = ptx::fma2(make_float2(__uint_as_float(dp[i + 2]), __uint_as_float(dp[i + 3])), sc2,
                                      make_float2(d4.z, d4.w));
          const float2 ds0 = ptx::mul2(p0, g0), ds1 = ptx::mul2(p1, g1);
          pk[(i >> 1) + 0] = pack2<BF16>(p0.x, p0.y);
          pk[(i >> 1) + 1] = pack2<BF16>(p1.x, p1.y);
          dk[(i >> 1) + 0] = pack2<BF16>(ds0.x, ds0.y);
          dk[(i >> 1) + 1] = pack2<BF16>(ds1.x, ds1.y);
        }
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
      if (wg == 0 && n + 1 < n_steps) {
        store_vec(n + 1, ln, dn);
        ptx::mbar_arrive(&ctl->vec_full[(n + 1) & 1]);
      }
      // dQ: of the previous step while this step's MMAs run (kPipe), else of this step
      if (kPipe) {
        if (wg < 2 && n >= 1) read_out_dq(n - 1);
      } else {
        read_out_dq(n);
      }
    }
    if (kPipe && n_steps > 0 && wg < 2) read_out_dq(n_steps - 1);
    if (r == 0) ptx::bulk_wait_all();

    // dV (warpgroup 0) and dK (warpgroup 1) of this key tile
    T* out = nullptr;
    if (wg == 0 && a.dv)
      out = reinterpret_cast<T*>(a.dv) + b * a.dvs.b + hk * a.dvs.h + static_cast<int64_t>(kv_row) * a.dvs.s;
    if (wg == 1 && a.dk)
      out = reinterpret_cast<T*>(a.dk) + b * a.dks.b + hk * a.dks.h + static_cast<int64_t>(kv_row) * a.dks.s;
    if (wg >= 2) {
      // warpgroups 2 and 3 have nothing to write
    } else if (n_steps > 0) {
      if (ok) ok = ptx::mbar_wait(&ctl->acc_full, 0, abort_flag);
      ptx::tc_fence_after();
      const uint32_t src = (wg == 0 ? tdV : tdK) + lane_addr;
#pragma unroll 1
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t v[32];
        ptx::tmem_ld32(src + cc * 32, v);
        ptx::tmem_wait_ld();
        if (ok && out && kv_row < a.Skv) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack2<BF16>(__uint_as_float(v[i + 0]), __uint_as_float(v[i + 1]));
            w.y = pack2<BF16>(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
            w.z = pack2<BF16>(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
            w.w = pack2<BF16>(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
            *reinterpret_cast<uint4*>(out + cc * 32 + i) = w;
          }
        }
      }
    } else if (out && kv_row < a.Skv) {
      // no query sees this key tile: zero gradients
#pragma unroll
      for (int i = 0; i < D; i += 8) *reinterpret_cast<uint4*>(out + i) = make_uint4(0, 0, 0, 0);
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 17) {
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
  CUtensorMap tq, tk, tv, tdo, tdq;
  if (!make_map(&tq, dtype, a.q, D, a.Lq, a.Hq, a.B, a.qs) || !make_map(&tk, dtype, a.k, D, a.Skv, a.Hkv, a.B, a.ks) ||
      !make_map(&tv, dtype, a.v, D, a.Skv, a.Hkv, a.B, a.vs) ||
      !make_map(&tdo, dtype, a.d_o, D, a.Lq, a.Hq, a.B, a.dos) ||
      !make_map_f32(&tdq, a.dq_accum, D, a.Lq, a.Hq, a.B))
    return cudaErrorInvalidValue;
  cudaError_t e;  // (dq_accum has been cleared by the delta pre-pass)
  auto kern = bwd_tc_kernel<D, BF16, GEN>;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::kSmem);
  if (e != cudaSuccess) return e;
  const int n_kt = (a.Skv + BM - 1) / BM;
  const long long n_ctas = static_cast<long long>(n_kt) * a.Hkv * a.B;
  if (n_ctas > 0x7fffffffll) return cudaErrorInvalidValue;
  dim3 grid(static_cast<unsigned>(n_ctas));
  BwdArgs ka = a;
  // two waves' worth of heads at the end of the grid (one CTA per SM); only worth it where walks differ in length
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
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = Cfg<D>::kSmem;
  cfg.stream = stream;
  cfg.attrs = attr, cfg.numAttrs = 1;  // early launch behind the delta pre-pass
  e = cudaLaunchKernelEx(&cfg, kern, tq, tk, tv, tdo, tdq, ka);
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
  cudaError_t e = launch_bwd_delta(dtype, D, pre, stream);
  if (e != cudaSuccess) return e;
  const bool general = a.mask.ptr != nullptr || a.causal == TT_ATTN_CAUSAL_BOTTOM_RIGHT;
  return general ? launch_g<true>(dtype, D, a, device, stream) : launch_g<false>(dtype, D, a, device, stream);
}

}  // namespace ttattn
