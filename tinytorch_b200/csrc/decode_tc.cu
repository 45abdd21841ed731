// Single-token decode for grouped-query attention on sm_100a tensor cores.
//
// With G query heads per kv head every cache row is used G times; beyond G = 1 the
// CUDA-core scan (decode.cu) runs out of FMA throughput long before HBM bandwidth
// (measured: 2.2 TB/s at G = 4, 1.5 TB/s at G = 8).  Here the G heads of a group
// become the N dimension of tcgen05 MMAs and everything is kept TRANSPOSED, so that
// a TMEM lane is a key (first MMA) or an output channel (second MMA):
//   S^T[128 keys x 16]  = K_tile[128 x D] . Q^T[D x 16]      (A, B K-major in shared memory)
//   O^T[D x 16]        += V_tile^T[D x 128 keys] . P[128 keys x 16]
//                                        (A = the V tile read MN-major, B = P K-major)
// Q of the group (rows beyond G are zero) is staged in shared memory one work item ahead.
//
// One CTA per SM (two for D = 64) draws work items (batch, kv head, split) from a global counter (sequences differ in
// length, and a fixed assignment left SMs idle at the end: 3.9 against 6.2 TB/s):
//   warp 8      producer: publishes the items that have keys through a small FIFO (one
//               item ahead of its loads), writes the empty result of items without keys
//               itself, and streams K / V tiles of 128 keys through a 3-stage TMA ring
//               that runs on across items, so HBM never waits for a prologue or epilogue
//   warp 9      issuer: one thread issues the MMAs, one first-MMA ahead of the softmax (with 16 small
//               MMAs behind three waits per tile a warp-wide loop with an elected lane was slower here)
//   warps 0-3,  two softmax warpgroups that take the tiles alternately (tile t belongs to
//   warps 4-7   warpgroup t & 1), each with its own S^T / P buffers, its own O^T
//               accumulator and its own running maximum and sum per head: two independent
//               online-softmax chains, merged once per item by warpgroup 0.  Thread r owns
//               key r of a tile (scores) and channel r of the output; the maximum of a head
//               over the 128 keys of a tile is one redux.sync per warp plus a small exchange
//               through shared memory.
// Partials of a split sequence have the layout of decode.cu and are folded by its
// combine kernel.  Every wait is bounded.
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace ttattn {
namespace {

constexpr int BK = 128, GP = 16, NFIFO = 4;
constexpr int kThreads = 320, kSoft = 128;
constexpr int kProducerWarp = 8, kIssuerWarp = 9;  // warps 0-3 and 4-7 are the softmax warpgroups
constexpr int kHalf = BK * 128;            // one 64-column half of a tile
constexpr int kPBytes = 2 * GP * 128;      // [16 heads][128 keys], two 64-key blocks (x 2 buffers)
constexpr int kMaxStages = 6;
// D = 128: 3 stages of 64 KB; D = 64: 6 stages of 32 KB (the same bytes in flight)
constexpr int kTmemCols = 64;              // S^T x 2 and O^T x 2, 16 columns each
constexpr int kItemConsumers = 1 + 2 * kSoft;  // issuer thread + both softmax warpgroups

struct ItemDesc {
  int b, hk, split, begin, end, n_tiles;  // n_tiles < 0: no more items
};

struct __align__(16) SmemCtl {
  uint64_t full[kMaxStages], empty[kMaxStages];
  uint64_t item_full[NFIFO], item_empty[NFIFO];
  uint64_t q_full[2], q_empty[2], s_full[2], s_free[2], p_full[2], pv_done[2];
  uint64_t b_done, o_free;
  ItemDesc item[NFIFO];
  alignas(16) float xmax[2][2][GP][4];  // per warpgroup, per tile parity: the four warps' maxima of a head
  float xsum[2][4][GP];     // per warpgroup: per-warp sums of an item
  float mb[GP], lb[GP]; // warpgroup 1's running maximum and total sum per head, for the merge
  uint32_t tmem_base;
  int abort_flag;
};

// OCC = 2 (D = 64 only): 3 stages of 32 KB, so that two CTAs share an SM and four softmax warpgroups
// work on its tiles; the bytes in flight per SM stay the same.
template <int D, int OCC>
struct Cfg {
  static constexpr int kTile = BK * D * 2;  // one K or V tile
  static constexpr int kStage = 2 * kTile;  // K + V
  static constexpr int NSTAGE = D == 128 ? 3 : (OCC == 2 ? 3 : 6);
  static constexpr int kQBytes = 2 * GP * D;  // [16 heads][D channels] in 64-channel blocks (x 2 buffers)
  static constexpr int kSmemBytes = NSTAGE * kStage + 2 * kQBytes + 2 * kPBytes + static_cast<int>(sizeof(SmemCtl));
};
static_assert(Cfg<128, 1>::kSmemBytes <= 232448, "exceeds the shared memory a CTA may request");
static_assert(2 * (Cfg<64, 2>::kSmemBytes + 1024) <= 233472, "two CTAs must fit the shared memory of an SM");

template <bool BF16>
__device__ __forceinline__ uint16_t to16(float x) {
  if constexpr (BF16) {
    __nv_bfloat16 t = __float2bfloat16_rn(x);
    return *reinterpret_cast<uint16_t*>(&t);
  } else {
    __half t = __float2half_rn(x);
    return *reinterpret_cast<uint16_t*>(&t);
  }
}

// maximum of a float over the warp with one redux.sync: floats are mapped to integers of the same order
__device__ __forceinline__ float warp_max(float x) {
  int i = __float_as_int(x);
  i ^= (i >> 31) & 0x7fffffff;
  int r;
  asm volatile("redux.sync.max.s32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(i));
  r ^= (r >> 31) & 0x7fffffff;
  return __int_as_float(r);
}

__device__ __forceinline__ ItemDesc item_of(const DecodeArgs& a, int w) {
  ItemDesc it;
  it.split = w % a.nsplit;
  const int bh = w / a.nsplit;
  it.hk = bh % a.Hkv;
  it.b = bh / a.Hkv;
  int len = a.capacity;
  if (a.kv_lens) {
    const int l = a.kv_lens[it.b];
    len = l < 0 ? 0 : (l < a.capacity ? l : a.capacity);
  }
  it.begin = it.split * a.chunk;
  it.end = len < it.begin + a.chunk ? len : it.begin + a.chunk;
  it.n_tiles = it.end > it.begin ? (it.end - it.begin + BK - 1) / BK : 0;
  return it;
}

// GH: the heads of a group rounded up to 4, 8 or 16.  The softmax loops run over GH heads without a test on the
// group size: every head's chain of reduction, exchange and exponentials is then scheduled next to the others'
// (with a test per head each chain ran alone, latency after latency: 2000 cycles per tile instead of 700).
// Heads beyond the group are rows of zeros in Q: their numbers are finite and nobody reads them.
template <bool BF16, int D, int OCC, int GH>
__global__ void __launch_bounds__(kThreads, OCC)
    decode_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const DecodeArgs a,
                     int n_items) {
  using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  constexpr int kTile = Cfg<D, OCC>::kTile, kStage = Cfg<D, OCC>::kStage, NSTAGE = Cfg<D, OCC>::NSTAGE;
  constexpr int kQBytes = Cfg<D, OCC>::kQBytes;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((ptx::smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0 && a.status) atomicOr(a.status, kStatusBadSmemAlign);
    return;
  }
  uint8_t* sQ = smem + NSTAGE * kStage;
  uint8_t* sP = sQ + 2 * kQBytes;
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(sP + 2 * kPBytes);
  volatile int* abort_flag = &ctl->abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = a.Hq / a.Hkv;

  if (warp == kProducerWarp && lane == 0) {
#pragma unroll
    for (int s = 0; s < NSTAGE; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
#pragma unroll
    for (int s = 0; s < NFIFO; ++s) {
      ptx::mbar_init(&ctl->item_full[s], 1);
      ptx::mbar_init(&ctl->item_empty[s], kItemConsumers);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&ctl->q_full[i], kSoft);
      ptx::mbar_init(&ctl->q_empty[i], 1);
      ptx::mbar_init(&ctl->s_full[i], 1);
      ptx::mbar_init(&ctl->s_free[i], kSoft);
      ptx::mbar_init(&ctl->p_full[i], kSoft);
      ptx::mbar_init(&ctl->pv_done[i], 1);
    }
    ptx::mbar_init(&ctl->b_done, kSoft);
    ptx::mbar_init(&ctl->o_free, kSoft);
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::tma_prefetch_desc(&tmK);
    ptx::tma_prefetch_desc(&tmV);
  }
  if (warp == kIssuerWarp) {
    ptx::tmem_alloc(&ctl->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tS = tmem, tO = tmem + 2 * GP;  // buffer i of each at + 16 i
  // Everything above touched no global memory.  In a chained launch the kernel before this one (rotation and
  // append) may still be running: wait for its results, then let the combine kernel's CTAs come up.
  ptx::grid_dep_wait();
  ptx::grid_dep_launch();

  if (warp == kProducerWarp) {
    // -------------------------------------------------------------- producer --
    // All 32 lanes walk the items (an item without keys gets its empty result from this warp);
    // lane 0 publishes the others and issues the loads.
    uint32_t g = 0, pub = 0;
    bool ok = true;
    // draws items from the counter until one has keys, publishes it (or the end marker)
    auto publish_next = [&](ItemDesc* out) {
      ItemDesc it;
      it.n_tiles = -1;
      for (;;) {
        int w = 0;
        if (lane == 0) w = atomicAdd(a.sched, 1);
        w = __shfl_sync(0xffffffffu, w, 0);
        if (w >= n_items) break;
        it = item_of(a, w);
        if (it.n_tiles > 0) break;
        for (int h = 0; h < group; ++h) {
          const int hq = it.hk * group + h;
          if (a.nsplit == 1) {
            for (int d = lane; d < D; d += 32) reinterpret_cast<T*>(a.o)[it.b * a.os.b + hq * a.os.h + d] = from_f32<T>(0.f);
            if (a.lse && lane == 0) a.lse[static_cast<int64_t>(it.b) * a.Hq + hq] = -INFINITY;
          } else {
            float* pp = a.partial + ((static_cast<int64_t>(it.b) * a.Hq + hq) * a.nsplit + it.split) * (D + 2);
            for (int d = lane; d < D; d += 32) pp[d] = 0.f;
            if (lane == 0) pp[D] = -INFINITY, pp[D + 1] = 0.f;
          }
        }
        it.n_tiles = -1;
      }
      if (lane == 0) {
        const int slot = pub % NFIFO;
        if (ok) ok = ptx::mbar_wait(&ctl->item_empty[slot], ((pub / NFIFO) & 1) ^ 1, abort_flag);
        ctl->item[slot] = it;
        ptx::mbar_arrive(&ctl->item_full[slot]);
      }
      ++pub;
      *out = it;
    };
    ItemDesc cur;
    publish_next(&cur);
    while (cur.n_tiles > 0) {
      ItemDesc nxt;
      publish_next(&nxt);  // one item ahead of the loads
      if (lane == 0) {
        for (int j = 0; j < cur.n_tiles && ok; ++j, ++g) {
          const int s = g % NSTAGE;
          if (!(ok = ptx::mbar_wait(&ctl->empty[s], ((g / NSTAGE) & 1) ^ 1, abort_flag))) break;
          uint8_t* st = smem + s * kStage;
          ptx::mbar_arrive_expect_tx(&ctl->full[s], kStage);
          const int row = cur.begin + j * BK;  // rows beyond the cache read as zero
#pragma unroll
          for (int hf = 0; hf < D / 64; ++hf) {
            ptx::tma_load_4d(st + hf * kHalf, &tmK, &ctl->full[s], hf * 64, row, cur.hk, cur.b);
            ptx::tma_load_4d(st + kTile + hf * kHalf, &tmV, &ctl->full[s], hf * 64, row, cur.hk, cur.b);
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      cur = nxt;
    }
    // A wait has expired: whatever a consumer still reads from the queue must be the end marker, not an old item.
    if (!ok && lane == 0) {
      for (int slot = 0; slot < NFIFO; ++slot) ctl->item[slot].n_tiles = -1;
    }
  } else if (warp == kIssuerWarp) {
    // ---------------------------------------------------------------- issuer --
    if (lane == 0) {
      constexpr uint32_t kHi = ptx::smem_desc_hi_sw128(1024);
      const uint32_t fmt = BF16 ? 1 : 0;
      const uint32_t idesc_s = ptx::make_idesc_f16(BK, GP, fmt, 0, 0);  // S^T: A = K tile, B = Q, both K-major
      // O^T: A = V tile MN-major (M = 128 channels; with D = 64 the second 64-channel block of the descriptor is the
      // first one again, so lanes 64-127 of O^T repeat lanes 0-63 and are ignored), B = P K-major
      const uint32_t idesc_o = ptx::make_idesc_f16(128, GP, fmt, 1, 0);
      uint32_t items = 0, tiles = 0;  // items / tiles so far (ring position = tiles)
      bool ok = true;
      // S^T = K_tile Q^T of global tile t (stage t % NSTAGE) into S^T buffer t & 1
      auto issue_s = [&](uint32_t t, uint32_t qb) {
        const int s = t % NSTAGE;
        if (!ptx::mbar_wait(&ctl->full[s], (t / NSTAGE) & 1, abort_flag)) return false;
        // the softmax warpgroup of this buffer has read what it held two tiles ago
        if (!ptx::mbar_wait(&ctl->s_free[t & 1], ((t >> 1) & 1) ^ 1, abort_flag)) return false;
        ptx::tc_fence_after();
        const uint32_t klo = ptx::smem_desc_lo(ptx::smem_u32(smem + s * kStage), 16);
        const uint32_t qlo = ptx::smem_desc_lo(ptx::smem_u32(sQ + qb * kQBytes), 16);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t oa = ((ks >> 2) * kHalf + (ks & 3) * 32) >> 4;       // 64-channel halves of the K tile
          const uint32_t ob = ((ks >> 2) * (GP * 128) + (ks & 3) * 32) >> 4;  // ... and of Q
          ptx::mma_ss2(tS + (t & 1) * GP, klo + oa, kHi, qlo + ob, kHi, idesc_s, ks > 0 ? 1u : 0u);
        }
        ptx::mma_commit(&ctl->s_full[t & 1]);
        return true;
      };
      for (;; ++items) {
        const int slot = items % NFIFO;
        if (!(ok = ptx::mbar_wait(&ctl->item_full[slot], (items / NFIFO) & 1, abort_flag))) break;
        const ItemDesc it = ctl->item[slot];
        ptx::mbar_arrive(&ctl->item_empty[slot]);
        if (it.n_tiles < 0) break;
        const uint32_t qb = items & 1;
        if (!(ok = ptx::mbar_wait(&ctl->q_full[qb], (items >> 1) & 1, abort_flag))) break;
        if (!(ok = issue_s(tiles, qb))) break;
        if (it.n_tiles == 1) ptx::mma_commit(&ctl->q_empty[qb]);
        bool first[2] = {true, true};  // the first second-MMA of each accumulator overwrites it
        for (int j = 0; j < it.n_tiles; ++j, ++tiles) {
          if (j + 1 < it.n_tiles) {
            // one first-MMA ahead: the softmax of tile j+1 need not wait for the second MMA of tile j
            if (!(ok = issue_s(tiles + 1, qb))) break;
            if (j + 2 == it.n_tiles) ptx::mma_commit(&ctl->q_empty[qb]);  // Q of this item has been read
          }
          const uint32_t wb = tiles & 1;  // warpgroup / buffers of this tile
          if (!(ok = ptx::mbar_wait(&ctl->p_full[wb], (tiles >> 1) & 1, abort_flag))) break;
          ptx::tc_fence_after();
          const int s = tiles % NSTAGE;
          const uint32_t vlo = ptx::smem_desc_lo(ptx::smem_u32(smem + s * kStage + kTile), D == 128 ? kHalf : 0);
          const uint32_t plo = ptx::smem_desc_lo(ptx::smem_u32(sP + wb * kPBytes), 16);
#pragma unroll
          for (int ks = 0; ks < BK / 16; ++ks) {  // 16 keys per step: 2048 bytes of the V tile, 32 bytes of a P row
            const uint32_t ob = ((ks >> 2) * (GP * 128) + (ks & 3) * 32) >> 4;
            ptx::mma_ss2(tO + wb * GP, vlo + ks * 128, kHi, plo + ob, kHi, idesc_o, (!first[wb] || ks > 0) ? 1u : 0u);
          }
          first[wb] = false;
          ptx::mma_commit(&ctl->empty[s]);
          ptx::mma_commit(&ctl->pv_done[wb]);
        }
        if (!ok) break;
      }
    }
  } else if (warp < 8) {
    // --------------------------------------------------------------- softmax --
    const int wg = warp >> 2;           // tiles t with (t & 1) == wg
    const int sw = warp & 3;
    const int r = tid & (kSoft - 1);        // key of the tile (scores) / output channel (O^T)
    const uint32_t lane_addr = static_cast<uint32_t>(sw * 32) << 16;
    const float c = a.scale * kLog2e;
    uint32_t items = 0, tiles = 0;  // items seen / global tile index at the start of the current item
    uint32_t mine = 0;              // tiles this warpgroup has processed (its barrier phases)
    uint32_t merges = 0;            // items merged so far (b_done / o_free phases)
    bool ok = true;

    auto next_desc = [&](uint32_t idx) {
      const int slot = idx % NFIFO;
      if (ok) ok = ptx::mbar_wait(&ctl->item_full[slot], (idx / NFIFO) & 1, abort_flag);
      const ItemDesc it = ctl->item[slot];
      ptx::mbar_arrive(&ctl->item_empty[slot]);
      return it;
    };
    // Q of a group: 16 rows x D/8 chunks of 16 bytes, D/64 chunks per thread (rows beyond the group are zero)
    constexpr int CPR = D / 8;  // chunks per row
    auto load_q = [&](const ItemDesc& it, uint4 (&qv)[2]) {
#pragma unroll
      for (int i = 0; i < D / 64; ++i) {
        const int idx = r + i * kSoft, n = idx / CPR, ch = idx % CPR;
        qv[i] = make_uint4(0, 0, 0, 0);
        if (n < group)
          qv[i] = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.q) + it.b * a.qs.b +
                                                  (it.hk * group + n) * a.qs.h + ch * 8);
      }
    };
    // ... into shared-memory buffer qb (K-major, 128-byte swizzle), then signalled to the issuer
    auto store_q = [&](uint32_t qb, const uint4 (&qv)[2]) {
#pragma unroll
      for (int i = 0; i < D / 64; ++i) {
        const int idx = r + i * kSoft, n = idx / CPR, ch = idx % CPR;
        *reinterpret_cast<uint4*>(sQ + qb * kQBytes + (ch >> 3) * (GP * 128) + n * 128 + (((ch & 7) ^ (n & 7)) << 4)) = qv[i];
      }
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(&ctl->q_full[qb]);
    };

    // warpgroup 0 stays one descriptor ahead (it stages the next item's Q); warpgroup 1 reads them in step
    // After an expired wait next_desc() no longer waits and may return an old item, and the threads of a
    // warpgroup meet at named barriers inside an item: so the warpgroup votes after every fetch and leaves
    // together, before it acts on a descriptor that some of its threads did not wait for.
    ItemDesc it = next_desc(0), nx;
    nx.n_tiles = -1;
    if (ptx::named_barrier_or(1 + wg, kSoft, !ok)) it.n_tiles = -1;
    if (wg == 0 && it.n_tiles > 0) {
      uint4 qv[2];
      load_q(it, qv);
      store_q(0, qv);
    }
    for (; it.n_tiles > 0; ++items) {
      const int h0 = it.hk * group;
      uint4 qn[2];
      if (wg == 0) {
        nx = next_desc(items + 1);
        if (nx.n_tiles > 0) load_q(nx, qn);  // in flight while the first tile is processed
      }
      float m[GH], l[GH];
#pragma unroll
      for (int h = 0; h < GH; ++h) m[h] = -INFINITY, l[h] = 0.f;
      int done = 0;  // tiles of this item processed by this warpgroup

      for (int j = 0; j < it.n_tiles; ++j) {
        const uint32_t t = tiles + j;
        if ((t & 1) != static_cast<uint32_t>(wg)) continue;
        if (ok) ok = ptx::mbar_wait(&ctl->s_full[wg], (t >> 1) & 1, abort_flag);
        ptx::tc_fence_after();
        uint32_t sv[GP];
        ptx::tmem_ld16(tS + wg * GP + lane_addr, sv);
        ptx::tmem_wait_ld();
        ptx::tc_fence_before();
        ptx::mbar_arrive(&ctl->s_free[wg]);
        const int key = it.begin + j * BK + r;
        const bool valid = key < it.end;
        // maximum per head over the 128 keys: one redux per head and warp, lane h keeps head h's and writes it;
        // the exchange buffer alternates with the tile, so one barrier per tile is enough (a warp cannot be two
        // tiles ahead of another)
        float x[GH], wm[GH];
#pragma unroll
        for (int h = 0; h < GH; ++h) x[h] = valid ? __uint_as_float(sv[h]) * c : -INFINITY;
#pragma unroll
        for (int h = 0; h < GH; ++h) wm[h] = warp_max(x[h]);
        float own = wm[0];
#pragma unroll
        for (int h = 1; h < GH; ++h) own = lane == h ? wm[h] : own;
        float(*xm)[4] = ctl->xmax[wg][mine & 1];
        if (lane < GH) xm[lane][sw] = own;
        ptx::named_barrier(1 + wg, kSoft);
        bool rescale = false;
        float alpha[GH], pv[GH];
        uint8_t* prow = sP + wg * kPBytes + (r >> 6) * (GP * 128) + (r & 7) * 2;
        const int pchunk = (r & 63) >> 3;
#pragma unroll
        for (int h = 0; h < GH; ++h) {
          const float4 w4 = *reinterpret_cast<const float4*>(xm[h]);
          const float mn = fmaxf(m[h], fmaxf(fmaxf(w4.x, w4.y), fmaxf(w4.z, w4.w)));
          // a head that has seen no valid key yet keeps m = -inf; its exponentials are taken against 0 (all 0)
          alpha[h] = mn == -INFINITY ? 1.f : ptx::ex2(m[h] - mn);
          pv[h] = ptx::ex2(x[h] - (mn == -INFINITY ? 0.f : mn));
          m[h] = mn;
        }
#pragma unroll
        for (int h = 0; h < GH; ++h) {
          rescale |= alpha[h] != 1.f;
          l[h] = l[h] * alpha[h] + pv[h];
          // P[h][key r]: K-major rows of 128 keys (two 64-key blocks), 128-byte swizzle.  Rows of heads
          // beyond GH are never written: they only feed output columns that nobody reads.
          *reinterpret_cast<uint16_t*>(prow + h * 128 + ((pchunk ^ (h & 7)) << 4)) = to16<BF16>(pv[h]);
        }
        // V rows at or beyond the length may hold anything; make them exact zeros so that 0 x garbage
        // cannot produce NaN
        if (!valid) {
          uint8_t* vt = smem + (t % NSTAGE) * kStage + kTile;
#pragma unroll
          for (int hf = 0; hf < D / 64; ++hf)
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
              *reinterpret_cast<uint4*>(vt + hf * kHalf + r * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        if (done == 0) {
          // the first tile of this warpgroup in this item overwrites its accumulator: warpgroup 0 must have
          // merged the previous item out of it
          if (wg == 1 && merges > 0 && ok) ok = ptx::mbar_wait(&ctl->o_free, (merges - 1) & 1, abort_flag);
        } else if (rescale) {
          // m is the same in every thread, so the decision is uniform; O^T holds the sum of this warpgroup's tiles so far
          if (ok) ok = ptx::mbar_wait(&ctl->pv_done[wg], (mine - 1) & 1, abort_flag);
          ptx::tc_fence_after();
          uint32_t ov[GP];
          ptx::tmem_ld16(tO + wg * GP + lane_addr, ov);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int h = 0; h < GH; ++h) ov[h] = __float_as_uint(__uint_as_float(ov[h]) * alpha[h]);
          ptx::tmem_st16(tO + wg * GP + lane_addr, ov);
          ptx::tmem_wait_st();
        }
        ptx::fence_proxy_async_smem();
        ptx::tc_fence_before();
        ptx::mbar_arrive(&ctl->p_full[wg]);
        ++done;
        ++mine;
        if (wg == 0 && done == 1 && nx.n_tiles > 0) {
          // stage the next item's Q: its buffer was last read by the item before this one
          if (items >= 1 && ok) ok = ptx::mbar_wait(&ctl->q_empty[(items + 1) & 1], ((items - 1) >> 1) & 1, abort_flag);
          store_q((items + 1) & 1, qn);
        }
      }
      if (wg == 0 && done == 0 && nx.n_tiles > 0) {
        // (an item whose only tile belongs to warpgroup 1) the next item's Q still has to be staged
        if (items >= 1 && ok) ok = ptx::mbar_wait(&ctl->q_empty[(items + 1) & 1], ((items - 1) >> 1) & 1, abort_flag);
        store_q((items + 1) & 1, qn);
      }

      // total sum per head of this warpgroup's keys
      ptx::named_barrier(1 + wg, kSoft);
      {
        float own = 0.f;
#pragma unroll
        for (int h = 0; h < GH; ++h) {
          float ls = l[h];
#pragma unroll
          for (int of = 16; of >= 1; of >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, of);
          own = lane == h ? ls : own;
        }
        if (lane < GH) ctl->xsum[wg][sw][lane] = own;
      }
      ptx::named_barrier(1 + wg, kSoft);
      if (wg == 1) {
        // hand maximum and sum to warpgroup 0; O^T buffer 1 is complete once pv_done says so
        if (done > 0 && ok) ok = ptx::mbar_wait(&ctl->pv_done[1], (mine - 1) & 1, abort_flag);
        // warpgroup 0 has taken the previous item's values out of mb / lb (and out of O^T buffer 1)
        if (merges > 0 && ok) ok = ptx::mbar_wait(&ctl->o_free, (merges - 1) & 1, abort_flag);
        if (r < GH) {
          float mv = m[0];
#pragma unroll
          for (int h = 1; h < GH; ++h) mv = r == h ? m[h] : mv;
          ctl->mb[r] = done > 0 ? mv : -INFINITY;
          ctl->lb[r] = ctl->xsum[1][0][r] + ctl->xsum[1][1][r] + ctl->xsum[1][2][r] + ctl->xsum[1][3][r];
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive(&ctl->b_done);
      } else {
        if (done > 0 && ok) ok = ptx::mbar_wait(&ctl->pv_done[0], (mine - 1) & 1, abort_flag);
        if (ok) ok = ptx::mbar_wait(&ctl->b_done, merges & 1, abort_flag);
        ptx::tc_fence_after();
        uint32_t oa[GP], ob[GP];
        ptx::tmem_ld16(tO + lane_addr, oa);
        ptx::tmem_ld16(tO + GP + lane_addr, ob);
        float mbr[GH], lbr[GH];  // (entries beyond the group are stale: they feed nothing that is stored)
#pragma unroll
        for (int h = 0; h < GH; ++h) mbr[h] = ctl->mb[h], lbr[h] = ctl->lb[h];
        ptx::tmem_wait_ld();
        ptx::tc_fence_before();
        ptx::mbar_arrive(&ctl->o_free);  // warpgroup 1 may reuse its accumulator and mb / lb
#pragma unroll
        for (int h = 0; h < GH; ++h) {
          {
            const float la = ctl->xsum[0][0][h] + ctl->xsum[0][1][h] + ctl->xsum[0][2][h] + ctl->xsum[0][3][h];
            const float ma = done > 0 ? m[h] : -INFINITY, mbv = mbr[h], lbv = lbr[h];
            const float mn = fmaxf(ma, mbv);
            // a side without tiles (or without valid keys) has maximum -inf and takes no part
            const float wa = ma == -INFINITY ? 0.f : ptx::ex2(ma - mn), wb = mbv == -INFINITY ? 0.f : ptx::ex2(mbv - mn);
            const float lt = la * wa + lbv * wb;
            float oh = (wa > 0.f ? __uint_as_float(oa[h]) * wa : 0.f) + (wb > 0.f ? __uint_as_float(ob[h]) * wb : 0.f);
            const int hq = h0 + h;
            if (r < D && h < group && ok) {  // D = 64: lanes 64-127 hold copies; heads beyond the group are padding
              // (nothing is stored after an expired wait: the status word reports it)
              if (a.nsplit == 1) {
                const float inv = lt > 0.f ? 1.f / lt : 0.f;
                reinterpret_cast<T*>(a.o)[it.b * a.os.b + hq * a.os.h + r] = from_f32<T>(oh * inv);
                if (a.lse && r == 0)
                  a.lse[static_cast<int64_t>(it.b) * a.Hq + hq] = lt > 0.f ? (mn + log2f(lt)) * kLn2 : -INFINITY;
              } else {
                float* pp = a.partial + ((static_cast<int64_t>(it.b) * a.Hq + hq) * a.nsplit + it.split) * (D + 2);
                pp[r] = oh;
                if (r == 0) pp[D] = lt > 0.f ? mn : -INFINITY, pp[D + 1] = lt;
              }
            }
          }
        }
      }
      ++merges;
      tiles += it.n_tiles;
      it = wg == 0 ? nx : next_desc(items + 1);
      if (ptx::named_barrier_or(1 + wg, kSoft, !ok)) break;
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kIssuerWarp) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
  if (tid == 0 && ctl->abort_flag && a.status) atomicOr(a.status, kStatusWaitExpired);
}

template <bool BF16, int D, int OCC, int GH>
cudaError_t launch_g(int dtype, const DecodeArgs& a, cudaStream_t stream) {
  constexpr int kSmem = Cfg<D, OCC>::kSmemBytes;
  CUtensorMap tk, tv;
  if (!make_map(&tk, dtype, a.k, D, a.capacity, a.Hkv, a.B, a.ks) || !make_map(&tv, dtype, a.v, D, a.capacity, a.Hkv, a.B, a.vs))
    return cudaErrorInvalidValue;
  auto kern = decode_tc_kernel<BF16, D, OCC, GH>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (e != cudaSuccess) return e;
  int device = 0;
  e = cudaGetDevice(&device);
  if (e != cudaSuccess) return e;
  const long long n_items = static_cast<long long>(a.B) * a.Hkv * a.nsplit;
  if (n_items > 0x7fffffffll || !a.sched) return cudaErrorInvalidValue;
  const int ctas = OCC * sm_count(device);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(n_items < ctas ? n_items : ctas));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  if (a.chained) {
    cfg.attrs = attr, cfg.numAttrs = 1;
  } else {
    e = cudaMemsetAsync(a.sched, 0, sizeof(int), stream);  // the work counter starts at zero for every launch
    if (e != cudaSuccess) return e;
  }
  return cudaLaunchKernelEx(&cfg, kern, tk, tv, a, static_cast<int>(n_items));
}

template <bool BF16, int D, int OCC>
cudaError_t launch_t(int dtype, const DecodeArgs& a, cudaStream_t stream) {
  const int group = a.Hq / a.Hkv;
  if (group <= 4) return launch_g<BF16, D, OCC, 4>(dtype, a, stream);
  if (group <= 8) return launch_g<BF16, D, OCC, 8>(dtype, a, stream);
  return launch_g<BF16, D, OCC, 16>(dtype, a, stream);
}

}  // namespace

bool decode_tc_applies(int dtype, int D, const DecodeArgs& a) {
  const int group = a.Hkv > 0 ? a.Hq / a.Hkv : 0;
  return dtype != TT_ATTN_F32 && (D == 64 || D == 128) && group >= 2 && group <= GP;
}

// The scan only; the caller folds the per-split partials (decode.cu's combine kernel).
cudaError_t launch_decode_tc(int dtype, int D, const DecodeArgs& a, cudaStream_t stream) {
  if (D == 128) return dtype == TT_ATTN_BF16 ? launch_t<true, 128, 1>(dtype, a, stream) : launch_t<false, 128, 1>(dtype, a, stream);
  // D = 64: a tile is half the bytes for the same count of MMAs and softmax steps, so two CTAs per SM
  // (measured 4.8 against 4.15 TB/s with one)
  return dtype == TT_ATTN_BF16 ? launch_t<true, 64, 2>(dtype, a, stream) : launch_t<false, 64, 2>(dtype, a, stream);
}

}  // namespace ttattn
