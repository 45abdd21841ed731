// Prefill forward for fp16 / bf16 on sm_100a tensor cores.
//
// Replaces the score-materialising composition of FuncSDPAttention::forward
// (reference: src/Function/FuncNNLayer.h:231-266) by one fused kernel that never
// writes the [L,S] score matrix to HBM.
//
// One CTA owns a 128-row query tile of one (batch, head) and walks the key/value
// sequence in 128-row tiles:
//   warp 4   producer : TMA tiled loads (128-byte swizzle, no multicast) of the Q
//                       tile once and of each K and V tile into shared memory
//   warp 5   issuer   : one thread issues tcgen05.mma; S = Q.K^T accumulates in
//                       TMEM columns [0,128), O += P.V in TMEM columns [128,128+D)
//   warps 0-3 softmax : thread t owns query row t (= TMEM lane t): reads its S
//                       row with tcgen05.ld, keeps the running max / sum in
//                       registers (no cross-thread reduction is needed in this
//                       layout), writes P as packed 16-bit pairs over the S
//                       columns with tcgen05.st, rescales O only when the row
//                       max grew by more than 2^8, and finally writes O and LSE
// P never leaves TMEM: the second MMA takes its A operand from TMEM.
// K and V are single-buffered so that two CTAs fit on one SM (96 KB + 256 TMEM
// columns each); the second CTA's MMAs fill the tensor pipe while the first is in
// its softmax.
#include <cuda.h>

#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace ttattn {
namespace {

constexpr int BM = 128;  // query rows per CTA
constexpr int BN = 128;  // keys per tile
constexpr int kThreads = 192;
constexpr int kTmemCols = 256;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct __align__(8) SmemCtl {
  uint64_t q_full, k_full, k_empty, v_full, v_empty, s_full, p_full, o_full;
  uint32_t tmem_base;
  int abort_flag;
};

template <int D>
constexpr int tile_bytes() {
  return BM * D * 2;
}
// Sized for D = 128 at every D: the request also caps residency at two CTAs
// per SM, which is what the 512 TMEM columns allow (256 per CTA).
template <int D>
constexpr int smem_bytes() {
  return 3 * tile_bytes<128>() + 1024 /*alignment slack*/ + 128 /*SmemCtl*/;
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
__global__ void __launch_bounds__(kThreads, 2)
    fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const FwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles must start on a 1024-byte boundary.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + tile_bytes<D>();
  uint8_t* sV = smem + 2 * tile_bytes<D>();
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(smem + 3 * tile_bytes<D>());
  volatile int* abort_flag = &ctl->abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // Heaviest (latest) causal tiles are launched first.
  const int mt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = h / (a.Hq / a.Hkv);
  const int row0 = mt * BM;

  int kv_len = a.Skv;
  if (a.kv_lens) {
    int l = a.kv_lens[b];
    kv_len = l < 0 ? 0 : (l < a.Skv ? l : a.Skv);
  }
  int kv_end = kv_len;
  if (a.causal && row0 + BM < kv_end) kv_end = row0 + BM;
  const int n_tiles = (kv_end + BN - 1) / BN;

  if (warp == 4 && lane == 0) {
    ptx::mbar_init(&ctl->q_full, 1);
    ptx::mbar_init(&ctl->k_full, 1);
    ptx::mbar_init(&ctl->k_empty, 1);
    ptx::mbar_init(&ctl->v_full, 1);
    ptx::mbar_init(&ctl->v_empty, 1);
    ptx::mbar_init(&ctl->s_full, 1);
    ptx::mbar_init(&ctl->p_full, 128);
    ptx::mbar_init(&ctl->o_full, 1);
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::tma_prefetch_desc(&tmQ);
    ptx::tma_prefetch_desc(&tmK);
    ptx::tma_prefetch_desc(&tmV);
  }
  if (warp == 5) {
    ptx::tmem_alloc(&ctl->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tS = tmem;        // S (fp32, 128 cols); P (16-bit pairs) overlays cols [0,64)
  const uint32_t tO = tmem + 128;  // O (fp32, D cols)

  constexpr int HALVES = D / 64;  // 64-element (128-byte) column blocks per row
  constexpr int HALF_BYTES = BM * 128;

  if (warp == 4) {
    // ------------------------------------------------------------ producer --
    if (lane == 0 && n_tiles > 0) {
      ptx::mbar_arrive_expect_tx(&ctl->q_full, tile_bytes<D>());
#pragma unroll
      for (int hf = 0; hf < HALVES; ++hf) ptx::tma_load_4d(sQ + hf * HALF_BYTES, &tmQ, &ctl->q_full, hf * 64, row0, h, b);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const uint32_t ph = static_cast<uint32_t>(j & 1);
        ok = ptx::mbar_wait(&ctl->k_empty, ph ^ 1, abort_flag);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(&ctl->k_full, tile_bytes<D>());
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf)
          ptx::tma_load_4d(sK + hf * HALF_BYTES, &tmK, &ctl->k_full, hf * 64, j * BN, hk, b);
        ok = ptx::mbar_wait(&ctl->v_empty, ph ^ 1, abort_flag);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(&ctl->v_full, tile_bytes<D>());
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf)
          ptx::tma_load_4d(sV + hf * HALF_BYTES, &tmV, &ctl->v_full, hf * 64, j * BN, hk, b);
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------- issuer --
    if (lane == 0 && n_tiles > 0) {
      // A negative scale is folded into the sign of Q so that the softmax
      // always works with a non-negative multiplier.
      const uint32_t neg = a.scale < 0.f ? (1u << 13) : 0u;
      const uint32_t idesc_qk = ptx::make_idesc_f16(BM, BN, BF16 ? 1 : 0, 0, 0) | neg;
      const uint32_t idesc_pv = ptx::make_idesc_f16(BM, D, BF16 ? 1 : 0, 0, 1);
      const uint32_t aQ = ptx::smem_u32(sQ), aK = ptx::smem_u32(sK), aV = ptx::smem_u32(sV);
      bool ok = ptx::mbar_wait(&ctl->q_full, 0, abort_flag);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const uint32_t ph = static_cast<uint32_t>(j & 1);
        ok = ptx::mbar_wait(&ctl->k_full, ph, abort_flag);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          // K-major operands: 64-element halves 16 KB apart, 32 bytes per k-step
          const uint32_t off = (ks >> 2) * HALF_BYTES + (ks & 3) * 32;
          ptx::mma_ss(tS, ptx::make_smem_desc_sw128(aQ + off, 16, 1024), ptx::make_smem_desc_sw128(aK + off, 16, 1024),
                      idesc_qk, ks > 0 ? 1u : 0u);
        }
        ptx::mma_commit(&ctl->k_empty);
        ptx::mma_commit(&ctl->s_full);
        ok = ptx::mbar_wait(&ctl->v_full, ph, abort_flag);
        if (!ok) break;
        ok = ptx::mbar_wait(&ctl->p_full, ph, abort_flag);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          // V is N(=D)-contiguous: 16 keys per k-step = 2048 bytes; the two
          // 64-wide column blocks of D=128 are HALF_BYTES apart (LBO).
          ptx::mma_ts(tO, tS + ks * 8, ptx::make_smem_desc_sw128(aV + ks * 2048, HALF_BYTES, 1024), idesc_pv,
                      (j > 0 || ks > 0) ? 1u : 0u);
        }
        ptx::mma_commit(&ctl->v_empty);
        if (j == n_tiles - 1) ptx::mma_commit(&ctl->o_full);
      }
    }
  } else {
    // ------------------------------------------------------------- softmax --
    const int row = row0 + tid;                                   // global query row of this thread
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;  // TMEM lane quarter of this warp
    const float c = fabsf(a.scale) * kLog2e;
    float m_ref = -INFINITY;  // reference max, in scaled log2 units
    float l = 0.f;
    bool ok = true;
    uint32_t r[32];

    for (int j = 0; j < n_tiles && ok; ++j) {
      const uint32_t ph = static_cast<uint32_t>(j & 1);
      ok = ptx::mbar_wait(&ctl->s_full, ph, abort_flag);
      if (!ok) break;
      ptx::tc_fence_after();
      const int col0 = j * BN;
      // Highest valid column of this row within the tile.
      int lim = kv_len - 1 - col0;
      if (a.causal && row - col0 < lim) lim = row - col0;
      const bool mask_tile = (col0 + BN > kv_len) || (a.causal && col0 + BN - 1 > row0);

      // pass 1: row max
      float mx = -INFINITY;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        ptx::tmem_ld32(tS + lane_addr + cc * 32, r);
        ptx::tmem_wait_ld();
        if (mask_tile) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (cc * 32 + i > lim) r[i] = 0xff800000u;  // -inf
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(r[i]), __uint_as_float(r[i + 1])));
      }
      const float x_max = mx * c;
      if (j == 0) {
        m_ref = x_max;
      } else {
        const bool grow = x_max - m_ref > kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = grow ? x_max : m_ref;
          const float alpha = grow ? ptx::ex2(m_ref - m_new) : 1.f;
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc) {
            ptx::tmem_ld32(tO + lane_addr + cc * 32, r);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            ptx::tmem_st32(tO + lane_addr + cc * 32, r);
          }
          l *= alpha;
          m_ref = m_new;
        }
      }
      // pass 2: P = 2^(c*s - m_ref), row sum, packed 16-bit P over the S columns
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        ptx::tmem_ld32(tS + lane_addr + cc * 32, r);
        ptx::tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ptx::ex2(fmaf(__uint_as_float(r[i]), c, -m_ref));
          float p1 = ptx::ex2(fmaf(__uint_as_float(r[i + 1]), c, -m_ref));
          if (mask_tile) {
            if (cc * 32 + i > lim) p0 = 0.f;
            if (cc * 32 + i + 1 > lim) p1 = 0.f;
          }
          l += p0 + p1;
          pk[i >> 1] = pack2<BF16>(p0, p1);
        }
        ptx::tmem_st16(tS + lane_addr + cc * 16, pk);
      }
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(&ctl->p_full);
    }

    // epilogue: O / l -> global, LSE
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    T* orow = reinterpret_cast<T*>(a.o) + b * a.os.b + h * a.os.h + static_cast<int64_t>(row) * a.os.s;
    if (n_tiles > 0) {
      if (ok) ok = ptx::mbar_wait(&ctl->o_full, 0, abort_flag);
      ptx::tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) {
        ptx::tmem_ld32(tO + lane_addr + cc * 32, r);
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

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
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
  dim3 grid((a.Lq + BM - 1) / BM, a.Hq, a.B);
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
