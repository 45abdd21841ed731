// y[M,N] = x[M,K] w[N,K]^T + bias[N] for fp16 / bf16 on sm_100a tensor cores: the
// projections either side of attention (reference: function::linear =
// op::matmul(input, weight, false, true, bias), src/Function/FuncNNLayer.h:14-19, which
// calls a library gemm and, for the bias, pre-fills C, src/Operation/OpLinalgCuda.cuh:141-215).
//
// Persistent kernel, one CTA per SM, output tiles of MT x 128 rows by 256 columns (MT = 1 or 2):
//   warp 0     producer: cp.async.bulk.tensor loads (128-byte swizzle) of the (MT x 128) x 64
//              slice of x and the 256 x 64 slice of w into a ring of 4 (MT = 1) or 3 (MT = 2) stages
//   warp 1     issuer: the warp runs the loop, one elected lane issues tcgen05.mma (kind::f16, M = 128, N = 256, both
//              operands K-major) into 256-column TMEM accumulators.  MT = 1: two accumulators used in
//              turn, so that the epilogue of a tile runs under the main loop of the next.  MT = 2: one
//              accumulator per 128-row half of the tile; both halves read the same slice of w from shared
//              memory, and the next tile's upper half starts while the lower half is still being drained.
//              Shared memory moves 128 bytes per clock, and the operands of an M = 128, N = 256 MMA are
//              12 KB per 128 clocks on top of the TMA writes that bring them in: with MT = 1 that is
//              192 bytes per clock of tensor time (the pipe cannot be busy more than two thirds of the
//              time; a profile showed 67 %), with MT = 2, where w is brought in once for two MMAs, 160.
//   warps 4-7  epilogue: thread r owns output row r (TMEM lane r); 64 columns at a time
//              are read with tcgen05.ld, get the bias (fp32), are rounded to the tensor
//              dtype and leave through a swizzled staging tile and a TMA store (rows and
//              columns beyond M, N are clipped by the tensor map; the K tail reads as zero)
// Tiles are ordered in groups of eight row-tiles so that CTAs running at the same time
// share slices of x and w in L2.  Every wait is bounded.
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"
#include "tma_host.cuh"

namespace ttattn {
namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kMaxStage = 4;
constexpr int kThreads = 256;
constexpr int kEpi = 128;
constexpr int kABytes = BM * BK * 2, kBBytes = BN * BK * 2;
constexpr int kOutBytes = BM * 128;  // staging: 128 rows x 64 columns of 16 bits

// MT: 128-row halves per output tile
template <int MT>
struct Cfg {
  static constexpr int kStages = MT == 1 ? 4 : 3;
  static constexpr int kStageBytes = MT * kABytes + kBBytes;
  static constexpr int kGroupM = 8 / MT;  // row-tiles per L2 group: 1024 rows either way
};

struct __align__(8) SmemCtl {
  uint64_t full[kMaxStage], empty[kMaxStage];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int MT>
constexpr int smem_bytes() {
  return Cfg<MT>::kStages * Cfg<MT>::kStageBytes + 2 * kOutBytes + BN * 4 + static_cast<int>(sizeof(SmemCtl));
}
static_assert(smem_bytes<1>() <= 232448 && smem_bytes<2>() <= 232448, "exceeds the shared memory a CTA may request");

struct LinArgs {
  const void* bias;  // [N] in the tensor dtype, or null
  int M, N, K;
  int32_t* status;
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

template <int kGroupM>
__device__ __forceinline__ void tile_of(int t, int tiles_m, int tiles_n, int* m_tile, int* n_tile) {
  const int per_group = kGroupM * tiles_n;
  const int g = t / per_group, in_g = t - g * per_group;
  const int first_m = g * kGroupM;
  const int gm = tiles_m - first_m < kGroupM ? tiles_m - first_m : kGroupM;
  *m_tile = first_m + in_g % gm;
  *n_tile = in_g / gm;
}

template <bool BF16, int MT>
__global__ void __launch_bounds__(kThreads, 1)
    linear_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                     const __grid_constant__ CUtensorMap tmY, const LinArgs a) {
  using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((ptx::smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte boundary
    if (threadIdx.x == 0 && a.status) atomicOr(a.status, kStatusBadSmemAlign);
    return;
  }
  constexpr int NSTAGE = Cfg<MT>::kStages, kStageBytes = Cfg<MT>::kStageBytes, kGroupM = Cfg<MT>::kGroupM;
  constexpr int TM = MT * BM;  // rows of an output tile
  uint8_t* sOut = smem + NSTAGE * kStageBytes;
  float* sBias = reinterpret_cast<float*>(sOut + 2 * kOutBytes);
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(sBias + BN);
  volatile int* abort_flag = &ctl->abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_m = (a.M + TM - 1) / TM, tiles_n = (a.N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;
  const int n_kb = (a.K + BK - 1) / BK;

  if (warp == 0 && lane == 0) {
#pragma unroll
    for (int s = 0; s < NSTAGE; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&ctl->acc_full[i], 1);
      ptx::mbar_init(&ctl->acc_empty[i], kEpi);
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::tma_prefetch_desc(&tmX);
    ptx::tma_prefetch_desc(&tmW);
    ptx::tma_prefetch_desc(&tmY);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&ctl->tmem_base, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;

  if (warp == 0) {
    // -------------------------------------------------------------- producer --
    if (lane == 0) {
      uint32_t g = 0;  // k-slices requested so far (ring position)
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        int mt, nt;
        tile_of<kGroupM>(t, tiles_m, tiles_n, &mt, &nt);
        for (int kb = 0; kb < n_kb; ++kb, ++g) {
          const int s = g % NSTAGE;
          if (!(ok = ptx::mbar_wait(&ctl->empty[s], ((g / NSTAGE) & 1) ^ 1, abort_flag))) break;
          uint8_t* sa = smem + s * kStageBytes;
          ptx::mbar_arrive_expect_tx(&ctl->full[s], kStageBytes);
#pragma unroll
          for (int h = 0; h < MT; ++h)  // rows beyond M read as zero
            ptx::tma_load_4d(sa + h * kABytes, &tmX, &ctl->full[s], kb * BK, mt * TM + h * BM, 0, 0);
          ptx::tma_load_4d(sa + MT * kABytes, &tmW, &ctl->full[s], kb * BK, nt * BN, 0, 0);
          ptx::tma_load_4d(sa + MT * kABytes + kBBytes / 2, &tmW, &ctl->full[s], kb * BK, nt * BN + 128, 0, 0);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- issuer --
    // the whole warp runs the loop (waits made uniform by a vote), one elected lane issues: addresses and
    // descriptors stay warp-uniform
    {
      const bool leader = ptx::elect_one();
      constexpr uint32_t kHi = ptx::smem_desc_hi_sw128(1024);
      const uint32_t idesc = ptx::make_idesc_f16(BM, BN, BF16 ? 1 : 0, 0, 0);
      const uint32_t alo = ptx::smem_desc_lo(ptx::smem_u32(smem), 16);
      const uint32_t blo = ptx::smem_desc_lo(ptx::smem_u32(smem + MT * kABytes), 16);
      uint32_t g = 0;
      bool ok = true;
      int i = 0;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++i) {
        // Accumulator of half h of tile i, and how often it has been used before: with MT = 1 the two
        // accumulators alternate between tiles, with MT = 2 each half of the tile has its own.
        auto acc_of = [&](int h) { return MT == 1 ? (i & 1) : h; };
        const uint32_t use = MT == 1 ? (i >> 1) : i;
        for (int kb = 0; kb < n_kb && ok; ++kb, ++g) {
          const int s = g % NSTAGE;
          if (!(ok = __all_sync(0xffffffffu, ptx::mbar_wait(&ctl->full[s], (g / NSTAGE) & 1, abort_flag)) != 0)) break;
          ptx::tc_fence_after();
          const uint32_t so = s * (kStageBytes >> 4);
#pragma unroll
          for (int h = 0; h < MT; ++h) {
            const int ai = acc_of(h);
            if (kb == 0) {
              // the epilogue has read what this accumulator held before
              if (!(ok = __all_sync(0xffffffffu, ptx::mbar_wait(&ctl->acc_empty[ai], (use & 1) ^ 1, abort_flag)) != 0)) break;
              ptx::tc_fence_after();
            }
            const uint32_t d = tmem + ai * BN, ah = alo + so + h * (kABytes >> 4);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)  // 32 bytes per k-step inside the 128-byte swizzled row
              if (leader) ptx::mma_ss2(d, ah + k * 2, kHi, blo + so + k * 2, kHi, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            if (leader && kb == n_kb - 1) ptx::mma_commit(&ctl->acc_full[ai]);
          }
          if (ok && leader) ptx::mma_commit(&ctl->empty[s]);
        }
      }
    }
  } else if (warp >= 4) {
    // -------------------------------------------------------------- epilogue --
    const int r = tid - 128;  // output row within the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    bool ok = true;
    int i = 0;
    uint32_t stores = 0;  // staging buffer toggle
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++i) {
      int mt, nt;
      tile_of<kGroupM>(t, tiles_m, tiles_n, &mt, &nt);
      const int n0 = nt * BN;
      const uint32_t use = MT == 1 ? (i >> 1) : i;
      // this tile's slice of the bias, as fp32 (threads that see an expired wait still meet the barriers)
      ptx::named_barrier(1, kEpi);  // the previous tile's readers of sBias are done
#pragma unroll
      for (int j = 0; j < BN / kEpi; ++j) {
        const int n = n0 + r + j * kEpi;
        sBias[r + j * kEpi] = (a.bias && n < a.N) ? to_f32<T>(reinterpret_cast<const T*>(a.bias)[n]) : 0.f;
      }
      ptx::named_barrier(1, kEpi);
#pragma unroll 1
      for (int h = 0; h < MT; ++h) {
      const int buf = MT == 1 ? (i & 1) : h, m0 = mt * TM + h * BM;
      if (ok) ok = ptx::mbar_wait(&ctl->acc_full[buf], use & 1, abort_flag);
      ptx::tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        uint32_t v[64];
        ptx::tmem_ld32p(tmem + buf * BN + lane_addr + c * 64, v);
        ptx::tmem_ld32p(tmem + buf * BN + lane_addr + c * 64 + 32, v + 32);
        ptx::tmem_wait_ld();
        if (c == BN / 64 - 1) {
          // the whole accumulator is in registers / already stored: the issuer may reuse it
          ptx::tc_fence_before();
          ptx::mbar_arrive(&ctl->acc_empty[buf]);
        }
        uint8_t* stage = sOut + (stores & 1) * kOutBytes;
        ++stores;
        // at most one earlier store (the other staging buffer) may still be reading shared memory
        if (r == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        ptx::named_barrier(1, kEpi);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const int e = ch * 8;
          const float4 b0 = *reinterpret_cast<const float4*>(sBias + c * 64 + e);
          const float4 b1 = *reinterpret_cast<const float4*>(sBias + c * 64 + e + 4);
          uint4 w;
          w.x = pack2<BF16>(__uint_as_float(v[e + 0]) + b0.x, __uint_as_float(v[e + 1]) + b0.y);
          w.y = pack2<BF16>(__uint_as_float(v[e + 2]) + b0.z, __uint_as_float(v[e + 3]) + b0.w);
          w.z = pack2<BF16>(__uint_as_float(v[e + 4]) + b1.x, __uint_as_float(v[e + 5]) + b1.y);
          w.w = pack2<BF16>(__uint_as_float(v[e + 6]) + b1.z, __uint_as_float(v[e + 7]) + b1.w);
          *reinterpret_cast<uint4*>(stage + r * 128 + ((ch ^ (r & 7)) << 4)) = w;
        }
        ptx::fence_proxy_async_smem();
        ptx::named_barrier(1, kEpi);
        if (r == 0 && ok && n0 + c * 64 < a.N && m0 < a.M) {
          ptx::tma_store_4d(&tmY, stage, n0 + c * 64, m0, 0, 0);
          ptx::bulk_commit();
        }
      }
      }
    }
    if (r == 0) ptx::bulk_wait_all();
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
  if (tid == 0 && ctl->abort_flag && a.status) atomicOr(a.status, kStatusWaitExpired);
}

template <bool BF16, int MT>
cudaError_t launch_t(int dtype, const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                     int64_t ldx, int64_t ldw, int64_t ldy, int32_t* status, int device, cudaStream_t stream) {
  CUtensorMap tx, tw, ty;
  // 2-D tensors as [1, 1, rows, cols] maps: box = 64 columns x 128 rows, 128-byte swizzle
  if (!make_map(&tx, dtype, x, K, M, 1, 1, Str3{ldx * M, ldx * M, ldx}) ||
      !make_map(&tw, dtype, w, K, N, 1, 1, Str3{ldw * N, ldw * N, ldw}) ||
      !make_map(&ty, dtype, y, N, M, 1, 1, Str3{ldy * M, ldy * M, ldy}))
    return cudaErrorInvalidValue;
  auto kern = linear_tc_kernel<BF16, MT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<MT>());
  if (e != cudaSuccess) return e;
  const long long tiles = static_cast<long long>((M + MT * BM - 1) / (MT * BM)) * ((N + BN - 1) / BN);
  const int sms = sm_count(device);
  LinArgs a{bias, M, N, K, status};
  kern<<<static_cast<unsigned>(tiles < sms ? tiles : sms), kThreads, smem_bytes<MT>(), stream>>>(tx, tw, ty, a);
  return cudaGetLastError();
}

// 256-row tiles when they still fill the machine at least once; otherwise 128-row tiles (twice the CTAs)
inline bool tall_tiles(int M, int N, int device) {
  const long long tiles = static_cast<long long>((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  return tiles >= sm_count(device);
}

}  // namespace

cudaError_t launch_linear_tc(int dtype, const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                             int64_t ldx, int64_t ldw, int64_t ldy, int32_t* status, int device, cudaStream_t stream) {
  if (dtype != TT_ATTN_BF16 && dtype != TT_ATTN_F16) return cudaErrorInvalidValue;
  const bool bf = dtype == TT_ATTN_BF16;
  if (tall_tiles(M, N, device))
    return bf ? launch_t<true, 2>(dtype, x, w, bias, y, M, N, K, ldx, ldw, ldy, status, device, stream)
              : launch_t<false, 2>(dtype, x, w, bias, y, M, N, K, ldx, ldw, ldy, status, device, stream);
  return bf ? launch_t<true, 1>(dtype, x, w, bias, y, M, N, K, ldx, ldw, ldy, status, device, stream)
            : launch_t<false, 1>(dtype, x, w, bias, y, M, N, K, ldx, ldw, ldy, status, device, stream);
}

}  // namespace ttattn
