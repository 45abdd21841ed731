// Attention backward on CUDA cores with fp32 arithmetic, for every dtype.
//
// The reference's FuncSDPAttention::backward is unimplemented
// (src/Function/FuncNNLayer.h:267); its gradient is defined by the chain
// linear -> mul -> add -> softmax -> linear (src/Function/FuncNNLayer.h:20-34,
// src/Function/FuncElemWise.h:77-87,113-123, src/Operation/OpNNLayerCpu.h:78-109):
//   dV = P^T dO          dP = dO V^T
//   dS = P o (dP - rowsum(P o dP)) * scale,   rowsum(P o dP) = rowsum(dO o O) = delta
//   dQ = dS K            dK = dS^T Q
// P is recomputed from Q, K and the forward's log-sum-exp, so no [L,S] matrix is
// ever stored.  Three kernels:
//   bwd_delta_kernel   delta[b,h,i] = sum_d dO[i,d] * O[i,d]           (fp32 workspace)
//   bwd_dkdv_kernel    one CTA per 64-key tile: loops over the query tiles (and
//                      over the query heads of the group), accumulates dK, dV in
//                      registers -> deterministic, no atomics
//   bwd_dq_kernel      one CTA per 64-query tile: loops over key tiles, accumulates dQ
#include "common.cuh"
#include "ptx.cuh"

namespace ttattn {
namespace {

constexpr int TM = 64, TN = 64, kThreads = 256;

template <typename T, int D>
__device__ __forceinline__ void load_tile(float* dst, const T* src, int64_t row_stride, int row0, int rows_valid,
                                          int tid) {
  constexpr int LD = D + 1;
  for (int idx = tid; idx < TM * (D / 4); idx += kThreads) {
    int r = idx / (D / 4), c4 = (idx % (D / 4)) * 4;
    float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
    if (row0 + r < rows_valid) {
      const T* p = src + static_cast<int64_t>(row0 + r) * row_stride + c4;
      v0 = to_f32<T>(p[0]), v1 = to_f32<T>(p[1]), v2 = to_f32<T>(p[2]), v3 = to_f32<T>(p[3]);
    }
    float* d = dst + r * LD + c4;
    d[0] = v0, d[1] = v1, d[2] = v2, d[3] = v3;
  }
}

// out[i][j] = sum_d A[(ty+16i)][d] * B[(tx+16j)][d]
template <int D>
__device__ __forceinline__ void tile_nt(const float* A, const float* B, int ty, int tx, float (&out)[4][4]) {
  constexpr int LD = D + 1;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) out[i][j] = 0.f;
#pragma unroll 8
  for (int d = 0; d < D; ++d) {
    float av[4], bv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) av[i] = A[(ty + 16 * i) * LD + d];
#pragma unroll
    for (int j = 0; j < 4; ++j) bv[j] = B[(tx + 16 * j) * LD + d];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) out[i][j] = fmaf(av[i], bv[j], out[i][j]);
  }
}

// delta[b,h,i] = sum_d dO[i,d] * O[i,d].  Each thread reads 16 bytes of a row of
// O and of dO; the D*sizeof(T)/16 threads of a row reduce with shuffles.  For the
// tensor-core backward the same pass clears the fp32 dQ accumulator (its TMA
// reductions need zeros to start from), which saves a separate memset of that size.
template <typename T, int D>
__global__ void __launch_bounds__(kThreads) bwd_delta_kernel(const BwdArgs a) {
  ptx::grid_dep_launch();  // the tensor-core backward kernel may set itself up and start on Q, K, V, dO meanwhile
  constexpr int N = 16 / sizeof(T);  // elements per thread
  constexpr int TPR = D / N;         // threads per row (8, 16 or 32)
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) / TPR;
  const int part = threadIdx.x % TPR;
  const int64_t total = static_cast<int64_t>(a.B) * a.Hq * a.Lq;
  float s = 0.f;
  if (row < total) {
    const int i = static_cast<int>(row % a.Lq);
    const int h = static_cast<int>((row / a.Lq) % a.Hq);
    const int b = static_cast<int>(row / (static_cast<int64_t>(a.Lq) * a.Hq));
    const T* o = reinterpret_cast<const T*>(a.o) + b * a.os.b + h * a.os.h + static_cast<int64_t>(i) * a.os.s + part * N;
    const T* g =
        reinterpret_cast<const T*>(a.d_o) + b * a.dos.b + h * a.dos.h + static_cast<int64_t>(i) * a.dos.s + part * N;
    const uint4 ov = *reinterpret_cast<const uint4*>(o), gv = *reinterpret_cast<const uint4*>(g);
    const T* op = reinterpret_cast<const T*>(&ov);
    const T* gp = reinterpret_cast<const T*>(&gv);
#pragma unroll
    for (int e = 0; e < N; ++e) s = fmaf(to_f32<T>(op[e]), to_f32<T>(gp[e]), s);
    if (a.zero_dq_accum) {
      float4* z = reinterpret_cast<float4*>(a.dq_accum + row * D + part * N);
#pragma unroll
      for (int e = 0; e < N / 4; ++e) z[e] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
#pragma unroll
  for (int of = TPR / 2; of >= 1; of >>= 1) s += __shfl_xor_sync(0xffffffffu, s, of);
  if (part == 0 && row < total) a.delta[row] = s;
}

// Computes P and dS for the (query tile, key tile) pair held in shared memory and
// writes them to Ps / dSs ([row][col], leading dimension TN+1).
// `shift` is the causal alignment (key j participates iff j <= i + shift), `mask_base` the
// mask offset of this (b, h).
template <typename T, int D>
__device__ __forceinline__ void tile_p_ds(const BwdArgs& a, const float* Qs, const float* Ks, const float* Vs,
                                          const float* dOs, const float* lse_s, const float* delta_s, float* Ps,
                                          float* dSs, int row0, int col0, int kv_len, int shift, int64_t mask_base,
                                          int ty, int tx) {
  constexpr int LP = TN + 1;
  const float c = a.scale * kLog2e;
  float s[4][4], dp[4][4];
  tile_nt<D>(Qs, Ks, ty, tx, s);
  tile_nt<D>(dOs, Vs, ty, tx, dp);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty + 16 * i, row = row0 + r;
    const float lse2 = lse_s[r] * kLog2e, dl = delta_s[r];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int cidx = tx + 16 * j, col = col0 + cidx;
      // a row without any participating key has LSE = -inf and P = 0
      const bool keep = row < a.Lq && col < kv_len && (!a.causal || col <= row + shift) && lse_s[r] != -INFINITY;
      float x = fmaf(s[i][j], c, -lse2);
      if (a.mask.ptr && keep) x += mask_bias2<T>(a.mask, mask_base + row * a.mask.sl + col);
      const float p = keep ? exp2f(x) : 0.f;
      if (Ps) Ps[r * LP + cidx] = p;
      dSs[r * LP + cidx] = p * (dp[i][j] - dl) * a.scale;
    }
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads) bwd_dkdv_kernel(const BwdArgs a) {
  constexpr int LD = D + 1, LP = TN + 1, DC = D / 16;
  extern __shared__ float sm[];
  float* Ks = sm;
  float* Vs = Ks + TN * LD;
  float* Qs = Vs + TN * LD;
  float* dOs = Qs + TM * LD;
  float* Ps = dOs + TM * LD;
  float* dSs = Ps + TM * LP;
  float* lse_s = dSs + TM * LP;
  float* delta_s = lse_s + TM;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int nt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int group = a.Hq / a.Hkv;
  const int col0 = nt * TN;
  int kv_len = a.Skv;
  if (a.kv_lens) {
    int l = a.kv_lens[b];
    kv_len = l < 0 ? 0 : (l < a.Skv ? l : a.Skv);
  }
  const T* k = reinterpret_cast<const T*>(a.k) + b * a.ks.b + hk * a.ks.h;
  const T* v = reinterpret_cast<const T*>(a.v) + b * a.vs.b + hk * a.vs.h;
  load_tile<T, D>(Ks, k, a.ks.s, col0, a.Skv, tid);
  load_tile<T, D>(Vs, v, a.vs.s, col0, a.Skv, tid);

  float dk[4][DC], dv[4][DC];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < DC; ++j) dk[i][j] = 0.f, dv[i][j] = 0.f;

  const int n_q_tiles = (a.Lq + TM - 1) / TM;
  const int shift = causal_shift(a.causal, kv_len, a.Lq);
  // first query tile with a row i such that col0 <= i + shift
  const int qt_begin = a.causal ? (col0 - shift > 0 ? (col0 - shift) / TM : 0) : 0;
  if (col0 < kv_len) {
    for (int g = 0; g < group; ++g) {
      const int h = hk * group + g;
      const T* q = reinterpret_cast<const T*>(a.q) + b * a.qs.b + h * a.qs.h;
      const T* dO = reinterpret_cast<const T*>(a.d_o) + b * a.dos.b + h * a.dos.h;
      const float* lse = a.lse + (static_cast<int64_t>(b) * a.Hq + h) * a.Lq;
      const float* delta = a.delta + (static_cast<int64_t>(b) * a.Hq + h) * a.Lq;
      for (int qt = qt_begin; qt < n_q_tiles; ++qt) {
        const int row0 = qt * TM;
        __syncthreads();
        load_tile<T, D>(Qs, q, a.qs.s, row0, a.Lq, tid);
        load_tile<T, D>(dOs, dO, a.dos.s, row0, a.Lq, tid);
        if (tid < TM) {
          const bool in = row0 + tid < a.Lq;
          lse_s[tid] = in ? lse[row0 + tid] : 0.f;
          delta_s[tid] = in ? delta[row0 + tid] : 0.f;
        }
        __syncthreads();
        tile_p_ds<T, D>(a, Qs, Ks, Vs, dOs, lse_s, delta_s, Ps, dSs, row0, col0, kv_len, shift,
                        b * a.mask.sb + h * a.mask.sh, ty, tx);
        __syncthreads();
        // dV[kv][d] += sum_row P[row][kv] dO[row][d];  dK[kv][d] += sum_row dS[row][kv] Q[row][d]
#pragma unroll 2
        for (int r = 0; r < TM; ++r) {
          float pv[4], sv[4], gv[DC], qv[DC];
#pragma unroll
          for (int i = 0; i < 4; ++i) pv[i] = Ps[r * LP + ty + 16 * i], sv[i] = dSs[r * LP + ty + 16 * i];
#pragma unroll
          for (int j = 0; j < DC; ++j) gv[j] = dOs[r * LD + tx + 16 * j], qv[j] = Qs[r * LD + tx + 16 * j];
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < DC; ++j) {
              dv[i][j] = fmaf(pv[i], gv[j], dv[i][j]);
              dk[i][j] = fmaf(sv[i], qv[j], dk[i][j]);
            }
        }
      }
    }
  }
  T* dK = a.dk ? reinterpret_cast<T*>(a.dk) + b * a.dks.b + hk * a.dks.h : nullptr;
  T* dV = a.dv ? reinterpret_cast<T*>(a.dv) + b * a.dvs.b + hk * a.dvs.h : nullptr;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int col = col0 + ty + 16 * i;
    if (col >= a.Skv) continue;
#pragma unroll
    for (int j = 0; j < DC; ++j) {
      if (dK) dK[static_cast<int64_t>(col) * a.dks.s + tx + 16 * j] = from_f32<T>(dk[i][j]);
      if (dV) dV[static_cast<int64_t>(col) * a.dvs.s + tx + 16 * j] = from_f32<T>(dv[i][j]);
    }
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads) bwd_dq_kernel(const BwdArgs a) {
  constexpr int LD = D + 1, LP = TN + 1, DC = D / 16;
  extern __shared__ float sm[];
  float* Qs = sm;
  float* dOs = Qs + TM * LD;
  float* Ks = dOs + TM * LD;
  float* Vs = Ks + TN * LD;
  float* dSs = Vs + TN * LD;
  float* lse_s = dSs + TM * LP;
  float* delta_s = lse_s + TM;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int mt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int h = blockIdx.y, b = blockIdx.z, hk = h / (a.Hq / a.Hkv);
  const int row0 = mt * TM;
  int kv_len = a.Skv;
  if (a.kv_lens) {
    int l = a.kv_lens[b];
    kv_len = l < 0 ? 0 : (l < a.Skv ? l : a.Skv);
  }
  const int shift = causal_shift(a.causal, kv_len, a.Lq);
  int kv_end = kv_len;
  if (a.causal && row0 + TM + shift < kv_end) kv_end = row0 + TM + shift > 0 ? row0 + TM + shift : 0;
  const int n_tiles = (kv_end + TN - 1) / TN;

  const T* q = reinterpret_cast<const T*>(a.q) + b * a.qs.b + h * a.qs.h;
  const T* dO = reinterpret_cast<const T*>(a.d_o) + b * a.dos.b + h * a.dos.h;
  const T* k = reinterpret_cast<const T*>(a.k) + b * a.ks.b + hk * a.ks.h;
  const T* v = reinterpret_cast<const T*>(a.v) + b * a.vs.b + hk * a.vs.h;
  load_tile<T, D>(Qs, q, a.qs.s, row0, a.Lq, tid);
  load_tile<T, D>(dOs, dO, a.dos.s, row0, a.Lq, tid);
  if (tid < TM) {
    const bool in = row0 + tid < a.Lq;
    const int64_t base = (static_cast<int64_t>(b) * a.Hq + h) * a.Lq + row0 + tid;
    lse_s[tid] = in ? a.lse[base] : 0.f;
    delta_s[tid] = in ? a.delta[base] : 0.f;
  }
  float dq[4][DC];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < DC; ++j) dq[i][j] = 0.f;

  for (int t = 0; t < n_tiles; ++t) {
    const int col0 = t * TN;
    __syncthreads();
    load_tile<T, D>(Ks, k, a.ks.s, col0, a.Skv, tid);
    load_tile<T, D>(Vs, v, a.vs.s, col0, a.Skv, tid);
    __syncthreads();
    tile_p_ds<T, D>(a, Qs, Ks, Vs, dOs, lse_s, delta_s, nullptr, dSs, row0, col0, kv_len, shift,
                    b * a.mask.sb + h * a.mask.sh, ty, tx);
    __syncthreads();
#pragma unroll 4
    for (int cc = 0; cc < TN; ++cc) {
      float sv[4], kv[DC];
#pragma unroll
      for (int i = 0; i < 4; ++i) sv[i] = dSs[(ty + 16 * i) * LP + cc];
#pragma unroll
      for (int j = 0; j < DC; ++j) kv[j] = Ks[cc * LD + tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < DC; ++j) dq[i][j] = fmaf(sv[i], kv[j], dq[i][j]);
    }
  }
  T* dQ = reinterpret_cast<T*>(a.dq) + b * a.dqs.b + h * a.dqs.h;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = row0 + ty + 16 * i;
    if (row >= a.Lq) continue;
#pragma unroll
    for (int j = 0; j < DC; ++j) dQ[static_cast<int64_t>(row) * a.dqs.s + tx + 16 * j] = from_f32<T>(dq[i][j]);
  }
}

template <typename T, int D>
cudaError_t launch_t(const BwdArgs& a, cudaStream_t stream) {
  const int64_t rows = static_cast<int64_t>(a.B) * a.Hq * a.Lq;
  bwd_delta_kernel<T, D><<<static_cast<unsigned>((rows * (D * sizeof(T) / 16) + kThreads - 1) / kThreads), kThreads, 0, stream>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (a.dk || a.dv) {
    constexpr int smem = (4 * TM * (D + 1) + 2 * TM * (TN + 1) + 2 * TM) * sizeof(float);
    auto kern = bwd_dkdv_kernel<T, D>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kern<<<dim3((a.Skv + TN - 1) / TN, a.Hkv, a.B), kThreads, smem, stream>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  if (a.dq) {
    constexpr int smem = (4 * TM * (D + 1) + TM * (TN + 1) + 2 * TM) * sizeof(float);
    auto kern = bwd_dq_kernel<T, D>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kern<<<dim3((a.Lq + TM - 1) / TM, a.Hq, a.B), kThreads, smem, stream>>>(a);
    e = cudaGetLastError();
  }
  return e;
}

template <typename T, int D>
cudaError_t launch_delta_t(const BwdArgs& a, cudaStream_t stream) {
  const int64_t rows = static_cast<int64_t>(a.B) * a.Hq * a.Lq;
  bwd_delta_kernel<T, D><<<static_cast<unsigned>((rows * (D * sizeof(T) / 16) + kThreads - 1) / kThreads), kThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_bwd_delta(int dtype, int D, const BwdArgs& a, cudaStream_t stream) {
  if (dtype == TT_ATTN_F32) return D == 64 ? launch_delta_t<float, 64>(a, stream) : launch_delta_t<float, 128>(a, stream);
  if (dtype == TT_ATTN_F16)
    return D == 64 ? launch_delta_t<__half, 64>(a, stream) : launch_delta_t<__half, 128>(a, stream);
  return D == 64 ? launch_delta_t<__nv_bfloat16, 64>(a, stream) : launch_delta_t<__nv_bfloat16, 128>(a, stream);
}

cudaError_t launch_bwd_simt(int dtype, int D, const BwdArgs& a, cudaStream_t stream) {
  if (dtype == TT_ATTN_F32) return D == 64 ? launch_t<float, 64>(a, stream) : launch_t<float, 128>(a, stream);
  if (dtype == TT_ATTN_F16) return D == 64 ? launch_t<__half, 64>(a, stream) : launch_t<__half, 128>(a, stream);
  return D == 64 ? launch_t<__nv_bfloat16, 64>(a, stream) : launch_t<__nv_bfloat16, 128>(a, stream);
}

}  // namespace ttattn
