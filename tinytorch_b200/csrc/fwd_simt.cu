// Prefill forward in full fp32 arithmetic (CUDA cores, FMA) for Float32 tensors.
//
// The reference's CUDA fp32 matmul runs in TF32 (src/Utils/CUDAUtils.cpp:148-155),
// which cannot meet a 1e-5 relative bound against its own CPU path
// (src/Operation/OpLinalgCpu.h:138-150); this kernel therefore keeps every
// product and sum in fp32.  Same fusion as the tensor-core kernel: one CTA owns a
// 64-row query tile of one (batch, head), streams 64-key tiles through shared
// memory, keeps an online softmax (warp-shuffle row max over the 16 lanes that
// share a row) and never writes scores to HBM.
#include "common.cuh"

namespace ttattn {
namespace {

constexpr int TM = 64, TN = 64, kThreads = 256;

template <typename T, int D>
__device__ __forceinline__ void load_tile(float* dst, const T* src, int64_t row_stride, int row0, int rows_valid,
                                          int tid) {
  // dst[r][D+1]; rows at or beyond rows_valid are zero
  constexpr int LD = D + 1;
  for (int idx = tid; idx < TM * (D / 4); idx += kThreads) {
    int r = idx / (D / 4), c4 = (idx % (D / 4)) * 4;
    float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
    if (row0 + r < rows_valid) {
      const T* p = src + static_cast<int64_t>(row0 + r) * row_stride + c4;
      v0 = to_f32<T>(p[0]);
      v1 = to_f32<T>(p[1]);
      v2 = to_f32<T>(p[2]);
      v3 = to_f32<T>(p[3]);
    }
    float* d = dst + r * LD + c4;
    d[0] = v0, d[1] = v1, d[2] = v2, d[3] = v3;
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads) fwd_simt_kernel(const FwdArgs a) {
  constexpr int LD = D + 1, LP = TN + 1, DC = D / 16;
  extern __shared__ float sm[];
  float* Qs = sm;
  float* Ks = Qs + TM * LD;
  float* Vs = Ks + TN * LD;
  float* Ps = Vs + TN * LD;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int mt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int h = blockIdx.y, b = blockIdx.z, hk = h / (a.Hq / a.Hkv);
  const int row0 = mt * TM;
  const T* q = reinterpret_cast<const T*>(a.q) + b * a.qs.b + h * a.qs.h;
  const T* k = reinterpret_cast<const T*>(a.k) + b * a.ks.b + hk * a.ks.h;
  const T* v = reinterpret_cast<const T*>(a.v) + b * a.vs.b + hk * a.vs.h;

  int kv_len = a.Skv;
  if (a.kv_lens) {
    int l = a.kv_lens[b];
    kv_len = l < 0 ? 0 : (l < a.Skv ? l : a.Skv);
  }
  const int shift = causal_shift(a.causal, kv_len, a.Lq);
  int kv_end = kv_len;
  if (a.causal && row0 + TM + shift < kv_end) kv_end = row0 + TM + shift > 0 ? row0 + TM + shift : 0;
  const int n_tiles = (kv_end + TN - 1) / TN;
  const float c = a.scale * kLog2e;
  const int64_t mask_base = b * a.mask.sb + h * a.mask.sh;

  load_tile<T, D>(Qs, q, a.qs.s, row0, a.Lq, tid);

  float m[4], l[4], acc[4][DC];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY, l[i] = 0.f;
#pragma unroll
    for (int j = 0; j < DC; ++j) acc[i][j] = 0.f;
  }

  for (int t = 0; t < n_tiles; ++t) {
    const int col0 = t * TN;
    __syncthreads();  // previous tile's K/V/P fully consumed (and Q visible on t == 0)
    load_tile<T, D>(Ks, k, a.ks.s, col0, kv_len, tid);
    load_tile<T, D>(Vs, v, a.vs.s, col0, kv_len, tid);
    __syncthreads();

    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll 8
    for (int d = 0; d < D; ++d) {
      float qa[4], kb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qa[i] = Qs[(ty + 16 * i) * LD + d];
#pragma unroll
      for (int j = 0; j < 4; ++j) kb[j] = Ks[(tx + 16 * j) * LD + d];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = fmaf(qa[i], kb[j], s[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = row0 + ty + 16 * i;
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = col0 + tx + 16 * j;
        const bool keep = col < kv_len && (!a.causal || col <= row + shift);
        s[i][j] = keep ? s[i][j] * c : -INFINITY;
        if (a.mask.ptr && keep && row < a.Lq) s[i][j] += mask_bias2<T>(a.mask, mask_base + row * a.mask.sl + col);
        mx = fmaxf(mx, s[i][j]);
      }
#pragma unroll
      for (int o = 8; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m[i], mx);
      // a row that has seen no participating key yet keeps m = -inf; its
      // exponentials are taken against 0 and are all 0
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m[i] - m_use);
      m[i] = m_new;
      l[i] *= alpha;
#pragma unroll
      for (int j = 0; j < DC; ++j) acc[i][j] *= alpha;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float p = exp2f(s[i][j] - m_use);
        l[i] += p;
        Ps[(ty + 16 * i) * LP + tx + 16 * j] = p;
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int kk = 0; kk < TN; ++kk) {
      float pa[4], vb[DC];
#pragma unroll
      for (int i = 0; i < 4; ++i) pa[i] = Ps[(ty + 16 * i) * LP + kk];
#pragma unroll
      for (int j = 0; j < DC; ++j) vb[j] = Vs[kk * LD + tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < DC; ++j) acc[i][j] = fmaf(pa[i], vb[j], acc[i][j]);
    }
  }

  T* o = reinterpret_cast<T*>(a.o) + b * a.os.b + h * a.os.h;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float ls = l[i];
#pragma unroll
    for (int of = 8; of >= 1; of >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, of);
    const int row = row0 + ty + 16 * i;
    if (row >= a.Lq) continue;
    const float inv = ls > 0.f ? 1.f / ls : 0.f;
#pragma unroll
    for (int j = 0; j < DC; ++j) o[static_cast<int64_t>(row) * a.os.s + tx + 16 * j] = from_f32<T>(acc[i][j] * inv);
    if (a.lse && tx == 0)
      a.lse[(static_cast<int64_t>(b) * a.Hq + h) * a.Lq + row] = ls > 0.f ? (m[i] + log2f(ls)) * kLn2 : -INFINITY;
  }
}

template <typename T, int D>
cudaError_t launch_t(const FwdArgs& a, cudaStream_t stream) {
  constexpr int smem = (3 * TM * (D + 1) + TM * (TN + 1)) * sizeof(float);
  auto kern = fwd_simt_kernel<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  dim3 grid((a.Lq + TM - 1) / TM, a.Hq, a.B);
  kern<<<grid, kThreads, smem, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fwd_simt(int dtype, int D, const FwdArgs& a, cudaStream_t stream) {
  if (dtype != TT_ATTN_F32) return cudaErrorInvalidValue;
  if (D == 64) return launch_t<float, 64>(a, stream);
  if (D == 128) return launch_t<float, 128>(a, stream);
  return cudaErrorInvalidValue;
}

}  // namespace ttattn
