// Fused add + RMS norm and SiLU-gated multiply: the two hand-fused transformer-block
// operators of the reference (src/Operation/OpFusedCuda.cuh:16-142), as HBM-bound
// streaming kernels.
//
// fusedAddRmsNorm: the reference's kernel makes two passes over a row and re-reads
// the residual it has just written.  Here a row (or a few short rows) lives in the
// registers of a thread group between the sum of squares and the scaling, so every
// byte crosses HBM once: read input, read residual, write residual, write input.
// All 16-byte loads of a thread are issued before the first use.
//
// siluMul: one pass, 16-byte streaming loads and stores, several vectors in flight
// per thread; long rows are tiled (row, chunk) so that indexing needs no division.
#include "common.cuh"

namespace ttattn {
namespace {

constexpr int kThreads = 256;

template <typename T>
struct Pack {
  static constexpr int N = 16 / sizeof(T);
  static __device__ __forceinline__ void unpack(const uint4& w, float (&f)[N]) {
    const T* t = reinterpret_cast<const T*>(&w);
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = to_f32<T>(t[i]);
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[N]) {
    uint4 w;
    T* t = reinterpret_cast<T*>(&w);
#pragma unroll
    for (int i = 0; i < N; ++i) t[i] = from_f32<T>(f[i]);
    return w;
  }
};

__device__ __forceinline__ uint4 ld_cs(const void* p) {
  uint4 r;
  asm volatile("ld.global.cs.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
__device__ __forceinline__ void st_cs(void* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// A group of `tpr` threads (a power of two, 32..256) owns one row; a CTA holds
// kThreads / tpr rows.  Each thread keeps VPT 16-byte vectors of the row.
template <typename T, int VPT>
__global__ void __launch_bounds__(kThreads) add_rms_norm_kernel(T* __restrict__ input, T* __restrict__ residual,
                                                                const T* __restrict__ weight, int64_t rows, int dim,
                                                                int tpr, float eps) {
  constexpr int N = Pack<T>::N;
  __shared__ float s_part[kThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rows_per_cta = kThreads / tpr;
  const int t_in_row = tid % tpr;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * rows_per_cta + tid / tpr;
  const bool row_ok = row < rows;
  const int vecs = dim / N;
  T* in_row = input + row * dim;
  T* res_row = residual + row * dim;

  uint4 a[VPT], b[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int idx = t_in_row + v * tpr;
    const bool ok = row_ok && idx < vecs;
    a[v] = ok ? ld_cs(in_row + idx * N) : make_uint4(0, 0, 0, 0);
    b[v] = ok ? ld_cs(res_row + idx * N) : make_uint4(0, 0, 0, 0);
  }
  float sum_sq = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int idx = t_in_row + v * tpr;
    float fa[N], fb[N];
    Pack<T>::unpack(a[v], fa);
    Pack<T>::unpack(b[v], fb);
#pragma unroll
    for (int i = 0; i < N; ++i) {
      fa[i] += fb[i];
      sum_sq = fmaf(fa[i], fa[i], sum_sq);  // of the unrounded sum, as the reference does
    }
    b[v] = Pack<T>::pack(fa);  // residual, rounded to T; the scaling below uses this rounded value
    if (row_ok && idx < vecs) st_cs(res_row + idx * N, b[v]);
  }
  // sum over the thread group: warp shuffles, then the group's warps through shared memory
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) sum_sq += __shfl_xor_sync(0xffffffffu, sum_sq, o);
  if (tpr > 32) {
    if (lane == 0) s_part[warp] = sum_sq;
    __syncthreads();
    const int w0 = (tid / tpr) * (tpr / 32);
    sum_sq = 0.f;
    for (int w = 0; w < tpr / 32; ++w) sum_sq += s_part[w0 + w];
  }
  const float inv_rms = rsqrtf(sum_sq / static_cast<float>(dim) + eps);
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int idx = t_in_row + v * tpr;
    if (!(row_ok && idx < vecs)) continue;
    float fr[N], fw[N];
    Pack<T>::unpack(b[v], fr);
    Pack<T>::unpack(__ldg(reinterpret_cast<const uint4*>(weight + idx * N)), fw);
#pragma unroll
    for (int i = 0; i < N; ++i) fr[i] = fr[i] * inv_rms * fw[i];
    st_cs(in_row + idx * N, Pack<T>::pack(fr));
  }
}

// Any dim and alignment: one CTA per row, two passes (the second re-reads the
// residual through the cache).
template <typename T>
__global__ void __launch_bounds__(kThreads) add_rms_norm_generic_kernel(T* input, T* residual, const T* weight, int64_t dim,
                                                                        float eps) {
  __shared__ float s_part[kThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  T* in_row = input + static_cast<int64_t>(blockIdx.x) * dim;
  T* res_row = residual + static_cast<int64_t>(blockIdx.x) * dim;
  float sum_sq = 0.f;
  for (int64_t i = tid; i < dim; i += kThreads) {
    const float r = to_f32<T>(in_row[i]) + to_f32<T>(res_row[i]);
    res_row[i] = from_f32<T>(r);
    sum_sq = fmaf(r, r, sum_sq);
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) sum_sq += __shfl_xor_sync(0xffffffffu, sum_sq, o);
  if (lane == 0) s_part[warp] = sum_sq;
  __syncthreads();
  sum_sq = 0.f;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) sum_sq += s_part[w];
  const float inv_rms = rsqrtf(sum_sq / static_cast<float>(dim) + eps);
  for (int64_t i = tid; i < dim; i += kThreads)
    in_row[i] = from_f32<T>(to_f32<T>(res_row[i]) * inv_rms * to_f32<T>(weight[i]));
}

constexpr int kSiluUnroll = 4;

// silu(g) * u with the fast exponential and reciprocal (the reference's kernel uses __expf as well)
__device__ __forceinline__ float silu_mul1(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

template <typename T>
__device__ __forceinline__ uint4 silu_vec(const uint4& g, const uint4& u) {
  constexpr int N = Pack<T>::N;
  float fg[N], fu[N];
  Pack<T>::unpack(g, fg);
  Pack<T>::unpack(u, fu);
#pragma unroll
  for (int i = 0; i < N; ++i) fg[i] = silu_mul1(fg[i], fu[i]);
  return Pack<T>::pack(fg);
}

// x [rows, 2d] -> out [rows, d], long rows: CTA (row, chunk) handles kThreads * kSiluUnroll
// vectors of one row, so that no index needs a division.  vecs_per_row = d / N.
template <typename T>
__global__ void __launch_bounds__(kThreads) silu_mul_rows_kernel(T* __restrict__ out, const T* __restrict__ x,
                                                                 int vecs_per_row) {
  constexpr int N = Pack<T>::N;
  const int64_t row = blockIdx.x;
  const int v0 = blockIdx.y * (kThreads * kSiluUnroll) + threadIdx.x;
  const T* gp = x + row * 2 * vecs_per_row * N;
  const T* up = gp + static_cast<int64_t>(vecs_per_row) * N;
  T* op = out + row * vecs_per_row * N;
  uint4 g[kSiluUnroll], u[kSiluUnroll];
#pragma unroll
  for (int k = 0; k < kSiluUnroll; ++k) {
    const int v = v0 + k * kThreads;
    if (v < vecs_per_row) g[k] = ld_cs(gp + v * N), u[k] = ld_cs(up + v * N);
  }
#pragma unroll
  for (int k = 0; k < kSiluUnroll; ++k) {
    const int v = v0 + k * kThreads;
    if (v < vecs_per_row) st_cs(op + v * N, silu_vec<T>(g[k], u[k]));
  }
}

// Short rows: a flat index over all vectors (32-bit arithmetic; the launcher checks the range).
template <typename T>
__global__ void __launch_bounds__(kThreads) silu_mul_kernel(T* __restrict__ out, const T* __restrict__ x, uint32_t total_vecs,
                                                            uint32_t vecs_per_row) {
  constexpr int N = Pack<T>::N;
  const uint32_t idx = blockIdx.x * kThreads + threadIdx.x;
  if (idx >= total_vecs) return;
  const uint32_t row = idx / vecs_per_row, col = idx - row * vecs_per_row;
  const T* gp = x + (static_cast<int64_t>(row) * 2 * vecs_per_row + col) * N;
  st_cs(out + static_cast<int64_t>(idx) * N, silu_vec<T>(ld_cs(gp), ld_cs(gp + static_cast<int64_t>(vecs_per_row) * N)));
}

template <typename T>
__global__ void __launch_bounds__(kThreads) silu_mul_generic_kernel(T* out, const T* x, int64_t n, int64_t d) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (i >= n) return;
  const int64_t row = i / d, col = i - row * d;
  const float g = to_f32<T>(x[row * 2 * d + col]), u = to_f32<T>(x[row * 2 * d + d + col]);
  out[i] = from_f32<T>(silu_mul1(g, u));
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
cudaError_t rms_t(void* input, void* residual, const void* weight, int64_t rows, int64_t dim, float eps,
                  cudaStream_t stream) {
  constexpr int N = Pack<T>::N;
  T* in = static_cast<T*>(input);
  T* res = static_cast<T*>(residual);
  const T* w = static_cast<const T*>(weight);
  const int64_t vecs = dim / N;
  const bool vec_ok = dim % N == 0 && vecs <= kThreads * 8 && aligned16(in) && aligned16(res) && aligned16(w);
  if (!vec_ok) {
    add_rms_norm_generic_kernel<T><<<static_cast<unsigned>(rows), kThreads, 0, stream>>>(in, res, w, dim, eps);
    return cudaGetLastError();
  }
  // threads per row: the fewest (>= 32) that keep a thread at <= 8 vectors ... but prefer
  // <= 4 so that enough loads are in flight without starving occupancy
  int tpr = 32;
  while (tpr < kThreads && vecs > static_cast<int64_t>(tpr) * 4) tpr <<= 1;
  const int vpt = static_cast<int>((vecs + tpr - 1) / tpr);
  const int rows_per_cta = kThreads / tpr;
  const unsigned grid = static_cast<unsigned>((rows + rows_per_cta - 1) / rows_per_cta);
  const int d = static_cast<int>(dim);
  if (vpt <= 1)
    add_rms_norm_kernel<T, 1><<<grid, kThreads, 0, stream>>>(in, res, w, rows, d, tpr, eps);
  else if (vpt <= 2)
    add_rms_norm_kernel<T, 2><<<grid, kThreads, 0, stream>>>(in, res, w, rows, d, tpr, eps);
  else if (vpt <= 4)
    add_rms_norm_kernel<T, 4><<<grid, kThreads, 0, stream>>>(in, res, w, rows, d, tpr, eps);
  else
    add_rms_norm_kernel<T, 8><<<grid, kThreads, 0, stream>>>(in, res, w, rows, d, tpr, eps);
  return cudaGetLastError();
}

template <typename T>
cudaError_t silu_t(void* out, const void* x, int64_t rows, int64_t d, cudaStream_t stream) {
  constexpr int N = Pack<T>::N;
  T* o = static_cast<T*>(out);
  const T* xi = static_cast<const T*>(x);
  const int64_t vpr = d / N, total = rows * vpr;
  const bool vec_ok = d % N == 0 && aligned16(o) && aligned16(xi);
  constexpr int kChunk = kThreads * kSiluUnroll;
  if (vec_ok && vpr >= kThreads && (vpr + kChunk - 1) / kChunk <= 65535 && rows <= 0x7fffffff) {
    dim3 grid(static_cast<unsigned>(rows), static_cast<unsigned>((vpr + kChunk - 1) / kChunk));
    silu_mul_rows_kernel<T><<<grid, kThreads, 0, stream>>>(o, xi, static_cast<int>(vpr));
  } else if (vec_ok && total < 0x7fffff00ll) {
    silu_mul_kernel<T><<<static_cast<unsigned>((total + kThreads - 1) / kThreads), kThreads, 0, stream>>>(
        o, xi, static_cast<uint32_t>(total), static_cast<uint32_t>(vpr));
  } else {
    const int64_t n = rows * d;
    silu_mul_generic_kernel<T><<<static_cast<unsigned>((n + kThreads - 1) / kThreads), kThreads, 0, stream>>>(o, xi, n, d);
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fused_add_rms_norm(int dtype, void* input, void* residual, const void* weight, int64_t rows,
                                      int64_t dim, float eps, cudaStream_t stream) {
  if (dtype == TT_ATTN_F32) return rms_t<float>(input, residual, weight, rows, dim, eps, stream);
  if (dtype == TT_ATTN_F16) return rms_t<__half>(input, residual, weight, rows, dim, eps, stream);
  return rms_t<__nv_bfloat16>(input, residual, weight, rows, dim, eps, stream);
}

cudaError_t launch_silu_mul(int dtype, void* out, const void* x, int64_t rows, int64_t d, cudaStream_t stream) {
  if (dtype == TT_ATTN_F32) return silu_t<float>(out, x, rows, d, stream);
  if (dtype == TT_ATTN_F16) return silu_t<__half>(out, x, rows, d, stream);
  return silu_t<__nv_bfloat16>(out, x, rows, d, stream);
}

}  // namespace ttattn
