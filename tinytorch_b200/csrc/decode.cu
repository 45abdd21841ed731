// Single-token decode against a KV cache: a streaming scan bounded by HBM bandwidth.
//
// The reference can only express this step as sdpAttention(q[B,H,1,D], Kc, Vc,
// false, boolmask) (src/Function/FuncNNLayer.h:249-252), which transposes the whole
// cache (src/Operation/OpTransformCpu.h:54-87) and materialises [B,H,1,S] scores.
// Here every valid cache byte is read exactly once with 128-bit loads and nothing
// else of that size touches HBM.
//
// Split-KV: CTA (split, kv head, batch) scans keys [split*chunk, (split+1)*chunk)
// below kv_len[b].  A cache row of D elements is covered by D*sizeof(T)/16 lanes,
// each holding one 16-byte slice of the row; the lanes of a row reduce the dot
// product with warp shuffles.  Every lane group keeps an independent online-softmax
// state (max, sum, D-slice of the weighted V sum) for each of the G query heads
// that share the kv head, so the loop has no cross-group dependency; states are
// merged across lane groups (shuffles), warps (shared memory) and, when the
// sequence was split, by a second small kernel over the per-split partials.
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace ttattn {
namespace {

constexpr int kThreads = 256, kWarps = 8, UNR = 4;

template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& w, float (&f)[4]) {
    f[0] = __uint_as_float(w.x), f[1] = __uint_as_float(w.y), f[2] = __uint_as_float(w.z), f[3] = __uint_as_float(w.w);
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& w, float (&f)[8]) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(u[i] << 16);
      f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
  }
};
template <>
struct Vec16<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& w, float (&f)[8]) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
      f[2 * i] = t.x, f[2 * i + 1] = t.y;
    }
  }
};

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.cs.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

template <typename T>
__device__ __forceinline__ uint4 pack16(const float (&f)[Vec16<T>::N]) {
  if constexpr (sizeof(T) == 4) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  } else {
    uint32_t u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      T lo = from_f32<T>(f[2 * i]), hi = from_f32<T>(f[2 * i + 1]);
      u[i] = static_cast<uint32_t>(*reinterpret_cast<uint16_t*>(&lo)) |
             (static_cast<uint32_t>(*reinterpret_cast<uint16_t*>(&hi)) << 16);
    }
    return make_uint4(u[0], u[1], u[2], u[3]);
  }
}

// Rotary position embedding of one row at position `pos`, applied to the lane's
// slice x[0..N) = elements [d0, d0+N) of the row.  Pairs are (i, i + D/2), the two
// halves living LPK/2 lanes apart (every lane of the warp must call this), or
// (2i, 2i+1) inside the slice when `interleaved`.  Pair i turns by the angle whose
// cosine / sine are cos[pos][i] / sin[pos][i].
template <int N, int LPK, int D>
__device__ __forceinline__ void rope_slice(float (&x)[N], const float* cos, const float* sin, int pos, int d0,
                                           bool interleaved) {
  const float* cp = cos + static_cast<int64_t>(pos) * (D / 2);
  const float* sp = sin + static_cast<int64_t>(pos) * (D / 2);
  if (interleaved) {
#pragma unroll
    for (int i = 0; i < N; i += 2) {
      const float c = cp[(d0 + i) >> 1], s = sp[(d0 + i) >> 1];
      const float a = x[i], b = x[i + 1];
      x[i] = a * c - b * s;
      x[i + 1] = b * c + a * s;
    }
  } else {
    const bool upper = d0 >= D / 2;
    const int f0 = upper ? d0 - D / 2 : d0;
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, x[i], LPK / 2);
      const float c = cp[f0 + i], s = sp[f0 + i];
      x[i] = upper ? x[i] * c + other * s : x[i] * c - other * s;
    }
  }
}

// G = query heads handled per pass (all share this CTA's kv head).  APPEND: the
// step's new key / value row is rotated, written to the cache at row kv_len[b] and
// attended to like any other row; q is rotated to the same position.
template <typename T, int D, int G, bool APPEND>
__global__ void __launch_bounds__(kThreads, G == 1 ? 3 : 1) decode_kernel(const DecodeArgs a) {
  ptx::grid_dep_launch();  // the combine kernel's CTAs may come up under the last wave of this grid
  constexpr int N = Vec16<T>::N;  // elements per 16-byte slice
  constexpr int LPK = D / N;      // lanes per cache row
  constexpr int KPW = 32 / LPK;   // rows per warp-wide load
  __shared__ float s_acc[kWarps][G][D];
  __shared__ float s_m[kWarps][G], s_l[kWarps][G];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sub = lane / LPK;        // which of the KPW rows this lane works on
  const int d0 = (lane % LPK) * N;   // first element of this lane's slice
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int group = a.Hq / a.Hkv;

  int len = a.capacity;
  if (a.kv_lens) {
    int l = a.kv_lens[b];
    len = l < 0 ? 0 : (l < a.capacity ? l : a.capacity);
  }
  const T* kbase = reinterpret_cast<const T*>(a.k) + b * a.ks.b + hk * a.ks.h + d0;
  const T* vbase = reinterpret_cast<const T*>(a.v) + b * a.vs.b + hk * a.vs.h + d0;

  int pos = 0;  // APPEND: position of the step's token
  bool rotate = false;
  if constexpr (APPEND) {
    pos = len;
    rotate = a.rope_cos != nullptr && pos < a.rope_positions;
    if (tid == 0 && a.status && a.rope_cos != nullptr && !rotate) atomicOr(a.status, kStatusRopeRange);
    if (pos < a.capacity) {
      // the one CTA of this (b, kv head) whose chunk holds row `pos` writes it;
      // no other CTA reads that row
      if (split == pos / a.chunk) {
        if (warp == 0) {
          const T* kn = reinterpret_cast<const T*>(a.k_new) + b * a.kn_b + hk * a.kn_h + d0;
          float kf[N];
          Vec16<T>::unpack(*reinterpret_cast<const uint4*>(kn), kf);
          if (rotate) rope_slice<N, LPK, D>(kf, a.rope_cos, a.rope_sin, pos, d0, a.rope_interleaved != 0);
          if (sub == 0) {
            const T* vn = reinterpret_cast<const T*>(a.v_new) + b * a.vn_b + hk * a.vn_h + d0;
            *reinterpret_cast<uint4*>(const_cast<T*>(kbase) + static_cast<int64_t>(pos) * a.ks.s) = pack16<T>(kf);
            *reinterpret_cast<uint4*>(const_cast<T*>(vbase) + static_cast<int64_t>(pos) * a.vs.s) =
                *reinterpret_cast<const uint4*>(vn);
          }
        }
        __syncthreads();  // the row is in the cache before this CTA scans it
      }
      len = pos + 1;
    } else if (tid == 0 && a.status) {
      atomicOr(a.status, kStatusCacheFull);  // nothing appended; the scan covers the full cache
    }
    if (split == 0 && hk == 0 && tid == 0 && a.new_lens) a.new_lens[b] = len;
  }
  const int begin = split * a.chunk;
  const int end = min(len, begin + a.chunk);
  const float c = a.scale * kLog2e;

  for (int g0 = 0; g0 < group; g0 += G) {
    const int h0 = hk * group + g0;
    float qf[G][N];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const T* qp = reinterpret_cast<const T*>(a.q) + b * a.qs.b + (h0 + g) * a.qs.h + d0;
      Vec16<T>::unpack(*reinterpret_cast<const uint4*>(qp), qf[g]);
      if constexpr (APPEND) {
        if (rotate) rope_slice<N, LPK, D>(qf[g], a.rope_cos, a.rope_sin, pos, d0, a.rope_interleaved != 0);
      }
#pragma unroll
      for (int i = 0; i < N; ++i) qf[g][i] *= c;
    }
    float m[G], l[G], acc[G][N];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      m[g] = -INFINITY, l[g] = 0.f;
#pragma unroll
      for (int i = 0; i < N; ++i) acc[g][i] = 0.f;
    }

    // warp w takes rows begin + (it*kWarps + w)*UNR*KPW + u*KPW + sub
    for (int base = begin + warp * UNR * KPW; base < end; base += kWarps * UNR * KPW) {
      uint4 kw[UNR], vw[UNR];
      bool valid[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int row = base + u * KPW + sub;
        valid[u] = row < end;
        kw[u] = valid[u] ? ld_stream(kbase + static_cast<int64_t>(row) * a.ks.s) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int row = base + u * KPW + sub;
        vw[u] = valid[u] ? ld_stream(vbase + static_cast<int64_t>(row) * a.vs.s) : make_uint4(0, 0, 0, 0);
      }
      float s[G][UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        float kf[N];
        Vec16<T>::unpack(kw[u], kf);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float t = 0.f;
#pragma unroll
          for (int i = 0; i < N; ++i) t = fmaf(qf[g][i], kf[i], t);
#pragma unroll
          for (int o = LPK / 2; o >= 1; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
          s[g][u] = valid[u] ? t : -INFINITY;
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float mx = m[g];
#pragma unroll
        for (int u = 0; u < UNR; ++u) mx = fmaxf(mx, s[g][u]);
        if (mx == -INFINITY) continue;  // nothing valid for this lane group yet
        const float alpha = exp2f(m[g] - mx);
        m[g] = mx;
        l[g] *= alpha;
#pragma unroll
        for (int i = 0; i < N; ++i) acc[g][i] *= alpha;
#pragma unroll
        for (int u = 0; u < UNR; ++u) s[g][u] = exp2f(s[g][u] - mx);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        float vf[N];
        Vec16<T>::unpack(vw[u], vf);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float p = (m[g] == -INFINITY) ? 0.f : s[g][u];
          l[g] += p;
#pragma unroll
          for (int i = 0; i < N; ++i) acc[g][i] = fmaf(p, vf[i], acc[g][i]);
        }
      }
    }

    // merge the KPW lane groups of the warp
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m[g], o);
        const float l2 = __shfl_xor_sync(0xffffffffu, l[g], o);
        const float mn = fmaxf(m[g], m2);
        const float w1 = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mn);
        const float w2 = (m2 == -INFINITY) ? 0.f : exp2f(m2 - mn);
        l[g] = l[g] * w1 + l2 * w2;
#pragma unroll
        for (int i = 0; i < N; ++i) {
          const float a2 = __shfl_xor_sync(0xffffffffu, acc[g][i], o);
          acc[g][i] = acc[g][i] * w1 + a2 * w2;
        }
        m[g] = mn;
      }
    }
    __syncthreads();  // shared arrays free (previous pass consumed)
    if (sub == 0) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int i = 0; i < N; ++i) s_acc[warp][g][d0 + i] = acc[g][i];
        if (lane == 0) s_m[warp][g] = m[g], s_l[warp][g] = l[g];
      }
    }
    __syncthreads();
    // merge the warps; thread t handles (head t / D, element t % D)
    for (int idx = tid; idx < G * D; idx += kThreads) {
      const int g = idx / D, d = idx % D;
      float mn = -INFINITY;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) mn = fmaxf(mn, s_m[w][g]);
      float lt = 0.f, at = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float wgt = (s_m[w][g] == -INFINITY) ? 0.f : exp2f(s_m[w][g] - mn);
        lt += s_l[w][g] * wgt;
        at += s_acc[w][g][d] * wgt;
      }
      const int h = h0 + g;
      if (a.nsplit == 1) {
        const float inv = lt > 0.f ? 1.f / lt : 0.f;
        reinterpret_cast<T*>(a.o)[b * a.os.b + h * a.os.h + d] = from_f32<T>(at * inv);
        if (a.lse && d == 0) a.lse[static_cast<int64_t>(b) * a.Hq + h] = lt > 0.f ? (mn + log2f(lt)) * kLn2 : -INFINITY;
      } else {
        float* pp = a.partial + ((static_cast<int64_t>(b) * a.Hq + h) * a.nsplit + split) * (D + 2);
        pp[d] = at;
        if (d == 0) pp[D] = mn, pp[D + 1] = lt;
      }
    }
  }
}

// One CTA per (head, batch): fold the per-split partials into O and LSE.
template <typename T, int D>
__global__ void __launch_bounds__(D) decode_combine_kernel(const DecodeArgs a) {
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  ptx::grid_dep_wait();  // (launched early after the tensor-core scan: its partials are complete from here on)
  const float* pp = a.partial + (static_cast<int64_t>(b) * a.Hq + h) * a.nsplit * (D + 2);
  float mn = -INFINITY;
  for (int s = 0; s < a.nsplit; ++s) mn = fmaxf(mn, pp[s * (D + 2) + D]);
  float lt = 0.f, at = 0.f;
  for (int s = 0; s < a.nsplit; ++s) {
    const float ms = pp[s * (D + 2) + D];
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - mn);
    lt += pp[s * (D + 2) + D + 1] * w;
    at += pp[s * (D + 2) + d] * w;
  }
  const float inv = lt > 0.f ? 1.f / lt : 0.f;
  reinterpret_cast<T*>(a.o)[b * a.os.b + h * a.os.h + d] = from_f32<T>(at * inv);
  if (a.lse && d == 0) a.lse[static_cast<int64_t>(b) * a.Hq + h] = lt > 0.f ? (mn + log2f(lt)) * kLn2 : -INFINITY;
}

// `early`: the scan kernel before it lets its dependents start; the combine kernel's CTAs
// then come up while the scan still runs and wait in grid_dep_wait() for its partials.
template <typename T, int D>
cudaError_t combine_t(const DecodeArgs& a, cudaStream_t stream, bool early = false) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.Hq, a.B);
  cfg.blockDim = dim3(D);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  if (early) cfg.attrs = attr, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, decode_combine_kernel<T, D>, a);
}

template <typename T, int D, bool APPEND>
cudaError_t launch_t(const DecodeArgs& a, cudaStream_t stream) {
  const int group = a.Hq / a.Hkv;
  dim3 grid(a.nsplit, a.Hkv, a.B);
  if (group % 8 == 0)
    decode_kernel<T, D, 8, APPEND><<<grid, kThreads, 0, stream>>>(a);
  else if (group % 4 == 0)
    decode_kernel<T, D, 4, APPEND><<<grid, kThreads, 0, stream>>>(a);
  else if (group % 2 == 0)
    decode_kernel<T, D, 2, APPEND><<<grid, kThreads, 0, stream>>>(a);
  else
    decode_kernel<T, D, 1, APPEND><<<grid, kThreads, 0, stream>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || a.nsplit == 1) return e;
  return combine_t<T, D>(a, stream, true);
}

}  // namespace

void decode_plan(int capacity, int* nsplit, int* chunk) {
  // 512-row chunks keep CTAs short enough that mixed sequence lengths balance
  // across the SMs; at most 64 splits per sequence.
  int ck = 512;
  if ((capacity + ck - 1) / ck > 64) ck = (((capacity + 63) / 64) + 63) / 64 * 64;
  *chunk = ck;
  *nsplit = capacity <= ck ? 1 : (capacity + ck - 1) / ck;
}

template <bool APPEND>
cudaError_t launch_d(int dtype, int D, const DecodeArgs& a, cudaStream_t stream) {
  if (dtype == TT_ATTN_F32)
    return D == 64 ? launch_t<float, 64, APPEND>(a, stream) : launch_t<float, 128, APPEND>(a, stream);
  if (dtype == TT_ATTN_F16)
    return D == 64 ? launch_t<__half, 64, APPEND>(a, stream) : launch_t<__half, 128, APPEND>(a, stream);
  return D == 64 ? launch_t<__nv_bfloat16, 64, APPEND>(a, stream) : launch_t<__nv_bfloat16, 128, APPEND>(a, stream);
}

// The plan a call with these sizes uses (the launcher, the workspace query and the entry points agree
// through this one function).  The tensor-core path pays a few thousand cycles at every item boundary
// (the two softmax chains are merged there), so its chunks are 2048 rows - 16 tiles - unless that would
// leave fewer than about two items per SM.
void decode_plan_for(int dtype, int D, int B, int Hq, int Hkv, int capacity, int* nsplit, int* chunk) {
  DecodeArgs probe{};
  probe.Hq = Hq, probe.Hkv = Hkv;
  if (!decode_tc_applies(dtype, D, probe)) {
    decode_plan(capacity, nsplit, chunk);
    return;
  }
  int ck = 2048;
  const long long want = D == 64 ? 592 : 296;  // two items per resident CTA (D = 64 runs two CTAs per SM)
  while (ck > 512 && static_cast<long long>(B) * Hkv * ((capacity + ck - 1) / ck) < want) ck >>= 1;
  if ((capacity + ck - 1) / ck > 64) ck = (((capacity + 63) / 64) + 127) / 128 * 128;
  *chunk = ck;
  *nsplit = capacity <= ck ? 1 : (capacity + ck - 1) / ck;
}

cudaError_t launch_decode(int dtype, int D, const DecodeArgs& a, cudaStream_t stream) {
  if (decode_tc_applies(dtype, D, a)) {
    // several query heads per kv head: the tensor-core scan, then the same combine kernel
    cudaError_t e = launch_decode_tc(dtype, D, a, stream);
    if (e != cudaSuccess || a.nsplit == 1) return e;
    if (D == 128) return dtype == TT_ATTN_F16 ? combine_t<__half, 128>(a, stream, true) : combine_t<__nv_bfloat16, 128>(a, stream, true);
    return dtype == TT_ATTN_F16 ? combine_t<__half, 64>(a, stream, true) : combine_t<__nv_bfloat16, 64>(a, stream, true);
  }
  return launch_d<false>(dtype, D, a, stream);
}

namespace {

// Grouped-query append on the tensor-core path, step 1: one CTA per (head, batch) rotates q into scratch
// (heads 0..Hq-1) or rotates the new key and writes it and the new value into the caches (heads Hq..Hq+Hkv-1);
// thread t handles the pair (t, t + D/2), or (2t, 2t+1) when interleaved.  The lengths after the append go to
// lens_out.  Step 2 is the ordinary tensor-core decode over q_rot and lens_out.
template <typename T, int D>
__global__ void __launch_bounds__(D / 2) rope_append_kernel(const DecodeArgs a, int32_t* lens_out) {
  const int hh = blockIdx.x, b = blockIdx.y, t = threadIdx.x;
  ptx::grid_dep_launch();  // the decode kernel may set itself up; it waits for this grid before it reads anything
  if (hh == 0 && b == 0 && t == 0 && a.sched) *a.sched = 0;  // its work counter
  int pos = a.kv_lens[b];
  pos = pos < 0 ? 0 : pos;
  const bool room = pos < a.capacity;
  const bool rotate = a.rope_cos != nullptr && pos < a.rope_positions;
  if (hh == 0 && t == 0) {
    const int len = room ? pos + 1 : a.capacity;
    lens_out[b] = len;
    if (a.new_lens) a.new_lens[b] = len;
    if (a.status && !room) atomicOr(a.status, kStatusCacheFull);
    if (a.status && a.rope_cos != nullptr && !rotate) atomicOr(a.status, kStatusRopeRange);
  }
  const bool is_q = hh < a.Hq;
  const int hk = hh - a.Hq;
  if (!is_q && !room) return;  // nothing is appended to a full cache
  const T* src = is_q ? reinterpret_cast<const T*>(a.q) + b * a.qs.b + hh * a.qs.h
                      : reinterpret_cast<const T*>(a.k_new) + b * a.kn_b + hk * a.kn_h;
  T* dst = is_q ? reinterpret_cast<T*>(a.q_rot) + (static_cast<int64_t>(b) * a.Hq + hh) * D
                : const_cast<T*>(reinterpret_cast<const T*>(a.k)) + b * a.ks.b + hk * a.ks.h + static_cast<int64_t>(pos) * a.ks.s;
  const int i0 = a.rope_interleaved ? 2 * t : t, i1 = a.rope_interleaved ? 2 * t + 1 : t + D / 2;
  float x0 = to_f32<T>(src[i0]), x1 = to_f32<T>(src[i1]);
  if (rotate) {
    const float c = a.rope_cos[static_cast<int64_t>(pos) * (D / 2) + t], s = a.rope_sin[static_cast<int64_t>(pos) * (D / 2) + t];
    const float y0 = x0 * c - x1 * s, y1 = x1 * c + x0 * s;
    x0 = y0, x1 = y1;
  }
  dst[i0] = from_f32<T>(x0);
  dst[i1] = from_f32<T>(x1);
  if (!is_q) {
    const T* vs = reinterpret_cast<const T*>(a.v_new) + b * a.vn_b + hk * a.vn_h;
    T* vd = const_cast<T*>(reinterpret_cast<const T*>(a.v)) + b * a.vs.b + hk * a.vs.h + static_cast<int64_t>(pos) * a.vs.s;
    vd[i0] = vs[i0];
    vd[i1] = vs[i1];
  }
}

template <typename T, int D>
cudaError_t append_tc_t(int dtype, const DecodeArgs& a, cudaStream_t stream) {
  rope_append_kernel<T, D><<<dim3(a.Hq + a.Hkv, a.B), D / 2, 0, stream>>>(a, a.lens_scratch);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  DecodeArgs d = a;
  d.q = a.q_rot;
  d.qs = Str3{static_cast<int64_t>(a.Hq) * D, D, D};
  d.kv_lens = a.lens_scratch;
  d.chained = 1;
  return launch_decode(dtype, D, d, stream);
}

}  // namespace

cudaError_t launch_decode_append(int dtype, int D, const DecodeArgs& a, cudaStream_t stream) {
  // several query heads per kv head: rotate / append in a small kernel, then the tensor-core decode
  if (decode_tc_applies(dtype, D, a) && a.q_rot && a.lens_scratch) {
    if (D == 128)
      return dtype == TT_ATTN_F16 ? append_tc_t<__half, 128>(dtype, a, stream) : append_tc_t<__nv_bfloat16, 128>(dtype, a, stream);
    return dtype == TT_ATTN_F16 ? append_tc_t<__half, 64>(dtype, a, stream) : append_tc_t<__nv_bfloat16, 64>(dtype, a, stream);
  }
  return launch_d<true>(dtype, D, a, stream);
}

// ---------------------------------------------------------------------------
// Allocation-free decode.  Some hosts may launch kernels but have no way to hand
// this library device memory: an embedding runtime that owns the whole heap and
// exposes neither an allocator callback nor a spare buffer, or a serving loop
// whose latency budget rules out allocator calls on the token path (cudaMalloc
// takes a process-wide lock and may synchronise the device).  For them the
// per-split partials live in a fixed array inside the library image instead of in
// caller-provided scratch.  Every GPU that loads the library carries the array
// until the process exits, hence the modest size.
//
// The array is shared by every call on a device and keeps the previous call's
// contents.  Each launch writes every (batch, head, split) slot before the combine
// kernel reads it; the only word that must start at zero, the tensor-core path's
// work counter in the last 256 bytes of what a call uses, is reset by a memset on
// the call's stream.  Two calls that overlap on the GPU (different streams) would
// race on the array.
namespace {

constexpr size_t kStaticScratchBytes = TT_ATTN_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_ptr[kMaxDevices] = {};

}  // namespace

// `device` must be the current device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel can use, so the device address
// is looked up once per device with cudaGetSymbolAddress and cached.
cudaError_t launch_decode_static(int dtype, int D, DecodeArgs a, size_t need, int device, cudaStream_t stream,
                                 bool* too_large) {
  *too_large = need > kStaticScratchBytes || device < 0 || device >= kMaxDevices;
  if (*too_large) return cudaSuccess;
  void* ptr = nullptr;
  if (need > 0) {
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[device]) {
      void* sym = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&sym, g_decode_scratch);
      if (e != cudaSuccess) return e;
      g_scratch_ptr[device] = sym;
    }
    ptr = g_scratch_ptr[device];
  }
  a.partial = static_cast<float*>(ptr);
  a.sched = need >= 256 ? reinterpret_cast<int*>(static_cast<char*>(ptr) + need - 256) : nullptr;
  return launch_decode(dtype, D, a, stream);
}

}  // namespace ttattn
