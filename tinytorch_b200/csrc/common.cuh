// Shared host/device declarations of the attention library's internal launchers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tt_attn.h"

namespace ttattn {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Status bits a kernel may OR into the caller's status word.
constexpr int kStatusWaitExpired = 1;
constexpr int kStatusBadSmemAlign = 2;   // dynamic shared memory did not start on a 1024-byte boundary
constexpr int kStatusCacheFull = 4;      // decode-append: no free row in the cache of some sequence
constexpr int kStatusRopeRange = 8;      // decode-append: position beyond the rotary tables

struct Str3 {
  int64_t b, h, s;
};

inline Str3 dense_or(const tt_attn_strides& st, int64_t H, int64_t S, int64_t D) {
  if (st.b == 0 && st.h == 0 && st.s == 0) return Str3{H * S * D, S * D, D};
  return Str3{st.b, st.h, st.s};
}

// Optional mask, broadcast against [B, Hq, Lq, Skv]; the key dimension is contiguous.
struct MaskArgs {
  const void* ptr;  // null: no mask
  int kind;         // tt_attn_mask_kind
  int64_t sb, sh, sl;
};

// Arguments common to the prefill kernels (SIMT and tensor-core).
struct FwdArgs {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;
  Str3 qs, ks, vs, os;
  int B, Hq, Hkv, Lq, Skv;
  int causal;  // tt_attn_causal
  float scale;
  const int32_t* kv_lens;
  int32_t* status;
  MaskArgs mask;
  int* sched;  // tensor-core path: work counter in scratch memory, zeroed by the launcher
};

struct BwdArgs {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* d_o;
  const float* lse;
  float* delta;     // workspace [B, Hq, Lq]
  float* dq_accum;  // workspace [B, Hq, Lq, D] fp32 (tensor-core path), zeroed by the delta pre-pass
  int zero_dq_accum;  // set by the tensor-core launcher: the delta kernel also clears dq_accum
  int tail_heads;     // tensor-core kernel: (batch, kv head) pairs at the end of the item order whose key tiles are
                      // ordered longest walk first across heads (set by its launcher)
  int* sched;         // tensor-core kernel: work counter in scratch memory, zeroed by its launcher
  void* dq;
  void* dk;
  void* dv;
  Str3 qs, ks, vs, os, dos, dqs, dks, dvs;
  int B, Hq, Hkv, Lq, Skv;
  int causal;  // tt_attn_causal
  float scale;
  const int32_t* kv_lens;
  int32_t* status;
  MaskArgs mask;
};

struct DecodeArgs {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;
  float* partial;  // workspace [B, Hq, nsplit, D + 2] when nsplit > 1
  Str3 qs, ks, vs, os;
  int B, Hq, Hkv, capacity;
  int nsplit, chunk;
  float scale;
  const int32_t* kv_lens;
  // append variant only: the step's new key / value row per (b, kv head), rotary tables, outputs
  const void* k_new;
  const void* v_new;
  int64_t kn_b, kn_h, vn_b, vn_h;  // element strides of k_new / v_new
  const float* rope_cos;           // [rope_positions, D/2] or null: no rotation
  const float* rope_sin;
  int rope_positions;
  int rope_interleaved;            // pairs (2i, 2i+1) instead of (i, i + D/2)
  int32_t* new_lens;               // optional [B]: kv_lens[b] + 1
  int32_t* status;
  int* sched;                      // tensor-core path: work counter in scratch memory, zeroed by the launcher
  void* q_rot;                     // append on the tensor-core path: scratch [B, Hq, D] for the rotated q
  int32_t* lens_scratch;           // ... and [B] for the lengths after the append
  int chained;                     // tensor-core path: the kernel before this one in the stream has zeroed the
                                   // work counter and lets its dependents start early (programmatic launch)
};

// Each returns a cudaError_t from the launch (no synchronisation).
cudaError_t launch_fwd_tc(int dtype, int D, const FwdArgs& a, int device, cudaStream_t stream);
cudaError_t launch_fwd_simt(int dtype, int D, const FwdArgs& a, cudaStream_t stream);
cudaError_t launch_bwd_simt(int dtype, int D, const BwdArgs& a, cudaStream_t stream);
// rowsum(dO o O) into a.delta only (first step of every backward)
cudaError_t launch_bwd_delta(int dtype, int D, const BwdArgs& a, cudaStream_t stream);
// fp16 / bf16 backward on the tensor cores; needs a.delta and a.dq_accum
cudaError_t launch_bwd_tc(int dtype, int D, const BwdArgs& a, int device, cudaStream_t stream);
cudaError_t launch_decode(int dtype, int D, const DecodeArgs& a, cudaStream_t stream);
// grouped-query decode on the tensor cores (decode_tc.cu): 16-bit tensors, 2..16 query heads per kv head
bool decode_tc_applies(int dtype, int D, const DecodeArgs& a);
cudaError_t launch_decode_tc(int dtype, int D, const DecodeArgs& a, cudaStream_t stream);
// rotary embedding of q and the new key, append of the new key / value row, then the same scan
cudaError_t launch_decode_append(int dtype, int D, const DecodeArgs& a, cudaStream_t stream);

cudaError_t launch_decode_static(int dtype, int D, DecodeArgs a, size_t need, int device, cudaStream_t stream,
                                 bool* too_large);

// The reference's two fused transformer-block operators (fused_ops.cu).
cudaError_t launch_fused_add_rms_norm(int dtype, void* input, void* residual, const void* weight, int64_t rows,
                                      int64_t dim, float eps, cudaStream_t stream);
cudaError_t launch_silu_mul(int dtype, void* out, const void* x, int64_t rows, int64_t d, cudaStream_t stream);

// y = x w^T + bias on the tensor cores (linear_tc.cu); ld* are row strides in elements
cudaError_t launch_linear_tc(int dtype, const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                             int64_t ldx, int64_t ldw, int64_t ldy, int32_t* status, int device, cudaStream_t stream);

// one CTA waiting `limit_ns` on an mbarrier nobody arrives on (selftest.cu)
cudaError_t launch_wait_expiry(int32_t* status, uint64_t limit_ns, unsigned long long* waited_ns, cudaStream_t stream);

// Split planning for decode, shared by the launcher and the workspace query.
void decode_plan(int capacity, int* nsplit, int* chunk);
// ... for the tensor-core path (several query heads per kv head): longer chunks, see decode.cu
void decode_plan_for(int dtype, int D, int B, int Hq, int Hkv, int capacity, int* nsplit, int* chunk);

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) {
  return x;
}
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) {
  return __half2float(x);
}
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) {
  return __bfloat162float(x);
}
template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) {
  return x;
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) {
  return __float2half_rn(x);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}


// Query i sees key j under a causal mask iff j <= i + causal_shift(...).
__host__ __device__ __forceinline__ int causal_shift(int causal, int kv_len, int Lq) {
  return causal == TT_ATTN_CAUSAL_BOTTOM_RIGHT ? kv_len - Lq : 0;
}

// What the mask adds to the scaled score of one (query, key) pair, in log2
// units: 0 or -inf for a boolean mask.  `off` is the element offset of the pair.
template <typename T>
__device__ __forceinline__ float mask_bias2(const MaskArgs& m, int64_t off) {
  if (m.kind == TT_ATTN_MASK_BOOL) return reinterpret_cast<const uint8_t*>(m.ptr)[off] ? 0.f : -INFINITY;
  if (m.kind == TT_ATTN_MASK_ADD_F32) return reinterpret_cast<const float*>(m.ptr)[off] * kLog2e;
  return to_f32<T>(reinterpret_cast<const T*>(m.ptr)[off]) * kLog2e;
}

}  // namespace ttattn
