// extern "C" entry points of libtt_attn.so: argument validation, workspace
// handling through the caller's allocator hook, device guard, kernel dispatch.
// See include/tt_attn.h for the contract of each function.
#include <cstddef>
#include <cstdio>
#include <cstring>

#include "../../include/tt_fused.h"
#include "common.cuh"
#include "tma_host.cuh"

namespace ttattn {
namespace {

thread_local char g_cuda_error[256] = "";

int launch_failed(cudaError_t e) {
  std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
  return TT_ATTN_ERR_LAUNCH;
}

// Equivalent of the reference's CudaDeviceGuard (src/Utils/CUDAUtils.h:100-113).
struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) return;
    ok = (prev == device) || cudaSetDevice(device) == cudaSuccess;
    if (prev == device) prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

inline size_t elem_size(int dtype) { return dtype == TT_ATTN_F32 ? 4 : 2; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline bool strides_ok(const Str3& s, size_t es) {
  return s.b >= 0 && s.h >= 0 && s.s > 0 && (s.b * es) % 16 == 0 && (s.h * es) % 16 == 0 && (s.s * es) % 16 == 0;
}
inline size_t round256(size_t n) { return (n + 255) & ~size_t(255); }

// Scratch memory for one call: the caller's buffer, or a block from the hook
// that is handed back when this object goes out of scope (after the launches
// have been enqueued; reuse is stream-ordered).
struct Workspace {
  void* ptr = nullptr;
  const tt_attn_alloc_hook* hook = nullptr;
  int device = 0;
  bool owned = false;
  int acquire(size_t need, void* user, size_t user_bytes, const tt_attn_alloc_hook* h, int dev) {
    if (need == 0) return TT_ATTN_OK;
    if (user) {
      if (user_bytes < need) return TT_ATTN_ERR_WORKSPACE;
      if (!aligned16(user)) return TT_ATTN_ERR_ALIGN;
      ptr = user;
      return TT_ATTN_OK;
    }
    if (!h || !h->alloc || !h->free) return TT_ATTN_ERR_WORKSPACE;
    ptr = h->alloc(h->ctx, need, dev);
    if (!ptr) return TT_ATTN_ERR_WORKSPACE;
    hook = h, device = dev, owned = true;
    return TT_ATTN_OK;
  }
  ~Workspace() {
    if (owned) hook->free(hook->ctx, ptr, device);
  }
};

int check_common(int dtype, int B, int Hq, int Hkv, int Lq, int Skv, int D) {
  if (dtype != TT_ATTN_F32 && dtype != TT_ATTN_F16 && dtype != TT_ATTN_BF16) return TT_ATTN_ERR_DTYPE;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Lq <= 0 || Skv <= 0 || Hq % Hkv != 0) return TT_ATTN_ERR_SHAPE;
  if (D != 64 && D != 128) return TT_ATTN_ERR_HEAD_DIM;
  if (B > 65535 || Hq > 65535) return TT_ATTN_ERR_TOO_LARGE;  // grid.y / grid.z
  return TT_ATTN_OK;
}

}  // namespace
}  // namespace ttattn

using namespace ttattn;

extern "C" {

int tt_attn_version(void) { return TT_ATTN_ABI_VERSION; }

const char* tt_attn_last_cuda_error(void) { return g_cuda_error; }

const char* tt_attn_strerror(int status) {
  switch (status) {
    case TT_ATTN_OK: return "ok";
    case TT_ATTN_ERR_NULL: return "a required pointer is NULL";
    case TT_ATTN_ERR_DTYPE: return "unsupported dtype (expected 0=Float32, 1=Float16, 2=BFloat16)";
    case TT_ATTN_ERR_SHAPE: return "invalid shape";
    case TT_ATTN_ERR_HEAD_DIM: return "head dimension must be 64 or 128";
    case TT_ATTN_ERR_ALIGN: return "pointers and strides must be 16-byte aligned";
    case TT_ATTN_ERR_WORKSPACE: return "workspace too small, or allocator hook missing / returned NULL";
    case TT_ATTN_ERR_LAUNCH: return "CUDA launch error (see tt_attn_last_cuda_error)";
    case TT_ATTN_ERR_STRUCT: return "parameter struct size mismatch";
    case TT_ATTN_ERR_NO_DEVICE: return "invalid device or CUDA driver entry point unavailable";
    case TT_ATTN_ERR_TOO_LARGE: return "size beyond a fixed limit of this library";
    default: return "unknown status";
  }
}

}  // extern "C"

namespace {
// Validates the optional mask of a prefill call.
int take_mask(const void* ptr, int kind, const int64_t st[3], MaskArgs* m) {
  *m = MaskArgs{};
  if (kind == TT_ATTN_MASK_NONE || !ptr) return (kind == TT_ATTN_MASK_NONE) ? TT_ATTN_OK : TT_ATTN_ERR_NULL;
  if (kind < 0 || kind > TT_ATTN_MASK_ADD_F32) return TT_ATTN_ERR_DTYPE;
  if (st[0] < 0 || st[1] < 0 || st[2] < 0) return TT_ATTN_ERR_SHAPE;
  m->ptr = ptr, m->kind = kind, m->sb = st[0], m->sh = st[1], m->sl = st[2];
  return TT_ATTN_OK;
}
}  // namespace

extern "C" {

size_t tt_attn_workspace_bytes(int kind, int dtype, int B, int Hq, int Hkv, int Lq, int Skv, int D) {
  (void)Hkv;
  if (B <= 0 || Hq <= 0 || D <= 0) return 0;
  // fp16 / bf16 forward: one work counter for the persistent kernel's scheduler
  if (kind == TT_ATTN_KIND_FWD) return dtype == TT_ATTN_F32 ? 0 : 256;
  if (kind == TT_ATTN_KIND_BWD) {
    // delta [B,Hq,Lq] fp32; the fp16 / bf16 path adds an fp32 dQ accumulator [B,Hq,Lq,D]
    const size_t rows = static_cast<size_t>(B) * Hq * (Lq > 0 ? Lq : 0);
    // and the persistent kernel's work counter
    return round256(rows * sizeof(float)) + (dtype == TT_ATTN_F32 ? 0 : round256(rows * D * sizeof(float)) + 256);
  }
  if (kind == TT_ATTN_KIND_DECODE_APPEND) {
    // the decode scratch; on the grouped-query tensor-core path also the rotated q and the new lengths
    const size_t base = tt_attn_workspace_bytes(TT_ATTN_KIND_DECODE, dtype, B, Hq, Hkv, Lq, Skv, D);
    DecodeArgs probe{};
    probe.Hq = Hq, probe.Hkv = Hkv;
    if (Skv <= 0 || !decode_tc_applies(dtype, D, probe)) return base;
    return base + round256(static_cast<size_t>(B) * Hq * D * elem_size(dtype)) + round256(static_cast<size_t>(B) * 4);
  }
  if (kind == TT_ATTN_KIND_DECODE) {
    if (Skv <= 0) return 0;
    int nsplit, chunk;
    decode_plan_for(dtype, D, B, Hq, Hkv, Skv, &nsplit, &chunk);
    // per-split partials, and for the tensor-core path (several query heads per kv head) a work counter
    DecodeArgs probe{};
    probe.Hq = Hq, probe.Hkv = Hkv;
    const size_t counter = decode_tc_applies(dtype, D, probe) ? 256 : 0;
    if (nsplit == 1) return counter;
    return round256(static_cast<size_t>(B) * Hq * nsplit * (D + 2) * sizeof(float)) + counter;
  }
  return 0;
}

int tt_attn_fwd(const tt_attn_fwd_params* p) {
  if (!p) return TT_ATTN_ERR_NULL;
  const bool v2 = p->struct_size == sizeof(tt_attn_fwd_params);
  if (!v2 && p->struct_size != offsetof(tt_attn_fwd_params, mask)) return TT_ATTN_ERR_STRUCT;
  if (int rc = check_common(p->dtype, p->B, p->Hq, p->Hkv, p->Lq, p->Skv, p->D)) return rc;
  if (!p->q || !p->k || !p->v || !p->o) return TT_ATTN_ERR_NULL;
  const size_t es = elem_size(p->dtype);
  FwdArgs a{};
  a.q = p->q, a.k = p->k, a.v = p->v, a.o = p->o, a.lse = p->lse;
  a.qs = dense_or(p->q_strides, p->Hq, p->Lq, p->D);
  a.ks = dense_or(p->k_strides, p->Hkv, p->Skv, p->D);
  a.vs = dense_or(p->v_strides, p->Hkv, p->Skv, p->D);
  a.os = dense_or(p->o_strides, p->Hq, p->Lq, p->D);
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->o) || !strides_ok(a.qs, es) ||
      !strides_ok(a.ks, es) || !strides_ok(a.vs, es) || !strides_ok(a.os, es))
    return TT_ATTN_ERR_ALIGN;
  a.B = p->B, a.Hq = p->Hq, a.Hkv = p->Hkv, a.Lq = p->Lq, a.Skv = p->Skv;
  if (p->is_causal < 0 || p->is_causal > TT_ATTN_CAUSAL_BOTTOM_RIGHT) return TT_ATTN_ERR_SHAPE;
  a.causal = p->is_causal;
  a.scale = p->scale;
  a.kv_lens = p->kv_lens;
  a.status = p->status;
  if (v2)
    if (int rc = take_mask(p->mask, p->mask_kind, p->mask_strides, &a.mask)) return rc;
  DeviceGuard guard(p->device);
  if (!guard.ok) return TT_ATTN_ERR_NO_DEVICE;
  Workspace ws;
  const size_t need = tt_attn_workspace_bytes(TT_ATTN_KIND_FWD, p->dtype, p->B, p->Hq, p->Hkv, p->Lq, p->Skv, p->D);
  if (int rc = ws.acquire(need, p->workspace, p->workspace_bytes, p->alloc, p->device)) return rc;
  a.sched = static_cast<int*>(ws.ptr);
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  cudaError_t e = p->dtype == TT_ATTN_F32 ? launch_fwd_simt(p->dtype, p->D, a, stream)
                                          : launch_fwd_tc(p->dtype, p->D, a, p->device, stream);
  return e == cudaSuccess ? TT_ATTN_OK : launch_failed(e);
}

int tt_attn_bwd(const tt_attn_bwd_params* p) {
  if (!p) return TT_ATTN_ERR_NULL;
  const bool v2 = p->struct_size == sizeof(tt_attn_bwd_params);
  if (!v2 && p->struct_size != offsetof(tt_attn_bwd_params, mask)) return TT_ATTN_ERR_STRUCT;
  if (int rc = check_common(p->dtype, p->B, p->Hq, p->Hkv, p->Lq, p->Skv, p->D)) return rc;
  if (!p->q || !p->k || !p->v || !p->o || !p->d_o || !p->lse) return TT_ATTN_ERR_NULL;
  if (!p->dq && !p->dk && !p->dv) return TT_ATTN_OK;
  const size_t es = elem_size(p->dtype);
  BwdArgs a{};
  a.q = p->q, a.k = p->k, a.v = p->v, a.o = p->o, a.d_o = p->d_o, a.lse = p->lse;
  a.dq = p->dq, a.dk = p->dk, a.dv = p->dv;
  a.qs = dense_or(p->q_strides, p->Hq, p->Lq, p->D);
  a.ks = dense_or(p->k_strides, p->Hkv, p->Skv, p->D);
  a.vs = dense_or(p->v_strides, p->Hkv, p->Skv, p->D);
  a.os = dense_or(p->o_strides, p->Hq, p->Lq, p->D);
  a.dos = dense_or(p->do_strides, p->Hq, p->Lq, p->D);
  a.dqs = dense_or(p->dq_strides, p->Hq, p->Lq, p->D);
  a.dks = dense_or(p->dk_strides, p->Hkv, p->Skv, p->D);
  a.dvs = dense_or(p->dv_strides, p->Hkv, p->Skv, p->D);
  const void* ptrs[] = {p->q, p->k, p->v, p->o, p->d_o, p->dq, p->dk, p->dv, p->lse};
  for (const void* q : ptrs)
    if (!aligned16(q)) return TT_ATTN_ERR_ALIGN;
  const Str3* sts[] = {&a.qs, &a.ks, &a.vs, &a.os, &a.dos, &a.dqs, &a.dks, &a.dvs};
  for (const Str3* s : sts)
    if (!strides_ok(*s, es)) return TT_ATTN_ERR_ALIGN;
  a.B = p->B, a.Hq = p->Hq, a.Hkv = p->Hkv, a.Lq = p->Lq, a.Skv = p->Skv;
  if (p->is_causal < 0 || p->is_causal > TT_ATTN_CAUSAL_BOTTOM_RIGHT) return TT_ATTN_ERR_SHAPE;
  a.causal = p->is_causal;
  a.scale = p->scale;
  a.kv_lens = p->kv_lens;
  a.status = p->status;
  if (v2)
    if (int rc = take_mask(p->mask, p->mask_kind, p->mask_strides, &a.mask)) return rc;
  DeviceGuard guard(p->device);
  if (!guard.ok) return TT_ATTN_ERR_NO_DEVICE;
  Workspace ws;
  const size_t need = tt_attn_workspace_bytes(TT_ATTN_KIND_BWD, p->dtype, p->B, p->Hq, p->Hkv, p->Lq, p->Skv, p->D);
  if (int rc = ws.acquire(need, p->workspace, p->workspace_bytes, p->alloc, p->device)) return rc;
  a.delta = static_cast<float*>(ws.ptr);
  a.dq_accum = reinterpret_cast<float*>(static_cast<char*>(ws.ptr) +
                                        round256(static_cast<size_t>(p->B) * p->Hq * p->Lq * sizeof(float)));
  a.sched = p->dtype == TT_ATTN_F32 ? nullptr : reinterpret_cast<int*>(static_cast<char*>(ws.ptr) + need - 256);
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  cudaError_t e = p->dtype == TT_ATTN_F32 ? launch_bwd_simt(p->dtype, p->D, a, stream)
                                          : launch_bwd_tc(p->dtype, p->D, a, p->device, stream);
  return e == cudaSuccess ? TT_ATTN_OK : launch_failed(e);
}

int tt_attn_decode(const tt_attn_decode_params* p) {
  if (!p) return TT_ATTN_ERR_NULL;
  if (p->struct_size != sizeof(tt_attn_decode_params)) return TT_ATTN_ERR_STRUCT;
  if (int rc = check_common(p->dtype, p->B, p->Hq, p->Hkv, 1, p->capacity, p->D)) return rc;
  if (!p->q || !p->k || !p->v || !p->o) return TT_ATTN_ERR_NULL;
  const size_t es = elem_size(p->dtype);
  DecodeArgs a{};
  a.q = p->q, a.k = p->k, a.v = p->v, a.o = p->o, a.lse = p->lse;
  a.qs = dense_or(p->q_strides, p->Hq, 1, p->D);
  a.ks = dense_or(p->k_strides, p->Hkv, p->capacity, p->D);
  a.vs = dense_or(p->v_strides, p->Hkv, p->capacity, p->D);
  a.os = dense_or(p->o_strides, p->Hq, 1, p->D);
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->o) || !strides_ok(a.qs, es) ||
      !strides_ok(a.ks, es) || !strides_ok(a.vs, es) || !strides_ok(a.os, es))
    return TT_ATTN_ERR_ALIGN;
  a.B = p->B, a.Hq = p->Hq, a.Hkv = p->Hkv, a.capacity = p->capacity;
  a.scale = p->scale;
  a.kv_lens = p->kv_lens;
  decode_plan_for(p->dtype, p->D, p->B, p->Hq, p->Hkv, p->capacity, &a.nsplit, &a.chunk);
  DeviceGuard guard(p->device);
  if (!guard.ok) return TT_ATTN_ERR_NO_DEVICE;
  Workspace ws;
  const size_t need =
      tt_attn_workspace_bytes(TT_ATTN_KIND_DECODE, p->dtype, p->B, p->Hq, p->Hkv, 1, p->capacity, p->D);
  if (int rc = ws.acquire(need, p->workspace, p->workspace_bytes, p->alloc, p->device)) return rc;
  a.partial = static_cast<float*>(ws.ptr);
  // the tensor-core path's work counter sits in the last 256 bytes (unused by the scan kernel)
  a.sched = need >= 256 ? reinterpret_cast<int*>(static_cast<char*>(ws.ptr) + need - 256) : nullptr;
  a.status = p->status;
  cudaError_t e = launch_decode(p->dtype, p->D, a, static_cast<cudaStream_t>(p->stream));
  return e == cudaSuccess ? TT_ATTN_OK : launch_failed(e);
}

int tt_attn_decode_append(const tt_attn_decode_append_params* p) {
  if (!p) return TT_ATTN_ERR_NULL;
  if (p->struct_size != sizeof(tt_attn_decode_append_params)) return TT_ATTN_ERR_STRUCT;
  if (int rc = check_common(p->dtype, p->B, p->Hq, p->Hkv, 1, p->capacity, p->D)) return rc;
  if (!p->q || !p->k_new || !p->v_new || !p->k_cache || !p->v_cache || !p->o || !p->kv_lens) return TT_ATTN_ERR_NULL;
  if ((p->rope_cos == nullptr) != (p->rope_sin == nullptr)) return TT_ATTN_ERR_NULL;
  if (p->rope_cos && p->rope_positions <= 0) return TT_ATTN_ERR_SHAPE;
  if (p->new_lens && p->new_lens == p->kv_lens) return TT_ATTN_ERR_SHAPE;
  const size_t es = elem_size(p->dtype);
  DecodeArgs a{};
  a.q = p->q, a.k = p->k_cache, a.v = p->v_cache, a.o = p->o, a.lse = p->lse;
  a.k_new = p->k_new, a.v_new = p->v_new;
  a.qs = dense_or(p->q_strides, p->Hq, 1, p->D);
  a.ks = dense_or(p->k_strides, p->Hkv, p->capacity, p->D);
  a.vs = dense_or(p->v_strides, p->Hkv, p->capacity, p->D);
  a.os = dense_or(p->o_strides, p->Hq, 1, p->D);
  const Str3 kn = dense_or(p->k_new_strides, p->Hkv, 1, p->D), vn = dense_or(p->v_new_strides, p->Hkv, 1, p->D);
  a.kn_b = kn.b, a.kn_h = kn.h, a.vn_b = vn.b, a.vn_h = vn.h;
  const void* ptrs[] = {p->q, p->k_new, p->v_new, p->k_cache, p->v_cache, p->o};
  for (const void* q : ptrs)
    if (!aligned16(q)) return TT_ATTN_ERR_ALIGN;
  const Str3* sts[] = {&a.qs, &a.ks, &a.vs, &a.os, &kn, &vn};
  for (const Str3* s : sts)
    if (!strides_ok(*s, es)) return TT_ATTN_ERR_ALIGN;
  a.B = p->B, a.Hq = p->Hq, a.Hkv = p->Hkv, a.capacity = p->capacity;
  a.scale = p->scale;
  a.kv_lens = p->kv_lens;
  a.new_lens = p->new_lens;
  a.rope_cos = p->rope_cos, a.rope_sin = p->rope_sin;
  a.rope_positions = p->rope_positions, a.rope_interleaved = p->rope_interleaved;
  a.status = p->status;
  decode_plan_for(p->dtype, p->D, p->B, p->Hq, p->Hkv, p->capacity, &a.nsplit, &a.chunk);
  DeviceGuard guard(p->device);
  if (!guard.ok) return TT_ATTN_ERR_NO_DEVICE;
  Workspace ws;
  const size_t base =
      tt_attn_workspace_bytes(TT_ATTN_KIND_DECODE, p->dtype, p->B, p->Hq, p->Hkv, 1, p->capacity, p->D);
  const size_t need =
      tt_attn_workspace_bytes(TT_ATTN_KIND_DECODE_APPEND, p->dtype, p->B, p->Hq, p->Hkv, 1, p->capacity, p->D);
  if (int rc = ws.acquire(need, p->workspace, p->workspace_bytes, p->alloc, p->device)) return rc;
  a.partial = static_cast<float*>(ws.ptr);
  a.sched = base >= 256 ? reinterpret_cast<int*>(static_cast<char*>(ws.ptr) + base - 256) : nullptr;
  if (need > base) {
    a.q_rot = static_cast<char*>(ws.ptr) + base;
    a.lens_scratch = reinterpret_cast<int32_t*>(static_cast<char*>(ws.ptr) + need - round256(static_cast<size_t>(p->B) * 4));
  }
  cudaError_t e = launch_decode_append(p->dtype, p->D, a, static_cast<cudaStream_t>(p->stream));
  return e == cudaSuccess ? TT_ATTN_OK : launch_failed(e);
}

int tt_attn_decode_static(const tt_attn_decode_params* p) {
  if (!p) return TT_ATTN_ERR_NULL;
  if (p->struct_size != sizeof(tt_attn_decode_params)) return TT_ATTN_ERR_STRUCT;
  if (int rc = check_common(p->dtype, p->B, p->Hq, p->Hkv, 1, p->capacity, p->D)) return rc;
  if (!p->q || !p->k || !p->v || !p->o) return TT_ATTN_ERR_NULL;
  const size_t es = elem_size(p->dtype);
  DecodeArgs a{};
  a.q = p->q, a.k = p->k, a.v = p->v, a.o = p->o, a.lse = p->lse;
  a.qs = dense_or(p->q_strides, p->Hq, 1, p->D);
  a.ks = dense_or(p->k_strides, p->Hkv, p->capacity, p->D);
  a.vs = dense_or(p->v_strides, p->Hkv, p->capacity, p->D);
  a.os = dense_or(p->o_strides, p->Hq, 1, p->D);
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->o) || !strides_ok(a.qs, es) ||
      !strides_ok(a.ks, es) || !strides_ok(a.vs, es) || !strides_ok(a.os, es))
    return TT_ATTN_ERR_ALIGN;
  a.B = p->B, a.Hq = p->Hq, a.Hkv = p->Hkv, a.capacity = p->capacity;
  a.scale = p->scale;
  a.kv_lens = p->kv_lens;
  a.status = p->status;
  decode_plan_for(p->dtype, p->D, p->B, p->Hq, p->Hkv, p->capacity, &a.nsplit, &a.chunk);
  const size_t need =
      tt_attn_workspace_bytes(TT_ATTN_KIND_DECODE, p->dtype, p->B, p->Hq, p->Hkv, 1, p->capacity, p->D);
  if (need > TT_ATTN_STATIC_SCRATCH_BYTES) return TT_ATTN_ERR_TOO_LARGE;
  DeviceGuard guard(p->device);
  if (!guard.ok) return TT_ATTN_ERR_NO_DEVICE;
  bool too_large = false;
  cudaError_t e =
      launch_decode_static(p->dtype, p->D, a, need, p->device, static_cast<cudaStream_t>(p->stream), &too_large);
  if (too_large) return TT_ATTN_ERR_TOO_LARGE;
  return e == cudaSuccess ? TT_ATTN_OK : launch_failed(e);
}

int tt_attn_selftest_wait_expiry(int device, void* stream, uint64_t limit_ns, int32_t* status,
                                 unsigned long long* waited_ns) {
  if (!status) return TT_ATTN_ERR_NULL;
  if (limit_ns == 0 || limit_ns > 2000000000ull) return TT_ATTN_ERR_SHAPE;  // the kernels' own limit is 2 s
  DeviceGuard guard(device);
  if (!guard.ok) return TT_ATTN_ERR_NO_DEVICE;
  cudaError_t e = launch_wait_expiry(status, limit_ns, waited_ns, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? TT_ATTN_OK : launch_failed(e);
}

int tt_fused_add_rms_norm(const tt_fused_add_rms_norm_params* p) {
  if (!p) return TT_ATTN_ERR_NULL;
  if (p->struct_size != sizeof(tt_fused_add_rms_norm_params)) return TT_ATTN_ERR_STRUCT;
  if (p->dtype < TT_ATTN_F32 || p->dtype > TT_ATTN_BF16) return TT_ATTN_ERR_DTYPE;
  if (p->rows < 0 || p->dim <= 0 || p->rows > 0x7fffffff) return TT_ATTN_ERR_SHAPE;
  if (p->rows == 0) return TT_ATTN_OK;  // an empty tensor has no storage to point to
  if (!p->input || !p->residual || !p->weight) return TT_ATTN_ERR_NULL;
  const size_t es = elem_size(p->dtype);
  if (reinterpret_cast<uintptr_t>(p->input) % es || reinterpret_cast<uintptr_t>(p->residual) % es ||
      reinterpret_cast<uintptr_t>(p->weight) % es)
    return TT_ATTN_ERR_ALIGN;
  DeviceGuard guard(p->device);
  if (!guard.ok) return TT_ATTN_ERR_NO_DEVICE;
  cudaError_t e = launch_fused_add_rms_norm(p->dtype, p->input, p->residual, p->weight, p->rows, p->dim, p->eps,
                                            static_cast<cudaStream_t>(p->stream));
  return e == cudaSuccess ? TT_ATTN_OK : launch_failed(e);
}

int tt_silu_mul(const tt_silu_mul_params* p) {
  if (!p) return TT_ATTN_ERR_NULL;
  if (p->struct_size != sizeof(tt_silu_mul_params)) return TT_ATTN_ERR_STRUCT;
  if (p->dtype < TT_ATTN_F32 || p->dtype > TT_ATTN_BF16) return TT_ATTN_ERR_DTYPE;
  if (p->rows < 0 || p->d <= 0) return TT_ATTN_ERR_SHAPE;
  if (p->rows == 0) return TT_ATTN_OK;
  if (!p->x || !p->out) return TT_ATTN_ERR_NULL;
  const size_t es = elem_size(p->dtype);
  if (reinterpret_cast<uintptr_t>(p->x) % es || reinterpret_cast<uintptr_t>(p->out) % es) return TT_ATTN_ERR_ALIGN;
  DeviceGuard guard(p->device);
  if (!guard.ok) return TT_ATTN_ERR_NO_DEVICE;
  cudaError_t e = launch_silu_mul(p->dtype, p->out, p->x, p->rows, p->d, static_cast<cudaStream_t>(p->stream));
  return e == cudaSuccess ? TT_ATTN_OK : launch_failed(e);
}

int tt_linear(const tt_linear_params* p) {
  if (!p) return TT_ATTN_ERR_NULL;
  if (p->struct_size != sizeof(tt_linear_params)) return TT_ATTN_ERR_STRUCT;
  if (p->dtype != TT_ATTN_F16 && p->dtype != TT_ATTN_BF16) return TT_ATTN_ERR_DTYPE;
  if (p->M < 0 || p->N <= 0 || p->K <= 0 || p->M > 0x7fffffff || p->N > 0x7fffffff || p->K > 0x7fffffff)
    return TT_ATTN_ERR_SHAPE;
  if (p->M == 0) return TT_ATTN_OK;
  if (!p->x || !p->w || !p->y) return TT_ATTN_ERR_NULL;
  const int64_t ldx = p->ldx ? p->ldx : p->K, ldw = p->ldw ? p->ldw : p->K, ldy = p->ldy ? p->ldy : p->N;
  if (ldx < p->K || ldw < p->K || ldy < p->N) return TT_ATTN_ERR_SHAPE;
  if (p->K % 8 || p->N % 8 || ldx % 8 || ldw % 8 || ldy % 8 || !aligned16(p->x) || !aligned16(p->w) ||
      !aligned16(p->y) || (p->bias && reinterpret_cast<uintptr_t>(p->bias) % 2))
    return TT_ATTN_ERR_ALIGN;
  DeviceGuard guard(p->device);
  if (!guard.ok) return TT_ATTN_ERR_NO_DEVICE;
  cudaError_t e = launch_linear_tc(p->dtype, p->x, p->w, p->bias, p->y, static_cast<int>(p->M), static_cast<int>(p->N),
                                   static_cast<int>(p->K), ldx, ldw, ldy, p->status, p->device,
                                   static_cast<cudaStream_t>(p->stream));
  return e == cudaSuccess ? TT_ATTN_OK : launch_failed(e);
}

}  // extern "C"
