/*
 * tt_attn.h - C ABI of libtt_attn.so: fused scaled-dot-product attention for
 * NVIDIA B200 (sm_100a).  Forward (prefill), single-token decode against a KV
 * cache, and the training backward.
 *
 * This is the launch layer a TinyTorch build binds in place of the generic-op
 * composition inside FuncSDPAttention::forward (src/Function/FuncNNLayer.h:231-266)
 * and of the unimplemented FuncSDPAttention::backward (src/Function/FuncNNLayer.h:267).
 *
 * Conventions shared by every entry point
 *  - Tensors are the reference's dense row-major layout [B, H, S, D] with D
 *    innermost and contiguous (src/Tensor/TensorImpl.cpp:13-31).  The strides of
 *    the three outer dimensions are passed explicitly, in ELEMENTS, so that a
 *    KV cache with capacity > valid length and head-sharded sub-views work; a
 *    stride triple of all zeros means "dense".
 *  - dtype uses the reference's enum values (src/Tensor/DType.h:20-24):
 *    0 = Float32, 1 = Float16, 2 = BFloat16.  Q, K, V, O (and dO, dQ, dK, dV)
 *    share one dtype.  Accumulation is always fp32.  LSE is fp32.
 *  - is_causal = 1 keeps key j for query i iff j <= i, top-left aligned for any
 *    Lq, Skv (src/Function/FuncNNLayer.h:243-246, src/Operation/OpTransformCpu.h:204).
 *    is_causal = 2 (no counterpart in the reference) aligns the triangle to the
 *    bottom right instead: j <= i + (len_b - Lq) with len_b = kv_lens[b] or Skv,
 *    which is what a chunk of Lq new queries at the end of a cache of len_b keys needs.
 *  - mask (optional, prefill forward and backward) is the reference's attnMask
 *    (src/Function/FuncNNLayer.h:249-256): a boolean mask (one byte per element,
 *    non-zero = the key participates) or an additive mask added to the scaled
 *    scores, broadcast against [B, Hq, Lq, Skv].  The key dimension is contiguous;
 *    the strides of (b, h, l) are given in elements and 0 broadcasts that
 *    dimension.  The mask receives no gradient.  It may be combined with
 *    is_causal and kv_lens (the reference allows only one of mask / isCausal,
 *    src/Function/FuncNNLayer.h:242).
 *  - scale multiplies Q.K^T before the softmax; the caller passes 1/sqrt(D) when
 *    the user gave none (src/Function/FuncNNLayer.h:235).
 *  - kv_lens (optional, device int32 [B]): key j of batch b participates iff
 *    j < kv_lens[b]; this is the reference's boolean mask [B,1,1,S] with
 *    mask[b,0,0,j] = (j < len_b) (src/Function/FuncNNLayer.h:249-252).  Cache
 *    rows at or beyond the length are never used in the result, but must hold
 *    finite values in the prefill path (they may be multiplied by an exact 0).
 *  - A query row with no participating key yields O = 0 and LSE = -inf (the
 *    reference yields NaN there, src/Operation/OpNNLayerCpu.h:28-54).
 *  - Grouped-query attention: Hq must be a multiple of Hkv; query head h reads
 *    kv head h / (Hq/Hkv), which equals op::repeatInterleave(kv, group, 1)
 *    (src/Operation/OpTransformCpu.h:399-442) without materialising the copy.
 *  - All work is enqueued on `stream` of `device`; no entry point synchronises
 *    the host, allocates device memory itself, or aborts.  Scratch memory comes
 *    from `workspace` (>= tt_attn_workspace_bytes) or, when that is NULL, from
 *    the allocator hook, which the TinyTorch shim backs with
 *    getCUDACachedAllocator(device) (src/Tensor/Allocator.cpp:117-139); blocks
 *    are handed back through the hook as soon as the last launch is enqueued,
 *    the stream-ordered reuse the reference itself relies on
 *    (src/Operation/OpNNLayerCuda.cuh:415-429).
 *  - Return value: 0 on success, a negative tt_attn_status otherwise (the
 *    reference has no return codes: its ops LOGE + trap, src/Utils/Macros.h:25;
 *    the shim turns a non-zero code into exactly that).
 *  - Every device-side wait in the kernels is bounded.  If one expires the
 *    kernel stores a non-zero word to `status` (optional device int32) and
 *    returns early; the output of that call is then undefined.
 */
#ifndef TT_ATTN_H_
#define TT_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TT_ATTN_ABI_VERSION 2

#if defined(__GNUC__)
#define TT_ATTN_API __attribute__((visibility("default")))
#else
#define TT_ATTN_API
#endif

enum tt_attn_dtype { TT_ATTN_F32 = 0, TT_ATTN_F16 = 1, TT_ATTN_BF16 = 2 };

enum tt_attn_status {
  TT_ATTN_OK = 0,
  TT_ATTN_ERR_NULL = -1,        /* a required pointer is NULL */
  TT_ATTN_ERR_DTYPE = -2,       /* dtype not 0/1/2 */
  TT_ATTN_ERR_SHAPE = -3,       /* non-positive dimension, Hq % Hkv != 0, Lq != 1 in decode ... */
  TT_ATTN_ERR_HEAD_DIM = -4,    /* D not in {64, 128} */
  TT_ATTN_ERR_ALIGN = -5,       /* pointer or stride not 16-byte aligned */
  TT_ATTN_ERR_WORKSPACE = -6,   /* workspace too small / hook returned NULL / no hook */
  TT_ATTN_ERR_LAUNCH = -7,      /* CUDA reported an error at launch (message: tt_attn_last_cuda_error) */
  TT_ATTN_ERR_STRUCT = -8,      /* struct_size does not match this library */
  TT_ATTN_ERR_NO_DEVICE = -9,   /* device index invalid or driver entry point unavailable */
  TT_ATTN_ERR_TOO_LARGE = -10   /* size beyond a documented fixed limit */
};

/* Workspace allocator hook; replaces direct cudaMalloc so that the reference's
 * caching allocator (src/Tensor/CachedAllocator.cpp:408-416) stays the only
 * owner of device memory. */
typedef struct tt_attn_alloc_hook {
  void* (*alloc)(void* ctx, size_t bytes, int device);
  void (*free)(void* ctx, void* ptr, int device);
  void* ctx;
} tt_attn_alloc_hook;

enum tt_attn_causal { TT_ATTN_CAUSAL_NONE = 0, TT_ATTN_CAUSAL_TOP_LEFT = 1, TT_ATTN_CAUSAL_BOTTOM_RIGHT = 2 };

enum tt_attn_mask_kind {
  TT_ATTN_MASK_NONE = 0,
  TT_ATTN_MASK_BOOL = 1,    /* uint8, non-zero = participate (the reference's Bool tensor) */
  TT_ATTN_MASK_ADD = 2,     /* additive, same dtype as q (the reference adds a mask of the tensors' dtype) */
  TT_ATTN_MASK_ADD_F32 = 3  /* additive, fp32 */
};

/* Strides in elements of dimensions (b, h, s); D is contiguous. */
typedef struct tt_attn_strides {
  int64_t b, h, s;
} tt_attn_strides;

/* Forward.  Replaces FuncSDPAttention::forward (src/Function/FuncNNLayer.h:231-266)
 * for dropoutP == 0. */
typedef struct tt_attn_fwd_params {
  uint32_t struct_size; /* sizeof(tt_attn_fwd_params) */
  int32_t dtype;
  int32_t B, Hq, Hkv, Lq, Skv, D;
  const void* q;  /* [B, Hq,  Lq,  D] */
  const void* k;  /* [B, Hkv, Skv, D] */
  const void* v;  /* [B, Hkv, Skv, D] */
  void* o;        /* [B, Hq,  Lq,  D] */
  float* lse;     /* [B, Hq, Lq] dense fp32, natural log; may be NULL */
  tt_attn_strides q_strides, k_strides, v_strides, o_strides;
  int32_t is_causal;
  float scale;
  const int32_t* kv_lens; /* device [B] or NULL */
  int32_t device;
  void* stream; /* cudaStream_t */
  void* workspace;
  size_t workspace_bytes;
  const tt_attn_alloc_hook* alloc;
  int32_t* status; /* device word, may be NULL */
  /* fields below were added with TT_ATTN_ABI_VERSION 2; a caller compiled against
   * version 1 passes the shorter struct_size and gets "no mask" */
  const void* mask;        /* device pointer or NULL */
  int32_t mask_kind;       /* tt_attn_mask_kind */
  int32_t reserved0;       /* must be 0 */
  int64_t mask_strides[3]; /* elements, for (b, h, l); 0 = broadcast; keys are contiguous */
} tt_attn_fwd_params;

/* Backward.  Supplies what FuncSDPAttention::backward (src/Function/FuncNNLayer.h:267)
 * leaves unimplemented; gradients equal those of the reference's differentiable
 * chain linear->mul->add->softmax->linear (src/Function/FuncNNLayer.h:14-35,
 * src/Function/FuncElemWise.h:71-124, src/Function/FuncActivation.h:42-63).
 * o and lse are the forward's outputs.  dq/dk/dv are overwritten (the caller
 * accumulates into .grad(), src/Tensor/AutogradMeta.cpp:29-43); any of the
 * three may be NULL to skip it. */
typedef struct tt_attn_bwd_params {
  uint32_t struct_size;
  int32_t dtype;
  int32_t B, Hq, Hkv, Lq, Skv, D;
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* d_o;
  const float* lse; /* [B, Hq, Lq] */
  void* dq;         /* [B, Hq,  Lq,  D] */
  void* dk;         /* [B, Hkv, Skv, D] */
  void* dv;         /* [B, Hkv, Skv, D] */
  tt_attn_strides q_strides, k_strides, v_strides, o_strides, do_strides, dq_strides, dk_strides, dv_strides;
  int32_t is_causal;
  float scale;
  const int32_t* kv_lens;
  int32_t device;
  void* stream;
  void* workspace;
  size_t workspace_bytes;
  const tt_attn_alloc_hook* alloc;
  int32_t* status;
  /* fields below were added with TT_ATTN_ABI_VERSION 2; a caller compiled against
   * version 1 passes the shorter struct_size and gets "no mask" */
  const void* mask;        /* device pointer or NULL */
  int32_t mask_kind;       /* tt_attn_mask_kind */
  int32_t reserved0;       /* must be 0 */
  int64_t mask_strides[3]; /* elements, for (b, h, l); 0 = broadcast; keys are contiguous */
} tt_attn_bwd_params;

/* Single-token decode: Lq == 1, one query per sequence against a KV cache
 * [B, Hkv, capacity, D] of which the first kv_lens[b] rows are valid.  The
 * reference can only express this as sdpAttention(q, Kc, Vc, false, boolmask)
 * (src/Function/FuncNNLayer.h:249-252, 298-302). */
typedef struct tt_attn_decode_params {
  uint32_t struct_size;
  int32_t dtype;
  int32_t B, Hq, Hkv, capacity, D;
  const void* q;  /* [B, Hq, 1, D] */
  const void* k;  /* [B, Hkv, capacity, D] */
  const void* v;
  void* o;        /* [B, Hq, 1, D] */
  float* lse;     /* [B, Hq] or NULL */
  tt_attn_strides q_strides, k_strides, v_strides, o_strides;
  float scale;
  const int32_t* kv_lens; /* device [B]; NULL means every row of the cache is valid */
  int32_t device;
  void* stream;
  void* workspace;
  size_t workspace_bytes;
  const tt_attn_alloc_hook* alloc;
  int32_t* status;
} tt_attn_decode_params;

/* One decode step of a token loop, fused (no counterpart in the reference, which has
 * neither a KV cache object nor rotary embeddings; its consumer keeps the cache as
 * plain tensors and would run these as separate ops before sdpAttention):
 *   1. rotary position embedding of q and of the step's new key at position
 *      p_b = kv_lens[b] (skipped when rope_cos is NULL);
 *   2. the rotated key and the new value are written to row p_b of the caches;
 *   3. attention of the rotated q over rows [0, p_b] as tt_attn_decode does.
 * rope_cos / rope_sin are fp32 tables [rope_positions, D/2]; pair i of a row at
 * position p turns by the angle whose cosine and sine are table[p][i].  The pairs
 * are elements (i, i + D/2), or (2i, 2i+1) when rope_interleaved is non-zero.
 * new_lens (optional, may not alias kv_lens) receives kv_lens[b] + 1.  A sequence
 * whose cache is full (kv_lens[b] >= capacity) appends nothing, attends over the
 * whole cache and sets bit 4 of *status; a position beyond the tables skips the
 * rotation and sets bit 8. */
typedef struct tt_attn_decode_append_params {
  uint32_t struct_size;
  int32_t dtype;
  int32_t B, Hq, Hkv, capacity, D;
  const void* q;      /* [B, Hq, 1, D] */
  const void* k_new;  /* [B, Hkv, 1, D] */
  const void* v_new;  /* [B, Hkv, 1, D] */
  void* k_cache;      /* [B, Hkv, capacity, D]; row kv_lens[b] is written */
  void* v_cache;
  void* o;            /* [B, Hq, 1, D] */
  float* lse;         /* [B, Hq] or NULL */
  tt_attn_strides q_strides, k_new_strides, v_new_strides, k_strides, v_strides, o_strides;
  float scale;
  const int32_t* kv_lens; /* device [B], required: valid rows before this step */
  int32_t* new_lens;      /* device [B] or NULL */
  const float* rope_cos;  /* device [rope_positions, D/2] or NULL */
  const float* rope_sin;
  int32_t rope_positions;
  int32_t rope_interleaved;
  int32_t device;
  void* stream;
  void* workspace; /* tt_attn_workspace_bytes(TT_ATTN_KIND_DECODE_APPEND, ...) */
  size_t workspace_bytes;
  const tt_attn_alloc_hook* alloc;
  int32_t* status;
} tt_attn_decode_append_params;

enum tt_attn_kind {
  TT_ATTN_KIND_FWD = 0,
  TT_ATTN_KIND_BWD = 1,
  TT_ATTN_KIND_DECODE = 2,
  TT_ATTN_KIND_DECODE_APPEND = 3 /* tt_attn_decode_append: the decode scratch, plus a rotated copy of q and the
                                    new lengths when the grouped-query tensor-core path is taken */
};

TT_ATTN_API int tt_attn_fwd(const tt_attn_fwd_params* p);
TT_ATTN_API int tt_attn_bwd(const tt_attn_bwd_params* p);
TT_ATTN_API int tt_attn_decode(const tt_attn_decode_params* p);
TT_ATTN_API int tt_attn_decode_append(const tt_attn_decode_append_params* p);

/* Decode for callers that cannot give this library any device memory: hosts
 * where an embedding runtime owns the whole device heap and offers neither an
 * allocator callback nor a spare buffer, and token loops that must not touch an
 * allocator at all (cudaMalloc takes a process-wide lock and may synchronise the
 * device).  Same arguments and result as tt_attn_decode, but `workspace`,
 * `workspace_bytes` and `alloc` are ignored and neither this call nor anything
 * it uses allocates or frees memory: the per-split partial results go to a fixed
 * TT_ATTN_STATIC_SCRATCH_BYTES array inside the library image (resident on every
 * GPU that loads the library, until the process exits).
 *  - A problem whose tt_attn_workspace_bytes(TT_ATTN_KIND_DECODE, ...) exceeds
 *    TT_ATTN_STATIC_SCRATCH_BYTES is refused with TT_ATTN_ERR_TOO_LARGE.
 *  - The first call on each device looks up the array's device address (once,
 *    with that device current); make that first call before starting any stream
 *    capture.
 *  - All calls on a device share the one array; calls that overlap in time on the
 *    same GPU race on it, so keep them on one stream or otherwise ordered.  It is
 *    never cleared as a whole: every launch writes what it later reads, and the one
 *    4-byte work counter that grouped-query shapes use is reset by a memset enqueued
 *    on the call's stream.
 * This entry point has no counterpart in the reference. */
#define TT_ATTN_STATIC_SCRATCH_BYTES (24u << 20)
TT_ATTN_API int tt_attn_decode_static(const tt_attn_decode_params* p);

/* Self-test of the bounded device-side waits: launches one CTA that waits `limit_ns` nanoseconds
 * (1 .. 2e9) on a barrier nothing arrives on.  The kernel returns by itself, ORs status bit 1
 * (a wait expired) into *status (device memory, required) and, if `waited_ns` (device memory) is
 * given, stores how long the wait lasted.  Enqueues on `stream` like every other entry point.
 * For tests of a host's handling of the status word; it has no counterpart in the reference. */
TT_ATTN_API int tt_attn_selftest_wait_expiry(int device, void* stream, uint64_t limit_ns, int32_t* status,
                                             unsigned long long* waited_ns);

/* Scratch bytes the given call needs (0 if none; the fp16/bf16 forward needs a
 * 256-byte block for its work counter).  Skv is the cache capacity
 * for TT_ATTN_KIND_DECODE. */
TT_ATTN_API size_t tt_attn_workspace_bytes(int kind, int dtype, int B, int Hq, int Hkv, int Lq, int Skv, int D);

TT_ATTN_API const char* tt_attn_strerror(int status);
/* Text of the CUDA error behind the calling thread's last TT_ATTN_ERR_LAUNCH. */
TT_ATTN_API const char* tt_attn_last_cuda_error(void);
TT_ATTN_API int tt_attn_version(void);

#ifdef __cplusplus
}
#endif
#endif /* TT_ATTN_H_ */
