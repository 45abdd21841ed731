/*
 * Header-only TinyTorch binding of libtt_attn.so.
 *
 * Compile this together with a CUDA-enabled TinyTorch build (USE_CUDA) and link
 * libtt_attn.so.  It adds, with TinyTorch's own mechanisms,
 *   - three dispatch-table ops (DEFINE_OP / REGISTER_OP_IMPL, src/Tensor/Dispatch.h:73-120):
 *       op::sdpAttentionFwd, op::sdpAttentionBwd, op::sdpAttentionDecode
 *     registered for CUDA x {Float32, Float16, BFloat16} from a STATIC_CALL
 *     initialiser (src/Utils/Macros.h:53-57), exactly like the built-in ops
 *     (e.g. src/Operation/OpNNLayerCuda.cu:11-36);
 *   - function::FuncSDPAttentionFused, the Function<> node with the same forward
 *     arguments as FuncSDPAttention (src/Function/FuncNNLayer.h:229-268) and the
 *     backward that class leaves as NOT_IMPLEMENTED();
 *   - function::sdpAttentionFused(query, key, value, isCausal, attnMask, dropoutP, scale),
 *     signature-identical to function::sdpAttention (src/Function/FuncNNLayer.h:298-302).
 *     Calls the fused path when it applies (CUDA tensors, D in {64,128}, no
 *     dropout, a mask that is absent or of a supported form) and otherwise forwards to the
 *     original composition.  Setting TINYTORCH_FUSED_ATTENTION=0 in the environment sends every
 *     call to the original composition (read once, at the first call): the switch for A/B runs.
 * Error convention: a non-zero status is logged with LOGE and then ASSERT(false)
 * fires, which is what every reference op does on failure (src/Utils/Macros.h:34-43).
 */
#pragma once

#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <optional>

#include "TinyTorch.h"
#include "Tensor/CachedAllocator.h"
#include "Utils/CUDAUtils.h"
#include "tt_attn.h"

namespace tinytorch {

namespace fused_detail {

inline void* hookAlloc(void*, size_t bytes, int device) {
  return getCUDACachedAllocator(device)->allocate(static_cast<int64_t>(bytes));
}
inline void hookFree(void*, void* ptr, int device) { getCUDACachedAllocator(device)->deallocate(ptr); }
inline const tt_attn_alloc_hook* allocHook() {
  static const tt_attn_alloc_hook hook = {&hookAlloc, &hookFree, nullptr};
  return &hook;
}

inline void check(int rc) {
  if (rc != TT_ATTN_OK) {
    LOGE("tt_attn: %s %s", tt_attn_strerror(rc), rc == TT_ATTN_ERR_LAUNCH ? tt_attn_last_cuda_error() : "");
    ASSERT(false && "tt_attn call failed");
  }
}

// Tensors are dense with an element storage offset (src/Tensor/TensorImpl.h:88-95),
// so the strides are the dense ones and only the base pointer may be offset.
inline tt_attn_strides denseStrides(const Tensor& t) {
  return tt_attn_strides{t.stride(0), t.stride(1), t.stride(2)};
}

// attnMask (src/Function/FuncNNLayer.h:249-256) runs fused when it is Bool, Float32 or the
// tensors' dtype, has at most 4 dimensions, spans all keys in its last dimension and
// broadcasts against [B, H, L, S] in the others.
inline bool maskApplicable(const Tensor& mask, const Tensor& q, const Tensor& k) {
  if (!mask.defined()) return true;
  if (mask.dim() < 1 || mask.dim() > 4 || mask.size(-1) != k.size(2)) return false;
  if (mask.dtype() != DType::Bool && mask.dtype() != DType::Float32 && mask.dtype() != q.dtype()) return false;
  const int64_t want[3] = {q.size(0), q.size(1), q.size(2)};
  for (int64_t i = 0; i < mask.dim() - 1; i++) {
    const int64_t have = mask.size(i), full = want[3 - (mask.dim() - 1) + i];
    if (have != 1 && have != full) return false;
  }
  return true;
}

// Fills the mask fields of a parameter struct (fwd and bwd share their names).
template <typename P>
inline void setMask(P& p, const Tensor& mask, const Tensor& /*q*/) {
  if (!mask.defined()) return;
  p.mask = mask.dataPtr<>();
  p.mask_kind = mask.dtype() == DType::Bool      ? TT_ATTN_MASK_BOOL
                : mask.dtype() == DType::Float32 ? TT_ATTN_MASK_ADD_F32
                                                 : TT_ATTN_MASK_ADD;  // the tensors' 16-bit dtype
  // trailing-dimension alignment (src/Tensor/TensorIterator.cpp:73-106); extent 1 broadcasts
  for (int64_t i = 0; i < mask.dim() - 1; i++)
    p.mask_strides[3 - (mask.dim() - 1) + i] = mask.size(i) == 1 ? 0 : mask.stride(i);
}

// TINYTORCH_FUSED_ATTENTION=0 turns the fused path off for the whole process.
inline bool fusedEnabled() {
  static const bool on = [] {
    const char* e = std::getenv("TINYTORCH_FUSED_ATTENTION");
    return !(e && e[0] == '0');
  }();
  return on;
}

// Calls that took the fused path so far (for tests and A/B runs).
inline std::atomic<long>& fusedCalls() {
  static std::atomic<long> n{0};
  return n;
}

// The kernels read 16-byte vectors and TMA tiles: a view whose storage offset breaks that
// alignment goes to the original composition instead of failing in the library.
inline bool aligned16(const Tensor& t) { return (reinterpret_cast<uintptr_t>(t.dataPtr<>()) & 15) == 0; }

inline bool applicable(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& mask, float dropoutP) {
  if (!fusedEnabled()) return false;
  if (!q.device().isCuda() || dropoutP > 0.f) return false;
  if (q.dim() == 4 && k.dim() == 4 && !maskApplicable(mask, q, k)) return false;
  if (q.dim() != 4 || k.dim() != 4 || v.dim() != 4) return false;
  if (q.dtype() != k.dtype() || q.dtype() != v.dtype()) return false;
  if (q.dtype() != DType::Float32 && q.dtype() != DType::Float16 && q.dtype() != DType::BFloat16) return false;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v)) return false;
  const auto D = q.size(-1);
  return (D == 64 || D == 128) && k.size(-1) == D && v.size(-1) == D && q.size(1) % k.size(1) == 0;
}

}  // namespace fused_detail

namespace op {

using SDPAttentionFwdOpFn = TensorPair (*)(const Tensor& q, const Tensor& k, const Tensor& v, bool isCausal,
                                           float scale, const Tensor& kvLens, const Tensor& mask);
using SDPAttentionBwdOpFn = TensorList (*)(const Tensor& dO, const Tensor& q, const Tensor& k, const Tensor& v,
                                           const Tensor& o, const Tensor& lse, bool isCausal, float scale,
                                           const Tensor& kvLens, const Tensor& mask);
using SDPAttentionDecodeOpFn = Tensor (*)(const Tensor& q, const Tensor& kCache, const Tensor& vCache,
                                          const Tensor& kvLens, float scale);

// one step of a token loop: rotary embedding of q / kNew at position kvLens[b], append of kNew / vNew to the
// caches (in place), attention over the appended cache; returns {O, kvLens + 1}
using SDPAttentionDecodeAppendOpFn = TensorPair (*)(const Tensor& q, const Tensor& kNew, const Tensor& vNew,
                                                    const Tensor& kCache, const Tensor& vCache, const Tensor& kvLens,
                                                    const Tensor& ropeCos, const Tensor& ropeSin, bool interleaved,
                                                    float scale);

DEFINE_OP(sdpAttentionFwd, SDPAttentionFwdOpFn)
DEFINE_OP(sdpAttentionDecodeAppend, SDPAttentionDecodeAppendOpFn)
DEFINE_OP(sdpAttentionBwd, SDPAttentionBwdOpFn)
DEFINE_OP(sdpAttentionDecode, SDPAttentionDecodeOpFn)

inline TensorPair sdpAttentionFwdCudaImpl(const Tensor& q, const Tensor& k, const Tensor& v, bool isCausal,
                                          float scale, const Tensor& kvLens, const Tensor& mask) {
  const int device = q.device().index;
  Tensor o(q.shape(), q.options().noGrad());
  Tensor lse({q.size(0), q.size(1), q.size(2)}, q.options().noGrad().dtype(DType::Float32));
  tt_attn_fwd_params p{};
  p.struct_size = sizeof(p);
  p.dtype = static_cast<int32_t>(q.dtype());  // enum values are the ABI (src/Tensor/DType.h:20-24)
  p.B = static_cast<int32_t>(q.size(0)), p.Hq = static_cast<int32_t>(q.size(1));
  p.Hkv = static_cast<int32_t>(k.size(1)), p.Lq = static_cast<int32_t>(q.size(2));
  p.Skv = static_cast<int32_t>(k.size(2)), p.D = static_cast<int32_t>(q.size(3));
  p.q = q.dataPtr<>(), p.k = k.dataPtr<>(), p.v = v.dataPtr<>(), p.o = o.dataPtr<>();
  p.lse = lse.dataPtr<float>();
  p.q_strides = fused_detail::denseStrides(q), p.k_strides = fused_detail::denseStrides(k);
  p.v_strides = fused_detail::denseStrides(v), p.o_strides = fused_detail::denseStrides(o);
  p.is_causal = isCausal ? 1 : 0;
  p.scale = scale;
  p.kv_lens = kvLens.defined() ? kvLens.dataPtr<int32_t>() : nullptr;
  fused_detail::setMask(p, mask, q);
  p.device = device;
  p.stream = cuda::getCurrentCUDAStream(device).stream();
  p.alloc = fused_detail::allocHook();
  fused_detail::check(tt_attn_fwd(&p));
  return {o, lse};
}

inline TensorList sdpAttentionBwdCudaImpl(const Tensor& dO, const Tensor& q, const Tensor& k, const Tensor& v,
                                          const Tensor& o, const Tensor& lse, bool isCausal, float scale,
                                          const Tensor& kvLens, const Tensor& mask) {
  const int device = q.device().index;
  Tensor dq(q.shape(), q.options().noGrad());
  Tensor dk(k.shape(), k.options().noGrad());
  Tensor dv(v.shape(), v.options().noGrad());
  tt_attn_bwd_params p{};
  p.struct_size = sizeof(p);
  p.dtype = static_cast<int32_t>(q.dtype());
  p.B = static_cast<int32_t>(q.size(0)), p.Hq = static_cast<int32_t>(q.size(1));
  p.Hkv = static_cast<int32_t>(k.size(1)), p.Lq = static_cast<int32_t>(q.size(2));
  p.Skv = static_cast<int32_t>(k.size(2)), p.D = static_cast<int32_t>(q.size(3));
  p.q = q.dataPtr<>(), p.k = k.dataPtr<>(), p.v = v.dataPtr<>(), p.o = o.dataPtr<>(), p.d_o = dO.dataPtr<>();
  p.lse = lse.dataPtr<float>();
  p.dq = dq.dataPtr<>(), p.dk = dk.dataPtr<>(), p.dv = dv.dataPtr<>();
  p.q_strides = fused_detail::denseStrides(q), p.k_strides = fused_detail::denseStrides(k);
  p.v_strides = fused_detail::denseStrides(v), p.o_strides = fused_detail::denseStrides(o);
  p.do_strides = fused_detail::denseStrides(dO), p.dq_strides = fused_detail::denseStrides(dq);
  p.dk_strides = fused_detail::denseStrides(dk), p.dv_strides = fused_detail::denseStrides(dv);
  p.is_causal = isCausal ? 1 : 0;
  p.scale = scale;
  p.kv_lens = kvLens.defined() ? kvLens.dataPtr<int32_t>() : nullptr;
  fused_detail::setMask(p, mask, q);
  p.device = device;
  p.stream = cuda::getCurrentCUDAStream(device).stream();
  p.alloc = fused_detail::allocHook();
  fused_detail::check(tt_attn_bwd(&p));
  return {dq, dk, dv};
}

inline Tensor sdpAttentionDecodeCudaImpl(const Tensor& q, const Tensor& kCache, const Tensor& vCache,
                                         const Tensor& kvLens, float scale) {
  const int device = q.device().index;
  ASSERT(q.size(2) == 1);
  Tensor o(q.shape(), q.options().noGrad());
  tt_attn_decode_params p{};
  p.struct_size = sizeof(p);
  p.dtype = static_cast<int32_t>(q.dtype());
  p.B = static_cast<int32_t>(q.size(0)), p.Hq = static_cast<int32_t>(q.size(1));
  p.Hkv = static_cast<int32_t>(kCache.size(1)), p.capacity = static_cast<int32_t>(kCache.size(2));
  p.D = static_cast<int32_t>(q.size(3));
  p.q = q.dataPtr<>(), p.k = kCache.dataPtr<>(), p.v = vCache.dataPtr<>(), p.o = o.dataPtr<>();
  p.q_strides = fused_detail::denseStrides(q), p.k_strides = fused_detail::denseStrides(kCache);
  p.v_strides = fused_detail::denseStrides(vCache), p.o_strides = fused_detail::denseStrides(o);
  p.scale = scale;
  p.kv_lens = kvLens.defined() ? kvLens.dataPtr<int32_t>() : nullptr;
  p.device = device;
  p.stream = cuda::getCurrentCUDAStream(device).stream();
  p.alloc = fused_detail::allocHook();
  fused_detail::check(tt_attn_decode(&p));
  return o;
}

inline TensorPair sdpAttentionDecodeAppendCudaImpl(const Tensor& q, const Tensor& kNew, const Tensor& vNew,
                                                   const Tensor& kCache, const Tensor& vCache, const Tensor& kvLens,
                                                   const Tensor& ropeCos, const Tensor& ropeSin, bool interleaved,
                                                   float scale) {
  const int device = q.device().index;
  ASSERT(q.size(2) == 1 && kNew.size(2) == 1 && vNew.size(2) == 1 && kvLens.defined());
  Tensor o(q.shape(), q.options().noGrad());
  Tensor newLens(kvLens.shape(), kvLens.options().noGrad());
  tt_attn_decode_append_params p{};
  p.struct_size = sizeof(p);
  p.dtype = static_cast<int32_t>(q.dtype());
  p.B = static_cast<int32_t>(q.size(0)), p.Hq = static_cast<int32_t>(q.size(1));
  p.Hkv = static_cast<int32_t>(kCache.size(1)), p.capacity = static_cast<int32_t>(kCache.size(2));
  p.D = static_cast<int32_t>(q.size(3));
  p.q = q.dataPtr<>(), p.k_new = kNew.dataPtr<>(), p.v_new = vNew.dataPtr<>();
  // the caches are updated in place (as the reference's *Inplace ops do through a const Tensor&)
  p.k_cache = const_cast<void*>(kCache.dataPtr<>()), p.v_cache = const_cast<void*>(vCache.dataPtr<>());
  p.o = o.dataPtr<>();
  p.q_strides = fused_detail::denseStrides(q), p.o_strides = fused_detail::denseStrides(o);
  p.k_new_strides = fused_detail::denseStrides(kNew), p.v_new_strides = fused_detail::denseStrides(vNew);
  p.k_strides = fused_detail::denseStrides(kCache), p.v_strides = fused_detail::denseStrides(vCache);
  p.scale = scale;
  p.kv_lens = kvLens.dataPtr<int32_t>();
  p.new_lens = newLens.dataPtr<int32_t>();
  if (ropeCos.defined()) {
    p.rope_cos = ropeCos.dataPtr<float>(), p.rope_sin = ropeSin.dataPtr<float>();
    p.rope_positions = static_cast<int32_t>(ropeCos.size(0));
  }
  p.rope_interleaved = interleaved ? 1 : 0;
  p.device = device;
  p.stream = cuda::getCurrentCUDAStream(device).stream();
  p.alloc = fused_detail::allocHook();
  fused_detail::check(tt_attn_decode_append(&p));
  return {o, newLens};
}

inline void registerFusedAttentionCuda() {
  const std::vector<DispatchDType> floats = {DispatchDType::Float32, DispatchDType::Float16, DispatchDType::BFloat16};
  REGISTER_OP_IMPL_MULTI(sdpAttentionFwd, {DispatchDevice::CUDA}, floats, &sdpAttentionFwdCudaImpl);
  REGISTER_OP_IMPL_MULTI(sdpAttentionBwd, {DispatchDevice::CUDA}, floats, &sdpAttentionBwdCudaImpl);
  REGISTER_OP_IMPL_MULTI(sdpAttentionDecode, {DispatchDevice::CUDA}, floats, &sdpAttentionDecodeCudaImpl);
  REGISTER_OP_IMPL_MULTI(sdpAttentionDecodeAppend, {DispatchDevice::CUDA}, floats, &sdpAttentionDecodeAppendCudaImpl);
}
STATIC_CALL(registerFusedAttentionCuda);

}  // namespace op

namespace function {

class FuncSDPAttentionFused : public Function<FuncSDPAttentionFused> {
 public:
  static Tensor forward(AutogradContext* ctx, const Tensor& query, const Tensor& key, const Tensor& value,
                        bool isCausal, const Tensor& attnMask, float dropoutP, std::optional<float> scale) {
    ASSERT(!(isCausal && attnMask.defined()) && dropoutP == 0.f);  // as src/Function/FuncNNLayer.h:242
    const float s = scale.has_value() ? scale.value() : (1.f / std::sqrt(static_cast<float>(query.size(-1))));
    fused_detail::fusedCalls()++;
    auto [o, lse] = op::sdpAttentionFwd(query, key, value, isCausal, s, Tensor{}, attnMask);
    if (ctx) {
      // savedInputs holds every Tensor argument in order: query, key, value, attnMask
      ctx->pushData(o);
      ctx->pushData(lse);
      ctx->pushData(isCausal);
      ctx->pushData(s);
    }
    return o;
  }

  static void backward(AutogradContext* ctx, const Tensor& grad) {
    auto& query = ctx->savedInputs[0];
    auto& key = ctx->savedInputs[1];
    auto& value = ctx->savedInputs[2];
    auto o = ctx->popData().toTensor();
    auto lse = ctx->popData().toTensor();
    const bool isCausal = ctx->popData().toBool();
    const float s = ctx->popData().toFloat();
    const Tensor mask = ctx->savedInputs.size() > 3 ? ctx->savedInputs[3] : Tensor{};
    // an upstream gradient that arrives as a misaligned view is copied once
    Tensor dO = grad;
    if (!fused_detail::aligned16(grad)) {
      dO = Tensor(grad.shape(), grad.options().noGrad());
      dO.copy_(grad);
    }
    auto grads = op::sdpAttentionBwd(dO, query, key, value, o, lse, isCausal, s, Tensor{}, mask);
    if (query.requiresGrad()) query.addGrad(std::move(grads[0]));
    if (key.requiresGrad()) key.addGrad(std::move(grads[1]));
    if (value.requiresGrad()) value.addGrad(std::move(grads[2]));
  }
};

inline Tensor sdpAttentionFused(const Tensor& query, const Tensor& key, const Tensor& value, bool isCausal = false,
                                const Tensor& attnMask = {}, float dropoutP = 0.f,
                                std::optional<float> scale = std::nullopt) {
  if (fused_detail::applicable(query, key, value, attnMask, dropoutP)) {
    return FuncSDPAttentionFused::apply(query, key, value, isCausal, attnMask, dropoutP, scale);
  }
  return FuncSDPAttention::apply(query, key, value, isCausal, attnMask, dropoutP, scale);
}

}  // namespace function
}  // namespace tinytorch
