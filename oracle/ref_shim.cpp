/*
 * TEST INFRASTRUCTURE ONLY.  Thin extern "C" driver around the UNMODIFIED
 * reference sources (compiled where they lie by the Makefile in this
 * directory into _ref/libref_attn.so).  It exists so that the parity tests and
 * the CPU-baseline leg of the benchmark can call the reference's own CPU
 * implementation on raw float arrays.  The product path never loads it.
 *
 * What each entry point runs in the reference:
 *   ref_sdpa_fwd            function::sdpAttention      src/Function/FuncNNLayer.h:298-302
 *   ref_sdpa_grad           linear->mul->add->softmax->linear, .backward(dO)
 *                           src/Function/FuncNNLayer.h:14-35,
 *                           src/Function/FuncElemWise.h:71-124,
 *                           src/Function/FuncActivation.h:42-63
 *   ref_sdpa_fwd_mask       function::sdpAttention with an attnMask of any broadcastable
 *                           shape, Bool or Float32      src/Function/FuncNNLayer.h:249-256
 *   ref_silu_mul            op::siluMul                 src/Operation/OpFused.h:19, OpFusedCpu.h:14-39
 *   ref_fused_add_rms_norm  op::fusedAddRmsNorm         src/Operation/OpFused.h:22, OpFusedCpu.h:42-72
 *   ref_linear              function::linear            src/Function/FuncNNLayer.h:270-272
 *   ref_linear_grad         FuncLinear::backward        src/Function/FuncNNLayer.h:20-34
 *   ref_repeat_interleave   op::repeatInterleave        src/Operation/OpTransform.h:168
 *   ref_lse                 op::logSoftmax on the scaled, biased scores the
 *                           forward builds              src/Function/FuncNNLayer.h:237-260
 */
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#include "TinyTorch.h"

using namespace tinytorch;

namespace {

Tensor fromHost(const float* p, std::vector<int64_t> shape) {
  Tensor t = Tensor::empty(IntArrayView(shape), Options(Device(DeviceType::CPU), DType::Float32));
  std::memcpy(t.dataPtr<float>(), p, static_cast<size_t>(t.numel()) * sizeof(float));
  return t;
}

void toHost(const Tensor& t, float* p) {
  std::memcpy(p, t.dataPtr<float>(), static_cast<size_t>(t.numel()) * sizeof(float));
}

}  // namespace

extern "C" {

/* mask: NULL, or uint8 [B,1,1,S] with 1 = attend (the reference's boolean
 * mask convention).  scale <= 0 selects the reference default 1/sqrt(D). */
int ref_sdpa_fwd(const float* q, const float* k, const float* v, int64_t B, int64_t H, int64_t L, int64_t S,
                 int64_t D, int isCausal, const uint8_t* mask, float scale, float* out) {
  NoGradGuard guard;
  Tensor tq = fromHost(q, {B, H, L, D});
  Tensor tk = fromHost(k, {B, H, S, D});
  Tensor tv = fromHost(v, {B, H, S, D});
  Tensor tm;
  if (mask) {
    std::vector<int64_t> ms = {B, 1, 1, S};
    tm = Tensor::empty(IntArrayView(ms), Options(Device(DeviceType::CPU), DType::Bool));
    std::memcpy(tm.dataPtr<uint8_t>(), mask, static_cast<size_t>(B * S));
  }
  std::optional<float> sc = scale > 0.f ? std::optional<float>(scale) : std::nullopt;
  Tensor y = function::sdpAttention(tq, tk, tv, isCausal != 0, tm, 0.f, sc);
  toHost(y, out);
  return 0;
}

/* Gradients of the composed chain, one (b,h) slice at a time. */
int ref_sdpa_grad(const float* q, const float* k, const float* v, const float* dout, int64_t B, int64_t H,
                  int64_t L, int64_t S, int64_t D, int isCausal, float scale, float* out, float* dq, float* dk,
                  float* dv) {
  Options leaf = Options(Device(DeviceType::CPU), DType::Float32);
  for (int64_t u = 0; u < B * H; u++) {
    Tensor tq = fromHost(q + u * L * D, {L, D});
    Tensor tk = fromHost(k + u * S * D, {S, D});
    Tensor tvT;
    {
      NoGradGuard guard;
      tvT = op::transpose(fromHost(v + u * S * D, {S, D}), 0, 1);
    }
    tq.setRequiresGrad(true);
    tk.setRequiresGrad(true);
    tvT.setRequiresGrad(true);
    Tensor s = function::linear(tq, tk);
    s = function::mul(s, Tensor::scalar(scale, leaf));
    if (isCausal) {
      Tensor bias = Tensor::zeros({L, S}, leaf);
      Tensor keep = op::tril(Tensor::ones({L, S}, Options(Device(DeviceType::CPU), DType::Bool)), 0);
      op::fillMaskedInplace(bias, op::logicNot(keep), -std::numeric_limits<float>::infinity());
      s = function::add(s, bias);
    }
    Tensor p = function::softmax(s, -1);
    Tensor o = function::linear(p, tvT);
    if (out) toHost(o, out + u * L * D);
    o.backward(fromHost(dout + u * L * D, {L, D}));
    toHost(tq.grad(), dq + u * L * D);
    toHost(tk.grad(), dk + u * S * D);
    {
      NoGradGuard guard;
      toHost(op::transpose(tvT.grad(), 0, 1), dv + u * S * D);
    }
  }
  return 0;
}

int ref_repeat_interleave(const float* kv, int64_t B, int64_t Hkv, int64_t S, int64_t D, int64_t group,
                          float* out) {
  NoGradGuard guard;
  Tensor t = fromHost(kv, {B, Hkv, S, D});
  Tensor r = op::repeatInterleave(t, group, 1);
  toHost(r, out);
  return 0;
}

/* log-sum-exp of the scaled (and causally biased) scores, via logSoftmax:
 * lse_i = s_i0 - logSoftmax(s)_i0 (key 0 is never masked under causal). */
int ref_lse(const float* q, const float* k, int64_t B, int64_t H, int64_t L, int64_t S, int64_t D, int isCausal,
            float scale, float* lse) {
  NoGradGuard guard;
  Tensor tq = fromHost(q, {B, H, L, D});
  Tensor tk = fromHost(k, {B, H, S, D});
  Tensor w = op::matmul(tq, op::transpose(tk, -2, -1), false, false, Tensor{});
  op::mulInplace(w, Tensor::scalar(scale, w.options()));
  if (isCausal) {
    Tensor bias = Tensor::zeros({L, S}, w.options());
    Tensor keep = op::tril(Tensor::ones({L, S}, Options(Device(DeviceType::CPU), DType::Bool)), 0);
    op::fillMaskedInplace(bias, op::logicNot(keep), -std::numeric_limits<float>::infinity());
    op::addInplace(w, bias, 1);
  }
  Tensor ls = op::logSoftmax(w, -1);
  const float* wp = w.dataPtr<float>();
  const float* lp = ls.dataPtr<float>();
  for (int64_t r = 0; r < B * H * L; r++) lse[r] = wp[r * S] - lp[r * S];
  return 0;
}

/* sdpAttention(q, k, v, false, mask): mask is [m0,m1,m2,m3] (each extent 1 or the
 * full one), uint8 (1 = attend) when is_float == 0, else float added to the scores. */
int ref_sdpa_fwd_mask(const float* q, const float* k, const float* v, int64_t B, int64_t H, int64_t L, int64_t S,
                      int64_t D, const void* mask, int is_float, const int64_t* mshape, float scale, float* out) {
  NoGradGuard guard;
  Tensor tq = fromHost(q, {B, H, L, D});
  Tensor tk = fromHost(k, {B, H, S, D});
  Tensor tv = fromHost(v, {B, H, S, D});
  std::vector<int64_t> ms = {mshape[0], mshape[1], mshape[2], mshape[3]};
  Tensor tm;
  if (is_float) {
    tm = fromHost(static_cast<const float*>(mask), ms);
  } else {
    tm = Tensor::empty(IntArrayView(ms), Options(Device(DeviceType::CPU), DType::Bool));
    std::memcpy(tm.dataPtr<uint8_t>(), mask, static_cast<size_t>(tm.numel()));
  }
  std::optional<float> sc = scale > 0.f ? std::optional<float>(scale) : std::nullopt;
  Tensor y = function::sdpAttention(tq, tk, tv, false, tm, 0.f, sc);
  toHost(y, out);
  return 0;
}

/* x [rows, last] fp32 -> out [rows, last/2] */
int ref_silu_mul(const float* x, int64_t rows, int64_t last, float* out) {
  NoGradGuard guard;
  Tensor y = op::siluMul(fromHost(x, {rows, last}));
  toHost(y, out);
  return 0;
}

/* in place on input / residual [rows, dim] */
int ref_fused_add_rms_norm(float* input, float* residual, const float* weight, int64_t rows, int64_t dim, float eps) {
  NoGradGuard guard;
  Tensor ti = fromHost(input, {rows, dim});
  Tensor tr = fromHost(residual, {rows, dim});
  Tensor tw = fromHost(weight, {dim});
  op::fusedAddRmsNorm(ti, tr, tw, eps);
  toHost(ti, input);
  toHost(tr, residual);
  return 0;
}

/* y[M,N] = linear(x[M,K], w[N,K], bias[N] or NULL) */
int ref_linear(const float* x, const float* w, const float* bias, int64_t M, int64_t N, int64_t K, float* y) {
  NoGradGuard guard;
  Tensor tb = bias ? fromHost(bias, {N}) : Tensor{};
  Tensor ty = function::linear(fromHost(x, {M, K}), fromHost(w, {N, K}), tb);
  toHost(ty, y);
  return 0;
}

/* gradients of linear(x, w, bias) for an upstream gradient dy[M,N] */
int ref_linear_grad(const float* x, const float* w, const float* bias, const float* dy, int64_t M, int64_t N,
                    int64_t K, float* dx, float* dw, float* db) {
  Tensor tx = fromHost(x, {M, K}), tw = fromHost(w, {N, K}), tb = fromHost(bias, {N});
  tx.setRequiresGrad(true);
  tw.setRequiresGrad(true);
  tb.setRequiresGrad(true);
  Tensor ty = function::linear(tx, tw, tb);
  ty.backward(fromHost(dy, {M, N}));
  toHost(tx.grad(), dx);
  toHost(tw.grad(), dw);
  toHost(tb.grad(), db);
  return 0;
}

int ref_abi_version(void) { return 4; }

}  // extern "C"
