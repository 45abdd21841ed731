"""Function layer: ``sdpAttention`` with the reference's signature and a working
backward.

Mirrors function::sdpAttention / FuncSDPAttention
(src/Function/FuncNNLayer.h:229-268, 298-302): same argument order and meaning
(query, key, value, isCausal, attnMask, dropoutP, scale), same default scale
1/sqrt(D), same top-left causal alignment, same assertion that isCausal and a
mask are mutually exclusive.  Differences, all forced by the fused path:
  * forward saves (O, LSE) for backward, as the reference's implemented
    backwards save what they need (AutogradContext::pushData,
    src/Tensor/Function.h:24-31);
  * backward exists (the reference traps, FuncNNLayer.h:267) and hands dQ, dK, dV
    to autograd, which accumulates them like AutogradMeta::addGrad
    (src/Tensor/AutogradMeta.cpp:29-43);
  * the mask, when given, must be the per-batch length form ``kvLens`` (int32
    [B]); dropoutP must be 0.  Other masks and dropout stay on the reference's
    generic-op composition, which this package does not contain.
"""
import torch

from . import op


class FuncSDPAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, key, value, isCausal, kvLens, scale):
        needs_grad = any(ctx.needs_input_grad[:3])
        o, lse = op.sdpAttentionFwd(query, key, value, isCausal, scale, kvLens, needLse=needs_grad)
        if needs_grad:
            ctx.save_for_backward(query, key, value, o, lse)
            ctx.isCausal, ctx.scale, ctx.kvLens = isCausal, scale, kvLens
        return o

    @staticmethod
    def backward(ctx, grad):
        query, key, value, o, lse = ctx.saved_tensors
        if grad.stride(3) != 1:
            grad = grad.contiguous()
        dq, dk, dv = op.sdpAttentionBwd(grad, query, key, value, o, lse, ctx.isCausal, ctx.scale, ctx.kvLens,
                                        needs=ctx.needs_input_grad[:3])
        return dq, dk, dv, None, None, None


def sdpAttention(query, key, value, isCausal=False, attnMask=None, dropoutP=0.0, scale=None, kvLens=None):
    """Drop-in for function::sdpAttention (src/Function/FuncNNLayer.h:298-302)."""
    if isCausal and attnMask is not None:
        raise AssertionError("isCausal and attnMask are mutually exclusive (FuncNNLayer.h:242)")
    if attnMask is not None:
        raise NotImplementedError("only causal and per-batch length (kvLens) masks run on the fused path")
    if dropoutP > 0.0:
        raise NotImplementedError("dropoutP > 0 is not on the fused path")
    if scale is None:
        scale = op.default_scale(query.shape[-1])
    return FuncSDPAttention.apply(query, key, value, bool(isCausal), kvLens, float(scale))
