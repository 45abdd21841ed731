"""Function layer: ``sdpAttention`` with the reference's signature and a working
backward.

Mirrors function::sdpAttention / FuncSDPAttention
(src/Function/FuncNNLayer.h:229-268, 298-302): same argument order and meaning
(query, key, value, isCausal, attnMask, dropoutP, scale), same default scale
1/sqrt(D), same top-left causal alignment, same assertion that isCausal and a
mask are mutually exclusive, same mask semantics (Bool: true = the key takes
part; otherwise added to the scaled scores; broadcast against [B, H, L, S],
src/Function/FuncNNLayer.h:249-256).  Differences, all forced by the fused path:
  * forward saves (O, LSE) for backward, as the reference's implemented
    backwards save what they need (AutogradContext::pushData,
    src/Tensor/Function.h:24-31);
  * backward exists (the reference traps, FuncNNLayer.h:267) and hands dQ, dK, dV
    to autograd, which accumulates them like AutogradMeta::addGrad
    (src/Tensor/AutogradMeta.cpp:29-43);
  * ``kvLens`` (int32 [B]) is the cheap form of the reference's per-batch length
    mask and may be combined with isCausal; isCausal may also be the string
    "bottom-right" (a chunk of new queries at the end of the keys);
  * a query row with no participating key gives O = 0 (the reference gives NaN);
  * the mask receives no gradient; dropoutP must be 0 (dropout stays on the
    reference's generic-op composition, which this package does not contain).
"""
import torch

from . import op


class FuncSDPAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, key, value, isCausal, kvLens, scale, attnMask=None):
        needs_grad = any(ctx.needs_input_grad[:3])
        o, lse = op.sdpAttentionFwd(query, key, value, isCausal, scale, kvLens, needLse=needs_grad, attnMask=attnMask)
        if needs_grad:
            ctx.save_for_backward(query, key, value, o, lse)
            ctx.isCausal, ctx.scale, ctx.kvLens, ctx.attnMask = isCausal, scale, kvLens, attnMask
        return o

    @staticmethod
    def backward(ctx, grad):
        query, key, value, o, lse = ctx.saved_tensors
        if grad.stride(3) != 1:
            grad = grad.contiguous()
        dq, dk, dv = op.sdpAttentionBwd(grad, query, key, value, o, lse, ctx.isCausal, ctx.scale, ctx.kvLens,
                                        needs=ctx.needs_input_grad[:3], attnMask=ctx.attnMask)
        return dq, dk, dv, None, None, None, None


def sdpAttention(query, key, value, isCausal=False, attnMask=None, dropoutP=0.0, scale=None, kvLens=None):
    """Drop-in for function::sdpAttention (src/Function/FuncNNLayer.h:298-302)."""
    if isCausal and attnMask is not None:
        raise AssertionError("isCausal and attnMask are mutually exclusive (FuncNNLayer.h:242)")
    if dropoutP > 0.0:
        raise NotImplementedError("dropoutP > 0 is not on the fused path")
    if scale is None:
        scale = op.default_scale(query.shape[-1])
    if not isinstance(isCausal, str):
        isCausal = bool(isCausal)
    if attnMask is not None:
        attnMask = attnMask.detach()
    return FuncSDPAttention.apply(query, key, value, isCausal, kvLens, float(scale), attnMask)
