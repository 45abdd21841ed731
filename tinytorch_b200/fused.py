"""The reference's two hand-fused transformer-block operators on B200, with the
reference's names, argument meaning and in-place behaviour:

  siluMul(x)                                   op::siluMul, function::siluMul
      (src/Operation/OpFused.h:19, src/Function/FuncFused.h:14-19,31)
  fusedAddRmsNorm(input, residual, weight, eps)  op::fusedAddRmsNorm, function::fusedAddRmsNorm
      (src/Operation/OpFused.h:22, src/Function/FuncFused.h:21-28,33-35)

  linear(input, weight, bias=None)            function::linear
      (src/Function/FuncNNLayer.h:14-35,270-272): input [..., K] x weight [N, K]^T + bias [N];
      float16 / bfloat16 on the tensor cores (float32 stays on the library gemm and is refused here),
      with the reference's backward (dX = dY W, dW = dY^T X, db = sum dY) through the same kernel

All go through the C ABI of libtt_attn.so (include/tt_fused.h) and launch on the
current CUDA stream of the tensors' device.  None has a CPU implementation here, and - as
in the reference (FuncFused.h:18,27) - siluMul and fusedAddRmsNorm have no backward.
"""
import ctypes as C

import torch

from . import _capi
from .op import _DTYPES


def _dev(t):
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def siluMul(x):
    """x [..., 2d] -> silu(x[..., :d]) * x[..., d:], a new tensor [..., d]."""
    if not x.is_cuda or x.dtype not in _DTYPES:
        raise ValueError("siluMul needs a CUDA tensor of dtype float32 / float16 / bfloat16 (no CPU path)")
    if x.shape[-1] % 2 != 0:
        raise AssertionError("last dimension must be even (OpFusedCpu.h:16)")
    x = x.contiguous()
    d = x.shape[-1] // 2
    out = torch.empty(x.shape[:-1] + (d,), dtype=x.dtype, device=x.device)
    p = _capi.SiluMulParams()
    p.struct_size = C.sizeof(_capi.SiluMulParams)
    p.dtype = _DTYPES[x.dtype]
    p.rows, p.d = x.numel() // (2 * d), d
    p.x, p.out = x.data_ptr(), out.data_ptr()
    p.device = _dev(x)
    p.stream = torch.cuda.current_stream(p.device).cuda_stream
    _capi.check(_capi.lib().tt_silu_mul(C.byref(p)))
    return out


def fusedAddRmsNorm(input, residual, weight, eps):
    """In place: residual += input; input = rmsnorm(residual) * weight.  Returns None, like the reference."""
    for t in (input, residual, weight):
        if not t.is_cuda or t.dtype != input.dtype or t.dtype not in _DTYPES:
            raise ValueError("fusedAddRmsNorm needs CUDA tensors of one dtype (float32 / float16 / bfloat16)")
    if input.shape != residual.shape:
        raise AssertionError("input and residual must have the same shape (OpFusedCpu.h:44)")
    if not (input.is_contiguous() and residual.is_contiguous() and weight.is_contiguous()):
        raise ValueError("fusedAddRmsNorm works in place on dense tensors")
    dim = input.shape[-1]
    if weight.numel() != dim:
        raise ValueError("weight must have input.size(-1) elements")
    p = _capi.AddRmsNormParams()
    p.struct_size = C.sizeof(_capi.AddRmsNormParams)
    p.dtype = _DTYPES[input.dtype]
    p.rows, p.dim = input.numel() // dim, dim
    p.input, p.residual, p.weight = input.data_ptr(), residual.data_ptr(), weight.data_ptr()
    p.eps = float(eps)
    p.device = _dev(input)
    p.stream = torch.cuda.current_stream(p.device).cuda_stream
    _capi.check(_capi.lib().tt_fused_add_rms_norm(C.byref(p)))


def _linear_raw(x2, w, bias, status=None):
    """x2 [M, K] @ w [N, K]^T (+ bias [N]) -> [M, N]; rows may be strided, columns are contiguous."""
    M, K = x2.shape
    N = w.shape[0]
    y = torch.empty((M, N), dtype=x2.dtype, device=x2.device)
    p = _capi.LinearParams()
    p.struct_size = C.sizeof(_capi.LinearParams)
    p.dtype = _DTYPES[x2.dtype]
    p.M, p.N, p.K = M, N, K
    p.x, p.w, p.y = x2.data_ptr(), w.data_ptr(), y.data_ptr()
    p.bias = bias.data_ptr() if bias is not None else None
    p.ldx, p.ldw, p.ldy = x2.stride(0), w.stride(0), N
    p.device = _dev(x2)
    p.stream = torch.cuda.current_stream(p.device).cuda_stream
    p.status = status.data_ptr() if status is not None else None
    _capi.check(_capi.lib().tt_linear(C.byref(p)))
    return y


def _check_linear(input, weight, bias):
    if not input.is_cuda or input.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("linear needs CUDA float16 / bfloat16 tensors (float32 stays on the library gemm; no CPU path)")
    if weight.dim() != 2 or weight.dtype != input.dtype or weight.device != input.device:
        raise ValueError("weight must be [N, K] with the dtype and device of input")
    if input.shape[-1] != weight.shape[1]:
        raise AssertionError("matmul error: shape not aligned (OpLinalg.cpp:251-254)")
    if bias is not None and (bias.dim() != 1 or bias.shape[0] != weight.shape[0] or bias.dtype != input.dtype):
        raise AssertionError("bias must be [N] (OpLinalg.cpp:261-263)")


class FuncLinear(torch.autograd.Function):
    """function::FuncLinear (src/Function/FuncNNLayer.h:14-35) on the tcgen05 kernel."""

    @staticmethod
    def forward(ctx, input, weight, bias):
        x2 = input.reshape(-1, input.shape[-1])
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        w = weight if weight.stride(1) == 1 else weight.contiguous()
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.in_shape = input.shape
        return _linear_raw(x2, w, bias).reshape(input.shape[:-1] + (weight.shape[0],))

    @staticmethod
    def backward(ctx, grad):
        x2, w = ctx.saved_tensors
        g2 = grad.reshape(-1, grad.shape[-1])
        if g2.stride(1) != 1:
            g2 = g2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            # dX[M,K] = dY[M,N] W[N,K] = dY (W^T)^T: the kernel contracts over the last dimension of both operands
            dx = _linear_raw(g2, w.t().contiguous(), None).reshape(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            # dW[N,K] = dY^T[N,M] X[M,K] = (dY^T) (X^T)^T
            dw = _linear_raw(g2.t().contiguous(), x2.t().contiguous(), None)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = g2.float().sum(0).to(grad.dtype)
        return dx, dw, db


def linear(input, weight, bias=None):
    """Drop-in for function::linear (src/Function/FuncNNLayer.h:270-272)."""
    _check_linear(input, weight, bias)
    return FuncLinear.apply(input, weight, bias)
