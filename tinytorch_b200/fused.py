"""The reference's two hand-fused transformer-block operators on B200, with the
reference's names, argument meaning and in-place behaviour:

  siluMul(x)                                   op::siluMul, function::siluMul
      (src/Operation/OpFused.h:19, src/Function/FuncFused.h:14-19,31)
  fusedAddRmsNorm(input, residual, weight, eps)  op::fusedAddRmsNorm, function::fusedAddRmsNorm
      (src/Operation/OpFused.h:22, src/Function/FuncFused.h:21-28,33-35)

Both go through the C ABI of libtt_attn.so (include/tt_fused.h) and launch on the
current CUDA stream of the tensors' device.  Neither has a CPU implementation here,
and - as in the reference (FuncFused.h:18,27) - neither has a backward.
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
