"""Operator layer: the three attention ops a TinyTorch build registers in its
dispatch tables (reference mechanism: DEFINE_OP / REGISTER_OP_IMPL,
src/Tensor/Dispatch.h:21-142), here bound to torch tensors used purely as
device-memory handles.  Every op goes through the C ABI of libtt_attn.so and
launches on the current CUDA stream of the tensors' device, as reference ops do
(src/Utils/CUDAUtils.cpp:123-135).  No op has a CPU implementation.
"""
import ctypes as C
import math

import torch

from . import _capi

_DTYPES = {torch.float32: _capi.F32, torch.float16: _capi.F16, torch.bfloat16: _capi.BF16}


def _alloc_cb(ctx, nbytes, device):
    return torch.cuda.caching_allocator_alloc(nbytes, device, torch.cuda.current_stream(device))


def _free_cb(ctx, ptr, device):
    torch.cuda.caching_allocator_delete(ptr)


# Workspace hook backed by torch's caching allocator: the stand-in for the
# reference's getCUDACachedAllocator(device) (src/Tensor/Allocator.cpp:117-139).
_HOOK = _capi.AllocHook(_capi.ALLOC_FN(_alloc_cb), _capi.FREE_FN(_free_cb), None)


def _check_tensor(t, name):
    if not t.is_cuda:
        raise ValueError("%s must be a CUDA tensor (this op has no CPU path)" % name)
    if t.dim() != 4:
        raise ValueError("%s must be [B, H, S, D]" % name)
    if t.stride(3) != 1:
        raise ValueError("%s: innermost dimension must be contiguous" % name)
    if t.dtype not in _DTYPES:
        raise ValueError("%s: dtype %s not supported" % (name, t.dtype))


def _strides(t):
    return _capi.Strides(t.stride(0), t.stride(1), t.stride(2))


def _common(p, ref):
    dev = ref.device.index if ref.device.index is not None else torch.cuda.current_device()
    p.device = dev
    p.stream = torch.cuda.current_stream(dev).cuda_stream
    p.workspace = None
    p.workspace_bytes = 0
    p.alloc = C.pointer(_HOOK)
    p.status = None


def _causal_mode(isCausal):
    """False/True as in the reference (top-left aligned triangle), or the string
    "bottom-right" for a chunk of new queries at the end of the key sequence."""
    if isCausal == "bottom-right":
        return _capi.CAUSAL_BOTTOM_RIGHT
    if isCausal in ("top-left", True, 1):
        return _capi.CAUSAL_TOP_LEFT
    if isCausal in (False, None, 0):
        return _capi.CAUSAL_NONE
    raise ValueError("isCausal must be a bool or 'top-left' / 'bottom-right'")


def _set_mask(p, mask, q, L, S):
    """attnMask of the reference (src/Function/FuncNNLayer.h:249-256): Bool -> keys that
    participate, otherwise added to the scaled scores; any shape that broadcasts against
    [B, Hq, L, S] by trailing-dimension alignment.  Returns the tensor to keep alive."""
    if mask is None:
        return None
    if not mask.is_cuda or mask.device != q.device:
        raise ValueError("attnMask must be on the device of q")
    if mask.dim() > 4:
        raise ValueError("attnMask has more than 4 dimensions")
    m = mask.reshape((1,) * (4 - mask.dim()) + tuple(mask.shape))
    B, Hq = q.shape[0], q.shape[1]
    for have, want in zip(m.shape, (B, Hq, L, S)):
        if have != want and have != 1:
            raise ValueError("attnMask shape %s does not broadcast against %s" % (tuple(mask.shape), (B, Hq, L, S)))
    if m.dtype == torch.bool:
        m = m.view(torch.uint8)
        kind = _capi.MASK_BOOL
    elif m.dtype == q.dtype and q.dtype != torch.float32:
        kind = _capi.MASK_ADD
    else:
        m = m.to(torch.float32)
        kind = _capi.MASK_ADD_F32
    if m.shape[3] != S or m.stride(3) != 1:
        # keys must be contiguous in memory; a mask broadcast over keys is expanded
        m = m.expand(m.shape[0], m.shape[1], m.shape[2], S).contiguous()
    p.mask = m.data_ptr()
    p.mask_kind = kind
    for i in range(3):
        p.mask_strides[i] = 0 if m.shape[i] == 1 else m.stride(i)
    return m


def default_scale(D):
    """1/sqrt(D) in fp32, the reference default (src/Function/FuncNNLayer.h:235)."""
    return 1.0 / math.sqrt(float(D))


def sdpAttentionFwd(q, k, v, isCausal=False, scale=None, kvLens=None, needLse=True, status=None, attnMask=None):
    """softmax(scale * Q K^T + bias) V  ->  (O [B,Hq,L,D], LSE [B,Hq,L] fp32 or None)."""
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_tensor(t, n)
    if not (q.dtype == k.dtype == v.dtype and q.device == k.device == v.device):
        raise ValueError("q, k, v must share dtype and device")
    B, Hq, L, D = q.shape
    _, Hkv, S, _ = k.shape
    o = torch.empty((B, Hq, L, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, L), dtype=torch.float32, device=q.device) if needLse else None
    p = _capi.FwdParams()
    p.struct_size = C.sizeof(_capi.FwdParams)
    p.dtype = _DTYPES[q.dtype]
    p.B, p.Hq, p.Hkv, p.Lq, p.Skv, p.D = B, Hq, Hkv, L, S, D
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.q_strides, p.k_strides, p.v_strides, p.o_strides = _strides(q), _strides(k), _strides(v), _strides(o)
    p.is_causal = _causal_mode(isCausal)
    p.scale = default_scale(D) if scale is None else float(scale)
    p.kv_lens = kvLens.data_ptr() if kvLens is not None else None
    keep = _set_mask(p, attnMask, q, L, S)  # noqa: F841 (alive until the launch is enqueued)
    _common(p, q)
    if status is not None:
        p.status = status.data_ptr()
    _capi.check(_capi.lib().tt_attn_fwd(C.byref(p)))
    return o, lse


def sdpAttentionBwd(dO, q, k, v, o, lse, isCausal=False, scale=None, kvLens=None, needs=(True, True, True),
                    attnMask=None):
    """Gradients (dQ, dK, dV); entries of `needs` that are False come back as None."""
    for t, n in ((dO, "dO"), (q, "q"), (k, "k"), (v, "v"), (o, "o")):
        _check_tensor(t, n)
    B, Hq, L, D = q.shape
    _, Hkv, S, _ = k.shape
    dq = torch.empty_like(q, memory_format=torch.contiguous_format) if needs[0] else None
    dk = torch.empty_like(k, memory_format=torch.contiguous_format) if needs[1] else None
    dv = torch.empty_like(v, memory_format=torch.contiguous_format) if needs[2] else None
    p = _capi.BwdParams()
    p.struct_size = C.sizeof(_capi.BwdParams)
    p.dtype = _DTYPES[q.dtype]
    p.B, p.Hq, p.Hkv, p.Lq, p.Skv, p.D = B, Hq, Hkv, L, S, D
    p.q, p.k, p.v, p.o, p.d_o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dO.data_ptr()
    p.lse = lse.data_ptr()
    p.dq = dq.data_ptr() if dq is not None else None
    p.dk = dk.data_ptr() if dk is not None else None
    p.dv = dv.data_ptr() if dv is not None else None
    p.q_strides, p.k_strides, p.v_strides = _strides(q), _strides(k), _strides(v)
    p.o_strides, p.do_strides = _strides(o), _strides(dO)
    if dq is not None:
        p.dq_strides = _strides(dq)
    if dk is not None:
        p.dk_strides = _strides(dk)
    if dv is not None:
        p.dv_strides = _strides(dv)
    p.is_causal = _causal_mode(isCausal)
    p.scale = default_scale(D) if scale is None else float(scale)
    p.kv_lens = kvLens.data_ptr() if kvLens is not None else None
    keep = _set_mask(p, attnMask, q, L, S)  # noqa: F841
    _common(p, q)
    _capi.check(_capi.lib().tt_attn_bwd(C.byref(p)))
    return dq, dk, dv


def sdpAttentionDecode(q, kCache, vCache, kvLens=None, scale=None, needLse=False, workspace=None):
    """One query per sequence against a KV cache [B,Hkv,capacity,D] -> (O [B,Hq,1,D], LSE [B,Hq] or None)."""
    for t, n in ((q, "q"), (kCache, "kCache"), (vCache, "vCache")):
        _check_tensor(t, n)
    B, Hq, L, D = q.shape
    if L != 1:
        raise ValueError("decode takes exactly one query per sequence")
    _, Hkv, cap, _ = kCache.shape
    o = torch.empty((B, Hq, 1, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq), dtype=torch.float32, device=q.device) if needLse else None
    p = _capi.DecodeParams()
    p.struct_size = C.sizeof(_capi.DecodeParams)
    p.dtype = _DTYPES[q.dtype]
    p.B, p.Hq, p.Hkv, p.capacity, p.D = B, Hq, Hkv, cap, D
    p.q, p.k, p.v, p.o = q.data_ptr(), kCache.data_ptr(), vCache.data_ptr(), o.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.q_strides, p.k_strides, p.v_strides, p.o_strides = _strides(q), _strides(kCache), _strides(vCache), _strides(o)
    p.scale = default_scale(D) if scale is None else float(scale)
    p.kv_lens = kvLens.data_ptr() if kvLens is not None else None
    _common(p, q)
    if workspace is not None:
        p.workspace = workspace.data_ptr()
        p.workspace_bytes = workspace.numel() * workspace.element_size()
    _capi.check(_capi.lib().tt_attn_decode(C.byref(p)))
    return o, lse


def ropeTables(positions, D, theta=10000.0, device="cuda"):
    """cos / sin tables [positions, D/2] fp32 of the usual rotary embedding: pair i at
    position p turns by p * theta^(-2i/D)."""
    inv = theta ** (-torch.arange(0, D, 2, dtype=torch.float64) / D)
    ang = torch.arange(positions, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


def sdpAttentionDecodeAppend(q, kNew, vNew, kCache, vCache, kvLens, ropeCos=None, ropeSin=None, interleaved=False,
                             scale=None, needLse=False, status=None):
    """One step of a token loop: rotate q and kNew to position kvLens[b], write kNew / vNew
    into row kvLens[b] of the caches (in place), attend over rows [0, kvLens[b]].
    Returns (O [B,Hq,1,D], LSE or None, newLens = kvLens + 1)."""
    for t, n in ((q, "q"), (kNew, "kNew"), (vNew, "vNew"), (kCache, "kCache"), (vCache, "vCache")):
        _check_tensor(t, n)
    B, Hq, L, D = q.shape
    _, Hkv, cap, _ = kCache.shape
    if L != 1 or kNew.shape != (B, Hkv, 1, D) or vNew.shape != (B, Hkv, 1, D):
        raise ValueError("decode-append takes one query and one new key / value row per sequence")
    if kvLens is None or kvLens.dtype != torch.int32:
        raise ValueError("kvLens (int32 [B]) is required")
    o = torch.empty((B, Hq, 1, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq), dtype=torch.float32, device=q.device) if needLse else None
    new_lens = torch.empty_like(kvLens)
    p = _capi.DecodeAppendParams()
    p.struct_size = C.sizeof(_capi.DecodeAppendParams)
    p.dtype = _DTYPES[q.dtype]
    p.B, p.Hq, p.Hkv, p.capacity, p.D = B, Hq, Hkv, cap, D
    p.q, p.k_new, p.v_new = q.data_ptr(), kNew.data_ptr(), vNew.data_ptr()
    p.k_cache, p.v_cache, p.o = kCache.data_ptr(), vCache.data_ptr(), o.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.q_strides, p.k_new_strides, p.v_new_strides = _strides(q), _strides(kNew), _strides(vNew)
    p.k_strides, p.v_strides, p.o_strides = _strides(kCache), _strides(vCache), _strides(o)
    p.scale = default_scale(D) if scale is None else float(scale)
    p.kv_lens = kvLens.data_ptr()
    p.new_lens = new_lens.data_ptr()
    if ropeCos is not None:
        if ropeCos.dtype != torch.float32 or ropeCos.shape != ropeSin.shape or ropeCos.shape[1] != D // 2 \
                or not ropeCos.is_contiguous() or not ropeSin.is_contiguous():
            raise ValueError("rope tables must be contiguous fp32 [positions, D/2]")
        p.rope_cos, p.rope_sin = ropeCos.data_ptr(), ropeSin.data_ptr()
        p.rope_positions = ropeCos.shape[0]
    p.rope_interleaved = 1 if interleaved else 0
    _common(p, q)
    if status is not None:
        p.status = status.data_ptr()
    _capi.check(_capi.lib().tt_attn_decode_append(C.byref(p)))
    return o, lse, new_lens


def workspaceBytes(kind, dtype, B, Hq, Hkv, Lq, Skv, D):
    return int(_capi.lib().tt_attn_workspace_bytes(kind, _DTYPES[dtype], B, Hq, Hkv, Lq, Skv, D))
