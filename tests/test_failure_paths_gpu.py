"""GPU: failure paths in their safe forms.  Nothing here faults, traps or hangs a GPU.

 - the allocator hook (include/tt_attn.h, tt_attn_alloc_hook): a hook that returns NULL gives
   TT_ATTN_ERR_WORKSPACE before anything is launched; a working hook gets each block back exactly once;
 - a device-side wait that runs out: the library's self-test kernel waits a millisecond on a barrier nothing
   arrives on, returns by itself and reports it in the status word; the stream and the context stay usable.
The reference's convention these map to is LOGE + ASSERT on the host (src/Utils/Macros.h:34-43), which the
TinyTorch binding applies to the return code.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import TOL_ABS_16BIT, make, to_np

pytestmark = pytest.mark.gpu


def _decode_params(q, k, v, o, hook):
    from tinytorch_b200 import _capi
    B, Hq, _, D = q.shape
    _, Hkv, cap, _ = k.shape
    p = _capi.DecodeParams()
    p.struct_size = C.sizeof(_capi.DecodeParams)
    p.dtype = _capi.BF16
    p.B, p.Hq, p.Hkv, p.capacity, p.D = B, Hq, Hkv, cap, D
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v), ("o_strides", o)):
        setattr(p, name, _capi.Strides(t.stride(0), t.stride(1), t.stride(2)))
    p.scale = 0.1
    p.device = torch.cuda.current_device()
    p.stream = torch.cuda.current_stream().cuda_stream
    p.workspace, p.workspace_bytes = None, 0
    p.alloc = C.pointer(hook) if hook is not None else None
    return p


def test_allocator_hook_failure_and_single_release(oracle):
    from tinytorch_b200 import _capi
    lib = _capi.lib()
    B, H, cap, D = 2, 4, 2048, 128   # four splits: the call needs scratch
    q, qn = make((B, H, 1, D), torch.bfloat16, 31)
    k, kn = make((B, H, cap, D), torch.bfloat16, 32)
    v, vn = make((B, H, cap, D), torch.bfloat16, 33)
    o = torch.zeros_like(q)
    log = {"alloc": [], "free": []}

    def failing_alloc(ctx, nbytes, device):
        log["alloc"].append(nbytes)
        return None  # NULL

    def alloc(ctx, nbytes, device):
        ptr = torch.cuda.caching_allocator_alloc(nbytes, device, torch.cuda.current_stream(device))
        log["alloc"].append(ptr)
        return ptr

    def free(ctx, ptr, device):
        log["free"].append(ptr)
        torch.cuda.caching_allocator_delete(ptr)

    bad = _capi.AllocHook(_capi.ALLOC_FN(failing_alloc), _capi.FREE_FN(free), None)
    assert lib.tt_attn_decode(C.byref(_decode_params(q, k, v, o, bad))) == -6   # TT_ATTN_ERR_WORKSPACE
    assert len(log["alloc"]) == 1 and log["free"] == []      # asked once, nothing to give back
    assert lib.tt_attn_decode(C.byref(_decode_params(q, k, v, o, None))) == -6  # no buffer and no hook at all
    torch.cuda.synchronize()
    assert float(o.float().abs().max()) == 0.0               # nothing was launched

    log["alloc"].clear()
    good = _capi.AllocHook(_capi.ALLOC_FN(alloc), _capi.FREE_FN(free), None)
    assert lib.tt_attn_decode(C.byref(_decode_params(q, k, v, o, good))) == 0
    torch.cuda.synchronize()
    assert len(log["alloc"]) == 1 and log["free"] == log["alloc"]   # the block came back exactly once
    wo, _ = oracle.fwd(qn, kn, vn, scale=0.1)
    assert np.abs(to_np(o) - wo).max() <= TOL_ABS_16BIT


def test_expired_device_wait_sets_status_and_leaves_the_context_usable(oracle):
    from tinytorch_b200 import _capi, op
    lib = _capi.lib()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    dev = torch.cuda.current_device()
    rc = lib.tt_attn_selftest_wait_expiry(dev, stream, 1_000_000, status.data_ptr(), waited.data_ptr())  # 1 ms
    assert rc == 0
    torch.cuda.synchronize()                      # the kernel returned by itself
    assert int(status.item()) & 1                 # kStatusWaitExpired
    assert 1_000_000 <= int(waited.item()) < 500_000_000
    assert lib.tt_attn_selftest_wait_expiry(dev, stream, 0, status.data_ptr(), None) == -3   # limit out of range
    assert lib.tt_attn_selftest_wait_expiry(dev, stream, 1000, None, None) == -1             # status is required
    # an ordinary call on the same stream afterwards: passes, and its own status word stays clear
    q, qn = make((1, 2, 200, 128), torch.bfloat16, 41)
    k, kn = make((1, 2, 200, 128), torch.bfloat16, 42)
    v, vn = make((1, 2, 200, 128), torch.bfloat16, 43)
    st2 = torch.zeros(1, dtype=torch.int32, device="cuda")
    o, _ = op.sdpAttentionFwd(q, k, v, isCausal=True, status=st2)
    torch.cuda.synchronize()
    assert int(st2.item()) == 0
    wo, _ = oracle.fwd(qn, kn, vn, causal=True)
    assert np.abs(to_np(o) - wo).max() <= TOL_ABS_16BIT
