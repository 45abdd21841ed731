"""GPU: the allocation-free decode entry point (tt_attn_decode_static).

It serves hosts that cannot give the library device memory (no allocator callback,
no spare buffer, or a token loop where allocator calls are off limits), so its
per-split partial results live in a fixed array inside the library.  The test
calls it directly through the C ABI, twice in a row with different inputs (the
array keeps the first call's contents, which must not leak into the second), and
compares each result with the regular tt_attn_decode entry point on the same
inputs.  Collected last so that a failure here cannot mask any other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import TOL_ABS_16BIT, make

pytestmark = pytest.mark.gpu


def _params(q, k, v, o, lens, scale):
    from tinytorch_b200 import _capi
    B, Hq, _, D = q.shape
    _, Hkv, cap, _ = k.shape
    p = _capi.DecodeParams()
    p.struct_size = C.sizeof(_capi.DecodeParams)
    p.dtype = _capi.BF16
    p.B, p.Hq, p.Hkv, p.capacity, p.D = B, Hq, Hkv, cap, D
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    p.lse = None
    for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v), ("o_strides", o)):
        setattr(p, name, _capi.Strides(t.stride(0), t.stride(1), t.stride(2)))
    p.scale = scale
    p.kv_lens = lens.data_ptr()
    p.device = torch.cuda.current_device()
    p.stream = torch.cuda.current_stream().cuda_stream
    p.workspace, p.workspace_bytes, p.alloc, p.status = None, 0, None, None
    return p


def test_static_scratch_matches_regular_decode_twice():
    from tinytorch_b200 import _capi, op
    lib = _capi.lib()
    B, Hq, Hkv, cap, D = 4, 8, 2, 3000, 128   # 6 splits -> partials are in use
    assert 0 < op.workspaceBytes(_capi.KIND_DECODE, torch.bfloat16, B, Hq, Hkv, 1, cap, D) <= _capi.STATIC_SCRATCH_BYTES
    for call, seed in enumerate((101, 202)):
        q, _ = make((B, Hq, 1, D), torch.bfloat16, seed)
        k, _ = make((B, Hkv, cap, D), torch.bfloat16, seed + 1)
        v, _ = make((B, Hkv, cap, D), torch.bfloat16, seed + 2)
        lens_np = np.array([cap, 1, 1777, 513] if call == 0 else [700, cap, 2, 2999], dtype=np.int32)
        lens = torch.from_numpy(lens_np).cuda()
        want, _ = op.sdpAttentionDecode(q, k, v, lens, scale=0.09)
        got = torch.full_like(want, float("nan"))
        p = _params(q, k, v, got, lens, 0.09)  # no workspace, no allocator hook
        rc = lib.tt_attn_decode_static(C.byref(p))
        torch.cuda.synchronize()
        assert rc == 0, lib.tt_attn_strerror(rc)
        assert bool(torch.isfinite(got.float()).all())
        assert float((got.float() - want.float()).abs().max()) <= TOL_ABS_16BIT
        assert torch.equal(got, want)  # same kernels, same reduction order


def test_static_scratch_rejects_oversize():
    from tinytorch_b200 import _capi, op
    lib = _capi.lib()
    B, Hq, Hkv, cap, D = 128, 32, 32, 8192, 128   # needs 34 MB of partials > 24 MiB
    assert op.workspaceBytes(_capi.KIND_DECODE, torch.bfloat16, B, Hq, Hkv, 1, cap, D) > _capi.STATIC_SCRATCH_BYTES
    t = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    p = _capi.DecodeParams()
    p.struct_size = C.sizeof(_capi.DecodeParams)
    p.dtype = _capi.BF16
    p.B, p.Hq, p.Hkv, p.capacity, p.D = B, Hq, Hkv, cap, D
    p.q = p.k = p.v = p.o = t.data_ptr()   # never dereferenced: the size check comes first
    p.scale = 0.1
    assert lib.tt_attn_decode_static(C.byref(p)) == -10
    assert b"limit" in lib.tt_attn_strerror(-10)
