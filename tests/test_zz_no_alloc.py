"""GPU: the allocation-free decode entry point (tt_attn_decode_static).

It serves hosts that cannot give the library device memory (no allocator callback,
no spare buffer, or a token loop where allocator calls are off limits), so its
per-split partial results live in a fixed array inside the library.  The test
calls it directly through the C ABI, twice in a row with different inputs (the
array keeps the first call's contents, which must not leak into the second), and
compares each result with the regular tt_attn_decode entry point on the same
inputs and with the CPU oracle, on every scan path the entry point can take.
Collected last so that a failure here cannot mask any other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import TOL_ABS_16BIT, make

pytestmark = pytest.mark.gpu


def _params(q, k, v, o, lens, scale, status=None):
    from tinytorch_b200 import _capi
    B, Hq, _, D = q.shape
    _, Hkv, cap, _ = k.shape
    p = _capi.DecodeParams()
    p.struct_size = C.sizeof(_capi.DecodeParams)
    p.dtype = {torch.bfloat16: _capi.BF16, torch.float16: _capi.F16, torch.float32: _capi.F32}[q.dtype]
    p.B, p.Hq, p.Hkv, p.capacity, p.D = B, Hq, Hkv, cap, D
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    p.lse = None
    for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v), ("o_strides", o)):
        setattr(p, name, _capi.Strides(t.stride(0), t.stride(1), t.stride(2)))
    p.scale = scale
    p.kv_lens = lens.data_ptr()
    p.device = torch.cuda.current_device()
    p.stream = torch.cuda.current_stream().cuda_stream
    p.workspace, p.workspace_bytes, p.alloc = None, 0, None
    p.status = status.data_ptr() if status is not None else None
    return p


# (query heads, kv heads, head dimension, dtype, cache capacity): the tensor-core scan (several query heads per
# kv head), the CUDA-core scan with its combine kernel (one query head per kv head, cache split), fp16 at D = 64,
# a cache short enough for a single split (no partials at all), and fp32
CASES = [
    (8, 2, 128, torch.bfloat16, 3000),
    (4, 4, 128, torch.bfloat16, 3000),
    (6, 2, 64, torch.float16, 2500),
    (4, 4, 64, torch.float16, 400),
    (2, 2, 128, torch.float32, 1500),
]


@pytest.mark.parametrize("Hq,Hkv,D,dt,cap", CASES)
def test_static_scratch_matches_regular_decode_twice(oracle, Hq, Hkv, D, dt, cap):
    from tinytorch_b200 import _capi, op
    lib = _capi.lib()
    B = 4
    assert op.workspaceBytes(_capi.KIND_DECODE, dt, B, Hq, Hkv, 1, cap, D) <= _capi.STATIC_SCRATCH_BYTES
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for call, seed in enumerate((101, 202)):
        q, qn = make((B, Hq, 1, D), dt, seed)
        k, kn = make((B, Hkv, cap, D), dt, seed + 1)
        v, vn = make((B, Hkv, cap, D), dt, seed + 2)
        lens_np = np.array([cap, 1, cap // 2 + 277, 513 % cap + 1] if call == 0 else [700 % cap + 1, cap, 2, cap - 1],
                           dtype=np.int32)
        lens = torch.from_numpy(lens_np).cuda()
        want, _ = op.sdpAttentionDecode(q, k, v, lens, scale=0.09)
        got = torch.full_like(want, float("nan"))
        p = _params(q, k, v, got, lens, 0.09, status)  # no workspace, no allocator hook
        rc = lib.tt_attn_decode_static(C.byref(p))
        torch.cuda.synchronize()
        assert rc == 0, lib.tt_attn_strerror(rc)
        assert int(status.item()) == 0  # the status word is passed on; no wait expired
        assert bool(torch.isfinite(got.float()).all())
        assert torch.equal(got, want)  # same kernels, same reduction order as the regular entry point
        # ... and both against the CPU oracle
        wo, _ = oracle.fwd(qn, kn, vn, kv_lens=lens_np, scale=0.09)
        if dt == torch.float32:
            assert np.abs(got.cpu().numpy() - wo).max() <= 1e-5 * np.abs(wo).max()
        else:
            assert np.abs(got.float().cpu().numpy() - wo).max() <= TOL_ABS_16BIT


def test_static_scratch_size_limit_both_sides():
    # the largest batch whose partials still fit the array runs; one more is refused
    from tinytorch_b200 import _capi, op
    lib = _capi.lib()
    Hq, Hkv = 16, 1   # many partial rows per byte of cache: the batch at the limit stays a few hundred MB
    cap, D, dt = 8192, 128, torch.bfloat16
    need = lambda B: op.workspaceBytes(_capi.KIND_DECODE, dt, B, Hq, Hkv, 1, cap, D)
    lo, hi = 1, 1 << 16
    while lo < hi:  # largest B with need(B) <= limit
        mid = (lo + hi + 1) // 2
        lo, hi = (mid, hi) if need(mid) <= _capi.STATIC_SCRATCH_BYTES else (lo, mid - 1)
    B = lo
    assert need(B) <= _capi.STATIC_SCRATCH_BYTES < need(B + 1)
    g = torch.Generator(device="cuda").manual_seed(9)
    for b, expect in ((B, 0), (B + 1, -10)):
        q = torch.randn((b, Hq, 1, D), generator=g, device="cuda").to(dt)
        k = torch.randn((b, Hkv, cap, D), generator=g, device="cuda").to(dt)
        v = torch.randn((b, Hkv, cap, D), generator=g, device="cuda").to(dt)
        lens = torch.full((b,), cap, dtype=torch.int32, device="cuda")
        got = torch.zeros((b, Hq, 1, D), dtype=dt, device="cuda")
        rc = lib.tt_attn_decode_static(C.byref(_params(q, k, v, got, lens, 0.09)))
        torch.cuda.synchronize()
        assert rc == expect, (b, rc)
        if expect == 0:
            want, _ = op.sdpAttentionDecode(q, k, v, lens, scale=0.09)
            assert torch.equal(got, want)


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
