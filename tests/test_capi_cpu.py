"""CPU: the C-ABI library loads without a GPU, exports every symbol the header
declares, and rejects bad arguments before touching CUDA."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT
from tinytorch_b200 import _capi


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_capi.LIB_PATH):
        from tinytorch_b200.build import build
        build()
    return _capi.lib()


def _declared():
    text = open(os.path.join(ROOT, "include", "tt_attn.h")).read()
    return re.findall(r"TT_ATTN_API\s+[\w\s\*]+?\b(tt_attn_\w+)\s*\(", text)


def test_exports_every_declared_symbol(lib):
    names = _declared()
    assert set(_capi.EXPORTS) <= set(names) and len(names) >= 7
    for n in names:
        assert hasattr(lib, n), n


def test_version_and_strerror(lib):
    assert lib.tt_attn_version() == 2  # 2: mask fields and the bottom-right causal alignment
    assert lib.tt_attn_strerror(0) == b"ok"
    for code in range(-10, 0):
        assert b"unknown" not in lib.tt_attn_strerror(code)


def test_struct_sizes_match_header_layout():
    # LP64 layout of the three parameter structs
    assert C.sizeof(_capi.Strides) == 24
    assert C.sizeof(_capi.AllocHook) == 24
    assert C.sizeof(_capi.FwdParams) % 8 == 0 and C.sizeof(_capi.BwdParams) > C.sizeof(_capi.FwdParams)


def _fwd(**kw):
    p = _capi.FwdParams()
    p.struct_size = C.sizeof(_capi.FwdParams)
    p.dtype, p.B, p.Hq, p.Hkv, p.Lq, p.Skv, p.D = 2, 1, 4, 2, 128, 128, 128
    p.q = p.k = p.v = p.o = 0x1000
    p.scale = 0.1
    for k, v in kw.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("kw,code", [
    (dict(struct_size=8), -8),
    (dict(dtype=3), -2),
    (dict(B=0), -3),
    (dict(Hq=3), -3),
    (dict(D=96), -4),
    (dict(q=None), -1),
    (dict(k=0x1004), -5),
    (dict(q_strides=_capi.Strides(4096, 1024, 4)), -5),
    (dict(B=70000), -10),
    (dict(is_causal=3), -3),
    (dict(mask=0x2000, mask_kind=4), -2),
    (dict(mask=None, mask_kind=1), -1),
])
def test_fwd_rejects_bad_arguments(lib, kw, code):
    p = _fwd(**kw)
    assert lib.tt_attn_fwd(C.byref(p)) == code


def test_version_1_struct_is_still_accepted(lib):
    # a caller compiled against ABI version 1 passes the struct without the mask fields; it must get past
    # the size check (and then fail on something else: here a misaligned pointer)
    p = _fwd(k=0x1004)
    p.struct_size = _capi.FwdParams.mask.offset
    assert lib.tt_attn_fwd(C.byref(p)) == -5
    p.struct_size = _capi.FwdParams.mask.offset + 8
    assert lib.tt_attn_fwd(C.byref(p)) == -8


def test_null_param_pointers(lib):
    assert lib.tt_attn_fwd(None) == -1
    assert lib.tt_attn_bwd(None) == -1
    assert lib.tt_attn_decode(None) == -1


def test_workspace_sizes(lib):
    w = lib.tt_attn_workspace_bytes
    assert w(_capi.KIND_FWD, 2, 4, 32, 32, 4096, 4096, 128) == 256  # work counter of the persistent kernel
    assert w(_capi.KIND_FWD, 0, 2, 4, 4, 128, 128, 64) == 0
    assert w(_capi.KIND_BWD, 0, 8, 16, 16, 2048, 2048, 64) == 8 * 16 * 2048 * 4
    # fp16 / bf16: plus the fp32 dQ accumulator
    assert w(_capi.KIND_BWD, 1, 8, 16, 16, 2048, 2048, 64) == 8 * 16 * 2048 * 4 * (1 + 64) + 256
    # decode: 512-row chunks -> 16 splits at capacity 8192; (D + 2) floats per (b, h, split)
    assert w(_capi.KIND_DECODE, 2, 64, 32, 32, 1, 8192, 128) == 64 * 32 * 16 * 130 * 4
    assert w(_capi.KIND_DECODE, 2, 64, 32, 32, 1, 512, 128) == 0
    # several query heads per kv head (16-bit, D = 128): the tensor-core path plans 2048-row chunks when there are
    # enough items to fill the GPU, and needs a 256-byte work counter besides the partials
    assert w(_capi.KIND_DECODE, 2, 64, 32, 8, 1, 8192, 128) == 64 * 32 * 4 * 130 * 4 + 256
    assert w(_capi.KIND_DECODE, 2, 64, 32, 8, 1, 1024, 128) == 256
    assert w(_capi.KIND_DECODE, 2, 1, 32, 8, 1, 8192, 128) == 1 * 32 * 16 * 130 * 4 + 256   # few items: 512-row chunks
    assert w(_capi.KIND_DECODE, 0, 64, 32, 8, 1, 8192, 128) == 64 * 32 * 16 * 130 * 4       # fp32 stays on the scan kernel
    # the fused decode step: same scratch, plus the rotated q and the new lengths on the tensor-core path
    assert w(_capi.KIND_DECODE_APPEND, 2, 64, 32, 32, 1, 8192, 128) == w(_capi.KIND_DECODE, 2, 64, 32, 32, 1, 8192, 128)
    assert w(_capi.KIND_DECODE_APPEND, 2, 64, 32, 8, 1, 8192, 128) == \
        w(_capi.KIND_DECODE, 2, 64, 32, 8, 1, 8192, 128) + 64 * 32 * 128 * 2 + 256


def test_ops_refuse_cpu_tensors():
    import torch
    from tinytorch_b200 import op
    x = torch.zeros(1, 1, 8, 64)
    with pytest.raises(ValueError):
        op.sdpAttentionFwd(x, x, x)


def test_function_signature_matches_reference():
    # function::sdpAttention(query, key, value, isCausal, attnMask, dropoutP, scale)
    import inspect
    from tinytorch_b200.function import sdpAttention
    names = list(inspect.signature(sdpAttention).parameters)
    assert names[:7] == ["query", "key", "value", "isCausal", "attnMask", "dropoutP", "scale"]
    import torch
    x = torch.zeros(1, 1, 8, 64)
    with pytest.raises(AssertionError):
        sdpAttention(x, x, x, True, torch.ones(8, 8, dtype=torch.bool))
