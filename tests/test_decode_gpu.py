"""GPU parity of single-token decode against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import rel_err
from gpu_util import DTYPES, TOL_ABS_16BIT, TOL_REL_FP32, make, to_np

pytestmark = pytest.mark.gpu


def _decode(q, k, v, lens, **kw):
    from tinytorch_b200 import op
    o, lse = op.sdpAttentionDecode(q, k, v, lens, needLse=True, **kw)
    torch.cuda.synchronize()
    return o, lse


def test_golden_decode_fixture(seeded):
    s = seeded
    q, k, v = (torch.from_numpy(s[n]).cuda() for n in ("d_q", "d_k", "d_v"))
    o, _ = _decode(q, k, v, torch.from_numpy(s["d_lens"]).cuda())
    assert rel_err(to_np(o), s["d_o"]) <= TOL_REL_FP32


@pytest.mark.parametrize("dt", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("Hq,Hkv,cap", [(4, 4, 100), (8, 2, 700), (8, 1, 1500), (6, 2, 513), (3, 1, 2049)])
def test_decode_shapes(oracle, dt, D, Hq, Hkv, cap):
    B = 3
    q, qn = make((B, Hq, 1, D), DTYPES[dt], 51)
    k, kn = make((B, Hkv, cap, D), DTYPES[dt], 52)
    v, vn = make((B, Hkv, cap, D), DTYPES[dt], 53)
    lens = np.array([cap, 1, max(1, cap // 2 + 3)], dtype=np.int32)
    o, lse = _decode(q, k, v, torch.from_numpy(lens).cuda())
    wo, wl = oracle.fwd(qn, kn, vn, kv_lens=lens)
    if dt == "f32":
        assert rel_err(to_np(o), wo) <= TOL_REL_FP32
    else:
        assert np.abs(to_np(o) - wo).max() <= TOL_ABS_16BIT
    assert np.abs(to_np(lse) - wl[:, :, 0]).max() <= 2e-3


def test_rows_beyond_length_are_ignored(oracle):
    B, H, cap, D = 2, 4, 1200, 128
    q, qn = make((B, H, 1, D), torch.bfloat16, 61)
    k, kn = make((B, H, cap, D), torch.bfloat16, 62)
    v, vn = make((B, H, cap, D), torch.bfloat16, 63)
    lens = np.array([600, 1100], dtype=np.int32)
    tl = torch.from_numpy(lens).cuda()
    o1, _ = _decode(q, k, v, tl)
    k2, v2 = k.clone(), v.clone()
    for b in range(B):
        k2[b, :, lens[b]:] = float("nan")
        v2[b, :, lens[b]:] = float("inf")
    o2, _ = _decode(q, k2, v2, tl)
    assert torch.equal(o1, o2)


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("Hq,Hkv,cap,lens", [
    (8, 4, 300, (300, 1, 129)),            # 2 heads per kv head, one split
    (8, 2, 4096, (4096, 513, 2000)),       # 4 per kv head, several splits, one of them empty for the short sequence
    (16, 2, 1000, (1000, 128, 999)),       # 8 per kv head
    (32, 2, 640, (640, 5, 600)),           # 16 per kv head (the most one MMA column block holds)
    (12, 4, 1536, (1536, 1024, 1)),        # 3 per kv head: rows of the Q tile beyond the group are zero
    (12, 2, 900, (900, 257, 3)),           # 6 per kv head (kernel instance for 8, two padding heads)
    (24, 2, 2300, (2300, 2049, 77)),       # 12 per kv head (kernel instance for 16)
])
def test_grouped_query_decode_on_tensor_cores(oracle, dt, Hq, Hkv, cap, lens):
    # several query heads per kv head, D = 128, 16-bit: the tcgen05 decode path; rows at or beyond the
    # lengths hold NaN / Inf and must not reach the result
    B, D = len(lens), 128
    q, qn = make((B, Hq, 1, D), DTYPES[dt], 91)
    k, kn = make((B, Hkv, cap, D), DTYPES[dt], 92)
    v, vn = make((B, Hkv, cap, D), DTYPES[dt], 93)
    ln = np.array(lens, dtype=np.int32)
    for b in range(B):
        k[b, :, int(ln[b]):] = float("nan")
        v[b, :, int(ln[b]):] = float("inf")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    from tinytorch_b200 import op
    o, lse = op.sdpAttentionDecode(q, k, v, torch.from_numpy(ln).cuda(), needLse=True)
    torch.cuda.synchronize()
    assert not bool(torch.isnan(o.float()).any())
    wo, wl = oracle.fwd(qn, kn, vn, kv_lens=ln)
    assert np.abs(to_np(o) - wo).max() <= TOL_ABS_16BIT
    assert np.abs(to_np(lse) - wl[:, :, 0]).max() <= 2e-2


def test_grouped_query_decode_agrees_with_the_scan_kernel(oracle):
    # the same cache read as 4 query heads per kv head (tensor cores) and, head by head, as 1 per kv head (scan)
    B, Hq, Hkv, cap, D = 3, 8, 2, 2500, 128
    q, _ = make((B, Hq, 1, D), torch.bfloat16, 95)
    k, _ = make((B, Hkv, cap, D), torch.bfloat16, 96)
    v, _ = make((B, Hkv, cap, D), torch.bfloat16, 97)
    lens = torch.tensor([2500, 700, 1], dtype=torch.int32, device="cuda")
    o, _ = _decode(q, k, v, lens)
    g = Hq // Hkv
    for h in range(Hq):
        oh, _ = _decode(q[:, h:h + 1].contiguous(), k[:, h // g:h // g + 1], v[:, h // g:h // g + 1], lens)
        assert float((o[:, h:h + 1].float() - oh.float()).abs().max()) <= 1e-2


def test_config4_full(oracle):
    # B=64 H=32 D=128 bf16, cache of 8192, lengths uniform in [1024, 8192]
    B, H, cap, D = 64, 32, 8192, 128
    g = torch.Generator(device="cuda").manual_seed(1238)
    q = torch.randn((B, H, 1, D), generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn((B, H, cap, D), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((B, H, cap, D), generator=g, device="cuda").to(torch.bfloat16)
    lens = np.random.default_rng(1238).integers(1024, 8193, size=B).astype(np.int32)
    tl = torch.from_numpy(lens).cuda()
    o, lse = _decode(q, k, v, tl)
    o2, _ = _decode(q, k, v, tl)
    assert torch.equal(o, o2)
    for b in (0, 17, 63):
        wo, wl = oracle.fwd(to_np(q[b:b + 1]), to_np(k[b:b + 1]), to_np(v[b:b + 1]), kv_lens=lens[b:b + 1])
        assert np.abs(to_np(o[b:b + 1]) - wo).max() <= TOL_ABS_16BIT
        assert np.abs(to_np(lse[b:b + 1]) - wl[:, :, 0]).max() <= 2e-3
    # decode must agree with the prefill kernel on the same inputs (L = 1, lengths)
    from tinytorch_b200 import op
    op_o, _ = op.sdpAttentionFwd(q, k, v, isCausal=False, kvLens=tl)
    torch.cuda.synchronize()
    assert float((op_o.float() - o.float()).abs().max()) <= TOL_ABS_16BIT


def test_caller_workspace_and_too_small(oracle):
    from tinytorch_b200 import _capi, op
    B, H, cap, D = 2, 4, 2048, 128
    q, qn = make((B, H, 1, D), torch.bfloat16, 71)
    k, kn = make((B, H, cap, D), torch.bfloat16, 72)
    v, vn = make((B, H, cap, D), torch.bfloat16, 73)
    need = op.workspaceBytes(_capi.KIND_DECODE, torch.bfloat16, B, H, H, 1, cap, D)
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    o, _ = op.sdpAttentionDecode(q, k, v, None, workspace=ws)
    torch.cuda.synchronize()
    wo, _ = oracle.fwd(qn, kn, vn)
    assert np.abs(to_np(o) - wo).max() <= TOL_ABS_16BIT
    with pytest.raises(_capi.AttnError) as e:
        op.sdpAttentionDecode(q, k, v, None, workspace=ws[:256])
    assert e.value.code == -6
