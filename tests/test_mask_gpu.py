"""GPU parity of masked attention (the reference's attnMask, src/Function/FuncNNLayer.h:249-256)
and of the bottom-right causal alignment against the CPU oracle, forward and backward,
through the C ABI and through the autograd hookup."""
import numpy as np
import pytest
import torch

from conftest import rel_err
from gpu_util import DTYPES, TOL_ABS_16BIT, TOL_REL_FP32, make, to_np

pytestmark = pytest.mark.gpu

NEG = np.float32(-np.inf)


def _close(got, want, dt, scale_by_max=False):
    got = to_np(got)
    if dt == "f32":
        assert rel_err(got, want) <= TOL_REL_FP32
    else:
        bound = TOL_ABS_16BIT * (max(1.0, np.abs(want).max()) if scale_by_max else 1.0)
        assert np.abs(got - want).max() <= bound


def _mask_case(kind, B, H, L, S, dtype, seed):
    """Returns (device mask tensor, additive fp32 bias broadcastable to [B,H,L,S] for the oracle).
    Every query row keeps key 0, so that no row is fully masked."""
    rng = np.random.default_rng(seed)
    if kind == "bool_b1ls":
        m = rng.random((B, 1, L, S)) < 0.6
        m[..., 0] = True
        return torch.from_numpy(m).cuda(), np.where(m, np.float32(0), NEG).astype(np.float32)
    if kind == "bool_ls":
        m = rng.random((L, S)) < 0.5
        m[..., 0] = True
        return torch.from_numpy(m).cuda(), np.where(m, np.float32(0), NEG).astype(np.float32)
    if kind == "add_1hls":  # additive, dtype of the tensors, with some -inf entries
        a = rng.standard_normal((1, H, L, S)).astype(np.float32)
        a[rng.random((1, H, L, S)) < 0.2] = NEG
        a[..., 0] = 0.5
        t = torch.from_numpy(a).to(dtype)
        return t.cuda(), t.float().numpy()
    if kind == "addf32_b11s":  # fp32 additive, broadcast over heads and queries
        a = (rng.standard_normal((B, 1, 1, S)) * 2).astype(np.float32)
        return torch.from_numpy(a).cuda(), a
    raise AssertionError(kind)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("kind", ["bool_b1ls", "bool_ls", "add_1hls", "addf32_b11s"])
@pytest.mark.parametrize("L,S", [(256, 384), (200, 328), (70, 130)])
def test_masked_forward(oracle, dt, D, kind, L, S):
    from tinytorch_b200 import op
    B, H = 2, 2
    q, qn = make((B, H, L, D), DTYPES[dt], 301)
    k, kn = make((B, H, S, D), DTYPES[dt], 302)
    v, vn = make((B, H, S, D), DTYPES[dt], 303)
    mask, bias = _mask_case(kind, B, H, L, S, DTYPES[dt], 304)
    o, lse = op.sdpAttentionFwd(q, k, v, attnMask=mask)
    torch.cuda.synchronize()
    wo, wl = oracle.fwd(qn, kn, vn, bias=bias)
    _close(o, wo, dt)
    assert np.abs(to_np(lse) - wl).max() <= (1e-4 if dt == "f32" else 2e-2)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("kind", ["bool_b1ls", "add_1hls", "addf32_b11s"])
@pytest.mark.parametrize("L,S,Hq,Hkv", [(256, 256, 2, 2), (100, 200, 4, 2)])
def test_masked_backward(oracle, dt, D, kind, L, S, Hq, Hkv):
    from tinytorch_b200 import op
    B = 2
    q, qn = make((B, Hq, L, D), DTYPES[dt], 311)
    k, kn = make((B, Hkv, S, D), DTYPES[dt], 312)
    v, vn = make((B, Hkv, S, D), DTYPES[dt], 313)
    do, don = make((B, Hq, L, D), DTYPES[dt], 314)
    mask, bias = _mask_case(kind, B, Hq, L, S, DTYPES[dt], 315)
    o, lse = op.sdpAttentionFwd(q, k, v, attnMask=mask)
    dq, dk, dv = op.sdpAttentionBwd(do, q, k, v, o, lse, attnMask=mask)
    torch.cuda.synchronize()
    wq, wk, wv = oracle.bwd(qn, kn, vn, don, bias=bias)
    for got, want in ((dq, wq), (dk, wk), (dv, wv)):
        _close(got, want, dt, scale_by_max=True)


def _bottom_right_bias(L, S, lens, B):
    """-inf where key j > i + (len_b - L), as an additive bias [B,1,L,S]."""
    i = np.arange(L)[:, None]
    j = np.arange(S)[None, :]
    out = np.zeros((B, 1, L, S), dtype=np.float32)
    for b in range(B):
        out[b, 0][j > i + (int(lens[b]) - L)] = NEG
    return out


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("L,S,lens", [(128, 384, None), (100, 300, (300, 177)), (256, 256, None), (1, 200, (200, 64))])
def test_bottom_right_causal_forward_backward(oracle, dt, D, L, S, lens):
    from tinytorch_b200 import op
    B, Hq, Hkv = 2, 4, 2
    q, qn = make((B, Hq, L, D), DTYPES[dt], 321)
    k, kn = make((B, Hkv, S, D), DTYPES[dt], 322)
    v, vn = make((B, Hkv, S, D), DTYPES[dt], 323)
    do, don = make((B, Hq, L, D), DTYPES[dt], 324)
    ln = np.array(lens if lens else (S, S), dtype=np.int32)
    kw = dict(isCausal="bottom-right", kvLens=torch.from_numpy(ln).cuda() if lens else None)
    o, lse = op.sdpAttentionFwd(q, k, v, **kw)
    dq, dk, dv = op.sdpAttentionBwd(do, q, k, v, o, lse, **kw)
    torch.cuda.synchronize()
    bias = _bottom_right_bias(L, S, ln, B)
    wo, wl = oracle.fwd(qn, kn, vn, kv_lens=ln if lens else None, bias=bias)
    wq, wk, wv = oracle.bwd(qn, kn, vn, don, kv_lens=ln if lens else None, bias=bias)
    _close(o, wo, dt)
    assert np.abs(to_np(lse) - wl).max() <= (1e-4 if dt == "f32" else 2e-2)
    for got, want in ((dq, wq), (dk, wk), (dv, wv)):
        _close(got, want, dt, scale_by_max=True)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_bottom_right_more_queries_than_keys(oracle, dt):
    # L > S: the first L - S queries see no key at all -> O = 0, LSE = -inf, zero gradients from them
    from tinytorch_b200 import op
    B, H, L, S, D = 1, 2, 300, 172, 64
    q, qn = make((B, H, L, D), DTYPES[dt], 331)
    k, kn = make((B, H, S, D), DTYPES[dt], 332)
    v, vn = make((B, H, S, D), DTYPES[dt], 333)
    do, don = make((B, H, L, D), DTYPES[dt], 334)
    o, lse = op.sdpAttentionFwd(q, k, v, isCausal="bottom-right")
    dq, dk, dv = op.sdpAttentionBwd(do, q, k, v, o, lse, isCausal="bottom-right")
    torch.cuda.synchronize()
    dead = L - S
    assert float(o[:, :, :dead].abs().max()) == 0.0
    assert bool(torch.isinf(lse[:, :, :dead]).all()) and float(lse[:, :, :dead].max()) < 0
    assert float(dq[:, :, :dead].float().abs().max()) == 0.0
    # the live rows equal top-left causal attention of those rows alone
    wo, wl = oracle.fwd(qn[:, :, dead:], kn, vn, causal=True)
    wq, wk, wv = oracle.bwd(qn[:, :, dead:], kn, vn, don[:, :, dead:], causal=True)
    _close(o[:, :, dead:], wo, dt)
    _close(dq[:, :, dead:], wq, dt, scale_by_max=True)
    _close(dk, wk, dt, scale_by_max=True)
    _close(dv, wv, dt, scale_by_max=True)
    assert not bool(torch.isnan(dk.float()).any() or torch.isnan(dv.float()).any())


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_fully_masked_rows_give_zero(dt):
    # the reference yields NaN for a row whose keys are all masked (src/Operation/OpNNLayerCpu.h:28-54);
    # the fused path documents O = 0, LSE = -inf, and keeps the other rows exact
    from tinytorch_b200 import op
    B, H, L, S, D = 1, 2, 192, 256, 128
    q, _ = make((B, H, L, D), DTYPES[dt], 341)
    k, _ = make((B, H, S, D), DTYPES[dt], 342)
    v, _ = make((B, H, S, D), DTYPES[dt], 343)
    m = torch.ones((L, S), dtype=torch.bool, device="cuda")
    m[5] = False          # fully masked row
    m[130, :200] = False  # first key tile fully masked for this row, later keys live
    o, lse = op.sdpAttentionFwd(q, k, v, attnMask=m)
    o_ref, lse_ref = op.sdpAttentionFwd(q, k, v)
    torch.cuda.synchronize()
    assert float(o[:, :, 5].abs().max()) == 0.0 and bool(torch.isinf(lse[:, :, 5]).all())
    keep = [i for i in range(L) if i not in (5, 130)]
    assert float((o[:, :, keep].float() - o_ref[:, :, keep].float()).abs().max()) <= (1e-6 if dt == "f32" else 2e-3)
    # row 130 against torch on the live keys only
    p = torch.softmax((q[:, :, 130:131].float() @ k[:, :, 200:].float().transpose(-1, -2)) / D ** 0.5, -1)
    want = p @ v[:, :, 200:].float()
    assert float((o[:, :, 130:131].float() - want).abs().max()) <= (1e-5 if dt == "f32" else 2e-2)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_golden_mask_fixture(dt):
    # inputs and outputs of the reference's own sdpAttention with a Bool and a float mask
    import os
    from conftest import GOLDEN
    from tinytorch_b200 import op
    g = np.load(os.path.join(GOLDEN, "ref_seeded_mask.npz"))
    q, k, v = (torch.from_numpy(g[n]).cuda().to(DTYPES[dt]) for n in ("q", "k", "v"))
    for mask, want, scale in ((g["mask_bool"], g["o_bool"], None), (g["mask_float"], g["o_float"], None),
                              (g["mask_float"], g["o_float_scale"], 0.2)):
        o, _ = op.sdpAttentionFwd(q, k, v, attnMask=torch.from_numpy(mask).cuda(), scale=scale)
        torch.cuda.synchronize()
        if dt == "f32":
            assert rel_err(to_np(o), want) <= TOL_REL_FP32
        else:
            # 16-bit inputs are rounded copies of the fixture's fp32 inputs: a loose bound
            assert np.abs(to_np(o) - want).max() <= 5e-2


def test_mask_combined_with_causal_and_lengths(oracle):
    from tinytorch_b200 import op
    B, H, L, S, D = 2, 2, 256, 256, 128
    dt = "bf16"
    q, qn = make((B, H, L, D), DTYPES[dt], 351)
    k, kn = make((B, H, S, D), DTYPES[dt], 352)
    v, vn = make((B, H, S, D), DTYPES[dt], 353)
    mask, bias = _mask_case("bool_b1ls", B, H, L, S, DTYPES[dt], 354)
    lens = np.array([256, 131], dtype=np.int32)
    o, lse = op.sdpAttentionFwd(q, k, v, isCausal=True, kvLens=torch.from_numpy(lens).cuda(), attnMask=mask)
    torch.cuda.synchronize()
    tri = np.where(np.arange(S)[None, :] > np.arange(L)[:, None], NEG, np.float32(0))
    wo, _ = oracle.fwd(qn, kn, vn, kv_lens=lens, bias=np.minimum(bias, tri[None, None]))
    _close(o, wo, dt)


def test_function_layer_with_mask_matches_reference_lib(reference):
    # function.sdpAttention(q, k, v, False, attnMask) against the reference's own sdpAttention with the same Bool mask
    from tinytorch_b200 import function
    B, H, L, S, D = 2, 2, 96, 160, 64
    q, qn = make((B, H, L, D), torch.float32, 361)
    k, kn = make((B, H, S, D), torch.float32, 362)
    v, vn = make((B, H, S, D), torch.float32, 363)
    rng = np.random.default_rng(364)
    m = rng.random((B, 1, L, S)) < 0.7
    m[..., 0] = True
    q.requires_grad_(True)
    o = function.sdpAttention(q, k, v, False, torch.from_numpy(m).cuda())
    o.sum().backward()
    torch.cuda.synchronize()
    want = reference.fwd_mask(qn, kn, vn, m)
    assert rel_err(to_np(o), want) <= TOL_REL_FP32
    assert q.grad is not None and not bool(torch.isnan(q.grad).any())
