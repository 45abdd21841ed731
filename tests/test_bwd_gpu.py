"""GPU parity of the attention backward against the CPU oracle (the reference's
composed differentiable chain), through the C ABI and through the autograd hookup."""
import numpy as np
import pytest
import torch

from conftest import rel_err
from gpu_util import DTYPES, TOL_ABS_16BIT, TOL_REL_FP32, assert_close_16bit, make, to_np

pytestmark = pytest.mark.gpu


def _fwd_bwd(q, k, v, do, **kw):
    from tinytorch_b200 import op
    o, lse = op.sdpAttentionFwd(q, k, v, **kw)
    dq, dk, dv = op.sdpAttentionBwd(do, q, k, v, o, lse, **kw)
    torch.cuda.synchronize()
    return o, dq, dk, dv


def test_config1_fp32_fwd_bwd(oracle):
    shp = (2, 4, 128, 64)
    (q, qn), (k, kn), (v, vn), (do, don) = (make(shp, torch.float32, 1235 + i) for i in range(4))
    o, dq, dk, dv = _fwd_bwd(q, k, v, do, isCausal=True)
    wq, wk, wv = oracle.bwd(qn, kn, vn, don, causal=True)
    assert rel_err(to_np(dq), wq) <= TOL_REL_FP32
    assert rel_err(to_np(dk), wk) <= TOL_REL_FP32
    assert rel_err(to_np(dv), wv) <= TOL_REL_FP32


def test_golden_fixture_gradients(seeded):
    s = seeded
    q, k, v, do = (torch.from_numpy(s[n]).cuda() for n in ("c_q", "c_k", "c_v", "c_do"))
    _, dq, dk, dv = _fwd_bwd(q, k, v, do, isCausal=True)
    assert rel_err(to_np(dq), s["c_dq"]) <= TOL_REL_FP32
    assert rel_err(to_np(dk), s["c_dk"]) <= TOL_REL_FP32
    assert rel_err(to_np(dv), s["c_dv"]) <= TOL_REL_FP32


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("L,S,causal,Hq,Hkv", [
    (64, 64, True, 2, 2), (100, 100, True, 4, 2), (130, 70, False, 2, 1), (70, 130, True, 2, 2), (1, 90, False, 2, 2),
])
def test_bwd_shapes(oracle, dt, D, L, S, causal, Hq, Hkv):
    B = 2
    q, qn = make((B, Hq, L, D), DTYPES[dt], 81)
    k, kn = make((B, Hkv, S, D), DTYPES[dt], 82)
    v, vn = make((B, Hkv, S, D), DTYPES[dt], 83)
    do, don = make((B, Hq, L, D), DTYPES[dt], 84)
    lens = np.array([S, max(1, S // 2)], dtype=np.int32)
    kw = dict(isCausal=causal, kvLens=torch.from_numpy(lens).cuda())
    _, dq, dk, dv = _fwd_bwd(q, k, v, do, **kw)
    wq, wk, wv = oracle.bwd(qn, kn, vn, don, causal=causal, kv_lens=lens)
    for name, got, want in (("dQ", dq, wq), ("dK", dk, wk), ("dV", dv, wv)):
        if dt == "f32":
            assert rel_err(to_np(got), want) <= TOL_REL_FP32
        else:
            # inputs to the backward (O, LSE) come from the 16-bit forward
            assert_close_16bit(to_np(got), want, dt, "%s %s D=%d L=%d S=%d" % (name, dt, D, L, S))


@pytest.mark.parametrize("dt,D", [("f16", 64), ("bf16", 64), ("bf16", 128)])
@pytest.mark.parametrize("causal,L,S", [(False, 640, 1536), (True, 640, 1536), ("bottom-right", 640, 1536),
                                        (True, 1536, 1536)])
def test_bwd_many_items_per_cta(oracle, dt, D, causal, L, S):
    """More key tiles (4 x 4 x 12 = 192 work items) than the persistent backward kernels have CTAs, several query
    heads per kv head, and key tiles that no query sees: whole runs of them behind short kv_lens and, under the
    top-left causal mask with L < S, behind the last query row.  Their dK / dV must come out as zeros, the items
    after them must still be walked, and every CTA goes through more than one item."""
    B, Hq, Hkv = 4, 8, 4
    q, qn = make((B, Hq, L, D), DTYPES[dt], 181)
    k, kn = make((B, Hkv, S, D), DTYPES[dt], 182)
    v, vn = make((B, Hkv, S, D), DTYPES[dt], 183)
    do, don = make((B, Hq, L, D), DTYPES[dt], 184)
    # (bottom-right: every length >= L, so that no query row is left without a key)
    lens = np.array([S, 700, 641, S - 77] if causal == "bottom-right" else [S, 200, 1, S - 77], dtype=np.int32)
    kw = dict(isCausal=causal, kvLens=torch.from_numpy(lens).cuda())
    from tinytorch_b200 import op
    o, lse = op.sdpAttentionFwd(q, k, v, **kw)
    dq, dk, dv = op.sdpAttentionBwd(do, q, k, v, o, lse, **kw)
    torch.cuda.synchronize()
    okw = dict(kv_lens=lens)
    if causal == "bottom-right":
        # the triangle's corner sits at each sequence's own (L, kv_len)
        bias = np.zeros((B, 1, L, S), dtype=np.float32)
        for b in range(B):
            i, j = np.arange(L)[:, None], np.arange(S)[None, :]
            bias[b, 0][j > i + (int(lens[b]) - L)] = -np.inf
        okw["bias"] = bias
    else:
        okw["causal"] = bool(causal)
    wq, wk, wv = oracle.bwd(qn, kn, vn, don, **okw)
    for name, got, want in (("dQ", dq, wq), ("dK", dk, wk), ("dV", dv, wv)):
        g = to_np(got)
        live = np.isfinite(want)  # (query rows without any visible key have no defined gradient in the oracle)
        assert_close_16bit(np.where(live, g, 0.0), np.where(live, want, 0.0), dt,
                           "%s %s D=%d causal=%s L=%d S=%d" % (name, dt, D, causal, L, S))
    # keys beyond a sequence's length get exact zeros
    assert float(np.abs(to_np(dk)[1, :, int(lens[1]):]).max()) == 0.0
    assert float(np.abs(to_np(dv)[2, :, int(lens[2]):]).max()) == 0.0


def test_config5_fp16_slices(oracle):
    # B=8 H=16 S=2048 D=64 fp16 causal fwd+bwd; oracle on two (b, h) slices
    B, H, S, D = 8, 16, 2048, 64
    g = torch.Generator(device="cuda").manual_seed(1239)
    q, k, v, do = (torch.randn((B, H, S, D), generator=g, device="cuda").half() for _ in range(4))
    o, dq, dk, dv = _fwd_bwd(q, k, v, do, isCausal=True)
    # the first unit, the last one and one from the middle of the grid
    for (b, h) in ((0, 0), (3, 9), (7, 15)):
        sl = (slice(b, b + 1), slice(h, h + 1))
        qn, kn, vn, don = (to_np(t[sl]) for t in (q, k, v, do))
        wo, _ = oracle.fwd(qn, kn, vn, causal=True)
        wq, wk, wv = oracle.bwd(qn, kn, vn, don, causal=True)
        assert np.abs(to_np(o[sl]) - wo).max() <= TOL_ABS_16BIT
        for name, got, want in (("dQ", dq, wq), ("dK", dk, wk), ("dV", dv, wv)):
            assert_close_16bit(to_np(got[sl]), want, "f16", "config 5 %s (b=%d, h=%d)" % (name, b, h))


def test_autograd_hookup_accumulates(oracle):
    # function.sdpAttention: gradients reach leaves and accumulate across two backward calls
    from tinytorch_b200.function import sdpAttention
    shp = (1, 2, 96, 64)
    (q, qn), (k, kn), (v, vn), (do, don) = (make(shp, torch.float32, 91 + i) for i in range(4))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    for _ in range(2):
        y = sdpAttention(q, k, v, True)
        y.backward(do)
    torch.cuda.synchronize()
    wq, wk, wv = oracle.bwd(qn, kn, vn, don, causal=True)
    assert rel_err(to_np(q.grad), 2 * wq) <= TOL_REL_FP32
    assert rel_err(to_np(k.grad), 2 * wk) <= TOL_REL_FP32
    assert rel_err(to_np(v.grad), 2 * wv) <= TOL_REL_FP32
    # only V requires grad: dQ / dK are skipped
    q2, k2, v2 = q.detach(), k.detach(), v.detach().requires_grad_(True)
    sdpAttention(q2, k2, v2, True).backward(do)
    assert rel_err(to_np(v2.grad), wv) <= TOL_REL_FP32
