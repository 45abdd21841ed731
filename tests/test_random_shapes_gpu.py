"""Seeded random shapes for the kernels with the most synchronisation (tensor-core decode, projection, prefill and
backward with ragged sizes), each against the CPU oracle."""
import numpy as np
import pytest
import torch

from gpu_util import DTYPES, TOL_ABS_16BIT, make, to_np

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", range(24))
def test_random_grouped_query_decode(oracle, seed):
    from tinytorch_b200 import op
    rng = np.random.default_rng(1000 + seed)
    D = int(rng.choice([64, 128]))
    group = int(rng.choice([2, 3, 4, 5, 8, 16]))
    Hkv = int(rng.integers(1, 5))
    B = int(rng.integers(1, 7))
    cap = int(rng.integers(1, 40)) * int(rng.choice([1, 7, 64, 128]))
    dt = str(rng.choice(["bf16", "f16"]))
    lens = rng.integers(0, cap + 1, size=B).astype(np.int32)   # 0: a sequence without any key
    if seed % 3 == 0:
        lens[0] = cap
    q, qn = make((B, Hkv * group, 1, D), DTYPES[dt], 2000 + seed)
    k, kn = make((B, Hkv, cap, D), DTYPES[dt], 3000 + seed)
    v, vn = make((B, Hkv, cap, D), DTYPES[dt], 4000 + seed)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o, lse = op.sdpAttentionDecode(q, k, v, torch.from_numpy(lens).cuda(), needLse=True)
    torch.cuda.synchronize()
    live = lens > 0
    if live.any():
        wo, wl = oracle.fwd(qn[live], kn[live], vn[live], kv_lens=lens[live])
        assert np.abs(to_np(o)[live] - wo).max() <= TOL_ABS_16BIT
        assert np.abs(to_np(lse)[live] - wl[:, :, 0]).max() <= 2e-2
    if (~live).any():
        assert float(o[torch.from_numpy(~live).cuda()].float().abs().max()) == 0.0


@pytest.mark.parametrize("seed", range(12))
def test_random_projection(seed):
    from oracle.loader import FusedOracle
    from tinytorch_b200 import fused as F
    rng = np.random.default_rng(5000 + seed)
    M = int(rng.integers(1, 700))
    N = 8 * int(rng.integers(1, 120))
    K = 8 * int(rng.integers(1, 90))
    dt = str(rng.choice(["bf16", "f16"]))
    x, xn = make((M, K), DTYPES[dt], 5100 + seed, std=0.5)
    w, wn = make((N, K), DTYPES[dt], 5200 + seed, std=0.5)
    b, bn = make((N,), DTYPES[dt], 5300 + seed)
    use_bias = bool(seed % 2)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = F._linear_raw(x, w, b if use_bias else None, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = FusedOracle().linear(xn, wn, bn if use_bias else None)
    assert np.abs(to_np(y) - want).max() <= TOL_ABS_16BIT * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("seed", range(12))
def test_random_prefill_and_backward(oracle, seed):
    from tinytorch_b200 import op
    rng = np.random.default_rng(6000 + seed)
    D = int(rng.choice([64, 128]))
    Hkv = int(rng.integers(1, 3))
    group = int(rng.choice([1, 2, 4]))
    B = int(rng.integers(1, 3))
    L = int(rng.integers(1, 400))
    S = int(rng.integers(1, 400))
    causal = [False, True, "bottom-right"][seed % 3]
    dt = str(rng.choice(["bf16", "f16"]))
    lens = rng.integers(1, S + 1, size=B).astype(np.int32)
    q, qn = make((B, Hkv * group, L, D), DTYPES[dt], 6100 + seed)
    k, kn = make((B, Hkv, S, D), DTYPES[dt], 6200 + seed)
    v, vn = make((B, Hkv, S, D), DTYPES[dt], 6300 + seed)
    do, don = make((B, Hkv * group, L, D), DTYPES[dt], 6400 + seed)
    kw = dict(isCausal=causal, kvLens=torch.from_numpy(lens).cuda())
    o, lse = op.sdpAttentionFwd(q, k, v, **kw)
    dq, dk, dv = op.sdpAttentionBwd(do, q, k, v, o, lse, **kw)
    torch.cuda.synchronize()
    if causal == "bottom-right":
        i, j = np.arange(L)[:, None], np.arange(S)[None, :]
        bias = np.zeros((B, 1, L, S), dtype=np.float32)
        for b in range(B):
            bias[b, 0][j > i + (int(lens[b]) - L)] = -np.inf
        okw = dict(kv_lens=lens, bias=bias)
    else:
        okw = dict(kv_lens=lens, causal=bool(causal))
    wo, _ = oracle.fwd(qn, kn, vn, **okw)
    wq, wk, wv = oracle.bwd(qn, kn, vn, don, **okw)
    dead = np.isnan(wo).any(axis=-1)          # rows without any participating key: NaN in the reference, 0 here
    got = to_np(o)
    assert np.abs(np.where(dead[..., None], 0, got - np.nan_to_num(wo))).max() <= TOL_ABS_16BIT
    assert float(np.abs(got[dead]).max()) == 0.0 if dead.any() else True
    if not dead.any():
        for g_, w_ in ((dq, wq), (dk, wk), (dv, wv)):
            assert np.abs(to_np(g_) - w_).max() <= TOL_ABS_16BIT * max(1.0, np.abs(w_).max())
