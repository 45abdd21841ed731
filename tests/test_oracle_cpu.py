"""CPU: pins the plain-C oracle against the reference's known answers, against
fixtures produced by the reference's own code, and (where the compiled reference
is present) against the reference live."""
import json
import os

import numpy as np
import pytest

from conftest import GOLDEN, rel_err


def _known():
    with open(os.path.join(GOLDEN, "ref_known_answers.json")) as f:
        return json.load(f)


def test_known_answers_of_reference_test(oracle):
    # test/test_function.cpp:393-419, abs 1e-3 (test/test.h:17-30)
    ka = _known()
    sh = ka["shape"]
    q, k, v = (np.array(ka[n], dtype=np.float32).reshape(sh) for n in ("q", "k", "v"))
    o, _ = oracle.fwd(q, k, v)
    assert np.abs(o.ravel() - np.array(ka["expect_plain"])).max() <= 1e-3
    o, _ = oracle.fwd(q, k, v, causal=True)
    assert np.abs(o.ravel() - np.array(ka["expect_causal"])).max() <= 1e-3
    # and bit-for-bit what the reference code itself produced for them
    assert np.array_equal(o.ravel(), np.array(ka["reference_causal"], dtype=np.float32))


def test_fully_masked_row_is_nan_like_reference(oracle):
    # third case of the reference test: rows with no kept key are NaN (0 * inf)
    ka = _known()
    sh = ka["shape"]
    q, k, v = (np.array(ka[n], dtype=np.float32).reshape(sh) for n in ("q", "k", "v"))
    bias = np.where(np.array([[0, 0], [1, 0]], dtype=bool), 0.0, -np.inf).astype(np.float32)
    o, _ = oracle.fwd(q, k, v, bias=bias)
    assert np.isnan(o[:, :, 0]).all()
    assert np.allclose(o[:, :, 1], v[:, :, 0], atol=1e-6)


def test_seeded_causal_fwd_bwd_bitexact(oracle, seeded):
    s = seeded
    o, lse = oracle.fwd(s["c_q"], s["c_k"], s["c_v"], causal=True)
    assert np.array_equal(o, s["c_o"])
    assert np.abs(lse - s["c_lse"]).max() < 5e-6
    dq, dk, dv = oracle.bwd(s["c_q"], s["c_k"], s["c_v"], s["c_do"], causal=True)
    assert np.array_equal(dq, s["c_dq"])
    assert np.array_equal(dk, s["c_dk"])
    assert np.array_equal(dv, s["c_dv"])


def test_seeded_decode_lengths_bitexact(oracle, seeded):
    s = seeded
    o, _ = oracle.fwd(s["d_q"], s["d_k"], s["d_v"], kv_lens=s["d_lens"])
    assert np.array_equal(o, s["d_o"])


def test_seeded_gqa_matches_repeat_path(oracle, seeded):
    s = seeded
    o, _ = oracle.fwd(s["g_q"], s["g_k"], s["g_v"], causal=True)
    assert np.array_equal(o, s["g_o"])


def test_seeded_scale_and_rectangular(oracle, seeded):
    s = seeded
    o, _ = oracle.fwd(s["s_q"], s["s_k"], s["s_v"], scale=float(s["s_scale"]))
    assert np.array_equal(o, s["s_o"])
    o, _ = oracle.fwd(s["s_q"], s["s_k"], s["s_v"], causal=True, scale=float(s["s_scale"]))
    assert np.array_equal(o, s["s_o_causal"])


def test_config1_live_against_reference(oracle, reference):
    # B=2 H=4 S=128 D=64 fp32 causal, N(0,1) inputs from a seed
    rng = np.random.default_rng(1235)
    q, k, v, do = (rng.standard_normal((2, 4, 128, 64), dtype=np.float32) for _ in range(4))
    o, lse = oracle.fwd(q, k, v, causal=True)
    ro, rdq, rdk, rdv = reference.grad(q, k, v, do, causal=True)
    assert np.array_equal(o, reference.fwd(q, k, v, causal=True))
    assert np.array_equal(o, ro)
    dq, dk, dv = oracle.bwd(q, k, v, do, causal=True)
    assert np.array_equal(dq, rdq) and np.array_equal(dk, rdk) and np.array_equal(dv, rdv)
    assert np.abs(lse - reference.lse(q, k, causal=True)).max() < 5e-6


def test_oracle_against_torch_fp64(oracle):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(7)
    q = rng.standard_normal((1, 4, 50, 64), dtype=np.float32)
    k, v = (rng.standard_normal((1, 2, 70, 64), dtype=np.float32) for _ in range(2))
    do = rng.standard_normal(q.shape, dtype=np.float32)
    lens = np.array([33], dtype=np.int32)
    tq, tk, tv = (torch.tensor(x, dtype=torch.float64, requires_grad=True) for x in (q, k, v))
    ke, ve = tk.repeat_interleave(2, 1), tv.repeat_interleave(2, 1)
    s = (tq @ ke.transpose(-1, -2)) / 8.0
    s = s.masked_fill(torch.arange(70)[None, None, None, :] >= 33, float("-inf"))
    p = torch.softmax(s, -1)
    y = p @ ve
    y.backward(torch.tensor(do, dtype=torch.float64))
    o, lse = oracle.fwd(q, k, v, kv_lens=lens)
    dq, dk, dv = oracle.bwd(q, k, v, do, kv_lens=lens)
    assert rel_err(o, y.detach().numpy()) < 1e-5
    assert rel_err(lse, torch.logsumexp(s, -1).detach().numpy()) < 1e-5
    assert rel_err(dq, tq.grad.numpy()) < 1e-5
    assert rel_err(dk, tk.grad.numpy()) < 1e-5
    assert rel_err(dv, tv.grad.numpy()) < 1e-5


def test_threads_do_not_change_results(oracle):
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal((2, 3, 40, 64), dtype=np.float32) for _ in range(3))
    n = oracle.threads
    oracle.set_threads(1)
    a, _ = oracle.fwd(q, k, v, causal=True)
    oracle.set_threads(4)
    b, _ = oracle.fwd(q, k, v, causal=True)
    oracle.set_threads(n)
    assert np.array_equal(a, b)


def _bias_of(mask):
    mask = np.asarray(mask)
    if mask.dtype == np.bool_:
        return np.where(mask, np.float32(0), np.float32(-np.inf)).astype(np.float32)
    return mask.astype(np.float32)


def test_seeded_masks_bitexact(oracle):
    # attnMask of the reference (src/Function/FuncNNLayer.h:249-256): Bool [B,1,L,S] and float [L,S]
    g = np.load(os.path.join(GOLDEN, "ref_seeded_mask.npz"))
    q, k, v = g["q"], g["k"], g["v"]
    o, _ = oracle.fwd(q, k, v, bias=_bias_of(g["mask_bool"]))
    assert np.array_equal(o, g["o_bool"])
    o, _ = oracle.fwd(q, k, v, bias=_bias_of(g["mask_float"]))
    assert np.array_equal(o, g["o_float"])
    o, _ = oracle.fwd(q, k, v, bias=_bias_of(g["mask_float"]), scale=0.2)
    assert np.array_equal(o, g["o_float_scale"])


def test_masks_live_against_reference(oracle, reference):
    rng = np.random.default_rng(77)
    B, H, L, S, D = 1, 3, 33, 50, 64
    q = rng.standard_normal((B, H, L, D), dtype=np.float32)
    k, v = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(2))
    m = rng.random((1, H, L, S)) < 0.5
    m[..., 0] = True
    o, _ = oracle.fwd(q, k, v, bias=_bias_of(m))
    assert np.array_equal(o, reference.fwd_mask(q, k, v, m))
