"""GPU parity of the prefill forward against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import rel_err
from gpu_util import DTYPES, TOL_ABS_16BIT, TOL_REL_FP32, check_status, make, to_np

pytestmark = pytest.mark.gpu


def _run(q, k, v, **kw):
    from tinytorch_b200 import op
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o, lse = op.sdpAttentionFwd(q, k, v, status=status, **kw)
    torch.cuda.synchronize()
    check_status(status)
    return o, lse


def test_config1_fp32_causal(oracle, seeded):
    # B=2 H=4 S=128 D=64 fp32 causal: <= 1e-5 relative against the CPU fp32 path
    q, qn = make((2, 4, 128, 64), torch.float32, 1235)
    k, kn = make((2, 4, 128, 64), torch.float32, 1236)
    v, vn = make((2, 4, 128, 64), torch.float32, 1237)
    o, lse = _run(q, k, v, isCausal=True)
    wo, wl = oracle.fwd(qn, kn, vn, causal=True)
    assert rel_err(to_np(o), wo) <= TOL_REL_FP32
    assert rel_err(to_np(lse), wl) <= TOL_REL_FP32


def test_golden_fixture_fp32(seeded):
    # outputs produced by the reference's own code (tests/golden/ref_seeded.npz)
    s = seeded
    q, k, v = (torch.from_numpy(s[n]).cuda() for n in ("c_q", "c_k", "c_v"))
    o, lse = _run(q, k, v, isCausal=True)
    assert rel_err(to_np(o), s["c_o"]) <= TOL_REL_FP32
    assert rel_err(to_np(lse), s["c_lse"]) <= TOL_REL_FP32
    q, k, v = (torch.from_numpy(s[n]).cuda() for n in ("s_q", "s_k", "s_v"))
    o, _ = _run(q, k, v, scale=float(s["s_scale"]))
    assert rel_err(to_np(o), s["s_o"]) <= TOL_REL_FP32
    o, _ = _run(q, k, v, isCausal=True, scale=float(s["s_scale"]))
    assert rel_err(to_np(o), s["s_o_causal"]) <= TOL_REL_FP32
    q, k, v = (torch.from_numpy(s[n]).cuda() for n in ("g_q", "g_k", "g_v"))
    o, _ = _run(q, k, v, isCausal=True)
    assert rel_err(to_np(o), s["g_o"]) <= TOL_REL_FP32


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("L,S,causal", [
    (128, 128, True), (128, 128, False), (256, 256, True), (1, 1, True), (1, 300, False),
    (63, 63, True), (129, 129, True), (200, 328, True), (328, 200, True), (384, 384, False), (130, 77, False),
])
def test_tensor_core_shapes(oracle, dt, D, L, S, causal):
    B, Hq, Hkv = 2, 4, 2
    q, qn = make((B, Hq, L, D), DTYPES[dt], 11)
    k, kn = make((B, Hkv, S, D), DTYPES[dt], 12)
    v, vn = make((B, Hkv, S, D), DTYPES[dt], 13)
    o, lse = _run(q, k, v, isCausal=causal)
    wo, wl = oracle.fwd(qn, kn, vn, causal=causal)
    assert np.abs(to_np(o) - wo).max() <= TOL_ABS_16BIT
    assert np.abs(to_np(lse) - wl).max() <= 2e-3


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("which", ["few_rows", "all_rows"])
def test_row_maximum_grows_in_later_key_tiles(oracle, dt, D, causal, which):
    # The tensor-core kernel keeps a row's reference maximum across key tiles and only takes a new one
    # (rescaling O and the running sum) when a tile's exponentials grow large.  Here late keys score far
    # above the first tile's maximum: for a few rows of a warp only, or for every row.
    B, H, L, S = 1, 2, 512, 512
    rng = np.random.default_rng(21)
    qn = (rng.standard_normal((B, H, L, D)) * 0.5).astype(np.float32)
    kn = (rng.standard_normal((B, H, S, D)) * 0.5).astype(np.float32)
    vn = rng.standard_normal((B, H, S, D)).astype(np.float32)
    if which == "few_rows":
        for row, key in ((300, 140), (305, 290), (420, 400), (511, 130)):
            kn[:, :, key] = qn[:, :, row] * (1200.0 / D)   # score * scale of (row, key) around 25-50
    else:
        kn[:, :, 256:] *= 12.0
        kn[:, :, 400:] *= 3.0
    q, k, v = (torch.from_numpy(x).to(DTYPES[dt]).cuda() for x in (qn, kn, vn))
    o, lse = _run(q, k, v, isCausal=causal)
    wo, wl = oracle.fwd(*(to_np(t) for t in (q, k, v)), causal=causal)
    assert np.abs(to_np(o) - wo).max() <= TOL_ABS_16BIT
    assert np.abs(to_np(lse) - wl).max() <= 2e-2


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_kv_lens_and_scale(oracle, dt):
    B, H, L, S, D = 3, 2, 150, 300, 128
    q, qn = make((B, H, L, D), DTYPES[dt], 21)
    k, kn = make((B, H, S, D), DTYPES[dt], 22)
    v, vn = make((B, H, S, D), DTYPES[dt], 23)
    lens = np.array([300, 1, 129], dtype=np.int32)
    tl = torch.from_numpy(lens).cuda()
    for scale in (0.05, -0.07):
        o, lse = _run(q, k, v, kvLens=tl, scale=scale)
        wo, wl = oracle.fwd(qn, kn, vn, kv_lens=lens, scale=scale)
        if dt == "f32":
            assert rel_err(to_np(o), wo) <= TOL_REL_FP32
        else:
            assert np.abs(to_np(o) - wo).max() <= TOL_ABS_16BIT
        assert np.abs(to_np(lse) - wl).max() <= 2e-3


def test_zero_length_rows_give_zero_and_minus_inf():
    q, _ = make((2, 2, 64, 128), torch.bfloat16, 31)
    k, _ = make((2, 2, 64, 128), torch.bfloat16, 32)
    v, _ = make((2, 2, 64, 128), torch.bfloat16, 33)
    tl = torch.tensor([0, 64], dtype=torch.int32, device="cuda")
    o, lse = _run(q, k, v, kvLens=tl)
    assert float(o[0].abs().max()) == 0.0 and bool(torch.isinf(lse[0]).all())
    assert bool(torch.isfinite(o[1].float()).all())


def test_strided_head_view(oracle):
    # a head-sharded sub-view: strides differ from the dense ones
    B, H, S, D = 2, 6, 192, 128
    q, qn = make((B, H, S, D), torch.bfloat16, 41)
    k, kn = make((B, H, S, D), torch.bfloat16, 42)
    v, vn = make((B, H, S, D), torch.bfloat16, 43)
    o, _ = _run(q[:, 2:4], k[:, 2:4], v[:, 2:4], isCausal=True)
    wo, _ = oracle.fwd(qn[:, 2:4], kn[:, 2:4], vn[:, 2:4], causal=True)
    assert np.abs(to_np(o) - wo).max() <= TOL_ABS_16BIT


def test_config2_full_size_slices(oracle):
    # B=4 H=32 S=4096 D=128 bf16 causal; the oracle checks a few (b, h) slices
    B, H, S, D = 4, 32, 4096, 128
    g = torch.Generator(device="cuda").manual_seed(1236)
    q, k, v = (torch.randn((B, H, S, D), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
               for _ in range(3))
    o, lse = _run(q, k, v, isCausal=True)
    o2, lse2 = _run(q, k, v, isCausal=True)
    assert torch.equal(o, o2) and torch.equal(lse, lse2)  # run-to-run determinism
    assert bool(torch.isfinite(o.float()).all())
    # the first unit, the last one, and one from the middle of the grid (where a CTA changes heads mid-way)
    for (b, h) in ((0, 0), (1, 19), (3, 31)):
        qn, kn, vn = (to_np(t[b:b + 1, h:h + 1]) for t in (q, k, v))
        wo, wl = oracle.fwd(qn, kn, vn, causal=True)
        assert np.abs(to_np(o[b:b + 1, h:h + 1]) - wo).max() <= TOL_ABS_16BIT
        assert np.abs(to_np(lse[b:b + 1, h:h + 1]) - wl).max() <= 2e-3
    # size-independent property: row 0 of a causal head attends key 0 only -> O[0] == V[0]
    assert torch.equal(o[:, :, 0], v[:, :, 0])
    # linearity in V: O(V) + O(V') == O(V + V') up to output rounding
    v2 = torch.randn((B, H, S, D), generator=g, device="cuda").to(torch.bfloat16)
    oa, _ = _run(q, k, v2, isCausal=True)
    ob, _ = _run(q, k, (v.float() + v2.float()).to(torch.bfloat16), isCausal=True)
    assert float((o.float() + oa.float() - ob.float()).abs().max()) <= 6e-2


def test_config3_gqa_fp16_slices(oracle):
    # B=8, 32 query heads on 8 kv heads, S=2048, D=128, fp16, causal, N(0, sigma=0.5)
    B, Hq, Hkv, S, D = 8, 32, 8, 2048, 128
    g = torch.Generator(device="cuda").manual_seed(1237)
    q = (torch.randn((B, Hq, S, D), generator=g, device="cuda") * 0.5).half()
    k = (torch.randn((B, Hkv, S, D), generator=g, device="cuda") * 0.5).half()
    v = (torch.randn((B, Hkv, S, D), generator=g, device="cuda") * 0.5).half()
    o, lse = _run(q, k, v, isCausal=True)
    for (b, hk) in ((0, 0), (4, 3), (7, 7)):
        qn = to_np(q[b:b + 1, hk * 4:hk * 4 + 4])
        kn, vn = to_np(k[b:b + 1, hk:hk + 1]), to_np(v[b:b + 1, hk:hk + 1])
        wo, wl = oracle.fwd(qn, kn, vn, causal=True)
        assert np.abs(to_np(o[b:b + 1, hk * 4:hk * 4 + 4]) - wo).max() <= TOL_ABS_16BIT
        assert np.abs(to_np(lse[b:b + 1, hk * 4:hk * 4 + 4]) - wl).max() <= 2e-3
