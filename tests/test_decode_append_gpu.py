"""GPU checks of the fused decode step (rotary embedding of q and the new key, append of the new
key / value row to the cache, attention over the appended cache) through the C ABI.

The attention itself is checked against the reference-pinned CPU oracle; the rotation and the
append have no counterpart in the reference and are checked against oracle/rope.py, a numpy
restatement of the published algorithm (parity unpinned for that part)."""
import numpy as np
import pytest
import torch

from conftest import rel_err
from gpu_util import DTYPES, TOL_ABS_16BIT, TOL_REL_FP32, make, to_np

pytestmark = pytest.mark.gpu


def _round(x, dtype):
    return torch.from_numpy(x).to(dtype).float().numpy()


def _step(oracle, dt, D, Hq, Hkv, cap, lens, interleaved, use_rope=True, seed=400):
    from oracle import rope
    from tinytorch_b200 import op
    B = len(lens)
    dtype = DTYPES[dt]
    q, qn = make((B, Hq, 1, D), dtype, seed + 1)
    kc, kcn = make((B, Hkv, cap, D), dtype, seed + 2)
    vc, vcn = make((B, Hkv, cap, D), dtype, seed + 3)
    kn_t, knn = make((B, Hkv, 1, D), dtype, seed + 4)
    vn_t, vnn = make((B, Hkv, 1, D), dtype, seed + 5)
    lens = np.asarray(lens, dtype=np.int32)
    cos_t = sin_t = None
    q_rot, k_rot = qn, knn
    if use_rope:
        cos_n, sin_n = rope.tables(cap, D)
        cos_t, sin_t = op.ropeTables(cap, D)
        assert np.abs(to_np(cos_t) - cos_n).max() <= 1e-6
        q_rot = rope.rotate(qn, lens, cos_n, sin_n, interleaved)
        k_rot = _round(rope.rotate(knn, lens, cos_n, sin_n, interleaved), dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    k_before, v_before = kc.clone(), vc.clone()
    o, lse, new_lens = op.sdpAttentionDecodeAppend(q, kn_t, vn_t, kc, vc, torch.from_numpy(lens).cuda(), cos_t, sin_t,
                                                   interleaved=interleaved, needLse=True, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert np.array_equal(new_lens.cpu().numpy(), lens + 1)
    # the caches: row lens[b] holds the rotated key / the new value, every other row is untouched
    tol = 1e-6 if dt == "f32" else 2e-2
    for b in range(B):
        p = int(lens[b])
        assert np.abs(to_np(kc[b, :, p]) - k_rot[b, :, 0]).max() <= tol * max(1.0, np.abs(k_rot).max())
        assert torch.equal(vc[b, :, p], vn_t[b, :, 0])
        keep = torch.ones(cap, dtype=torch.bool, device="cuda")
        keep[p] = False
        assert torch.equal(kc[b][:, keep], k_before[b][:, keep]) and torch.equal(vc[b][:, keep], v_before[b][:, keep])
    # attention of the rotated query over the appended cache, by the attention oracle
    wo, wl = oracle.fwd(q_rot, to_np(kc), to_np(vc), kv_lens=lens + 1)
    if dt == "f32":
        assert rel_err(to_np(o), wo) <= 2 * TOL_REL_FP32
    else:
        assert np.abs(to_np(o) - wo).max() <= TOL_ABS_16BIT
    assert np.abs(to_np(lse) - wl[:, :, 0]).max() <= (1e-4 if dt == "f32" else 2e-2)


@pytest.mark.parametrize("dt", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("Hq,Hkv,cap,lens", [
    (4, 4, 100, (0, 99, 37)),          # empty cache, last free row
    (8, 2, 1500, (511, 512, 1499)),    # either side of a split boundary, last row of the last split
    (6, 2, 2049, (2048, 1024, 5)),
    (8, 1, 700, (1, 350, 698)),
])
def test_decode_append_with_rope(oracle, dt, D, interleaved, Hq, Hkv, cap, lens):
    _step(oracle, dt, D, Hq, Hkv, cap, lens, interleaved)


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_decode_append_without_rope(oracle, dt):
    _step(oracle, dt, 128, 8, 2, 900, (0, 600, 899), False, use_rope=False)


def test_token_loop_matches_prefill(oracle):
    # eight steps of the loop from an empty cache equal causal prefill over the same eight tokens
    # (keys rotated to their own positions, queries to theirs)
    from oracle import rope
    from tinytorch_b200 import op
    B, Hq, Hkv, D, cap, T = 2, 4, 2, 64, 64, 8
    q, qn = make((B, Hq, T, D), torch.float32, 411)
    k, kn = make((B, Hkv, T, D), torch.float32, 412)
    v, vn = make((B, Hkv, T, D), torch.float32, 413)
    cos_t, sin_t = op.ropeTables(cap, D)
    cos_n, sin_n = rope.tables(cap, D)
    kc = torch.zeros((B, Hkv, cap, D), device="cuda")
    vc = torch.zeros((B, Hkv, cap, D), device="cuda")
    lens = torch.zeros(B, dtype=torch.int32, device="cuda")
    outs = []
    for t in range(T):
        o, _, lens = op.sdpAttentionDecodeAppend(q[:, :, t:t + 1].contiguous(), k[:, :, t:t + 1].contiguous(),
                                                 v[:, :, t:t + 1].contiguous(), kc, vc, lens, cos_t, sin_t)
        outs.append(o)
    torch.cuda.synchronize()
    got = to_np(torch.cat(outs, dim=2))
    pos = np.zeros(B, dtype=np.int32)
    q_rot = np.concatenate([rope.rotate(qn[:, :, t:t + 1], pos + t, cos_n, sin_n) for t in range(T)], axis=2)
    k_rot = np.concatenate([rope.rotate(kn[:, :, t:t + 1], pos + t, cos_n, sin_n) for t in range(T)], axis=2)
    want, _ = oracle.fwd(q_rot, k_rot, vn, causal=True)
    assert rel_err(got, want) <= 2 * TOL_REL_FP32
    assert np.array_equal(lens.cpu().numpy(), np.full(B, T, dtype=np.int32))


def test_full_cache_and_table_range_are_reported(oracle):
    from tinytorch_b200 import op
    B, H, D, cap = 2, 2, 64, 40
    q, qn = make((B, H, 1, D), torch.bfloat16, 421)
    kc, kcn = make((B, H, cap, D), torch.bfloat16, 422)
    vc, vcn = make((B, H, cap, D), torch.bfloat16, 423)
    kn_t, _ = make((B, H, 1, D), torch.bfloat16, 424)
    vn_t, _ = make((B, H, 1, D), torch.bfloat16, 425)
    lens = np.array([cap, 3], dtype=np.int32)  # sequence 0 has no free row
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    k_before = kc.clone()
    o, _, new_lens = op.sdpAttentionDecodeAppend(q, kn_t, vn_t, kc, vc, torch.from_numpy(lens).cuda(), status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & 4
    assert torch.equal(kc[0], k_before[0])                       # nothing written for the full sequence
    assert list(new_lens.cpu().numpy()) == [cap, 4]
    wo, _ = oracle.fwd(qn[:1], kcn[:1], vcn[:1])                  # ... which attends over its whole cache
    assert np.abs(to_np(o[:1]) - wo).max() <= TOL_ABS_16BIT
    # a position beyond the rotary tables: rotation skipped, bit 8
    cos_t, sin_t = op.ropeTables(2, D)
    status.zero_()
    op.sdpAttentionDecodeAppend(q, kn_t, vn_t, kc, vc, torch.from_numpy(np.array([1, 5], dtype=np.int32)).cuda(),
                                cos_t, sin_t, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & 8
