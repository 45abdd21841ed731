"""Regenerates the committed golden fixtures from the reference itself.

Needs oracle/_ref/libref_attn.so, i.e. the reference's own CPU sources compiled
by oracle/Makefile where the reference tree is mounted.  Run from the repo root:

    python tests/golden/make_golden.py

Outputs (both committed):
  ref_known_answers.json   inputs / expected values of the reference's attention
                           known-answer test (test/test_function.cpp:393-419, 1e-3
                           absolute as in test/test.h:17-30) plus what the reference
                           code computes for them here
  ref_seeded.npz           seeded inputs and the reference's outputs for small
                           causal fwd+bwd, length-masked decode and GQA cases
  ref_seeded_fused.npz     seeded inputs and the reference's outputs of op::siluMul and
                           op::fusedAddRmsNorm (src/Operation/OpFusedCpu.h:14-72)
  ref_seeded_linear.npz    function::linear: the reference's known-answer vectors
                           (test/test_function.cpp:234-248, asserted here) and a seeded
                           forward / backward case
  ref_seeded_mask.npz      the same for attnMask: a Bool mask [B,1,L,S] and a float
                           mask [L,S] (src/Function/FuncNNLayer.h:249-256)
"""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from oracle.loader import Reference  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ref = Reference()
    # --- the reference's own known-answer vectors (test/test_function.cpp:394-418)
    q = [0.6201, 0.5199, 0.2614, 0.9816, 0.9369, 0.8059, 0.8578, 0.7864, 0.8947, 0.4272, 0.7566, 0.2975, 0.4676,
         0.1170, 0.1046, 0.7130]
    k = [0.8691, 0.8571, 0.9015, 0.3962, 0.7809, 0.0260, 0.7946, 0.6102, 0.0999, 0.9367, 0.3174, 0.1418, 0.6388,
         0.4654, 0.5967, 0.3617]
    v = [0.9904, 0.8726, 0.8662, 0.3096, 0.4391, 0.9327, 0.5259, 0.6763, 0.6314, 0.8901, 0.6936, 0.2933, 0.0599,
         0.3249, 0.3593, 0.8228]
    expect_plain = [0.9331, 0.6129, 0.9380, 0.6349, 0.4899, 0.7828, 0.4897, 0.7833, 0.6609, 0.6070, 0.6617, 0.5993,
                    0.2079, 0.5711, 0.2054, 0.5670]
    expect_causal = [0.9904, 0.8726, 0.9380, 0.6349, 0.4391, 0.9327, 0.4897, 0.7833, 0.6314, 0.8901, 0.6617, 0.5993,
                     0.0599, 0.3249, 0.2055, 0.5670]
    sh = (2, 2, 2, 2)
    qa, ka, va = (np.array(x, dtype=np.float32).reshape(sh) for x in (q, k, v))
    got_plain = ref.fwd(qa, ka, va, causal=False)
    got_causal = ref.fwd(qa, ka, va, causal=True)
    assert np.abs(got_plain.ravel() - expect_plain).max() <= 1e-3
    assert np.abs(got_causal.ravel() - expect_causal).max() <= 1e-3
    with open(os.path.join(HERE, "ref_known_answers.json"), "w") as f:
        json.dump({
            "source": "test/test_function.cpp:393-419 (abs tolerance 1e-3, test/test.h:17-30)",
            "shape": list(sh), "q": q, "k": k, "v": v,
            "expect_plain": expect_plain, "expect_causal": expect_causal,
            "reference_plain": [float(x) for x in got_plain.ravel()],
            "reference_causal": [float(x) for x in got_causal.ravel()],
            "note": "the test's third case (bool mask with fully masked rows) yields NaN in the reference "
                    "(src/Operation/OpNNLayerCpu.h:28-54) and is not a usable vector",
        }, f, indent=1)

    # --- seeded cases through the reference
    rng = np.random.default_rng(20240607)
    out = {}
    B, H, S, D = 1, 2, 96, 64
    Q, K, V, dO = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(4))
    o, dq, dk, dv = ref.grad(Q, K, V, dO, causal=True)
    assert np.array_equal(o, ref.fwd(Q, K, V, causal=True))
    out.update(c_q=Q, c_k=K, c_v=V, c_do=dO, c_o=o, c_dq=dq, c_dk=dk, c_dv=dv, c_lse=ref.lse(Q, K, causal=True))
    # decode-shaped: one query, bool length mask (src/Function/FuncNNLayer.h:249-252)
    B, H, S, D = 3, 1, 120, 64
    Q = rng.standard_normal((B, H, 1, D), dtype=np.float32)
    K, V = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(2))
    lens = np.array([120, 1, 77], dtype=np.int32)
    out.update(d_q=Q, d_k=K, d_v=V, d_lens=lens, d_o=ref.fwd(Q, K, V, kv_lens=lens))
    # grouped-query: the reference's repeat path (src/Operation/OpTransform.h:168)
    B, Hq, Hkv, S, D = 1, 4, 2, 64, 64
    Q = rng.standard_normal((B, Hq, S, D), dtype=np.float32)
    K, V = (rng.standard_normal((B, Hkv, S, D), dtype=np.float32) for _ in range(2))
    Ke, Ve = ref.repeat_interleave(K, Hq // Hkv), ref.repeat_interleave(V, Hq // Hkv)
    out.update(g_q=Q, g_k=K, g_v=V, g_o=ref.fwd(Q, Ke, Ve, causal=True))
    # non-default scale, non-causal, L != S
    B, H, L, S, D = 1, 1, 40, 72, 64
    Q = rng.standard_normal((B, H, L, D), dtype=np.float32)
    K, V = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(2))
    out.update(s_q=Q, s_k=K, s_v=V, s_scale=np.float32(0.3), s_o=ref.fwd(Q, K, V, scale=0.3),
               s_o_causal=ref.fwd(Q, K, V, causal=True, scale=0.3))
    np.savez_compressed(os.path.join(HERE, "ref_seeded.npz"), **out)

    # --- attnMask through the reference's sdpAttention (its own generator, so that
    # ref_seeded.npz stays byte-identical when this part changes)
    rng = np.random.default_rng(20240608)
    B, H, L, S, D = 2, 2, 72, 136, 64
    Q = rng.standard_normal((B, H, L, D), dtype=np.float32)
    K, V = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(2))
    mb = rng.random((B, 1, L, S)) < 0.6
    mb[..., 0] = True  # no fully masked row (those are NaN in the reference)
    mf = rng.standard_normal((L, S)).astype(np.float32)
    mf[rng.random((L, S)) < 0.15] = -np.inf
    mf[:, 0] = 0.25
    np.savez_compressed(os.path.join(HERE, "ref_seeded_mask.npz"), q=Q, k=K, v=V, mask_bool=mb, mask_float=mf,
                        o_bool=ref.fwd_mask(Q, K, V, mb), o_float=ref.fwd_mask(Q, K, V, mf),
                        o_float_scale=ref.fwd_mask(Q, K, V, mf, scale=0.2))

    # --- the two fused transformer-block operators
    rng = np.random.default_rng(20240609)
    x = (rng.standard_normal((3, 5, 176)) * 2).astype(np.float32)
    inp = rng.standard_normal((7, 200)).astype(np.float32)
    res = rng.standard_normal((7, 200)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(200)).astype(np.float32)
    n_in, n_res = ref.fused_add_rms_norm(inp, res, w, 1e-5)
    # function::linear: the reference's own known answer (test/test_function.cpp:234-248) and a seeded case
    kx = np.array([[-0.3089, 0.5301, -0.0245], [1.5852, 0.8954, 0.7485]], dtype=np.float32)
    kw = np.array([[0.8397, 1.7990, -0.2738], [-0.8910, -0.6746, 0.3419]], dtype=np.float32)
    kb = np.array([-0.9601, -1.4163], dtype=np.float32)
    ky = ref.linear(kx, kw, kb)
    assert abs(float(ky.sum()) - (-3.1661377)) <= 1e-5
    kdx, kdw, kdb = ref.linear_grad(kx, kw, kb, np.ones_like(ky))
    assert np.abs(kdx.ravel() - [-0.0512999892, 1.1244, 0.0681000054] * 2).max() <= 1e-4
    assert np.abs(kdw.ravel() - [1.2763, 1.42549992, 0.724] * 2).max() <= 1e-4 and list(kdb) == [2.0, 2.0]
    lx = rng.standard_normal((37, 72)).astype(np.float32)
    lw = rng.standard_normal((40, 72)).astype(np.float32)
    lb = rng.standard_normal(40).astype(np.float32)
    ldy = rng.standard_normal((37, 40)).astype(np.float32)
    ldx, ldw, ldb = ref.linear_grad(lx, lw, lb, ldy)
    np.savez_compressed(os.path.join(HERE, "ref_seeded_linear.npz"), known_x=kx, known_w=kw, known_b=kb, known_y=ky,
                        x=lx, w=lw, b=lb, y=ref.linear(lx, lw, lb), y_nobias=ref.linear(lx, lw), dy=ldy, dx=ldx, dw=ldw,
                        db=ldb)
    np.savez_compressed(os.path.join(HERE, "ref_seeded_fused.npz"), silu_x=x, silu_out=ref.silu_mul(x),
                        rms_input=inp, rms_residual=res, rms_weight=w, rms_eps=np.float32(1e-5),
                        rms_out_input=n_in, rms_out_residual=n_res)
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main()
