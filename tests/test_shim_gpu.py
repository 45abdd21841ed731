"""GPU: the C++ binding (tinytorch_b200/shim/TinyTorchFusedAttention.h) run inside the reference itself.

oracle/_ref/shim_driver is the UNMODIFIED reference (its .cpp and .cu sources compiled with USE_CUDA for
sm_100a by `make -C oracle refcuda`), the binding header, tests/cxx/shim_driver.cpp and libtt_attn.so.  The
driver calls function::sdpAttentionFused exactly as the patched call site of the reference would
(src/Function/FuncNNLayer.h:298-302): Function<>::apply (src/Tensor/Function.h:106-144), the dispatch table
(src/Tensor/Dispatch.h:110-142), AutogradMeta::addGrad (src/Tensor/AutogradMeta.cpp:29-43).  Tensors travel as
raw float32 files; this module makes the inputs and checks what comes back against the CPU oracle.
"""
import json
import os
import re
import subprocess

import numpy as np
import pytest

from conftest import GOLDEN, ROOT, rel_err

pytestmark = pytest.mark.gpu

DRIVER = os.path.join(ROOT, "oracle", "_ref", "shim_driver")


@pytest.fixture(scope="module")
def driver():
    if not os.path.exists(DRIVER):
        pytest.skip("oracle/_ref/shim_driver not built (`make -C oracle refcuda` needs the reference tree)")

    def run(args, env=None):
        e = dict(os.environ)
        e.update(env or {})
        r = subprocess.run([DRIVER] + [str(a) for a in args], capture_output=True, text=True, timeout=600, env=e)
        assert r.returncode == 0, "shim_driver failed (%d):\n%s\n%s" % (r.returncode, r.stdout[-2000:], r.stderr[-2000:])
        m = re.search(r"fused_calls=(\d+) ms=([0-9.]+)", r.stdout)
        assert m, r.stdout
        return int(m.group(1)), float(m.group(2))

    return run


def _save(tmp, name, arr):
    p = os.path.join(str(tmp), name)
    np.ascontiguousarray(arr, dtype=np.float32).tofile(p)
    return p


def _load(tmp, name, shape):
    return np.fromfile(os.path.join(str(tmp), name), dtype=np.float32).reshape(shape)


def _fwd(driver, tmp, q, k, v, dtype, causal, impl="fused", chunk=1, offset=0, env=None):
    N, Hq, L, D = q.shape
    Hkv, S = k.shape[1], k.shape[2]
    files = [_save(tmp, n, a) for n, a in (("q.bin", q), ("k.bin", k), ("v.bin", v))]
    out = os.path.join(str(tmp), "o.bin")
    calls, ms = driver(["fwd", dtype, N, Hq, Hkv, L, S, D, int(causal), impl, chunk, offset] + files + [out], env=env)
    return _load(tmp, "o.bin", q.shape), calls, ms


def _round(x, dtype):
    import torch
    dt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[dtype]
    return torch.from_numpy(x).to(dt).float().numpy()


def test_reference_known_answers_through_the_drop_in(driver, tmp_path):
    # test/test_function.cpp:393-419 (abs 1e-3): head dimension 2, so the drop-in must hand these to the
    # original composition and leave the answers as they were
    with open(os.path.join(GOLDEN, "ref_known_answers.json")) as f:
        ka = json.load(f)
    q, k, v = (np.array(ka[n], dtype=np.float32).reshape(ka["shape"]) for n in ("q", "k", "v"))
    o, calls, _ = _fwd(driver, tmp_path, q, k, v, "f32", False)
    assert calls == 0
    assert np.abs(o.ravel() - np.array(ka["expect_plain"])).max() <= 1e-3
    o, calls, _ = _fwd(driver, tmp_path, q, k, v, "f32", True)
    assert calls == 0
    assert np.abs(o.ravel() - np.array(ka["expect_causal"])).max() <= 1e-3


def test_config1_forward_and_autograd_through_function_apply(driver, oracle, seeded, tmp_path):
    # config 1 (fp32, B2 H4 S128 D64, causal): y.backward(dO) through FuncSDPAttentionFused against the CPU
    # oracle at 1e-5; run twice, the leaves must hold twice the gradient (AutogradMeta::addGrad)
    s = seeded
    q, k, v, do = s["c_q"], s["c_k"], s["c_v"], s["c_do"]
    wo, _ = oracle.fwd(q, k, v, causal=True)
    wdq, wdk, wdv = oracle.bwd(q, k, v, do, causal=True)
    files = [_save(tmp_path, n, a) for n, a in (("q.bin", q), ("k.bin", k), ("v.bin", v), ("do.bin", do))]
    outs = [os.path.join(str(tmp_path), n) for n in ("o.bin", "dq.bin", "dk.bin", "dv.bin")]
    N, H, L, D = q.shape
    for reps in (1, 2):
        calls, _ = driver(["fwdbwd", "f32", N, H, H, L, L, D, 1, reps, 1, 1, 1] + files + outs)
        assert calls == reps
        assert rel_err(_load(tmp_path, "o.bin", q.shape), wo) <= 1e-5
        for name, want in (("dq.bin", wdq), ("dk.bin", wdk), ("dv.bin", wdv)):
            assert rel_err(_load(tmp_path, name, q.shape), reps * want) <= 1e-5, (name, reps)
    # only V requires a gradient: dV as before, and the driver fails if q or k were marked or given one
    calls, _ = driver(["fwdbwd", "f32", N, H, H, L, L, D, 1, 1, 0, 0, 1] + files + outs)
    assert calls == 1
    assert rel_err(_load(tmp_path, "dv.bin", q.shape), wdv) <= 1e-5


def test_runtime_switch_forces_the_original_composition(driver, oracle, tmp_path):
    rng = np.random.default_rng(5)
    q, k, v = (rng.standard_normal((2, 2, 96, 64)).astype(np.float32) for _ in range(3))
    want, _ = oracle.fwd(q, k, v, causal=True)
    o, calls, _ = _fwd(driver, tmp_path, q, k, v, "f32", True)
    assert calls == 2 and rel_err(o, want) <= 1e-5          # warm-up + timed call, both fused
    o, calls, _ = _fwd(driver, tmp_path, q, k, v, "f32", True, env={"TINYTORCH_FUSED_ATTENTION": "0"})
    assert calls == 0                                        # same call site, reference composition
    assert rel_err(o, want) <= 2e-3                          # (its fp32 matmul runs in TF32 on the GPU)


def test_misaligned_view_falls_back_instead_of_failing(driver, oracle, tmp_path):
    rng = np.random.default_rng(6)
    q, k, v = (rng.standard_normal((1, 2, 64, 64)).astype(np.float32) for _ in range(3))
    want, _ = oracle.fwd(q, k, v)
    o, calls, _ = _fwd(driver, tmp_path, q, k, v, "f32", False, offset=1)   # q starts 4 bytes into its storage
    assert calls == 0
    assert rel_err(o, want) <= 2e-3
    o, calls, _ = _fwd(driver, tmp_path, q, k, v, "f32", False, offset=4)   # 16 bytes: aligned again
    assert calls == 2
    assert rel_err(o, want) <= 1e-5


@pytest.mark.parametrize("dtype,L,D,std", [("bf16", 4096, 128, 1.0), ("f16", 2048, 128, 0.5), ("f16", 2048, 64, 1.0)])
def test_fused_kernels_against_the_reference_cuda_composition(driver, tmp_path, dtype, L, D, std):
    # The reference's own GPU path (cuBLAS batched gemm + its generic kernels) in the tensors' dtype, on a
    # few (batch, head) slices of configs 2, 3 and 5.  Its large-row softmax launch puts B*H*L on gridDim.y
    # (src/Operation/OpNNLayerCuda.cuh:375), so it is called on chunks with B*H*L <= 65535.
    n = 3
    rng = np.random.default_rng(7)
    q, k, v = ((rng.standard_normal((n, 1, L, D)) * std).astype(np.float32) for _ in range(3))
    q, k, v = (_round(x, dtype) for x in (q, k, v))
    chunk = max(1, 65535 // L)
    ref, calls, _ = _fwd(driver, tmp_path, q, k, v, dtype, True, impl="ref", chunk=min(chunk, n))
    assert calls == 0
    got, calls, _ = _fwd(driver, tmp_path, q, k, v, dtype, True)
    assert calls == 2
    err = float(np.abs(got - ref).max())
    print("fused vs reference CUDA composition, %s L=%d D=%d: max abs diff %.3e" % (dtype, L, D, err))
    assert err <= 2e-2


@pytest.mark.parametrize("N,Hq,Hkv,S,D,dtype", [(4, 8, 8, 8192, 128, "bf16"), (3, 8, 2, 3000, 64, "f16")])
def test_decode_op_against_the_reference_mask_composition(driver, oracle, tmp_path, N, Hq, Hkv, S, D, dtype):
    # config 4's shape on a few sequences: op::sdpAttentionDecode through the dispatch table against what a
    # TinyTorch caller writes without it (sdpAttention with a Bool length mask, the reference's own CUDA kernels),
    # and both against the CPU oracle
    rng = np.random.default_rng(8)
    q = _round(rng.standard_normal((N, Hq, 1, D)).astype(np.float32), dtype)
    k = _round(rng.standard_normal((N, Hkv, S, D)).astype(np.float32), dtype)
    v = _round(rng.standard_normal((N, Hkv, S, D)).astype(np.float32), dtype)
    lens = rng.integers(S // 8, S + 1, size=N).astype(np.int32)
    lens[0] = S
    files = [_save(tmp_path, n, a) for n, a in (("lens.bin", lens.astype(np.float32)), ("q.bin", q), ("k.bin", k), ("v.bin", v))]
    res = {}
    for impl in ("fused", "ref"):
        out = os.path.join(str(tmp_path), impl + ".bin")
        driver(["decode", dtype, N, Hq, Hkv, S, D, impl] + files + [out])
        res[impl] = _load(tmp_path, impl + ".bin", q.shape)
    want, _ = oracle.fwd(q, k, v, kv_lens=lens)
    print("decode %s: fused vs oracle %.3e, reference composition vs oracle %.3e" % (
        dtype, float(np.abs(res["fused"] - want).max()), float(np.abs(res["ref"] - want).max())))
    assert np.abs(res["fused"] - want).max() <= 2e-2
    assert np.abs(res["fused"] - res["ref"]).max() <= 2e-2


@pytest.mark.parametrize("dtype,rows,dim,nout", [("bf16", 300, 1024, 512), ("f16", 64, 4096, 256), ("f32", 33, 200, 0)])
def test_block_operators_replace_the_reference_cuda_entries(dtype, rows, dim, nout):
    # tinytorch_b200/shim/TinyTorchFusedOps.h: after registerFusedOpsB200() the same op::siluMul /
    # op::fusedAddRmsNorm calls reach the B200 kernels; the projection through linearOpB200.  Each against the
    # reference's own CUDA implementation of the same operator on the same tensors (both compute in fp32 and
    # round once, so they differ by at most a unit or two in the last place of the 16-bit result).
    if not os.path.exists(DRIVER):
        pytest.skip("oracle/_ref/shim_driver not built")
    if dtype == "f32":
        nout = 8
    r = subprocess.run([DRIVER, "fusedops", dtype, str(rows), str(dim), str(nout)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr[-1000:])
    d = {k: float(v) for k, v in re.findall(r"(\w+)=(-?[0-9.eE+-]+|nan|inf)", r.stdout)}
    print(r.stdout.strip())
    ulp = {"bf16": 2.0 ** -7, "f16": 2.0 ** -10, "f32": 2.0 ** -23}[dtype]
    assert d["silu"] <= 2 * ulp * 8            # |silu(gate) * up| stays below ~8 for N(0,1) inputs
    assert d["rms_residual"] <= 2 * ulp * 8
    assert d["rms_input"] <= 2 * ulp * 16
    if dtype == "f32":
        assert d["linear"] == -1.0             # linearOpB200 declines fp32: the caller falls back to op::matmul
    else:
        # cuBLAS and the tensor-core kernel sum in different orders; outputs reach |y| ~ 8, where one unit in the
        # last place of bf16 is 0.03
        assert d["linear"] <= 2e-2 + 2 * ulp * 8
