"""CPU checks of the fused-operator oracle (fused_oracle.c) against the reference's own code and
the committed fixture, and of the C ABI's argument validation (no GPU work)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from conftest import GOLDEN, ROOT
from tinytorch_b200 import _capi


@pytest.fixture(scope="module")
def fused():
    from oracle.loader import FusedOracle
    return FusedOracle()


def test_oracle_matches_fixture_bitexact(fused):
    g = np.load(os.path.join(GOLDEN, "ref_seeded_fused.npz"))
    assert np.array_equal(fused.silu_mul(g["silu_x"]), g["silu_out"])
    n_in, n_res = fused.fused_add_rms_norm(g["rms_input"], g["rms_residual"], g["rms_weight"], float(g["rms_eps"]))
    assert np.array_equal(n_res, g["rms_out_residual"])
    assert np.array_equal(n_in, g["rms_out_input"])


def test_oracle_live_against_reference(fused, reference):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((4, 3, 130)) * 3).astype(np.float32)
    assert np.array_equal(fused.silu_mul(x), reference.silu_mul(x))
    inp, res = (rng.standard_normal((5, 77)).astype(np.float32) for _ in range(2))
    w = rng.standard_normal(77).astype(np.float32)
    a = fused.fused_add_rms_norm(inp, res, w, 1e-6)
    b = reference.fused_add_rms_norm(inp, res, w, 1e-6)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_oracle_against_numpy_fp64(fused):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((6, 64)).astype(np.float32)
    g, u = x[:, :32].astype(np.float64), x[:, 32:].astype(np.float64)
    assert np.abs(fused.silu_mul(x) - g / (1 + np.exp(-g)) * u).max() <= 1e-6
    inp, res = (rng.standard_normal((3, 48)).astype(np.float32) for _ in range(2))
    w = rng.standard_normal(48).astype(np.float32)
    n_in, n_res = fused.fused_add_rms_norm(inp, res, w, 1e-5)
    r = inp.astype(np.float64) + res
    want = r / np.sqrt((r * r).mean(-1, keepdims=True) + 1e-5) * w
    assert np.abs(n_res - r).max() <= 1e-6 and np.abs(n_in - want).max() <= 1e-5


def test_linear_oracle_matches_fixture_and_reference_known_answer(fused):
    g = np.load(os.path.join(GOLDEN, "ref_seeded_linear.npz"))
    # the reference's own test vector (test/test_function.cpp:234-241): sum of linear(x, w, b) = -3.1661377
    y = fused.linear(g["known_x"], g["known_w"], g["known_b"])
    assert np.array_equal(y, g["known_y"]) and abs(float(y.sum()) + 3.1661377) <= 1e-5
    assert np.array_equal(fused.linear(g["x"], g["w"], g["b"]), g["y"])
    assert np.array_equal(fused.linear(g["x"], g["w"]), g["y_nobias"])
    # gradients of the fixture are those of three more linear maps: dX = dY W, dW = dY^T X, db = column sums
    assert np.abs(fused.linear(g["dy"], g["w"].T.copy()) - g["dx"]).max() <= 1e-4
    assert np.abs(fused.linear(g["dy"].T.copy(), g["x"].T.copy()) - g["dw"]).max() <= 1e-4
    assert np.abs(g["dy"].sum(0) - g["db"]).max() <= 1e-4


def test_linear_oracle_live_against_reference(fused, reference):
    rng = np.random.default_rng(6)
    x, w, b = rng.standard_normal((9, 50)), rng.standard_normal((13, 50)), rng.standard_normal(13)
    assert np.array_equal(fused.linear(x, w, b), reference.linear(x, w, b))
    assert np.array_equal(fused.linear(x, w), reference.linear(x, w))


def test_linear_rejects_bad_arguments():
    lib = _capi.lib()
    assert lib.tt_linear(None) == -1
    p = _capi.LinearParams()
    p.struct_size = C.sizeof(p)
    p.dtype, p.M, p.N, p.K = 2, 128, 256, 64
    assert lib.tt_linear(C.byref(p)) == -1            # null tensors
    p.x = p.w = p.y = 0x1000
    p.dtype = 0
    assert lib.tt_linear(C.byref(p)) == -2            # Float32 is not served by this kernel
    p.dtype, p.K = 2, 60
    assert lib.tt_linear(C.byref(p)) == -5            # K not a multiple of 8
    p.K, p.ldx = 64, 32
    assert lib.tt_linear(C.byref(p)) == -3            # row stride shorter than a row
    p.ldx, p.N = 0, 0
    assert lib.tt_linear(C.byref(p)) == -3
    p.N, p.M = 256, 0
    assert lib.tt_linear(C.byref(p)) == 0             # nothing to do


def test_library_exports_every_symbol_of_tt_fused_h():
    text = open(os.path.join(ROOT, "include", "tt_fused.h")).read()
    names = re.findall(r"TT_ATTN_API\s+[\w\s\*]+?\b(tt_\w+)\s*\(", text)
    assert set(names) == set(_capi.FUSED_EXPORTS)
    lib = _capi.lib()
    for n in names:
        assert hasattr(lib, n), n


def test_fused_entry_points_reject_bad_arguments():
    lib = _capi.lib()
    assert lib.tt_fused_add_rms_norm(None) == -1 and lib.tt_silu_mul(None) == -1
    p = _capi.AddRmsNormParams()
    p.struct_size = C.sizeof(p)
    p.dtype, p.rows, p.dim = 2, 4, 128
    assert lib.tt_fused_add_rms_norm(C.byref(p)) == -1   # null tensors
    p.input = p.residual = p.weight = 0x1000
    p.dtype = 5
    assert lib.tt_fused_add_rms_norm(C.byref(p)) == -2
    p.dtype, p.dim = 2, 0
    assert lib.tt_fused_add_rms_norm(C.byref(p)) == -3
    p.dim, p.struct_size = 128, 12
    assert lib.tt_fused_add_rms_norm(C.byref(p)) == -8
    s = _capi.SiluMulParams()
    s.struct_size = C.sizeof(s)
    s.dtype, s.rows, s.d = 1, 2, 64
    assert lib.tt_silu_mul(C.byref(s)) == -1
    s.x, s.out = 0x1001, 0x2000
    assert lib.tt_silu_mul(C.byref(s)) == -5             # not even element-aligned
    s.x, s.out, s.rows = None, None, 0
    assert lib.tt_silu_mul(C.byref(s)) == 0              # empty input: nothing to do, no storage needed


def test_python_ops_refuse_cpu_tensors():
    import torch
    from tinytorch_b200 import fused as F
    with pytest.raises(ValueError):
        F.siluMul(torch.zeros(2, 8))
    with pytest.raises(ValueError):
        F.fusedAddRmsNorm(torch.zeros(2, 8), torch.zeros(2, 8), torch.zeros(8), 1e-5)
