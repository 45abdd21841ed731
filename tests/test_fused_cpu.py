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
