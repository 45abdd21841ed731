"""GPU parity of siluMul and fusedAddRmsNorm (src/Operation/OpFusedCuda.cuh:16-142) against the CPU
oracle of the reference's fp32 implementation, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, rel_err
from gpu_util import DTYPES, TOL_ABS_16BIT, TOL_REL_FP32, make, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fused():
    from oracle.loader import FusedOracle
    return FusedOracle()


def test_golden_fixture(fused):
    from tinytorch_b200 import fused as F
    g = np.load(os.path.join(GOLDEN, "ref_seeded_fused.npz"))
    out = F.siluMul(torch.from_numpy(g["silu_x"]).cuda())
    inp, res = torch.from_numpy(g["rms_input"]).cuda(), torch.from_numpy(g["rms_residual"]).cuda()
    F.fusedAddRmsNorm(inp, res, torch.from_numpy(g["rms_weight"]).cuda(), float(g["rms_eps"]))
    torch.cuda.synchronize()
    assert rel_err(to_np(out), g["silu_out"]) <= TOL_REL_FP32
    assert np.array_equal(to_np(res), g["rms_out_residual"])      # one fp32 add: identical
    assert rel_err(to_np(inp), g["rms_out_input"]) <= TOL_REL_FP32


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", [
    (4, 128), (3, 5, 4096), (1, 8192), (300, 1024), (7, 200), (5, 33), (2, 16384), (2, 40000), (1025, 64), (0, 128),
])
def test_fused_add_rms_norm(fused, dt, shape):
    from tinytorch_b200 import fused as F
    inp, inp_n = make(shape, DTYPES[dt], 501)
    res, res_n = make(shape, DTYPES[dt], 502)
    w, w_n = make((shape[-1],), DTYPES[dt], 503)
    F.fusedAddRmsNorm(inp, res, w, 1e-5)
    torch.cuda.synchronize()
    if inp.numel() == 0:
        return
    want_in, want_res = fused.fused_add_rms_norm(inp_n, res_n, w_n, 1e-5)
    if dt == "f32":
        assert np.array_equal(to_np(res), want_res)
        assert rel_err(to_np(inp), want_in) <= TOL_REL_FP32
    else:
        # the residual is the fp32 sum rounded once to the 16-bit dtype
        assert np.array_equal(to_np(res), torch.from_numpy(want_res).to(DTYPES[dt]).float().numpy())
        # the oracle normalises the unrounded residual; the kernel (like the reference's CUDA kernel)
        # the rounded one: one 16-bit rounding of difference, relative to the value
        assert np.abs(to_np(inp) - want_in).max() <= TOL_ABS_16BIT * max(1.0, np.abs(want_in).max())


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", [(4, 256), (3, 5, 8192), (1000, 2048), (7, 200), (5, 34), (2, 3, 22016), (0, 64)])
def test_silu_mul(fused, dt, shape):
    from tinytorch_b200 import fused as F
    x, xn = make(shape, DTYPES[dt], 511, std=2.0)
    out = F.siluMul(x)
    torch.cuda.synchronize()
    assert out.shape == shape[:-1] + (shape[-1] // 2,)
    if x.numel() == 0:
        return
    want = fused.silu_mul(xn)
    if dt == "f32":
        assert rel_err(to_np(out), want) <= TOL_REL_FP32
    else:
        assert np.abs(to_np(out) - want).max() <= TOL_ABS_16BIT * max(1.0, np.abs(want).max())


def test_unaligned_views_take_the_generic_path(fused):
    # a storage offset of one element breaks the 16-byte alignment; results must not change
    from tinytorch_b200 import fused as F
    base = torch.randn(4 * 512 + 1, device="cuda")
    x = base[1:].view(4, 512)
    want = fused.silu_mul(to_np(x))
    assert rel_err(to_np(F.siluMul(x)), want) <= TOL_REL_FP32
    inp = torch.randn(3 * 256 + 1, device="cuda")[1:].view(3, 256)
    res = torch.randn(3, 256, device="cuda")
    w = torch.randn(256, device="cuda")
    want_in, want_res = fused.fused_add_rms_norm(to_np(inp), to_np(res), to_np(w), 1e-6)
    F.fusedAddRmsNorm(inp, res, w, 1e-6)
    torch.cuda.synchronize()
    assert rel_err(to_np(inp), want_in) <= TOL_REL_FP32 and np.array_equal(to_np(res), want_res)
