"""GPU parity of the tensor-core projection y = x w^T + bias (function::linear,
src/Function/FuncNNLayer.h:14-35,270-272) against the CPU oracle of the reference's gemm, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from gpu_util import DTYPES, TOL_ABS_16BIT, make, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fused():
    from oracle.loader import FusedOracle
    return FusedOracle()


def _close(got, want):
    # fp32 accumulation, one rounding to 16 bits: the error scales with the magnitude of the output
    assert np.abs(to_np(got) - want).max() <= TOL_ABS_16BIT * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K,bias", [
    (128, 256, 64, True), (128, 256, 64, False), (256, 512, 256, True), (1, 8, 8, True), (100, 200, 72, True),
    (129, 264, 136, False), (300, 1000, 520, True), (1024, 768, 2048, True), (37, 40, 72, True), (640, 256, 8, True),
])
def test_linear_shapes(fused, dt, M, N, K, bias):
    from tinytorch_b200 import fused as F
    x, xn = make((M, K), DTYPES[dt], 601, std=0.5)
    w, wn = make((N, K), DTYPES[dt], 602, std=0.5)
    b, bn = make((N,), DTYPES[dt], 603)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = F._linear_raw(x, w, b if bias else None, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    _close(y, fused.linear(xn, wn, bn if bias else None))


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", [(2100, 4712, 200), (4096, 2560, 72), (2304, 4352, 1032)])
def test_linear_tall_tiles(fused, dt, M, N, K):
    # enough 256 x 256 tiles to fill the machine: the kernel takes 256-row tiles (two accumulators sharing a
    # slice of w).  Ragged in every dimension; in the first shape the last tile's lower half lies wholly beyond M.
    # The oracle runs on a band of rows from every part of the tile grid.
    from tinytorch_b200 import fused as F
    x, xn = make((M, K), DTYPES[dt], 631, std=0.5)
    w, wn = make((N, K), DTYPES[dt], 632, std=0.5)
    b, bn = make((N,), DTYPES[dt], 633)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = F._linear_raw(x, w, b, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    rows = sorted(set([0, 1, 127, 128, 129, 255, 256, 257, 383, 384, M // 2, M // 2 + 131, M - 130, M - 129, M - 2, M - 1]))
    _close(y[rows], fused.linear(xn[rows], wn, bn))
    # and the whole result against an fp32 product on the GPU
    want = x.float() @ w.float().t() + b.float()
    assert float((y.float() - want).abs().max()) <= TOL_ABS_16BIT * max(1.0, float(want.abs().max()))


def test_golden_fixture(fused):
    from tinytorch_b200 import fused as F
    g = np.load(os.path.join(GOLDEN, "ref_seeded_linear.npz"))
    x, w, b = (torch.from_numpy(g[n]).cuda().bfloat16() for n in ("x", "w", "b"))
    y = F.linear(x, w, b)
    torch.cuda.synchronize()
    # the fixture is fp32; with inputs rounded to bf16 the bound is loose
    assert np.abs(to_np(y) - g["y"]).max() <= 0.25
    _close(y, fused.linear(to_np(x), to_np(w), to_np(b)))


def test_leading_dimensions_and_strided_rows(fused):
    # input [B, S, K] flattened to rows; a weight that is a row-slice of a larger matrix (fused QKV weight)
    from tinytorch_b200 import fused as F
    x, xn = make((2, 50, 128), torch.bfloat16, 611, std=0.5)
    wbig, wn = make((3 * 64, 256), torch.bfloat16, 612, std=0.5)
    w = wbig[64:128, :128]           # rows 64..127, first 128 columns: row stride 256
    y = F.linear(x, w)
    torch.cuda.synchronize()
    assert y.shape == (2, 50, 64)
    _close(y.reshape(100, 64), fused.linear(xn.reshape(100, 128), wn[64:128, :128]))


def test_full_size_projection_rows(fused):
    # QKV projection of the bench: 16384 tokens x 4096 -> 12288; the oracle on a few rows (rows are independent)
    from tinytorch_b200 import fused as F
    g = torch.Generator(device="cuda").manual_seed(621)
    M, K, N = 16384, 4096, 12288
    x = (torch.randn((M, K), generator=g, device="cuda") * 0.5).bfloat16()
    w = (torch.randn((N, K), generator=g, device="cuda") * 0.05).bfloat16()
    b = torch.randn((N,), generator=g, device="cuda").bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = F._linear_raw(x, w, b, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    rows = [0, 127, 128, 5000, 16383]
    want = fused.linear(to_np(x[rows]), to_np(w), to_np(b))
    _close(y[rows], want)
    # linearity in x: linear(2x) - bias = 2 (linear(x) - bias), exactly representable scaling
    y2 = F._linear_raw((x * 2).contiguous(), w, None)
    y0 = F._linear_raw(x, w, None)
    assert float((y2.float() - 2 * y0.float()).abs().max()) <= 2e-2 * float(y0.float().abs().max())


def test_autograd_matches_reference_gradients(fused):
    from tinytorch_b200 import fused as F
    g = np.load(os.path.join(GOLDEN, "ref_seeded_linear.npz"))
    # pad the fixture (M=37, N=40, K=72) is fine for the forward; the backward contracts over M and N, which must be
    # multiples of 8 for the kernel: use the leading 32 rows
    x = torch.from_numpy(g["x"][:32]).cuda().bfloat16().requires_grad_(True)
    w = torch.from_numpy(g["w"]).cuda().bfloat16().requires_grad_(True)
    b = torch.from_numpy(g["b"]).cuda().bfloat16().requires_grad_(True)
    dy = torch.from_numpy(g["dy"][:32]).cuda().bfloat16()
    F.linear(x, w, b).backward(dy)
    torch.cuda.synchronize()
    xn, wn, dyn = to_np(x), to_np(w), to_np(dy)
    _close(x.grad, fused.linear(dyn, wn.T.copy()))
    _close(w.grad, fused.linear(dyn.T.copy(), xn.T.copy()))
    _close(b.grad, dyn.sum(0))
