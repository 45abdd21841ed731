"""Helpers shared by the GPU parity tests (test infrastructure)."""
import numpy as np
import torch

TOL_ABS_16BIT = 2e-2   # absolute bound for fp16 / bf16 outputs and gradients
TOL_REL_FP32 = 1e-5    # max|a-b| / max|b| bound for fp32

DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def make(shape, dtype, seed, std=1.0):
    """Seeded N(0, std) host array rounded to `dtype`; returns (device tensor, fp32 numpy of the rounded values)."""
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(shape, dtype=np.float32) * np.float32(std))
    t = torch.from_numpy(x).to(dtype)
    return t.cuda(), t.float().numpy()


def to_np(t):
    return t.detach().float().cpu().numpy()


# relative spacing of the 16-bit formats (one unit in the last place of a value near 1)
ULP = {"f16": 2.0 ** -10, "bf16": 2.0 ** -7, torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}


def assert_close_16bit(got, want, dtype, what=""):
    """Element-wise bound for 16-bit outputs and gradients: 2e-2 absolute plus two units in the last place of
    the element's own magnitude.  Prints the largest error and the largest error relative to that bound, so that a
    passing run (pytest -rA / -s) shows the head-room as well."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    bound = TOL_ABS_16BIT + 2.0 * ULP[dtype] * np.abs(want)
    err = np.abs(got - want)
    worst = int(np.argmax(err / bound))
    print("%s: max |err| %.3e, max err/bound %.3f (max |want| %.3e)" % (
        what, float(err.max()), float((err / bound).ravel()[worst]), float(np.abs(want).max())))
    assert bool((err <= bound).all()), "%s: |err| %.4e > bound %.4e at flat index %d (want %.4e)" % (
        what, float(err.ravel()[worst]), float(bound.ravel()[worst]), worst, float(want.ravel()[worst]))


def check_status(status):
    assert int(status.item()) == 0, "a device-side wait expired (status %d)" % int(status.item())
