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


def check_status(status):
    assert int(status.item()) == 0, "a device-side wait expired (status %d)" % int(status.item())
