"""TEST INFRASTRUCTURE ONLY: numpy restatement of the rotary position embedding and of
the cache append that the fused decode step performs before attention.

The reference (keith2018/TinyTorch) has no rotary embedding and no KV-cache object, so
nothing in its tree pins this part: PARITY UNPINNED for the rotation and the append.  The
restated algorithm is the published one (Su et al., "RoFormer", 2021): the pair
(x_a, x_b) of a row at position p turns by the angle p * theta^(-2i/D),
    x_a' = x_a cos - x_b sin,   x_b' = x_b cos + x_a sin,
with (a, b) = (i, i + D/2) in the half-split layout and (2i, 2i+1) in the interleaved
one.  The attention over the appended cache is then checked with the reference-pinned
attention oracle (oracle/attn_oracle.c).
"""
import numpy as np


def tables(positions, D, theta=10000.0):
    """cos / sin [positions, D/2] in fp32, computed in fp64."""
    inv = theta ** (-np.arange(0, D, 2, dtype=np.float64) / D)
    ang = np.arange(positions, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def rotate(x, pos, cos, sin, interleaved=False):
    """x [B, H, 1, D] fp32, pos [B] -> rotated copy, fp32 arithmetic."""
    x = np.asarray(x, dtype=np.float32)
    out = np.empty_like(x)
    D = x.shape[-1]
    for b in range(x.shape[0]):
        c, s = cos[int(pos[b])], sin[int(pos[b])]
        if interleaved:
            xa, xb = x[b, ..., 0::2], x[b, ..., 1::2]
            out[b, ..., 0::2] = xa * c - xb * s
            out[b, ..., 1::2] = xb * c + xa * s
        else:
            xa, xb = x[b, ..., : D // 2], x[b, ..., D // 2:]
            out[b, ..., : D // 2] = xa * c - xb * s
            out[b, ..., D // 2:] = xb * c + xa * s
    return out


def append(cache, new, pos):
    """Writes new[b, h, 0, :] into cache[b, h, pos[b], :] (in place) and returns the cache."""
    for b in range(cache.shape[0]):
        cache[b, :, int(pos[b]), :] = new[b, :, 0, :]
    return cache
