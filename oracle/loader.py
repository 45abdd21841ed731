"""TEST INFRASTRUCTURE ONLY: ctypes loaders for the two CPU checkers.

``Oracle``     wraps liboracle.so, the plain-C restatement (attn_oracle.c) of the
               reference's attention arithmetic (src/Function/FuncNNLayer.h:231-266).
``Reference``  wraps _ref/libref_attn.so, the reference's own CPU sources compiled
               unmodified plus ref_shim.cpp; present only where the Makefile had the
               reference tree to compile (the built file travels with the repo).

Nothing in the product package imports this module.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libref_attn.so")

BIAS_NONE, BIAS_CAUSAL, BIAS_ADDITIVE = 0, 1, 2


class _Dims(C.Structure):
    _fields_ = [
        ("B", C.c_int64), ("Hq", C.c_int64), ("Hkv", C.c_int64),
        ("L", C.c_int64), ("S", C.c_int64), ("D", C.c_int64),
        ("bias_kind", C.c_int32), ("scale", C.c_float),
        ("kv_lens", C.c_void_p), ("bias", C.c_void_p),
        ("bias_stride", C.c_int64 * 4),
    ]


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def build(ref_root=None):
    """Compile both checkers with the Makefile beside this file.  The reference tree is taken from
    `ref_root`, else from $TT_REFERENCE_ROOT, else the Makefile looks for a directory named "reference"
    beside this repository; without one only the plain-C oracle is built."""
    import subprocess
    cmd = ["make", "-C", HERE, "-j8", "all"]
    if ref_root:
        cmd.append(f"REF={ref_root}")
    subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL)


class Oracle:
    def __init__(self, threads=None):
        if not os.path.exists(ORACLE_SO):
            build()
        self.lib = C.CDLL(ORACLE_SO)
        self.lib.oracle_sdpa_fwd.restype = C.c_int
        self.lib.oracle_sdpa_bwd.restype = C.c_int
        self.lib.oracle_sdpa_fwd.argtypes = [C.POINTER(_Dims)] + [C.c_void_p] * 5
        self.lib.oracle_sdpa_bwd.argtypes = [C.POINTER(_Dims)] + [C.c_void_p] * 7
        self.set_threads(threads if threads else (os.cpu_count() or 1))

    def set_threads(self, n):
        self.lib.oracle_set_threads(int(n))
        self.threads = int(self.lib.oracle_num_threads())

    @staticmethod
    def _dims(q, k, causal, scale, kv_lens, bias):
        B, Hq, L, D = q.shape
        _, Hkv, S, _ = k.shape
        d = _Dims(B, Hq, Hkv, L, S, D)
        d.scale = float(scale) if scale is not None else 1.0 / np.sqrt(np.float32(D))
        d.bias_kind = BIAS_CAUSAL if causal else BIAS_NONE
        keep = []
        if kv_lens is not None:
            kl = np.ascontiguousarray(kv_lens, dtype=np.int32)
            keep.append(kl)
            d.kv_lens = kl.ctypes.data
        if bias is not None:
            assert not causal
            bb = _f32(np.broadcast_to(bias, (B, Hq, L, S)))
            keep.append(bb)
            d.bias_kind = BIAS_ADDITIVE
            d.bias = bb.ctypes.data
            d.bias_stride[:] = [Hq * L * S, L * S, S, 1]
        return d, keep

    def fwd(self, q, k, v, causal=False, scale=None, kv_lens=None, bias=None):
        """q [B,Hq,L,D], k/v [B,Hkv,S,D] float32 -> (out [B,Hq,L,D], lse [B,Hq,L])."""
        q, k, v = _f32(q), _f32(k), _f32(v)
        d, keep = self._dims(q, k, causal, scale, kv_lens, bias)
        out = np.empty_like(q)
        lse = np.empty(q.shape[:3], dtype=np.float32)
        rc = self.lib.oracle_sdpa_fwd(C.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse))
        assert rc == 0
        return out, lse

    def bwd(self, q, k, v, dout, causal=False, scale=None, kv_lens=None, bias=None):
        q, k, v, dout = _f32(q), _f32(k), _f32(v), _f32(dout)
        d, keep = self._dims(q, k, causal, scale, kv_lens, bias)
        dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
        rc = self.lib.oracle_sdpa_bwd(C.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(dout),
                                      _ptr(dq), _ptr(dk), _ptr(dv))
        assert rc == 0
        return dq, dk, dv


class FusedOracle:
    """fused_oracle.c: the reference's CPU fp32 siluMul / fusedAddRmsNorm, restated."""

    def __init__(self):
        self.lib = C.CDLL(ORACLE_SO)
        self.lib.oracle_silu_mul.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
        self.lib.oracle_silu_mul.restype = None
        self.lib.oracle_fused_add_rms_norm.argtypes = [C.c_void_p] * 3 + [C.c_int64, C.c_int64, C.c_float]
        self.lib.oracle_fused_add_rms_norm.restype = None

    def linear(self, x, w, bias=None):
        x, w = _f32(x), _f32(w)
        bias = _f32(bias) if bias is not None else None
        M, K = x.shape
        N = w.shape[0]
        y = np.empty((M, N), dtype=np.float32)
        self.lib.oracle_linear.argtypes = [C.c_void_p] * 3 + [C.c_int64] * 3 + [C.c_void_p]
        self.lib.oracle_linear.restype = None
        self.lib.oracle_linear(_ptr(x), _ptr(w), _ptr(bias), M, N, K, _ptr(y))
        return y

    def silu_mul(self, x):
        x = _f32(x)
        rows, last = int(np.prod(x.shape[:-1])), x.shape[-1]
        out = np.empty(x.shape[:-1] + (last // 2,), dtype=np.float32)
        self.lib.oracle_silu_mul(_ptr(x), rows, last, _ptr(out))
        return out

    def fused_add_rms_norm(self, inp, residual, weight, eps):
        """Returns (new input, new residual); the arguments are not modified."""
        inp, residual, weight = _f32(inp).copy(), _f32(residual).copy(), _f32(weight)
        dim = inp.shape[-1]
        self.lib.oracle_fused_add_rms_norm(_ptr(inp), _ptr(residual), _ptr(weight), inp.size // dim, dim, float(eps))
        return inp, residual


class Reference:
    """The reference's own CPU code.  Single-threaded, like the reference."""

    @staticmethod
    def available():
        return os.path.exists(REF_SO)

    def __init__(self):
        self.lib = C.CDLL(REF_SO)
        for n in ("ref_sdpa_fwd", "ref_sdpa_grad", "ref_repeat_interleave", "ref_lse", "ref_sdpa_fwd_mask"):
            getattr(self.lib, n).restype = C.c_int
        i64 = C.c_int64
        self.lib.ref_sdpa_fwd.argtypes = [C.c_void_p] * 3 + [i64] * 5 + [C.c_int, C.c_void_p, C.c_float,
                                                                          C.c_void_p]
        self.lib.ref_sdpa_grad.argtypes = [C.c_void_p] * 4 + [i64] * 5 + [C.c_int, C.c_float] + [C.c_void_p] * 4
        self.lib.ref_repeat_interleave.argtypes = [C.c_void_p] + [i64] * 5 + [C.c_void_p]
        self.lib.ref_lse.argtypes = [C.c_void_p] * 2 + [i64] * 5 + [C.c_int, C.c_float, C.c_void_p]
        self.lib.ref_sdpa_fwd_mask.argtypes = [C.c_void_p] * 3 + [i64] * 5 + [C.c_void_p, C.c_int, C.c_void_p,
                                                                               C.c_float, C.c_void_p]

    def fwd(self, q, k, v, causal=False, scale=None, kv_lens=None):
        q, k, v = _f32(q), _f32(k), _f32(v)
        B, H, L, D = q.shape
        S = k.shape[2]
        mask = None
        if kv_lens is not None:
            mask = np.ascontiguousarray(
                (np.arange(S)[None, :] < np.asarray(kv_lens)[:, None]).astype(np.uint8).reshape(B, 1, 1, S))
        out = np.empty_like(q)
        self.lib.ref_sdpa_fwd(_ptr(q), _ptr(k), _ptr(v), B, H, L, S, D, int(causal), _ptr(mask),
                              float(scale) if scale is not None else 0.0, _ptr(out))
        return out

    def fwd_mask(self, q, k, v, mask, scale=None):
        """sdpAttention(q, k, v, false, mask): bool mask (True = attend) or float mask (added),
        any shape of up to 4 dimensions that broadcasts against [B, H, L, S]."""
        q, k, v = _f32(q), _f32(k), _f32(v)
        B, H, L, D = q.shape
        S = k.shape[2]
        mask = np.asarray(mask)
        m4 = mask.reshape((1,) * (4 - mask.ndim) + mask.shape)
        is_float = m4.dtype != np.bool_
        m4 = np.ascontiguousarray(m4.astype(np.float32 if is_float else np.uint8))
        shape = (C.c_int64 * 4)(*m4.shape)
        out = np.empty_like(q)
        self.lib.ref_sdpa_fwd_mask(_ptr(q), _ptr(k), _ptr(v), B, H, L, S, D, _ptr(m4), int(is_float), shape,
                                   float(scale) if scale is not None else 0.0, _ptr(out))
        return out

    def silu_mul(self, x):
        x = _f32(x)
        rows, last = int(np.prod(x.shape[:-1])), x.shape[-1]
        out = np.empty(x.shape[:-1] + (last // 2,), dtype=np.float32)
        self.lib.ref_silu_mul.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
        self.lib.ref_silu_mul(_ptr(x), rows, last, _ptr(out))
        return out

    def fused_add_rms_norm(self, inp, residual, weight, eps):
        inp, residual, weight = _f32(inp).copy(), _f32(residual).copy(), _f32(weight)
        dim = inp.shape[-1]
        self.lib.ref_fused_add_rms_norm.argtypes = [C.c_void_p] * 3 + [C.c_int64, C.c_int64, C.c_float]
        self.lib.ref_fused_add_rms_norm(_ptr(inp), _ptr(residual), _ptr(weight), inp.size // dim, dim, float(eps))
        return inp, residual

    def linear(self, x, w, bias=None):
        x, w = _f32(x), _f32(w)
        bias = _f32(bias) if bias is not None else None
        M, K = x.shape
        N = w.shape[0]
        y = np.empty((M, N), dtype=np.float32)
        self.lib.ref_linear.argtypes = [C.c_void_p] * 3 + [C.c_int64] * 3 + [C.c_void_p]
        self.lib.ref_linear(_ptr(x), _ptr(w), _ptr(bias), M, N, K, _ptr(y))
        return y

    def linear_grad(self, x, w, bias, dy):
        x, w, bias, dy = _f32(x), _f32(w), _f32(bias), _f32(dy)
        M, K = x.shape
        N = w.shape[0]
        dx, dw, db = np.empty_like(x), np.empty_like(w), np.empty_like(bias)
        self.lib.ref_linear_grad.argtypes = [C.c_void_p] * 4 + [C.c_int64] * 3 + [C.c_void_p] * 3
        self.lib.ref_linear_grad(_ptr(x), _ptr(w), _ptr(bias), _ptr(dy), M, N, K, _ptr(dx), _ptr(dw), _ptr(db))
        return dx, dw, db

    def grad(self, q, k, v, dout, causal=False, scale=None):
        q, k, v, dout = _f32(q), _f32(k), _f32(v), _f32(dout)
        B, H, L, D = q.shape
        S = k.shape[2]
        sc = float(scale) if scale is not None else float(1.0 / np.sqrt(np.float32(D)))
        out, dq, dk, dv = np.empty_like(q), np.empty_like(q), np.empty_like(k), np.empty_like(v)
        self.lib.ref_sdpa_grad(_ptr(q), _ptr(k), _ptr(v), _ptr(dout), B, H, L, S, D, int(causal), sc,
                               _ptr(out), _ptr(dq), _ptr(dk), _ptr(dv))
        return out, dq, dk, dv

    def repeat_interleave(self, kv, group):
        kv = _f32(kv)
        B, Hkv, S, D = kv.shape
        out = np.empty((B, Hkv * group, S, D), dtype=np.float32)
        self.lib.ref_repeat_interleave(_ptr(kv), B, Hkv, S, D, group, _ptr(out))
        return out

    def lse(self, q, k, causal=False, scale=None):
        q, k = _f32(q), _f32(k)
        B, H, L, D = q.shape
        S = k.shape[2]
        sc = float(scale) if scale is not None else float(1.0 / np.sqrt(np.float32(D)))
        lse = np.empty((B, H, L), dtype=np.float32)
        self.lib.ref_lse(_ptr(q), _ptr(k), B, H, L, S, D, int(causal), sc, _ptr(lse))
        return lse
