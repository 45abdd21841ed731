"""ctypes binding of libtt_attn.so (declared in include/tt_attn.h).

This is the only route from Python to the kernels.  There is no fallback: if the
shared library is missing or fails to load, importing the ops raises.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# TT_ATTN_LIB selects another build of the same library (e.g. a tuning variant).
LIB_PATH = os.environ.get("TT_ATTN_LIB") or os.path.join(HERE, "lib", "libtt_attn.so")

F32, F16, BF16 = 0, 1, 2
KIND_FWD, KIND_BWD, KIND_DECODE, KIND_DECODE_APPEND = 0, 1, 2, 3
CAUSAL_NONE, CAUSAL_TOP_LEFT, CAUSAL_BOTTOM_RIGHT = 0, 1, 2
MASK_NONE, MASK_BOOL, MASK_ADD, MASK_ADD_F32 = 0, 1, 2, 3

_MASK_FIELDS = [("mask", C.c_void_p), ("mask_kind", C.c_int32), ("reserved0", C.c_int32),
                ("mask_strides", C.c_int64 * 3)]
STATIC_SCRATCH_BYTES = 24 << 20  # TT_ATTN_STATIC_SCRATCH_BYTES

ALLOC_FN = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_size_t, C.c_int)
FREE_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_int)


class AllocHook(C.Structure):
    _fields_ = [("alloc", ALLOC_FN), ("free", FREE_FN), ("ctx", C.c_void_p)]


class Strides(C.Structure):
    _fields_ = [("b", C.c_int64), ("h", C.c_int64), ("s", C.c_int64)]


class FwdParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Lq", C.c_int32), ("Skv", C.c_int32),
        ("D", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("lse", C.c_void_p),
        ("q_strides", Strides), ("k_strides", Strides), ("v_strides", Strides), ("o_strides", Strides),
        ("is_causal", C.c_int32), ("scale", C.c_float),
        ("kv_lens", C.c_void_p),
        ("device", C.c_int32), ("stream", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("alloc", C.POINTER(AllocHook)), ("status", C.c_void_p),
    ] + _MASK_FIELDS


class BwdParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Lq", C.c_int32), ("Skv", C.c_int32),
        ("D", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("d_o", C.c_void_p),
        ("lse", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("q_strides", Strides), ("k_strides", Strides), ("v_strides", Strides), ("o_strides", Strides),
        ("do_strides", Strides), ("dq_strides", Strides), ("dk_strides", Strides), ("dv_strides", Strides),
        ("is_causal", C.c_int32), ("scale", C.c_float),
        ("kv_lens", C.c_void_p),
        ("device", C.c_int32), ("stream", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("alloc", C.POINTER(AllocHook)), ("status", C.c_void_p),
    ] + _MASK_FIELDS


class DecodeParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("capacity", C.c_int32), ("D", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("lse", C.c_void_p),
        ("q_strides", Strides), ("k_strides", Strides), ("v_strides", Strides), ("o_strides", Strides),
        ("scale", C.c_float),
        ("kv_lens", C.c_void_p),
        ("device", C.c_int32), ("stream", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("alloc", C.POINTER(AllocHook)), ("status", C.c_void_p),
    ]


class DecodeAppendParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("capacity", C.c_int32), ("D", C.c_int32),
        ("q", C.c_void_p), ("k_new", C.c_void_p), ("v_new", C.c_void_p),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("o", C.c_void_p), ("lse", C.c_void_p),
        ("q_strides", Strides), ("k_new_strides", Strides), ("v_new_strides", Strides),
        ("k_strides", Strides), ("v_strides", Strides), ("o_strides", Strides),
        ("scale", C.c_float),
        ("kv_lens", C.c_void_p), ("new_lens", C.c_void_p),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
        ("rope_positions", C.c_int32), ("rope_interleaved", C.c_int32),
        ("device", C.c_int32), ("stream", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("alloc", C.POINTER(AllocHook)), ("status", C.c_void_p),
    ]


class AddRmsNormParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32), ("rows", C.c_int64), ("dim", C.c_int64),
        ("input", C.c_void_p), ("residual", C.c_void_p), ("weight", C.c_void_p),
        ("eps", C.c_float), ("device", C.c_int32), ("stream", C.c_void_p),
    ]


class SiluMulParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32), ("rows", C.c_int64), ("d", C.c_int64),
        ("x", C.c_void_p), ("out", C.c_void_p), ("device", C.c_int32), ("stream", C.c_void_p),
    ]


class LinearParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32), ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("x", C.c_void_p), ("w", C.c_void_p), ("bias", C.c_void_p), ("y", C.c_void_p),
        ("ldx", C.c_int64), ("ldw", C.c_int64), ("ldy", C.c_int64),
        ("device", C.c_int32), ("stream", C.c_void_p), ("status", C.c_void_p),
    ]


FUSED_EXPORTS = ("tt_fused_add_rms_norm", "tt_silu_mul", "tt_linear")  # include/tt_fused.h

EXPORTS = ("tt_attn_fwd", "tt_attn_bwd", "tt_attn_decode", "tt_attn_decode_append", "tt_attn_decode_static",
           "tt_attn_selftest_wait_expiry", "tt_attn_workspace_bytes", "tt_attn_strerror",
           "tt_attn_last_cuda_error", "tt_attn_version")

_lib = None


class AttnError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("tt_attn status %d: %s" % (code, text))
        self.code = code


def lib():
    """Load libtt_attn.so once.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "%s not found: build it with `python -m tinytorch_b200.build` "
                "(there is no CPU or PyTorch fallback for these ops)" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        L.tt_attn_fwd.argtypes = [C.POINTER(FwdParams)]
        L.tt_attn_bwd.argtypes = [C.POINTER(BwdParams)]
        L.tt_attn_decode.argtypes = [C.POINTER(DecodeParams)]
        L.tt_attn_decode_append.argtypes = [C.POINTER(DecodeAppendParams)]
        L.tt_attn_decode_append.restype = C.c_int
        L.tt_fused_add_rms_norm.argtypes = [C.POINTER(AddRmsNormParams)]
        L.tt_fused_add_rms_norm.restype = C.c_int
        L.tt_silu_mul.argtypes = [C.POINTER(SiluMulParams)]
        L.tt_silu_mul.restype = C.c_int
        L.tt_linear.argtypes = [C.POINTER(LinearParams)]
        L.tt_linear.restype = C.c_int
        L.tt_attn_decode_static.argtypes = [C.POINTER(DecodeParams)]
        L.tt_attn_decode_static.restype = C.c_int
        L.tt_attn_selftest_wait_expiry.argtypes = [C.c_int, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]
        L.tt_attn_selftest_wait_expiry.restype = C.c_int
        for n in ("tt_attn_fwd", "tt_attn_bwd", "tt_attn_decode", "tt_attn_version"):
            getattr(L, n).restype = C.c_int
        L.tt_attn_workspace_bytes.argtypes = [C.c_int] * 8
        L.tt_attn_workspace_bytes.restype = C.c_size_t
        L.tt_attn_strerror.argtypes = [C.c_int]
        L.tt_attn_strerror.restype = C.c_char_p
        L.tt_attn_last_cuda_error.restype = C.c_char_p
        _lib = L
    return _lib


def check(rc):
    if rc != 0:
        L = lib()
        text = L.tt_attn_strerror(rc).decode()
        if rc == -7:
            text += " [" + L.tt_attn_last_cuda_error().decode() + "]"
        raise AttnError(rc, text)
