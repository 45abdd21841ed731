"""B200-native fused attention behind TinyTorch's sdpAttention interface.

``function.sdpAttention`` mirrors the reference's function-layer entry point,
``op`` the dispatch-layer ops, ``shard`` the batch x head partitioning across
GPUs.  All compute goes through the C ABI of lib/libtt_attn.so (include/tt_attn.h).
"""
from . import _capi  # noqa: F401

__all__ = ["function", "op", "shard"]
