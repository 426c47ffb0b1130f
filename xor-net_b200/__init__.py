"""B200 (sm_100a) implementation of xor-net's causal GQA attention path.

The compute lives in ``libxn_attn.so`` (hand-written CUDA + C ABI, see ``include/xn_attn.h``);
this package is the Python host side.  Importing it never falls back to a CPU path: calls raise
if the library is not built or no sm_100 device is present.
"""
from ._build import LIB_PATH, build_host_tool, build_library
from .api import (Context, DeviceKvCache, FastTensor, Group, Stream, TernaryLinear, XnError,
                  close_default_contexts, default_context, default_group, fast_attention, place_stream,
                  rope_tables)
from . import sharding
from ._ffi import (PLACE_LEAST_LOADED, PLACE_ROUND_ROBIN, KV_F32, KV_U8, PACK4, PACK5, SPARSE, REQ_DEVICE_PTRS, REQ_HOST_PINNED, REQ_OUT_PROJ, REQ_QKV_PROJ, REQ_ROPE,
                   REQ_SEQ_MAJOR, SIGNATURES, load)

__all__ = [
    "Context", "Stream", "Group", "default_group", "place_stream", "PLACE_LEAST_LOADED", "PLACE_ROUND_ROBIN",
    "DeviceKvCache", "FastTensor", "XnError", "fast_attention", "rope_tables",
    "default_context", "close_default_contexts", "build_library", "build_host_tool", "load", "LIB_PATH", "SIGNATURES",
    "REQ_DEVICE_PTRS", "REQ_ROPE", "REQ_SEQ_MAJOR", "REQ_HOST_PINNED", "REQ_OUT_PROJ", "REQ_QKV_PROJ", "KV_F32", "KV_U8", "SPARSE", "PACK4",
    "PACK5", "TernaryLinear", "sharding",
]
