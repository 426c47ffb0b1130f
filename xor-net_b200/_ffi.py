"""ctypes declarations of the C ABI in ``include/xn_attn.h`` (one entry per exported symbol)."""
from __future__ import annotations

import ctypes as C
import os

from . import _build

c_f32p = C.POINTER(C.c_float)
c_i32p = C.POINTER(C.c_int32)


class CtxDesc(C.Structure):
    _fields_ = [
        ("device", C.c_int32), ("num_layers", C.c_int32), ("num_heads", C.c_int32),
        ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("page_tokens", C.c_int32),
        ("pool_pages", C.c_int64), ("pool_bytes", C.c_int64), ("shuffle_seed", C.c_uint64),
        ("max_pos", C.c_int32), ("prefill_mode", C.c_int32),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p), ("cuda_stream", C.c_void_p),
        ("batch_window_us", C.c_int32), ("kv_format", C.c_int32),
    ]


class Req(C.Structure):
    _fields_ = [
        ("stream", C.c_void_p), ("layer", C.c_int32), ("seq_len", C.c_int32),
        ("index_pos", C.c_int64), ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("out", C.c_void_p), ("flags", C.c_uint32), ("reserved", C.c_uint32),
    ]


class Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "calls", "batches", "kernel_launches", "decode_launches", "prefill_launches", "h2d_bytes",
        "d2h_bytes", "pages_total", "pages_in_use", "streams_live", "device_wait_errors",
        "coalesced_max", "out_proj_rows", "plan_reuses", "out_transfers")]


class QkvProjDesc(C.Structure):
    _fields_ = [("layer", C.c_int32), ("in_dim", C.c_int32), ("pack_type", C.c_int32),
                ("reserved", C.c_int32), ("q_packed", C.c_void_p), ("q_scales", C.c_void_p),
                ("k_packed", C.c_void_p), ("k_scales", C.c_void_p), ("v_packed", C.c_void_p),
                ("v_scales", C.c_void_p)]


class OutProjDesc(C.Structure):
    _fields_ = [("layer", C.c_int32), ("in_dim", C.c_int32), ("out_dim", C.c_int32),
                ("pack_type", C.c_int32), ("packed", C.c_void_p), ("w_scales", C.c_void_p),
                ("norm_weight", C.c_void_p), ("norm_eps", C.c_float), ("reserved", C.c_uint32)]


REQ_DEVICE_PTRS, REQ_ROPE, REQ_SEQ_MAJOR, REQ_HOST_PINNED, REQ_OUT_PROJ, REQ_QKV_PROJ = 1, 2, 4, 8, 16, 32
PACK4, PACK5, SPARSE = 4, 5, 64
KV_F32, KV_U8 = 0, 1   # xn_ctx_desc.kv_format
PLACE_LEAST_LOADED, PLACE_ROUND_ROBIN = 0, 1

STATUS_NAMES = {
    0: "XN_OK", 1: "XN_ERR_ARG", 2: "XN_ERR_SHAPE", 3: "XN_ERR_HANDLE", 4: "XN_ERR_OUT_OF_PAGES",
    5: "XN_ERR_CAPACITY", 6: "XN_ERR_CUDA", 7: "XN_ERR_DEVICE_WAIT", 8: "XN_ERR_NO_TABLES",
    9: "XN_ERR_NOMEM", 10: "XN_ERR_NO_DEVICE", 11: "XN_ERR_GUARD",
}

# symbol -> (restype, argtypes); must list every XN_API function of include/xn_attn.h
SIGNATURES = {
    "xn_ctx_create": (C.c_int32, [C.POINTER(CtxDesc), C.POINTER(C.c_void_p)]),
    "xn_ctx_destroy": (C.c_int32, [C.c_void_p]),
    "xn_ctx_synchronize": (C.c_int32, [C.c_void_p]),
    "xn_ctx_cuda_stream": (C.c_void_p, [C.c_void_p]),
    "xn_stats_get": (C.c_int32, [C.c_void_p, C.POINTER(Stats)]),
    "xn_last_error": (C.c_char_p, [C.c_void_p]),
    "xn_profile_enable": (C.c_int32, [C.c_void_p, C.c_int32]),
    "xn_profile_read": (C.c_int32, [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_uint64),
                                    C.POINTER(C.c_double), C.POINTER(C.c_uint64)]),
    "xn_stream_create": (C.c_int32, [C.c_void_p, C.c_int64, C.POINTER(C.c_void_p)]),
    "xn_stream_reset": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "xn_stream_destroy": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "xn_attention": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "xn_attention_rope": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32,
                                      C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "xn_attention_batch": (C.c_int32, [C.c_void_p, C.c_int32, C.POINTER(Req)]),
    "xn_decode_attention_static": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                               C.c_int32, C.c_int32, C.c_int32, C.c_int64,
                                               C.c_int64, C.c_void_p]),
    "xn_rope_tables": (C.c_int32, [C.c_float, C.c_int32, C.c_int32, C.c_float, C.c_float,
                                   C.c_float, C.c_int32, c_f32p, c_f32p]),
    "xn_kv_read": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int64,
                               C.c_void_p, C.c_void_p]),
    "xn_kv_read_range": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64,
                                     C.c_void_p, C.c_void_p]),
    "xn_kv_read_u8": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64,
                                  C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "xn_kv_fill_normal": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64,
                                      C.c_uint64]),
    "xn_fill_normal": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_uint64]),
    "xn_stream_len": (C.c_int64, [C.c_void_p, C.c_void_p, C.c_int32]),
    "xn_stream_pages": (C.c_int64, [C.c_void_p, C.c_void_p, c_i32p, C.c_int64]),
    "xn_plan_split": (C.c_int32, [C.c_int32, c_i32p, C.c_int32, C.c_int32, C.c_int32, c_i32p,
                                  c_i32p, c_i32p, c_i32p, c_i32p, c_i32p, c_i32p]),
    "xn_debug_expire_wait": (C.c_int32, [C.c_void_p, C.c_int32]),
    "xn_debug_check_guards": (C.c_int32, [C.c_void_p]),
    "xn_debug_drop_plan": (C.c_int32, [C.c_void_p]),
    "xn_profile_read_all": (C.c_int32, [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]),
    "xn_qkv_proj_set": (C.c_int32, [C.c_void_p, C.POINTER(QkvProjDesc)]),
    "xn_out_proj_set": (C.c_int32, [C.c_void_p, C.POINTER(OutProjDesc)]),
    "xn_out_proj": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_uint32]),
    "xn_ternary_pack": (C.c_int32, [C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_float,
                                    C.c_void_p, C.c_void_p]),
    "xn_ternary_pack_sparse": (C.c_int32, [C.c_int32, C.c_int32, C.c_void_p, C.c_float, C.c_void_p,
                                           C.c_int64, C.POINTER(C.c_int64), C.c_void_p]),
    "xn_group_create": (C.c_int32, [C.POINTER(CtxDesc), c_i32p, C.c_int32, C.POINTER(C.c_void_p)]),
    "xn_group_destroy": (C.c_int32, [C.c_void_p]),
    "xn_group_size": (C.c_int32, [C.c_void_p]),
    "xn_group_ctx": (C.c_void_p, [C.c_void_p, C.c_int32]),
    "xn_group_stream_create": (C.c_int32, [C.c_void_p, C.c_int64, C.c_int64, C.c_int32,
                                           C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "xn_place_stream": (C.c_int32, [C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_uint64,
                                    C.c_int32]),
    "xn_version": (C.c_char_p, []),
}

_lib = None


def load() -> C.CDLL:
    """Loads the in-tree CUDA library; raises if it is missing (there is no fallback)."""
    global _lib
    if _lib is None:
        path = os.environ.get("XORNET_ATTN_LIB") or _build.LIB_PATH  # override: a tuning build
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with __graft_entry__.build() "
                "(nvcc, sm_100a). This package has no CPU or PyTorch fallback.")
        lib = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
