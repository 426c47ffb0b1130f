"""ctypes binding of the CPU oracle (``xn_oracle.c``).

TEST INFRASTRUCTURE ONLY: the checker for the CUDA library and the timed CPU
baseline.  The product package never imports this module.

The oracle restates the reference's ``fast_attention`` path
(src/nn/fast_attention.rs:75-204, src/nn/fast_attention_simd.rs,
src/tensor.rs:295-376, src/models/llama/mod.rs:210-265) in C with the same x86
intrinsics; see the header of ``xn_oracle.c`` for the parity status.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libxn_oracle.so")
_lib = None

ISA_AUTO, ISA_SCALAR, ISA_AVX2, ISA_AVX512 = 0, 1, 2, 3

_f32p = C.POINTER(C.c_float)
_i8p = C.POINTER(C.c_int8)
_u8p = C.POINTER(C.c_uint8)
_sz = C.c_size_t

PACK4, PACK5, SPARSE = 4, 5, 64


def build(force: bool = False) -> str:
    """Compile ``libxn_oracle.so`` beside the source if it is missing or stale."""
    srcs = [os.path.join(_HERE, f) for f in ("xn_oracle.c", "xn_oracle_outproj.c", "Makefile")]
    stale = (not os.path.exists(_LIB_PATH)) or \
        os.path.getmtime(_LIB_PATH) < max(os.path.getmtime(f) for f in srcs)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libxn_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.xo_set_isa.argtypes = [C.c_int]
        L.xo_set_isa.restype = C.c_int
        L.xo_active_isa.restype = C.c_int
        L.xo_max_threads.restype = C.c_int
        L.xo_batched_dot_product.argtypes = [_f32p, _f32p, _sz, _sz, _sz, _sz, _sz, _f32p]
        L.xo_batched_dot_product.restype = None
        L.xo_softmax_inplace.argtypes = [_f32p, _sz]
        L.xo_softmax_inplace.restype = None
        L.xo_weighted_sum.argtypes = [_f32p, _f32p, _f32p, _sz, _sz, _sz, _sz]
        L.xo_weighted_sum.restype = None
        L.xo_rope_vec.argtypes = [_f32p, _f32p, _f32p, _sz]
        L.xo_rope_vec.restype = None
        L.xo_tensor_rope_inplace.argtypes = [_f32p, _sz, _sz, _sz, _f32p, _f32p, _sz]
        L.xo_tensor_rope_inplace.restype = None
        L.xo_rope_tables.argtypes = [C.c_float, _sz, _sz, C.c_float, C.c_float, C.c_float, _sz,
                                     _f32p, _f32p]
        L.xo_rope_tables.restype = None
        L.xo_transpose_seq_to_heads.argtypes = [_f32p, _f32p, _sz, _sz, _sz]
        L.xo_transpose_seq_to_heads.restype = None
        L.xo_transpose_heads_to_seq.argtypes = [_f32p, _f32p, _sz, _sz, _sz]
        L.xo_transpose_heads_to_seq.restype = None
        L.xo_cache_new.argtypes = [_sz, _sz, _sz, _sz]
        L.xo_cache_new.restype = C.c_void_p
        L.xo_cache_free.argtypes = [C.c_void_p]
        L.xo_cache_free.restype = None
        L.xo_cache_k.argtypes = [C.c_void_p, _sz]
        L.xo_cache_k.restype = _f32p
        L.xo_cache_v.argtypes = [C.c_void_p, _sz]
        L.xo_cache_v.restype = _f32p
        L.xo_cache_append.argtypes = [C.c_void_p, _sz, _sz, _sz, _f32p, _f32p]
        L.xo_cache_append.restype = None
        L.xo_quantize_to_u8.argtypes = [_f32p, _sz, _sz, C.c_void_p, _f32p]
        L.xo_quantize_to_u8.restype = None
        L.xo_dequantize_u8.argtypes = [C.c_void_p, _f32p, _sz, _sz, _f32p]
        L.xo_dequantize_u8.restype = None
        L.xo_fast_attention.argtypes = [_f32p, _f32p, _f32p, _sz, _sz, C.c_void_p, _sz, _sz, _sz,
                                        _sz, C.c_int, _sz, _f32p, C.c_int]
        L.xo_fast_attention.restype = C.c_int
        L.xo_fast_attention_streams.argtypes = [
            _sz, C.POINTER(_f32p), C.POINTER(_f32p), C.POINTER(_f32p), _sz, C.POINTER(_sz),
            C.POINTER(_sz), C.POINTER(C.c_void_p), _sz, _sz, _sz, C.POINTER(_f32p), C.c_int]
        L.xo_fast_attention_streams.restype = C.c_int
        L.xo_set_quant_body.argtypes = [C.c_int]
        L.xo_set_quant_body.restype = C.c_int
        # attention output block (xn_oracle_outproj.c)
        L.xo_rms_norm.argtypes = [_f32p, _f32p, C.c_float, _sz]
        L.xo_rms_norm.restype = None
        L.xo_tensor_rmsnorm.argtypes = [_f32p, _f32p, _f32p, C.c_float, _sz, _sz]
        L.xo_tensor_rmsnorm.restype = None
        L.xo_quantize_f32_to_i8.argtypes = [_f32p, _sz, _i8p]
        L.xo_quantize_f32_to_i8.restype = C.c_float
        L.xo_packed_row_bytes.argtypes = [_sz, C.c_int]
        L.xo_packed_row_bytes.restype = _sz
        for name in ("xo_pack4", "xo_pack5"):
            getattr(L, name).argtypes = [_f32p, _sz, C.c_float, _u8p]
            getattr(L, name).restype = None
        for name in ("xo_unpack4", "xo_unpack5"):
            getattr(L, name).argtypes = [_u8p, _sz, _f32p]
            getattr(L, name).restype = None
        for name in ("xo_ternary_dot_pack4", "xo_ternary_dot_pack5"):
            getattr(L, name).argtypes = [_i8p, _u8p, _sz]
            getattr(L, name).restype = C.c_int32
        L.xo_ternary_linear_pack.argtypes = [_sz, _sz, _f32p, C.c_int, C.c_float, _u8p, _f32p]
        L.xo_ternary_linear_pack.restype = None
        L.xo_sparse_encode_row.argtypes = [_i8p, _sz, _u8p]
        L.xo_sparse_encode_row.restype = _sz
        L.xo_sparse_decode_row.argtypes = [_u8p, _sz, _i8p]
        L.xo_sparse_decode_row.restype = _sz
        L.xo_ternary_dot_sparse.argtypes = [_i8p, _u8p, _sz]
        L.xo_ternary_dot_sparse.restype = C.c_int32
        L.xo_ternary_linear_pack_sparse.argtypes = [_sz, _sz, _f32p, C.c_float, _u8p, _f32p]
        L.xo_ternary_linear_pack_sparse.restype = _sz
        L.xo_ternary_linear_forward.argtypes = [_f32p, _sz, _sz, _sz, C.c_int, _u8p, _f32p, _f32p,
                                                C.c_int]
        L.xo_ternary_linear_forward.restype = None
        L.xo_attention_out_block.argtypes = [_f32p, _sz, _sz, _sz, _f32p, C.c_float, _sz, C.c_int,
                                             _u8p, _f32p, _f32p, C.c_int]
        L.xo_attention_out_block.restype = None
        _lib = L
    return _lib


def _p(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f32p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def set_isa(isa: int) -> int:
    return lib().xo_set_isa(isa)


def active_isa() -> int:
    return lib().xo_active_isa()


def max_threads() -> int:
    return lib().xo_max_threads()


# --- primitives (fast_attention_simd.rs) ------------------------------------------------------

def batched_dot_product(q, k_buf, h_kv, max_seq_len, head_dim, t_start, t_end) -> np.ndarray:
    q, k_buf = _f32(q), _f32(k_buf)
    out = np.zeros(max(16, t_end - t_start), dtype=np.float32)
    lib().xo_batched_dot_product(_p(q), _p(k_buf), h_kv, max_seq_len, head_dim, t_start, t_end,
                                 _p(out))
    return out[: t_end - t_start]


def softmax_inplace(scores) -> np.ndarray:
    s = _f32(scores).copy()
    lib().xo_softmax_inplace(_p(s), s.size)
    return s


def weighted_sum(scores, v_buf, h_kv, max_seq_len, head_dim, total_kv_len) -> np.ndarray:
    scores, v_buf = _f32(scores), _f32(v_buf)
    out = np.zeros(head_dim, dtype=np.float32)
    lib().xo_weighted_sum(_p(out), _p(scores), _p(v_buf), h_kv, max_seq_len, head_dim, total_kv_len)
    return out


def rope_tables(theta, head_dim, max_pos, scaling=None):
    """cos, sin tables ``[max_pos, head_dim // 2]`` (mod.rs:210-265).

    ``scaling`` = (factor, low_freq_factor, high_freq_factor, original_max_pos) or None.
    """
    half = head_dim // 2
    cos = np.zeros((max_pos, half), dtype=np.float32)
    sin = np.zeros((max_pos, half), dtype=np.float32)
    f, lo, hi, orig = scaling if scaling else (0.0, 1.0, 1.0, 0)
    lib().xo_rope_tables(theta, head_dim, max_pos, f, lo, hi, orig, _p(cos), _p(sin))
    return cos, sin


def tensor_rope(x, cos, sin, index_pos) -> np.ndarray:
    """FastTensor::rope_inplace (tensor.rs:295-316); x is [1, H, S, D].  Raises on non-4-D."""
    x = _f32(x)
    if x.ndim != 4:
        raise ValueError(
            f"rope_inplace: input must be 4D shape [b_sz, num_heads, seq_len, head_dim], got {list(x.shape)}")
    out = x.copy()
    _, H, S, D = out.shape
    cos, sin = _f32(cos), _f32(sin)
    lib().xo_tensor_rope_inplace(_p(out), H * out.shape[0], S, D, _p(cos), _p(sin), index_pos)
    return out


def transpose_seq_to_heads(x, num_heads, head_dim) -> np.ndarray:
    x = _f32(x)
    b, S, hidden = x.shape
    if hidden != num_heads * head_dim:
        raise ValueError("transpose_seq_to_heads: hidden_size must equal num_heads * head_dim")
    out = np.empty((b, num_heads, S, head_dim), dtype=np.float32)
    lib().xo_transpose_seq_to_heads(_p(x), _p(out), S, num_heads, head_dim)
    return out


def transpose_heads_to_seq(x) -> np.ndarray:
    x = _f32(x)
    b, H, S, D = x.shape
    out = np.empty((b, S, H * D), dtype=np.float32)
    lib().xo_transpose_heads_to_seq(_p(x), _p(out), S, H, D)
    return out


# --- cache + attention (fast_attention.rs) ----------------------------------------------------

class RingCache:
    """CpuRingCache (fast_attention.rs:18-60) without the write-only u8 shadow."""

    def __init__(self, num_layers, num_kv_heads, max_seq_len, head_dim, use_u8=False):
        self.num_layers, self.num_kv_heads = num_layers, num_kv_heads
        self.max_seq_len, self.head_dim = max_seq_len, head_dim
        self._h = lib().xo_cache_new(num_layers, num_kv_heads, max_seq_len, head_dim)
        if not self._h:
            raise MemoryError("xo_cache_new failed")

    def _view(self, fn, layer):
        n = self.num_kv_heads * self.max_seq_len * self.head_dim
        return np.ctypeslib.as_array(fn(self._h, layer), shape=(n,))

    def k_buffer(self, layer) -> np.ndarray:
        """The reference's pub field ``k_buffers[layer]``: index h*cap*D + t*D + d."""
        return self._view(lib().xo_cache_k, layer)

    def v_buffer(self, layer) -> np.ndarray:
        return self._view(lib().xo_cache_v, layer)

    def append(self, layer, index_pos, k, v):
        k, v = _f32(k), _f32(v)
        S = k.shape[-2]
        lib().xo_cache_append(self._h, layer, index_pos, S, _p(k), _p(v))

    def close(self):
        if self._h:
            lib().xo_cache_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def quantize_to_u8(rows):
    """CpuRingCache::quantize_to_u8 (fast_attention.rs:62-71) on every row (last axis) of ``rows``:
    returns (bytes uint8 of the same shape, scales float32 of the leading shape)."""
    x = _f32(rows)
    n = x.shape[-1]
    r = x.size // n if n else 0
    q = np.zeros(x.shape, dtype=np.uint8)
    sc = np.zeros(x.shape[:-1], dtype=np.float32)
    lib().xo_quantize_to_u8(_p(x), r, n, q.ctypes.data_as(C.c_void_p), _p(sc))
    return q, sc


def dequantize_u8(q, scales) -> np.ndarray:
    """(byte - 128) * scale per row: what a reader of the u8 cache format sees."""
    q = np.ascontiguousarray(q, dtype=np.uint8)
    sc = _f32(scales)
    n = q.shape[-1]
    out = np.zeros(q.shape, dtype=np.float32)
    lib().xo_dequantize_u8(q.ctypes.data_as(C.c_void_p), _p(sc), q.size // n if n else 0, n, _p(out))
    return out


def u8_round_trip(rows) -> np.ndarray:
    """Rows as the u8 cache format returns them: quantise, then dequantise."""
    q, sc = quantize_to_u8(rows)
    return dequantize_u8(q, sc)


def fast_attention(q, k, v, layer_idx, index_pos, cache: RingCache, num_heads, num_kv_heads,
                   head_dim, threads: int = 0) -> np.ndarray:
    """fast_attention (fast_attention.rs:75-204).  Raises ValueError with the reference's
    messages for the two checked shape errors (:86-92)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    if q.ndim != 4:
        raise ValueError("fast_attention: Q shape must be 4D")
    if q.shape[0] != 1:
        raise ValueError(
            f"fast_attention currently only supports batch size 1, got {q.shape[0]}")
    S = q.shape[2]
    out = np.zeros((1, num_heads, S, head_dim), dtype=np.float32)
    rc = lib().xo_fast_attention(_p(q), _p(k), _p(v), layer_idx, index_pos, cache._h, num_heads,
                                 num_kv_heads, head_dim, S, 4, 1, _p(out), threads)
    assert rc == 0
    return out


def fast_attention_streams(qs, ks, vs, layer_idx, index_pos, caches, num_heads, num_kv_heads,
                           head_dim, threads: int = 0):
    """One fast_attention call per stream, (stream, KV head) pairs spread over host threads."""
    n = len(qs)
    qs = [_f32(a) for a in qs]
    ks = [_f32(a) for a in ks]
    vs = [_f32(a) for a in vs]
    seq = [int(a.shape[-2]) for a in qs]
    outs = [np.zeros((1, num_heads, s, head_dim), dtype=np.float32) for s in seq]
    PA = _f32p * n
    rc = lib().xo_fast_attention_streams(
        n, PA(*[_p(a) for a in qs]), PA(*[_p(a) for a in ks]), PA(*[_p(a) for a in vs]), layer_idx,
        (_sz * n)(*[int(p) for p in index_pos]), (_sz * n)(*seq),
        (C.c_void_p * n)(*[c._h for c in caches]), num_heads, num_kv_heads, head_dim,
        PA(*[_p(a) for a in outs]), threads)
    assert rc == 0
    return outs


# --- attention output block: sub-norm + ternary o_proj (attention.rs:103-108) --------------------

def rms_norm(x, weight, eps) -> np.ndarray:
    """rms_norm (fast_attention_simd.rs:502-521) on one row; returns the normalised copy."""
    x, weight = _f32(x).copy(), _f32(weight)
    lib().xo_rms_norm(_p(x), _p(weight), eps, x.size)
    return x


def tensor_rmsnorm(x, weight, eps) -> np.ndarray:
    """FastTensor::rmsnorm (tensor.rs:242-265): every row of the last dimension."""
    x, weight = _f32(x), _f32(weight)
    if weight.size != x.shape[-1]:
        raise ValueError(f"FastTensor::rmsnorm weight size mismatch: expected {x.shape[-1]}, got {weight.size}")
    out = np.empty_like(x)
    lib().xo_tensor_rmsnorm(_p(x), _p(out), _p(weight), eps, x.size // x.shape[-1], x.shape[-1])
    return out


def set_quant_body(body: int) -> int:
    """-1: the quantiser follows the ISA level; 0: scalar body; 1: AVX-512 body (any CPU)."""
    return lib().xo_set_quant_body(body)


def quantize_f32_to_i8(acts):
    """quantize_f32_to_i8 (bit1_58/quantization.rs:95-187) -> (i8 array, inv_scale)."""
    acts = _f32(acts).ravel()
    q = np.zeros(acts.size, dtype=np.int8)
    inv = lib().xo_quantize_f32_to_i8(_p(acts), acts.size, q.ctypes.data_as(_i8p))
    return q, float(np.float32(inv))


def pack_ternary(weights, w_scale, pack_type=PACK4) -> np.ndarray:
    w = _f32(weights).ravel()
    out = np.zeros(lib().xo_packed_row_bytes(w.size, pack_type), dtype=np.uint8)
    (lib().xo_pack5 if pack_type == PACK5 else lib().xo_pack4)(_p(w), w.size, w_scale,
                                                               out.ctypes.data_as(_u8p))
    return out


def unpack_ternary(packed, n, pack_type=PACK4) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.zeros(n, dtype=np.float32)
    (lib().xo_unpack5 if pack_type == PACK5 else lib().xo_unpack4)(packed.ctypes.data_as(_u8p), n,
                                                                   _p(out))
    return out


def ternary_dot(acts_i8, packed, n, pack_type=PACK4) -> int:
    a = np.ascontiguousarray(acts_i8, dtype=np.int8)
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    fn = lib().xo_ternary_dot_pack5 if pack_type == PACK5 else lib().xo_ternary_dot_pack4
    return int(fn(a.ctypes.data_as(_i8p), packed.ctypes.data_as(_u8p), n))


def sparse_encode_row(vals_i8, in_dim) -> np.ndarray:
    """encode_sparse_row_into (bit1_58/sparse.rs:62-89)."""
    v = np.ascontiguousarray(vals_i8, dtype=np.int8)
    out = np.zeros(4 + ((in_dim + 63) // 64) * 16, dtype=np.uint8)
    n = lib().xo_sparse_encode_row(v.ctypes.data_as(_i8p), in_dim, out.ctypes.data_as(_u8p))
    return out[:n].copy()


def sparse_decode_row(row_bytes, in_dim):
    """SparseTernary::decode_row (bit1_58/sparse.rs:206-249) -> (i8 values, bytes of the row)."""
    row = np.ascontiguousarray(row_bytes, dtype=np.uint8)
    out = np.zeros(in_dim, dtype=np.int8)
    n = lib().xo_sparse_decode_row(row.ctypes.data_as(_u8p), in_dim, out.ctypes.data_as(_i8p))
    return out, int(n)


def ternary_dot_sparse(acts_i8, row_bytes, in_dim) -> int:
    a = np.ascontiguousarray(acts_i8, dtype=np.int8)
    row = np.ascontiguousarray(row_bytes, dtype=np.uint8)
    return int(lib().xo_ternary_dot_sparse(a.ctypes.data_as(_i8p), row.ctypes.data_as(_u8p), in_dim))


class TernaryLinear:
    """TernaryLinear (bit1_58/layers.rs:34-313) with the dense packed representation, or with
    ``pack_type=SPARSE`` the XorSparse one of ``new_sparse`` (:151-181): ``packed`` is then the blob
    and the forward pass runs over the rows decoded from it (the format is lossless)."""

    def __init__(self, in_dim, out_dim, weights_f32, pack_type=PACK4, provided_scale=None):
        w = _f32(weights_f32).ravel()
        if w.size != in_dim * out_dim:
            raise ValueError("Weight length must match in_dim * out_dim")
        if pack_type == SPARSE:
            self.in_dim, self.out_dim, self.pack_type = in_dim, out_dim, SPARSE
            blob = np.zeros(out_dim * (4 + ((in_dim + 63) // 64) * 16) + 16, dtype=np.uint8)
            self.w_scales = np.zeros(out_dim, dtype=np.float32)
            n = lib().xo_ternary_linear_pack_sparse(in_dim, out_dim, _p(w),
                                                    float("nan") if provided_scale is None else provided_scale,
                                                    blob.ctypes.data_as(_u8p), _p(self.w_scales))
            self.packed = blob[:n].copy()
            rows, off = [], 0
            for _ in range(out_dim):
                vals, used = sparse_decode_row(self.packed[off:], in_dim)
                rows.append(vals.astype(np.float32))
                off += used
            assert off == self.packed.size
            # the dense twin the forward pass uses: exactly the decoded rows, original scales
            self._dense = TernaryLinear(in_dim, out_dim, np.stack(rows) if rows else np.zeros((0, in_dim)), PACK4, 1.0)
            self._dense.w_scales = self.w_scales
            self.row_bytes = 0
            return
        self.in_dim, self.out_dim, self.pack_type = in_dim, out_dim, pack_type
        self.row_bytes = int(lib().xo_packed_row_bytes(in_dim, pack_type))
        self.packed = np.zeros(out_dim * self.row_bytes, dtype=np.uint8)
        self.w_scales = np.zeros(out_dim, dtype=np.float32)
        lib().xo_ternary_linear_pack(in_dim, out_dim, _p(w), pack_type,
                                     float("nan") if provided_scale is None else provided_scale,
                                     self.packed.ctypes.data_as(_u8p), _p(self.w_scales))

    def forward(self, x, threads: int = 0) -> np.ndarray:
        if self.pack_type == SPARSE:
            return self._dense.forward(x, threads)
        x = _f32(x)
        if x.ndim == 0:
            raise ValueError("Input must have at least 1 dimension")
        if x.shape[-1] != self.in_dim:
            raise ValueError(f"Input dimension mismatch: expected {self.in_dim}, got {x.shape[-1]}")
        rows = x.size // self.in_dim
        out = np.empty(x.shape[:-1] + (self.out_dim,), dtype=np.float32)
        lib().xo_ternary_linear_forward(_p(x), rows, self.in_dim, self.out_dim, self.pack_type,
                                        self.packed.ctypes.data_as(_u8p), _p(self.w_scales), _p(out),
                                        threads)
        return out


def attention_out_block(y, norm_weight, eps, o_proj: TernaryLinear, threads: int = 0) -> np.ndarray:
    """y [1,Hq,S,D] -> heads_to_seq -> optional sub-norm -> o_proj -> [1,S,out_dim]
    (models/llama/attention.rs:103-108)."""
    y = _f32(y)
    _, H, S, D = y.shape
    out = np.empty((1, S, o_proj.out_dim), dtype=np.float32)
    nw = _f32(norm_weight) if norm_weight is not None else None
    lib().xo_attention_out_block(_p(y), H, S, D, _p(nw) if nw is not None else None, eps,
                                 o_proj.out_dim, o_proj.pack_type,
                                 o_proj.packed.ctypes.data_as(_u8p), _p(o_proj.w_scales), _p(out),
                                 threads)
    return out


def causal_self_attention_forward(x, index_pos, layer_idx, cache: "RingCache", cos, sin,
                                  q_proj: TernaryLinear, k_proj: TernaryLinear, v_proj: TernaryLinear,
                                  num_heads, num_kv_heads, head_dim, sub_norm_weight, eps,
                                  o_proj: TernaryLinear, threads: int = 0, kv_u8: bool = False):
    """CausalSelfAttention::forward (models/llama/attention.rs:40-108) for ternary projections:
    x [1,S,hidden] -> q/k/v projections (each quantises the rows of x the same way, as the fused
    single-token path of bit1_58/layers.rs:347-424 does once) -> heads layout -> RoPE ->
    fast_attention -> heads_to_seq -> optional sub-norm -> o_proj.  Returns (y [1,S,out], attention
    output [1,Hq,S,D])."""
    x = _f32(x)
    q = transpose_seq_to_heads(q_proj.forward(x, threads), num_heads, head_dim)
    k = transpose_seq_to_heads(k_proj.forward(x, threads), num_kv_heads, head_dim)
    v = transpose_seq_to_heads(v_proj.forward(x, threads), num_kv_heads, head_dim)
    q = tensor_rope(q, cos, sin, index_pos)
    k = tensor_rope(k, cos, sin, index_pos)
    if kv_u8:   # checker of the u8 cache format: the cache holds (and returns) the round-tripped rows
        k, v = u8_round_trip(k), u8_round_trip(v)
    attn = fast_attention(q, k, v, layer_idx, index_pos, cache, num_heads, num_kv_heads, head_dim, threads)
    return attention_out_block(attn, sub_norm_weight, eps, o_proj, threads), attn


# --- independent f64 arbiter -------------------------------------------------------------------

def naive_attention_f64(q, k_all, v_all, index_pos, num_heads, num_kv_heads, head_dim):
    """Textbook causal GQA attention in float64 over the first index_pos+S cached tokens.

    q [Hq, S, D]; k_all, v_all [Hkv, L, D] with L = index_pos + S.  Independent of the
    restated code; plays the role candle plays in tests/fast_attention_tests.rs:15-91.
    """
    q = np.asarray(q, dtype=np.float64)
    k_all = np.asarray(k_all, dtype=np.float64)
    v_all = np.asarray(v_all, dtype=np.float64)
    Hq, S, D = q.shape
    G = num_heads // num_kv_heads
    L = index_pos + S
    scale = np.float64(np.float32(1.0) / np.sqrt(np.float32(head_dim)))
    out = np.zeros((Hq, S, D), dtype=np.float64)
    mask = np.arange(L)[None, :] > (index_pos + np.arange(S))[:, None]
    for h in range(Hq):
        kk, vv = k_all[h // G, :L], v_all[h // G, :L]
        s = (q[h] @ kk.T) * scale
        s[mask] = -np.inf
        s -= s.max(axis=1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(axis=1, keepdims=True)
        out[h] = p @ vv
    return out
