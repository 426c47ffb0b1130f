"""Python host side over the C ABI.

Two layers:

* ``Context`` / ``Stream``: thin handles over ``xn_ctx`` / ``xn_stream`` with numpy (host) and
  raw-pointer (device) calls.  Used by the benchmark and the batch tests.
* ``FastTensor`` / ``DeviceKvCache`` / ``fast_attention``: the reference's operator interface for
  this path with the same names, argument order and error behaviour
  (src/nn/fast_attention.rs:18-60, :75-85; src/tensor.rs:6-40), so that tests written against the
  reference read the same here.  ``DeviceKvCache`` stands where ``CpuRingCache`` stood.

All compute happens in the CUDA library; nothing here falls back to numpy or torch.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from typing import Optional, Sequence

import numpy as np

from . import _ffi
from ._ffi import (KV_F32, KV_U8, PACK4, PACK5, SPARSE, REQ_DEVICE_PTRS, REQ_HOST_PINNED, REQ_OUT_PROJ, REQ_QKV_PROJ, REQ_ROPE,
                   REQ_SEQ_MAJOR, CtxDesc, OutProjDesc, QkvProjDesc, Req, Stats)


class XnError(RuntimeError):
    """A non-zero xn_status; ``code`` is the status, the text comes from xn_last_error."""

    def __init__(self, code: int, text: str):
        super().__init__(f"{_ffi.STATUS_NAMES.get(code, code)}: {text}")
        self.code = code
        self.text = text


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def rope_tables(theta: float, head_dim: int, max_pos: int, scaling=None):
    """cos, sin ``[max_pos, head_dim // 2]`` as Cache::new builds them (models/llama/mod.rs:210-265).

    ``scaling`` = (factor, low_freq_factor, high_freq_factor, original_max_position_embeddings).
    """
    lib = _ffi.load()
    half = head_dim // 2
    cos = np.zeros((max_pos, half), dtype=np.float32)
    sin = np.zeros((max_pos, half), dtype=np.float32)
    f, lo, hi, orig = scaling if scaling else (0.0, 1.0, 1.0, 0)
    rc = lib.xn_rope_tables(theta, head_dim, max_pos, f, lo, hi, orig,
                            cos.ctypes.data_as(_ffi.c_f32p), sin.ctypes.data_as(_ffi.c_f32p))
    if rc != 0:
        raise XnError(rc, "xn_rope_tables: bad argument")
    return cos, sin


def _ctx_desc(num_layers, num_heads, num_kv_heads, head_dim, pool_pages, pool_bytes, device, shuffle_seed,
              rope, cuda_stream, prefill_mode, batch_window_us, kv_format):
    """(xn_ctx_desc, arrays it points at)."""
    d = CtxDesc()
    d.device, d.num_layers, d.num_heads = device, num_layers, num_heads
    d.num_kv_heads, d.head_dim, d.page_tokens = num_kv_heads, head_dim, 64
    d.pool_pages, d.pool_bytes, d.shuffle_seed = pool_pages, pool_bytes, shuffle_seed
    d.prefill_mode, d.batch_window_us = prefill_mode, batch_window_us
    d.kv_format = kv_format
    d.cuda_stream = cuda_stream or None
    keep = None
    if rope is not None:
        cos, sin = _f32(rope[0]), _f32(rope[1])
        keep = (cos, sin)
        d.max_pos, d.rope_cos, d.rope_sin = cos.shape[0], _ptr(cos), _ptr(sin)
    return d, keep


def place_stream(tokens, live_streams, ticket: int, policy: int = _ffi.PLACE_LEAST_LOADED) -> int:
    """xn_place_stream: the device a new stream goes to, given every device's cached (or announced)
    tokens and live streams and the number of streams placed so far.  Needs no GPU."""
    n = len(tokens)
    t = (C.c_int64 * n)(*[int(x) for x in tokens])
    l = (C.c_int64 * n)(*[int(x) for x in live_streams])
    where = _ffi.load().xn_place_stream(n, t, l, ticket, policy)
    if where < 0:
        raise XnError(-where, "xn_place_stream: bad argument")
    return where


class Stream:
    """One sequence's KV cache (one reference ``Cache``)."""

    def __init__(self, ctx: "Context", handle: int, max_seq_len: int):
        self.ctx, self.handle, self.max_seq_len = ctx, handle, max_seq_len

    def reset(self):
        self.ctx._check(self.ctx.lib.xn_stream_reset(self.ctx.handle, self.handle))

    def destroy(self):
        if self.handle and self.ctx.handle:
            self.ctx._check(self.ctx.lib.xn_stream_destroy(self.ctx.handle, self.handle))
        self.handle = None

    def length(self, layer: int) -> int:
        return int(self.ctx.lib.xn_stream_len(self.ctx.handle, self.handle, layer))

    def pages(self) -> np.ndarray:
        n = int(self.ctx.lib.xn_stream_pages(self.ctx.handle, self.handle, None, 0))
        out = np.zeros(max(n, 1), dtype=np.int32)
        self.ctx.lib.xn_stream_pages(self.ctx.handle, self.handle, out.ctypes.data_as(_ffi.c_i32p), n)
        return out[:n]

    def fill_normal(self, layer: int, t0: int, n: int, seed: int):
        """N(0,1) fill of slots [t0, t0+n) on the device; layer -1 fills every layer."""
        self.ctx._check(self.ctx.lib.xn_kv_fill_normal(self.ctx.handle, self.handle, layer, t0, n, seed))

    def read_range(self, layer: int, t0: int, n: int):
        """(k, v) each ``[Hkv, n, D]``: slots t0..t0+n of the logical ring."""
        c = self.ctx
        k = np.zeros((c.num_kv_heads, n, c.head_dim), dtype=np.float32)
        v = np.zeros_like(k)
        c._check(c.lib.xn_kv_read_range(c.handle, self.handle, layer, t0, n, _ptr(k), _ptr(v)))
        return k, v

    def read_u8(self, layer: int, t0: int, n: int):
        """``KV_U8`` contexts: the stored (k_u8, v_u8, k_scales, v_scales) of slots t0..t0+n, shaped
        ``[Hkv, n, D]`` (uint8) and ``[Hkv, n]`` (float32) like the reference's ``U8CacheLayer``."""
        c = self.ctx
        k8 = np.zeros((c.num_kv_heads, n, c.head_dim), dtype=np.uint8)
        v8 = np.zeros_like(k8)
        ks = np.zeros((c.num_kv_heads, n), dtype=np.float32)
        vs = np.zeros_like(ks)
        c._check(c.lib.xn_kv_read_u8(c.handle, self.handle, layer, t0, n, k8.ctypes.data, v8.ctypes.data,
                                     _ptr(ks), _ptr(vs)))
        return k8, v8, ks, vs

    def read(self, layer: int, kv_head: int, t: int):
        c = self.ctx
        k = np.zeros(c.head_dim, dtype=np.float32)
        v = np.zeros_like(k)
        c._check(c.lib.xn_kv_read(c.handle, self.handle, layer, kv_head, t, _ptr(k), _ptr(v)))
        return k, v


class Context:
    """One GPU's page pool and launch state (``xn_ctx``)."""

    def __init__(self, num_layers: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 pool_pages: int = 0, pool_bytes: int = 0, device: int = 0, shuffle_seed: int = 0,
                 rope: Optional[tuple] = None, cuda_stream: int = 0, prefill_mode: int = 0,
                 batch_window_us: int = 0, kv_format: int = KV_F32):
        self.lib = _ffi.load()
        self.num_layers, self.num_heads = num_layers, num_heads
        self.num_kv_heads, self.head_dim = num_kv_heads, head_dim
        self.device = device
        self.kv_format = kv_format
        self._owner = None
        d, self._rope = _ctx_desc(num_layers, num_heads, num_kv_heads, head_dim, pool_pages, pool_bytes, device,
                                  shuffle_seed, rope, cuda_stream, prefill_mode, batch_window_us, kv_format)
        h = C.c_void_p()
        rc = self.lib.xn_ctx_create(C.byref(d), C.byref(h))
        if rc != 0:
            raise XnError(rc, (self.lib.xn_last_error(None) or b"").decode())
        self.handle = h.value

    @classmethod
    def _adopt(cls, owner, handle, device, num_layers, num_heads, num_kv_heads, head_dim, kv_format):
        """A context that a ``Group`` created and destroys."""
        self = cls.__new__(cls)
        self.lib = _ffi.load()
        self.num_layers, self.num_heads = num_layers, num_heads
        self.num_kv_heads, self.head_dim = num_kv_heads, head_dim
        self.device, self.kv_format = device, kv_format
        self._owner, self._rope, self.handle = owner, None, handle
        return self

    def _check(self, rc: int):
        if rc != 0:
            raise XnError(rc, (self.lib.xn_last_error(self.handle) or b"").decode())

    def drop_plan(self):
        """xn_debug_drop_plan: the next decode submission plans afresh (what a new position does)."""
        self._check(self.lib.xn_debug_drop_plan(self.handle))

    def check_guards(self):
        """xn_debug_check_guards: raises if a kernel wrote outside one of the context's device buffers."""
        self._check(self.lib.xn_debug_check_guards(self.handle))

    def close(self, check_guards: bool = True):
        """Destroys the context.  The guard areas around its device buffers are verified first (a
        few small copies), so that every test that closes its context also checks memory safety."""
        if getattr(self, "handle", None) and self._owner is None:
            rc = self.lib.xn_debug_check_guards(self.handle) if check_guards else 0
            text = (self.lib.xn_last_error(self.handle) or b"").decode() if rc else ""
            self.lib.xn_ctx_destroy(self.handle)
            self.handle = None
            if rc == 11:
                raise XnError(rc, text)
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def new_stream(self, max_seq_len: int) -> Stream:
        h = C.c_void_p()
        self._check(self.lib.xn_stream_create(self.handle, max_seq_len, C.byref(h)))
        return Stream(self, h.value, max_seq_len)

    def synchronize(self):
        self._check(self.lib.xn_ctx_synchronize(self.handle))

    def cuda_stream(self) -> int:
        return int(self.lib.xn_ctx_cuda_stream(self.handle) or 0)

    def stats(self) -> dict:
        s = Stats()
        self._check(self.lib.xn_stats_get(self.handle, C.byref(s)))
        return {n: int(getattr(s, n)) for n, _ in Stats._fields_}

    def fill_normal(self, device_ptr: int, n: int, seed: int):
        self._check(self.lib.xn_fill_normal(self.handle, device_ptr, n, seed))

    def profile_enable(self, on: bool = True):
        self._check(self.lib.xn_profile_enable(self.handle, 1 if on else 0))

    def profile_read(self, which: str = "splitkv"):
        """(milliseconds, launches) of the split-KV kernel (or "prefill") since the last read;
        "both" returns the two pairs."""
        ms, n, pms, pn = C.c_double(), C.c_uint64(), C.c_double(), C.c_uint64()
        self._check(self.lib.xn_profile_read(self.handle, C.byref(ms), C.byref(n), C.byref(pms),
                                             C.byref(pn)))
        if which == "both":
            return (ms.value, int(n.value)), (pms.value, int(pn.value))
        return (pms.value, int(pn.value)) if which == "prefill" else (ms.value, int(n.value))

    def profile_read_all(self):
        """[(milliseconds, launches)] per timed kind: split-KV, tensor-core prefill, output block,
        q/k/v block."""
        ms, n = (C.c_double * 4)(), (C.c_uint64 * 4)()
        self._check(self.lib.xn_profile_read_all(self.handle, ms, n))
        return [(ms[i], int(n[i])) for i in range(4)]

    # -- attention output block (sub-norm + ternary o_proj) ------------------------------------

    def set_out_proj(self, layer: int, linear: "TernaryLinear", norm_weight=None, eps: float = 1e-5):
        """xn_out_proj_set: the o_proj weights (and optional sub-norm) of one layer."""
        d = OutProjDesc()
        d.layer, d.in_dim, d.out_dim, d.pack_type = layer, linear.in_dim, linear.out_dim, linear.pack_type
        d.packed, d.w_scales = linear.packed.ctypes.data, _ptr(linear.w_scales)
        nw = _f32(norm_weight) if norm_weight is not None else None
        d.norm_weight, d.norm_eps = (_ptr(nw) if nw is not None else None), eps
        self._check(self.lib.xn_out_proj_set(self.handle, C.byref(d)))
        self._out_dims = getattr(self, "_out_dims", {})
        self._out_dims[layer] = linear.out_dim

    def set_qkv_proj(self, layer: int, q_proj: "TernaryLinear", k_proj: "TernaryLinear",
                     v_proj: "TernaryLinear"):
        """xn_qkv_proj_set: the three input projections of one layer (same in_dim and packing)."""
        if not (q_proj.in_dim == k_proj.in_dim == v_proj.in_dim and
                q_proj.pack_type == k_proj.pack_type == v_proj.pack_type):
            raise ValueError("q, k, v projections must share in_dim and pack_type")
        d = QkvProjDesc()
        d.layer, d.in_dim, d.pack_type = layer, q_proj.in_dim, q_proj.pack_type
        d.q_packed, d.q_scales = q_proj.packed.ctypes.data, _ptr(q_proj.w_scales)
        d.k_packed, d.k_scales = k_proj.packed.ctypes.data, _ptr(k_proj.w_scales)
        d.v_packed, d.v_scales = v_proj.packed.ctypes.data, _ptr(v_proj.w_scales)
        self._check(self.lib.xn_qkv_proj_set(self.handle, C.byref(d)))

    def out_proj(self, layer: int, y) -> np.ndarray:
        """xn_out_proj on host arrays: y [..., in_dim] -> [..., out_dim]."""
        y = _f32(y)
        out = np.empty(y.shape[:-1] + (self._out_dims[layer],), dtype=np.float32)
        rows = y.size // y.shape[-1] if y.size else 0
        self._check(self.lib.xn_out_proj(self.handle, layer, rows, _ptr(y), _ptr(out), 0))
        return out

    # -- blocking single-stream calls (host arrays) ------------------------------------------

    def attention(self, stream: Stream, layer: int, index_pos: int, q, k, v, rope: bool = False):
        """xn_attention / xn_attention_rope.  q [1,Hq,S,D], k,v [1,Hkv,S,D] -> out [1,Hq,S,D]."""
        q, k, v = _f32(q), _f32(k), _f32(v)
        S = q.shape[-2]
        out = np.empty((1, self.num_heads, S, self.head_dim), dtype=np.float32)
        fn = self.lib.xn_attention_rope if rope else self.lib.xn_attention
        self._check(fn(self.handle, stream.handle, layer, index_pos, S, _ptr(q), _ptr(k), _ptr(v),
                       _ptr(out)))
        return out

    # -- explicit batches -------------------------------------------------------------------

    def make_batch(self, entries: Sequence[tuple], flags: int = 0):
        """entries: (stream, layer, index_pos, seq_len, q_ptr, k_ptr, v_ptr, out_ptr) -> Req array."""
        arr = (Req * len(entries))()
        for i, (st, layer, pos, S, q, k, v, o) in enumerate(entries):
            r = arr[i]
            r.stream, r.layer, r.seq_len, r.index_pos = st.handle, layer, S, pos
            r.q, r.k, r.v, r.out, r.flags = q, k, v, o, flags
        return arr

    def submit(self, reqs, n: Optional[int] = None):
        self._check(self.lib.xn_attention_batch(self.handle, len(reqs) if n is None else n, reqs))

    def attention_batch(self, streams, layer, index_pos, qs, ks=None, vs=None, rope=False,
                        seq_major=False, out_proj=False, qkv_proj=False):
        """Host-array batch: one request per stream; returns the list of outputs
        ([1,S,out_dim] each with ``out_proj``: the layer's output block applied on the device).
        With ``qkv_proj`` the entries of ``qs`` are the hidden states x [1,S,hidden] and the layer's
        q/k/v projections, the heads layout and the rotation run on the device; the attention output
        then comes back sequence-major, [1,S,Hq*D]."""
        qs = [_f32(a) for a in qs]
        ks = [_f32(a) for a in ks] if not qkv_proj else [None] * len(qs)
        vs = [_f32(a) for a in vs] if not qkv_proj else [None] * len(qs)
        seq = [a.shape[-2] for a in qs]  # [1,H,S,D] and [1,S,H*D] both keep S there
        layers = layer if isinstance(layer, (list, tuple)) else [layer] * len(streams)
        if out_proj:
            outs = [np.empty((1, seq[i], self._out_dims[layers[i]]), dtype=np.float32)
                    for i in range(len(qs))]
        elif qkv_proj:
            outs = [np.empty((1, seq[i], self.num_heads * self.head_dim), dtype=np.float32)
                    for i in range(len(qs))]
        else:
            outs = [np.empty_like(a) for a in qs]
        flags = (REQ_ROPE if rope else 0) | (REQ_SEQ_MAJOR if seq_major else 0) | \
            (REQ_OUT_PROJ if out_proj else 0) | (REQ_QKV_PROJ if qkv_proj else 0)
        reqs = self.make_batch(
            [(st, layers[i], int(index_pos[i]), int(seq[i]), _ptr(qs[i]),
              _ptr(ks[i]) if ks[i] is not None else None, _ptr(vs[i]) if vs[i] is not None else None,
              _ptr(outs[i])) for i, st in enumerate(streams)], flags)
        self.submit(reqs)
        return outs


# =============================================================================================
# The reference's operator interface for this path
# =============================================================================================

class TernaryLinear:
    """Host mirror of ``TernaryLinear`` with the dense packed representation
    (src/bit1_58/layers.rs:34-149): ternarises and packs f32 weights exactly like
    ``TernaryLinear::new``; the forward pass runs on the device through a Context
    (``Context.set_out_proj`` / ``Context.out_proj`` / ``REQ_OUT_PROJ``)."""

    def __init__(self, in_dim: int, out_dim: int, weights_f32, pack_type: int = PACK4,
                 provided_scale: Optional[float] = None):
        w = _f32(weights_f32).ravel()
        if w.size != in_dim * out_dim:
            raise ValueError("Weight length must match in_dim * out_dim")
        if pack_type not in (PACK4, PACK5, SPARSE):
            raise ValueError("pack_type must be PACK4, PACK5 or SPARSE")
        self.in_dim, self.out_dim, self.pack_type = in_dim, out_dim, pack_type
        self.w_scales = np.zeros(max(1, out_dim), dtype=np.float32)
        scale = float("nan") if provided_scale is None else provided_scale
        if pack_type == SPARSE:   # TernaryLinear::new_sparse: the XorSparse blob, rows back to back
            cap = out_dim * (4 + ((in_dim + 63) // 64) * 16) + 16
            self.packed = np.zeros(cap, dtype=np.uint8)
            n = C.c_int64(0)
            rc = _ffi.load().xn_ternary_pack_sparse(in_dim, out_dim, _ptr(w), scale, self.packed.ctypes.data,
                                                    cap, C.byref(n), _ptr(self.w_scales))
            self.packed = self.packed[: n.value].copy()
            self.row_bytes = 0
        else:
            self.row_bytes = (in_dim + 4) // 5 if pack_type == PACK5 else (in_dim + 3) // 4
            self.packed = np.zeros(max(1, out_dim * self.row_bytes), dtype=np.uint8)
            rc = _ffi.load().xn_ternary_pack(in_dim, out_dim, _ptr(w), pack_type, scale,
                                             self.packed.ctypes.data, _ptr(self.w_scales))
        if rc != 0:
            raise XnError(rc, "xn_ternary_pack")
        self.w_scales = self.w_scales[:out_dim]


class FastTensor:
    """``FastTensor { data: Vec<f32>, shape: Vec<usize> }`` (src/tensor.rs:6-33)."""

    def __init__(self, data, shape):
        self.data = _f32(data).reshape(-1)
        self.shape = list(int(s) for s in shape)
        assert self.data.size == int(np.prod(self.shape)) if self.shape else True, \
            f"FastTensor::new shape mismatch: data len is {self.data.size}"

    @staticmethod
    def new(data, shape) -> "FastTensor":
        return FastTensor(data, shape)

    @staticmethod
    def zeros(shape) -> "FastTensor":
        return FastTensor(np.zeros(int(np.prod(shape)), np.float32), shape)

    def dims(self):
        return self.shape

    def array(self) -> np.ndarray:
        return self.data.reshape(self.shape)


class Group:
    """One context per GPU behind one handle (``xn_group``): what a single server process uses to
    reach every GPU of the box.  ``new_stream`` places the stream on the least-loaded device (or
    round-robin) and returns a ``Stream`` bound to that device's ``Context``."""

    def __init__(self, num_layers: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 devices: Optional[Sequence[int]] = None, pool_pages: int = 0, pool_bytes: int = 0,
                 shuffle_seed: int = 0, rope: Optional[tuple] = None, prefill_mode: int = 0,
                 batch_window_us: int = 0, kv_format: int = KV_F32):
        self.lib = _ffi.load()
        d, self._rope = _ctx_desc(num_layers, num_heads, num_kv_heads, head_dim, pool_pages, pool_bytes, 0,
                                  shuffle_seed, rope, 0, prefill_mode, batch_window_us, kv_format)
        devs = list(devices) if devices else []
        arr = (C.c_int32 * max(1, len(devs)))(*devs)
        h = C.c_void_p()
        rc = self.lib.xn_group_create(C.byref(d), arr if devs else None, len(devs), C.byref(h))
        if rc != 0:
            raise XnError(rc, (self.lib.xn_last_error(None) or b"").decode())
        self.handle = h.value
        n = self.lib.xn_group_size(self.handle)
        self.contexts = [Context._adopt(self, self.lib.xn_group_ctx(self.handle, i), devs[i] if devs else i,
                                        num_layers, num_heads, num_kv_heads, head_dim, kv_format)
                         for i in range(n)]
        self._by_handle = {c.handle: c for c in self.contexts}

    def __len__(self):
        return len(self.contexts)

    def new_stream(self, max_seq_len: int, expected_tokens: int = 0,
                   policy: int = _ffi.PLACE_LEAST_LOADED) -> Stream:
        ch, sh = C.c_void_p(), C.c_void_p()
        rc = self.lib.xn_group_stream_create(self.handle, max_seq_len, expected_tokens, policy,
                                             C.byref(ch), C.byref(sh))
        if rc != 0:
            raise XnError(rc, (self.lib.xn_last_error(None) or b"").decode())
        return Stream(self._by_handle[ch.value], sh.value, max_seq_len)

    def close(self):
        if getattr(self, "handle", None):
            for c in self.contexts:
                if c.handle:
                    c.check_guards()
            self.lib.xn_group_destroy(self.handle)
            for c in self.contexts:
                c.handle = None
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_contexts: dict = {}
_contexts_lock = threading.Lock()
_groups: dict = {}


def default_group(num_layers, num_heads, num_kv_heads, head_dim) -> Group:
    """Process-wide group per model shape over the devices of ``XORNET_ATTN_DEVICES`` (default: all
    visible), created on first use.  Pool per device: ``XORNET_ATTN_POOL_PAGES`` pages if set, else
    ``XORNET_ATTN_POOL_MB`` (default 1024) megabytes."""
    key = (num_layers, num_heads, num_kv_heads, head_dim)
    with _contexts_lock:
        g = _groups.get(key)
        if g is None or g.handle is None:
            pages = int(os.environ.get("XORNET_ATTN_POOL_PAGES", "0"))
            mb = int(os.environ.get("XORNET_ATTN_POOL_MB", "1024"))
            g = Group(num_layers, num_heads, num_kv_heads, head_dim, pool_pages=pages,
                      pool_bytes=0 if pages else mb << 20)
            _groups[key] = g
        return g



def default_context(num_layers, num_heads, num_kv_heads, head_dim, device: int = 0) -> Context:
    """Process-wide context per (device, model shape), created on first use.

    Pool size: ``XORNET_ATTN_POOL_PAGES`` pages if set, else ``XORNET_ATTN_POOL_MB`` (default 1024)
    megabytes.
    """
    key = (device, num_layers, num_heads, num_kv_heads, head_dim)
    with _contexts_lock:
        ctx = _contexts.get(key)
        if ctx is None or ctx.handle is None:
            pages = int(os.environ.get("XORNET_ATTN_POOL_PAGES", "0"))
            mb = int(os.environ.get("XORNET_ATTN_POOL_MB", "1024"))
            ctx = Context(num_layers, num_heads, num_kv_heads, head_dim, pool_pages=pages,
                          pool_bytes=0 if pages else mb << 20, device=device)
            _contexts[key] = ctx
        return ctx


def close_default_contexts():
    with _contexts_lock:
        for ctx in _contexts.values():
            ctx.close()
        _contexts.clear()
        for g in _groups.values():
            g.close()
        _groups.clear()


class DeviceKvCache:
    """Stands where ``CpuRingCache`` stood (src/nn/fast_attention.rs:18-60).

    Same constructor arguments.  Storage is pages of a device pool; the reference's pub fields
    ``k_buffers`` / ``v_buffers`` are read-back views with the reference's index
    ``h*cap*D + t*D + d``.  ``use_u8`` is accepted and ignored: the reference's u8 shadow
    (:62-71, :117-128) is written but never read, so it cannot influence any result.
    """

    def __init__(self, num_layers, num_kv_heads, max_seq_len, head_dim, use_u8=False, device=None):
        self.num_layers, self.num_kv_heads = num_layers, num_kv_heads
        self.max_seq_len, self.head_dim = max_seq_len, head_dim
        self.device = device   # None: whichever GPU of the process-wide group is least loaded
        self._ctx: Optional[Context] = None
        self._stream: Optional[Stream] = None

    @staticmethod
    def new(num_layers, num_kv_heads, max_seq_len, head_dim, use_u8=False) -> "DeviceKvCache":
        return DeviceKvCache(num_layers, num_kv_heads, max_seq_len, head_dim, use_u8)

    def _bind(self, num_heads: int):
        if self._stream is None:
            if self.device is None:
                # one process, every GPU: the cache lands on the device with the fewest cached tokens
                # (XORNET_ATTN_PLACEMENT=rr: stream number mod number of devices)
                rr = os.environ.get("XORNET_ATTN_PLACEMENT", "least").lower() in ("rr", "round_robin")
                group = default_group(self.num_layers, num_heads, self.num_kv_heads, self.head_dim)
                self._stream = group.new_stream(self.max_seq_len, 0,
                                                _ffi.PLACE_ROUND_ROBIN if rr else _ffi.PLACE_LEAST_LOADED)
                self._ctx = self._stream.ctx
                self.device = self._ctx.device
            else:
                self._ctx = default_context(self.num_layers, num_heads, self.num_kv_heads,
                                            self.head_dim, self.device)
                self._stream = self._ctx.new_stream(self.max_seq_len)
        return self._ctx, self._stream

    def _buffers(self, which: int):
        n = self.num_kv_heads * self.max_seq_len * self.head_dim
        if self._stream is None:
            return [np.zeros(n, np.float32) for _ in range(self.num_layers)]
        return [self._stream.read_range(l, 0, self.max_seq_len)[which].reshape(-1)
                for l in range(self.num_layers)]

    @property
    def k_buffers(self):
        return self._buffers(0)

    @property
    def v_buffers(self):
        return self._buffers(1)

    def close(self):
        if self._stream is not None:
            self._stream.destroy()
            self._stream = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def fast_attention(q: FastTensor, k: FastTensor, v: FastTensor, layer_idx: int, index_pos: int,
                   cache: DeviceKvCache, num_heads: int, num_kv_heads: int,
                   head_dim: int) -> FastTensor:
    """``fast_attention`` (src/nn/fast_attention.rs:75-204) on the GPU.

    Raises ``ValueError`` with the reference's messages for its two checked errors (:86-92);
    anything the library rejects raises ``XnError``.
    """
    if len(q.shape) != 4:
        raise ValueError("fast_attention: Q shape must be 4D")
    b_sz, _, seq_len, _ = q.shape
    if b_sz != 1:
        raise ValueError(f"fast_attention currently only supports batch size 1, got {b_sz}")
    ctx, stream = cache._bind(num_heads)
    out = ctx.attention(stream, layer_idx, index_pos, q.data.reshape(1, num_heads, seq_len, head_dim),
                        k.data.reshape(1, num_kv_heads, seq_len, head_dim),
                        v.data.reshape(1, num_kv_heads, seq_len, head_dim))
    return FastTensor(out, [b_sz, num_heads, seq_len, head_dim])
