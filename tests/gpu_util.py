"""Helpers shared by the GPU tests (parity metrics, paired device/oracle caches)."""
import numpy as np

import oracle as xo

# Tolerances of the f32 path: max abs error and relative L2 error against the CPU oracle.
ABS_TOL = 1e-4
REL_TOL = 1e-5


def errs(got, want):
    got = np.asarray(got, np.float64).ravel()
    want = np.asarray(want, np.float64).ravel()
    n = np.linalg.norm(want)
    return float(np.max(np.abs(got - want))), float(np.linalg.norm(got - want) / (n if n > 0 else 1.0))


def assert_parity(got, want, what="", abs_tol=ABS_TOL, rel_tol=REL_TOL):
    a, r = errs(got, want)
    assert a <= abs_tol and r <= rel_tol, f"{what}: max abs {a:.3e} (<= {abs_tol}), rel {r:.3e} (<= {rel_tol})"
    return a, r


class Pair:
    """A device stream and an oracle ring cache fed with the same bytes."""

    def __init__(self, ctx, cap):
        self.ctx, self.cap = ctx, cap
        self.st = ctx.new_stream(cap)
        self.ref = xo.RingCache(ctx.num_layers, ctx.num_kv_heads, cap, ctx.head_dim)

    def step(self, layer, pos, q, k, v, **kw):
        got = self.ctx.attention(self.st, layer, pos, q, k, v, **kw)
        want = xo.fast_attention(q, k, v, layer, pos, self.ref, self.ctx.num_heads,
                                 self.ctx.num_kv_heads, self.ctx.head_dim)
        return got, want

    def check_cache(self, layer):
        k, v = self.st.read_range(layer, 0, self.cap)
        assert np.array_equal(k.ravel(), self.ref.k_buffer(layer))
        assert np.array_equal(v.ravel(), self.ref.v_buffer(layer))


def rand_qkv(rng, Hq, Hkv, S, D):
    return (rng.standard_normal((1, Hq, S, D)).astype(np.float32),
            rng.standard_normal((1, Hkv, S, D)).astype(np.float32),
            rng.standard_normal((1, Hkv, S, D)).astype(np.float32))
