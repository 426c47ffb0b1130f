"""Generates the golden fixtures of this directory with the CPU oracle.

    python tests/golden/make_golden.py

The reference publishes no fixture files (its tests build their vectors from formulas, which
tests/test_oracle_golden.py reproduces), and it cannot be run where this repository is built (it
is Rust).  These fixtures therefore freeze the *oracle's* outputs on seeded inputs: the CPU tests
re-run the oracle against them (so a change in the oracle, the compiler flags or libm shows up),
and the GPU tests compare the CUDA path with them.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle as xo  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    # name: (Hq, Hkv, D, theta, steps as (index_pos, seq_len), capacity)
    "gqa_2b_small": (20, 5, 128, 500000.0, [(0, 9), (9, 1), (10, 1), (11, 3)], 16),
    "mha_d100": (4, 4, 100, 10000.0, [(0, 7), (7, 1), (8, 1)], 12),
    "gqa_d8_reference_test_shape": (4, 2, 8, 10000.0, [(0, 4), (4, 1)], 32),
    "ring_fold": (4, 2, 16, 10000.0, [(0, 20), (20, 10), (30, 9), (39, 1)], 33),
}


def build(name):
    Hq, Hkv, D, theta, steps, cap = CASES[name]
    rng = np.random.default_rng(sum(map(ord, name)))  # a seed that depends only on the case name
    max_pos = max(p + s for p, s in steps)
    cos, sin = xo.rope_tables(theta, D, max_pos)
    cache = xo.RingCache(1, Hkv, cap, D)
    out = {"meta": np.array([Hq, Hkv, D, cap, len(steps)], np.int64), "theta": np.float64(theta),
           "steps": np.array(steps, np.int64)}
    for i, (pos, S) in enumerate(steps):
        q = rng.standard_normal((1, Hq, S, D)).astype(np.float32)
        k = rng.standard_normal((1, Hkv, S, D)).astype(np.float32)
        v = rng.standard_normal((1, Hkv, S, D)).astype(np.float32)
        qr, kr = xo.tensor_rope(q, cos, sin, pos), xo.tensor_rope(k, cos, sin, pos)
        o = xo.fast_attention(qr, kr, v, 0, pos, cache, Hq, Hkv, D)
        out[f"q{i}"], out[f"k{i}"], out[f"v{i}"], out[f"out{i}"] = q, k, v, o
    out["k_cache"] = cache.k_buffer(0).copy()
    out["v_cache"] = cache.v_buffer(0).copy()
    return out


# Whole attention block (ternary q/k/v projections, RoPE, attention, sub-norm, ternary o_proj):
# name: (Hq, Hkv, D, hidden, out_dim, pack, theta, steps, capacity)
BLOCK_CASES = {
    "block_pack4": (4, 2, 16, 48, 40, xo.PACK4, 10000.0, [(0, 5), (5, 1), (6, 1)], 16),
    "block_pack5": (3, 1, 32, 60, 20, xo.PACK5, 500000.0, [(0, 3), (3, 1)], 8),
}


def block_layers(z_or_rng, Hq, Hkv, D, hidden, out_dim, pack):
    """The four TernaryLinears of a block case, from stored f32 weights or fresh from a generator."""
    shapes = {"wq": (Hq * D, hidden), "wk": (Hkv * D, hidden), "wv": (Hkv * D, hidden), "wo": (out_dim, Hq * D)}
    ws = {n: (z_or_rng[n] if not hasattr(z_or_rng, "standard_normal")
              else z_or_rng.standard_normal(sh).astype(np.float32)) for n, sh in shapes.items()}
    scale = {n: (float(hidden) ** -0.5 if n != "wo" else None) for n in ws}   # q, k, v rows stay O(1)
    return ws, scale


def build_block(name):
    Hq, Hkv, D, hidden, out_dim, pack, theta, steps, cap = BLOCK_CASES[name]
    rng = np.random.default_rng(sum(map(ord, name)))
    xo.set_quant_body(1)   # the AVX-512 quantiser body, whatever CPU generates the fixture
    ws, scale = block_layers(rng, Hq, Hkv, D, hidden, out_dim, pack)
    lin = {n: xo.TernaryLinear(w.shape[1], w.shape[0], w, pack, scale[n]) for n, w in ws.items()}
    norm_w = (1.0 + 0.2 * rng.standard_normal(Hq * D)).astype(np.float32)
    cos, sin = xo.rope_tables(theta, D, max(p + s for p, s in steps))
    cache = xo.RingCache(1, Hkv, cap, D)
    out = {"meta": np.array([Hq, Hkv, D, hidden, out_dim, pack, cap, len(steps)], np.int64),
           "theta": np.float64(theta), "steps": np.array(steps, np.int64), "norm_w": norm_w,
           "eps": np.float32(1e-5), **ws}
    for i, (pos, S) in enumerate(steps):
        x = rng.standard_normal((1, S, hidden)).astype(np.float32)
        y, attn = xo.causal_self_attention_forward(x, pos, 0, cache, cos, sin, lin["wq"], lin["wk"], lin["wv"],
                                                   Hq, Hkv, D, norm_w, 1e-5, lin["wo"])
        out[f"x{i}"], out[f"y{i}"], out[f"attn{i}"] = x, y, attn
    out["k_cache"] = cache.k_buffer(0).copy()
    out["v_cache"] = cache.v_buffer(0).copy()
    xo.set_quant_body(-1)
    return out


if __name__ == "__main__":
    xo.set_isa(xo.ISA_AVX512) if xo.set_isa(xo.ISA_AVX512) == 0 else None
    for name in CASES:
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **build(name))
        print("wrote", name)
    for name in BLOCK_CASES:
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **build_block(name))
        print("wrote", name)
