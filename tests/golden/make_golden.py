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


if __name__ == "__main__":
    xo.set_isa(xo.ISA_AVX512) if xo.set_isa(xo.ISA_AVX512) == 0 else None
    for name in CASES:
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **build(name))
        print("wrote", name)
