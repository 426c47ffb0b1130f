"""Golden fixtures (tests/golden/*.npz, made by tests/golden/make_golden.py with the CPU oracle).

CPU: the oracle still reproduces them bit for bit (AVX-512 body) or within 1e-6 (other bodies).
GPU: the CUDA path, through the C ABI with fused RoPE, matches them within the f32 tolerances and
leaves a bit-identical cache.
"""
import glob
import os

import numpy as np
import pytest

import oracle as xo

HERE = os.path.dirname(os.path.abspath(__file__))
FIXTURES = sorted(p for p in glob.glob(os.path.join(HERE, "golden", "*.npz"))
                  if not os.path.basename(p).startswith("block_"))
BLOCK_FIXTURES = sorted(glob.glob(os.path.join(HERE, "golden", "block_*.npz")))


def load(path):
    z = np.load(path)
    Hq, Hkv, D, cap, n = (int(x) for x in z["meta"])
    return z, Hq, Hkv, D, cap, n, float(z["theta"]), [tuple(int(x) for x in s) for s in z["steps"]]


def test_fixtures_exist():
    assert len(FIXTURES) >= 4


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p) for p in FIXTURES])
def test_oracle_reproduces_fixture(path):
    z, Hq, Hkv, D, cap, n, theta, steps = load(path)
    exact = xo.set_isa(xo.ISA_AVX512) == 0  # the fixtures were made with the AVX-512 body
    if not exact:
        xo.set_isa(xo.ISA_AUTO)
    cos, sin = xo.rope_tables(theta, D, max(p + s for p, s in steps))
    cache = xo.RingCache(1, Hkv, cap, D)
    for i, (pos, S) in enumerate(steps):
        out = xo.fast_attention(xo.tensor_rope(z[f"q{i}"], cos, sin, pos), xo.tensor_rope(z[f"k{i}"], cos, sin, pos),
                                z[f"v{i}"], 0, pos, cache, Hq, Hkv, D)
        if exact:
            assert np.array_equal(out, z[f"out{i}"]), f"step {i}"
        else:
            assert np.max(np.abs(out - z[f"out{i}"])) < 1e-6
    assert np.array_equal(cache.k_buffer(0), z["k_cache"]) and np.array_equal(cache.v_buffer(0), z["v_cache"])
    xo.set_isa(xo.ISA_AUTO)


@pytest.mark.gpu
@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p) for p in FIXTURES])
def test_gpu_matches_fixture(path):
    import xor_net_b200 as xn
    from gpu_util import assert_parity

    z, Hq, Hkv, D, cap, n, theta, steps = load(path)
    cos, sin = xn.rope_tables(theta, D, max(p + s for p, s in steps))
    ctx = xn.Context(1, Hq, Hkv, D, pool_pages=8, rope=(cos, sin), prefill_mode=1)
    st = ctx.new_stream(cap)
    for i, (pos, S) in enumerate(steps):
        got = ctx.attention(st, 0, pos, z[f"q{i}"], z[f"k{i}"], z[f"v{i}"], rope=True)
        assert_parity(got, z[f"out{i}"], f"{os.path.basename(path)} step {i}")
    k, v = st.read_range(0, 0, cap)
    assert np.array_equal(k.ravel(), z["k_cache"]) and np.array_equal(v.ravel(), z["v_cache"])
    ctx.close()


# ---- whole attention block (ternary projections around the attention) ---------------------------

def load_block(path):
    z = np.load(path)
    Hq, Hkv, D, hidden, out_dim, pack, cap, n = (int(x) for x in z["meta"])
    steps = [tuple(int(x) for x in s) for s in z["steps"]]
    scale = {n_: (float(hidden) ** -0.5 if n_ != "wo" else None) for n_ in ("wq", "wk", "wv", "wo")}
    return z, Hq, Hkv, D, hidden, out_dim, pack, cap, float(z["theta"]), steps, scale


@pytest.mark.parametrize("path", BLOCK_FIXTURES, ids=[os.path.basename(p) for p in BLOCK_FIXTURES])
def test_oracle_reproduces_block_fixture(path):
    z, Hq, Hkv, D, hidden, out_dim, pack, cap, theta, steps, scale = load_block(path)
    exact = xo.set_isa(xo.ISA_AVX512) == 0
    if not exact:
        xo.set_isa(xo.ISA_AUTO)
    xo.set_quant_body(1)
    try:
        lin = {n: xo.TernaryLinear(z[n].shape[1], z[n].shape[0], z[n], pack, scale[n]) for n in scale}
        cos, sin = xo.rope_tables(theta, D, max(p + s for p, s in steps))
        cache = xo.RingCache(1, Hkv, cap, D)
        for i, (pos, S) in enumerate(steps):
            y, attn = xo.causal_self_attention_forward(z[f"x{i}"], pos, 0, cache, cos, sin, lin["wq"], lin["wk"],
                                                       lin["wv"], Hq, Hkv, D, z["norm_w"], float(z["eps"]), lin["wo"])
            if exact:
                assert np.array_equal(y, z[f"y{i}"]) and np.array_equal(attn, z[f"attn{i}"]), f"step {i}"
            else:
                assert np.linalg.norm(y - z[f"y{i}"]) <= 1e-3 * np.linalg.norm(z[f"y{i}"])
        # the projections and the rotation do not depend on the attention's ISA body: always exact
        assert np.array_equal(cache.k_buffer(0), z["k_cache"]) and np.array_equal(cache.v_buffer(0), z["v_cache"])
    finally:
        xo.set_quant_body(-1)
        xo.set_isa(xo.ISA_AUTO)


@pytest.mark.gpu
@pytest.mark.parametrize("path", BLOCK_FIXTURES, ids=[os.path.basename(p) for p in BLOCK_FIXTURES])
def test_gpu_matches_block_fixture(path):
    import xor_net_b200 as xn
    from gpu_util import assert_parity, errs

    z, Hq, Hkv, D, hidden, out_dim, pack, cap, theta, steps, scale = load_block(path)
    cos, sin = xn.rope_tables(theta, D, max(p + s for p, s in steps))
    ctx = xn.Context(1, Hq, Hkv, D, pool_pages=4, rope=(cos, sin), prefill_mode=1)
    lin = {n: xn.TernaryLinear(z[n].shape[1], z[n].shape[0], z[n], pack, scale[n]) for n in scale}
    ctx.set_qkv_proj(0, lin["wq"], lin["wk"], lin["wv"])
    ctx.set_out_proj(0, lin["wo"], z["norm_w"], float(z["eps"]))
    st = ctx.new_stream(cap)
    for i, (pos, S) in enumerate(steps):
        attn = ctx.attention_batch([st], 0, [pos], [z[f"x{i}"]], qkv_proj=True)[0]
        y = ctx.attention_batch([st], 0, [pos], [z[f"x{i}"]], qkv_proj=True, out_proj=True)[0]
        assert_parity(attn, xo.transpose_heads_to_seq(z[f"attn{i}"]), f"{os.path.basename(path)} attention {i}")
        assert errs(y, z[f"y{i}"])[1] <= 1e-3, f"{os.path.basename(path)} block {i}"
    k, v = st.read_range(0, 0, cap)
    assert np.array_equal(k.ravel(), z["k_cache"]) and np.array_equal(v.ravel(), z["v_cache"])
    ctx.close()
