"""Pins the CPU oracle against the reference's own known-answer tests.

Each test regenerates the vectors of one reference test from the formula that test
uses (the reference ships no fixture files) and checks the oracle to the reference's
tolerance.  Reference files cited per test.
"""
import math

import numpy as np
import pytest

import oracle as xo

ISAS = [xo.ISA_SCALAR, xo.ISA_AVX2, xo.ISA_AVX512]


@pytest.fixture(params=ISAS, ids=["scalar", "avx2", "avx512"])
def isa(request):
    if xo.set_isa(request.param) != 0:
        pytest.skip("ISA level not available on this CPU")
    yield request.param
    xo.set_isa(xo.ISA_AUTO)


def ft(data, shape):
    return np.asarray(data, dtype=np.float32).reshape(shape)


# ---- tests/attention_numerics_tests.rs ---------------------------------------------------------

def test_attention_single_token_is_identity(isa):
    # attention_numerics_tests.rs:10-30
    H, Hkv, D = 2, 2, 4
    cache = xo.RingCache(1, Hkv, 32, D, False)
    q = ft(np.ones(H * D), (1, H, 1, D))
    k = ft(np.ones(Hkv * D), (1, Hkv, 1, D))
    v_data = np.arange(Hkv * D, dtype=np.float32)
    v = ft(v_data, (1, Hkv, 1, D))
    out = xo.fast_attention(q, k, v, 0, 0, cache, H, Hkv, D)
    assert out.shape == (1, H, 1, D)
    assert np.all(np.abs(out.ravel() - v_data) < 1e-4)


def test_attention_causal_mask_second_token_no_future(isa):
    # attention_numerics_tests.rs:33-70 -> [5, 10]
    cache = xo.RingCache(1, 1, 32, 2, False)
    xo.fast_attention(ft([1, 0], (1, 1, 1, 2)), ft([1, 0], (1, 1, 1, 2)), ft([10, 0], (1, 1, 1, 2)),
                      0, 0, cache, 1, 1, 2)
    out = xo.fast_attention(ft([1, 1], (1, 1, 1, 2)), ft([0, 1], (1, 1, 1, 2)),
                            ft([0, 20], (1, 1, 1, 2)), 0, 1, cache, 1, 1, 2)
    assert np.all(np.abs(out.ravel() - np.array([5.0, 10.0], dtype=np.float32)) < 1e-4)


def test_attention_output_finite(isa):
    # attention_numerics_tests.rs:73-99
    H, Hkv, D, S = 4, 2, 8, 6
    cache = xo.RingCache(1, Hkv, 64, D, False)
    q = ft([math.sin(np.float32(i) * np.float32(0.1)) for i in range(H * S * D)], (1, H, S, D))
    k = ft([math.cos(np.float32(i) * np.float32(0.07)) for i in range(Hkv * S * D)], (1, Hkv, S, D))
    v = ft([np.float32(i) * np.float32(0.03) - 1.0 for i in range(Hkv * S * D)], (1, Hkv, S, D))
    out = xo.fast_attention(q, k, v, 0, 0, cache, H, Hkv, D)
    assert np.all(np.isfinite(out))
    ref = xo.naive_attention_f64(q[0], k[0], v[0], 0, H, Hkv, D)
    assert np.max(np.abs(out[0] - ref)) < 1e-5


def test_cache_write_correctness(isa):
    # attention_numerics_tests.rs:102-116: reads the pub field k_buffers[0]
    cache = xo.RingCache(1, 1, 8, 2, False)
    xo.fast_attention(ft([1, 1], (1, 1, 1, 2)), ft([5, 6], (1, 1, 1, 2)), ft([0, 0], (1, 1, 1, 2)),
                      0, 0, cache, 1, 1, 2)
    kb = cache.k_buffer(0)
    assert kb[0] == 5.0 and kb[1] == 6.0


def test_shape_errors():
    # fast_attention.rs:86-92
    cache = xo.RingCache(1, 1, 8, 2, False)
    with pytest.raises(ValueError, match="Q shape must be 4D"):
        xo.fast_attention(np.zeros((1, 1, 2), np.float32), np.zeros((1, 1, 1, 2), np.float32),
                          np.zeros((1, 1, 1, 2), np.float32), 0, 0, cache, 1, 1, 2)
    with pytest.raises(ValueError, match="only supports batch size 1, got 2"):
        xo.fast_attention(np.zeros((2, 1, 1, 2), np.float32), np.zeros((2, 1, 1, 2), np.float32),
                          np.zeros((2, 1, 1, 2), np.float32), 0, 0, cache, 1, 1, 2)


# ---- tests/fast_attention_tests.rs -------------------------------------------------------------

def test_fast_attention_parity_single_token(isa):
    # fast_attention_tests.rs:94-188: Hq=4, Hkv=2, D=8; prefill S=4 then decode at pos 4, each
    # within 1e-5 of textbook attention (candle there, float64 numpy here).  The reference draws
    # unseeded U(-1,1) inputs; several seeds are used here.
    H, Hkv, D, cap = 4, 2, 8, 32
    for seed in range(8):
        rng = np.random.default_rng(seed)
        cache = xo.RingCache(1, Hkv, cap, D, False)
        qp = rng.uniform(-1, 1, (1, H, 4, D)).astype(np.float32)
        kp = rng.uniform(-1, 1, (1, Hkv, 4, D)).astype(np.float32)
        vp = rng.uniform(-1, 1, (1, Hkv, 4, D)).astype(np.float32)
        out = xo.fast_attention(qp, kp, vp, 0, 0, cache, H, Hkv, D)
        ref = xo.naive_attention_f64(qp[0], kp[0], vp[0], 0, H, Hkv, D)
        assert np.max(np.abs(out[0] - ref)) < 1e-5
        qt = rng.uniform(-1, 1, (1, H, 1, D)).astype(np.float32)
        kt = rng.uniform(-1, 1, (1, Hkv, 1, D)).astype(np.float32)
        vt = rng.uniform(-1, 1, (1, Hkv, 1, D)).astype(np.float32)
        out = xo.fast_attention(qt, kt, vt, 0, 4, cache, H, Hkv, D)
        k_all = np.concatenate([kp[0], kt[0]], axis=1)
        v_all = np.concatenate([vp[0], vt[0]], axis=1)
        ref = xo.naive_attention_f64(qt[0], k_all, v_all, 4, H, Hkv, D)
        assert np.max(np.abs(out[0] - ref)) < 1e-5


def test_ring_wrapping_correctness(isa):
    # fast_attention_tests.rs:191-241: cap 4, positions 0..3 written with ones, then position 4
    # with zeros lands in slot 0; layout h_kv*cap*D + t*D + d.
    H, Hkv, cap, D = 2, 1, 4, 4
    cache = xo.RingCache(1, Hkv, cap, D, False)
    ones_q, ones_kv = np.ones((1, H, 1, D), np.float32), np.ones((1, Hkv, 1, D), np.float32)
    for pos in range(4):
        xo.fast_attention(ones_q, ones_kv, ones_kv, 0, pos, cache, H, Hkv, D)
    assert np.array_equal(cache.k_buffer(0), np.ones(Hkv * cap * D, np.float32))
    out = xo.fast_attention(np.zeros_like(ones_q), np.zeros_like(ones_kv), np.zeros_like(ones_kv),
                            0, 4, cache, H, Hkv, D)
    kb = cache.k_buffer(0)
    assert np.all(kb[0:D] == 0.0) and np.all(kb[D:2 * D] == 1.0)
    # logical positions 0..4 fold onto slots 0,1,2,3,0: slot 0 (now zero) is counted twice, all
    # scores are 0 (q = 0), so every output element is (0+1+1+1+0)/5.
    assert np.allclose(out, 0.6, atol=1e-6)


# ---- tests/tensor_ops_tests.rs:226-315 ---------------------------------------------------------

def test_softmax_matches_naive(isa):
    # tensor_ops_tests.rs:226-250
    for n in [1, 2, 3, 7, 8, 9, 15, 16, 17, 31, 32, 33, 64, 100, 128, 256]:
        scores = np.array([np.float32(i) - np.float32(n) / np.float32(2.0) for i in range(n)],
                          dtype=np.float32)
        got = xo.softmax_inplace(scores)
        m = scores.max()
        e = np.zeros(n, np.float32)
        s = np.float32(0)
        for i in range(n):
            e[i] = np.float32(math.exp(np.float64(np.float32(scores[i] - m))))
            s = np.float32(s + e[i])
        ref = e * (np.float32(1.0) / s)
        assert np.max(np.abs(got - ref)) < 1e-5, n
        assert abs(float(got.sum()) - 1.0) < 1e-5


def test_weighted_sum_matches_naive(isa):
    # tensor_ops_tests.rs:253-283
    for D in [4, 7, 8, 9, 15, 16, 17, 32, 64, 100, 128]:
        for L in [1, 2, 3, 5, 10, 20]:
            scores = np.array([(np.float32(i) + np.float32(1.0)) / np.float32(L) for i in range(L)],
                              dtype=np.float32)
            v_buf = np.sin(np.arange(2 * 64 * D, dtype=np.float32) * np.float32(0.01)).astype(np.float32)
            got = xo.weighted_sum(scores, v_buf, 0, 64, D, L)
            ref = np.zeros(D, np.float32)
            for i in range(D):
                s = np.float32(0)
                for t in range(L):
                    s = np.float32(s + np.float32(scores[t] * v_buf[(t % 64) * D + i]))
                ref[i] = s
            assert np.max(np.abs(got - ref)) < 1e-4, (D, L)


def test_batched_dot_product_matches_naive(isa):
    # tensor_ops_tests.rs:286-315
    for D in [4, 7, 8, 9, 15, 16, 17, 31, 32, 33, 64, 100]:
        for L in [1, 2, 3, 5, 10, 16, 20]:
            q = (np.arange(D, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
            k_buf = np.cos(np.arange(2 * 64 * D, dtype=np.float32) * np.float32(0.01)).astype(np.float32)
            # the reference passes out of len max(L,16) and one call for all L keys
            got = np.zeros(max(L, 16), np.float32)
            xo.lib().xo_batched_dot_product(xo._p(q), xo._p(k_buf), 0, 64, D, 0, L, xo._p(got))
            for t in range(L):
                s = np.float32(0)
                for i in range(D):
                    s = np.float32(s + np.float32(q[i] * k_buf[(t % 64) * D + i]))
                assert abs(got[t] - s) < 1e-4, (D, L, t)


def test_fast_tensor_rope_rotate_half():
    # tensor_ops_tests.rs:126-164: [1,2,3,4] tensor, explicit cos/sin tables, rotate-half pairs
    x = ft([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12,
            -1, -2, -3, -4, -5, -6, -7, -8, -9, -10, -11, -12], (1, 2, 3, 4))
    cos = ft([0.9, 0.8, 0.7, 0.6, 0.5, 0.4], (3, 2))
    sin = ft([0.1, 0.2, 0.3, 0.4, 0.5, 0.6], (3, 2))
    got = xo.tensor_rope(x, cos, sin, 0)
    ref = np.empty_like(x)
    for h in range(2):
        for t in range(3):
            x1, x2 = x[0, h, t, :2], x[0, h, t, 2:]
            ref[0, h, t, :2] = x1 * cos[t] - x2 * sin[t]
            ref[0, h, t, 2:] = x1 * sin[t] + x2 * cos[t]
    assert np.array_equal(got, ref)


def test_fast_tensor_transposes():
    # tensor_ops_tests.rs:167-193
    x = np.arange(24, dtype=np.float32).reshape(1, 3, 8)
    heads = xo.transpose_seq_to_heads(x, 2, 4)
    assert np.array_equal(heads, x.reshape(1, 3, 2, 4).transpose(0, 2, 1, 3))
    assert np.array_equal(xo.transpose_heads_to_seq(heads), x)


# ---- tests/tensor_layout_tests.rs:18-38 --------------------------------------------------------

def test_transpose_known_layout():
    t = np.arange(8, dtype=np.float32).reshape(1, 2, 4)
    h = xo.transpose_seq_to_heads(t, 2, 2)
    assert h.shape == (1, 2, 2, 2)
    assert h.ravel().tolist() == [0.0, 1.0, 4.0, 5.0, 2.0, 3.0, 6.0, 7.0]
    data = np.arange(24, dtype=np.float32).reshape(1, 3, 8)
    back = xo.transpose_heads_to_seq(xo.transpose_seq_to_heads(data, 2, 4))
    assert back.shape == (1, 3, 8) and np.array_equal(back, data)


# ---- tests/tensor_rope_tests.rs ----------------------------------------------------------------

@pytest.mark.parametrize("x,cos,sin,expected", [
    ([1, 2, 3, 4], [1, 1], [0, 0], [1, 2, 3, 4]),            # :10-20 identity
    ([3, 5, 7, 11], [0, 0], [1, 1], [-7, -11, 3, 5]),        # :23-37 90 degrees
    ([1, 2, 3, 4], [-1, -1], [0, 0], [-1, -2, -3, -4]),      # :40-50 180 degrees
])
def test_rope_known_answers(x, cos, sin, expected):
    out = xo.tensor_rope(ft(x, (1, 1, 1, 4)), ft(cos, (1, 2)), ft(sin, (1, 2)), 0)
    assert np.all(np.abs(out.ravel() - np.array(expected, np.float32)) < 1e-5)


def test_rope_preserves_norm():
    # tensor_rope_tests.rs:53-69
    x = [3.0, 4.0, 1.0, 2.0]
    a = np.float32(np.pi) / np.float32(6.0)
    c, s = np.float32(np.cos(a)), np.float32(np.sin(a))
    out = xo.tensor_rope(ft(x, (1, 1, 1, 4)), ft([c, c], (1, 2)), ft([s, s], (1, 2)), 0).ravel()
    assert abs(math.hypot(x[0], x[2]) - math.hypot(out[0], out[2])) < 1e-5
    assert abs(math.hypot(x[1], x[3]) - math.hypot(out[1], out[3])) < 1e-5


def test_rope_invalid_shape():
    # tensor_rope_tests.rs:72-77
    with pytest.raises(ValueError):
        xo.tensor_rope(ft([1, 2, 3], (3,)), ft([1, 1], (1, 2)), ft([0, 0], (1, 2)), 0)


def test_rope_multi_head():
    # tensor_rope_tests.rs:80-96
    out = xo.tensor_rope(ft([1, 0, 0, 1, 0, 1, 1, 0], (1, 2, 1, 4)), ft([0, 0], (1, 2)),
                         ft([1, 1], (1, 2)), 0)
    assert np.all(np.abs(out.ravel() - np.array([0, -1, 1, 0, -1, 0, 0, 1], np.float32)) < 1e-5)


# ---- RoPE tables (src/models/llama/mod.rs:210-265) ---------------------------------------------

@pytest.mark.parametrize("theta,D", [(500000.0, 128), (10000.0, 100)])
def test_rope_tables_against_f64(theta, D):
    cos, sin = xo.rope_tables(theta, D, 256)
    j = np.arange(0, D, 2, dtype=np.float64)
    inv = 1.0 / np.float64(theta) ** (j / D)
    ang = np.arange(256, dtype=np.float64)[:, None] * inv[None, :]
    # f32 angle rounding grows with position; 256 * 2^-24 bounds it
    assert np.max(np.abs(cos - np.cos(ang))) < 5e-5
    assert np.max(np.abs(sin - np.sin(ang))) < 5e-5
    assert np.all(cos[0] == 1.0) and np.all(sin[0] == 0.0)


def test_rope_tables_llama3_scaling():
    # mod.rs:226-249 with the Llama-3.1 constants: high frequencies untouched, low ones / factor
    plain_c, _ = xo.rope_tables(500000.0, 128, 4)
    sc_c, sc_s = xo.rope_tables(500000.0, 128, 4, scaling=(8.0, 1.0, 4.0, 8192))
    assert np.array_equal(plain_c[:, :8], sc_c[:, :8])
    inv_last = np.float32(1.0) / np.float32(500000.0) ** (np.float32(126) / np.float32(128))
    assert abs(sc_s[1, 63] - np.sin(np.float64(inv_last) / 8.0)) < 1e-9


# ---- ISA bodies agree with one another and with f64 at the benchmark shapes --------------------

@pytest.mark.parametrize("Hq,Hkv,D,L", [(20, 5, 128, 1024), (32, 32, 100, 300)])
def test_decode_shapes_vs_f64(Hq, Hkv, D, L):
    rng = np.random.default_rng(7)
    k_all = rng.standard_normal((Hkv, L, D)).astype(np.float32)
    v_all = rng.standard_normal((Hkv, L, D)).astype(np.float32)
    q = rng.standard_normal((1, Hq, 1, D)).astype(np.float32)
    ref = xo.naive_attention_f64(q[0], k_all, v_all, L - 1, Hq, Hkv, D)
    outs = []
    for isa in ISAS:
        if xo.set_isa(isa) != 0:
            continue
        cache = xo.RingCache(1, Hkv, L, D)
        cache.append(0, 0, k_all[:, :L - 1], v_all[:, :L - 1])
        out = xo.fast_attention(q, k_all[None, :, L - 1:], v_all[None, :, L - 1:], 0, L - 1, cache,
                                Hq, Hkv, D)
        outs.append(out)
        rel = np.linalg.norm(out[0] - ref) / np.linalg.norm(ref)
        assert rel < 2e-6, (isa, rel)
    xo.set_isa(xo.ISA_AUTO)
    assert len(outs) >= 1


def test_streams_entry_matches_single_calls():
    rng = np.random.default_rng(3)
    Hq, Hkv, D = 8, 2, 16
    lens = [5, 17, 64, 1]
    mk = lambda: [xo.RingCache(2, Hkv, 128, D) for _ in lens]
    ca, cb = mk(), mk()
    qs, ks, vs = [], [], []
    for i, L in enumerate(lens):
        kk = rng.standard_normal((Hkv, L - 1, D)).astype(np.float32) if L > 1 else np.zeros((Hkv, 0, D), np.float32)
        for c in (ca[i], cb[i]):
            if L > 1:
                c.append(1, 0, kk, kk * 0.5)
        qs.append(rng.standard_normal((1, Hq, 1, D)).astype(np.float32))
        ks.append(rng.standard_normal((1, Hkv, 1, D)).astype(np.float32))
        vs.append(rng.standard_normal((1, Hkv, 1, D)).astype(np.float32))
    outs = xo.fast_attention_streams(qs, ks, vs, 1, [L - 1 for L in lens], ca, Hq, Hkv, D)
    for i, L in enumerate(lens):
        single = xo.fast_attention(qs[i], ks[i], vs[i], 1, L - 1, cb[i], Hq, Hkv, D)
        assert np.array_equal(outs[i], single)
