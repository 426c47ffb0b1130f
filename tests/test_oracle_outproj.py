"""Pins the CPU oracle of the attention output block (sub-norm + ternary o_proj) against the
reference's own known-answer tests.  Every case regenerates the vectors of one reference test
from the formula or the literals that test holds; the file and line are cited per case.

The reference's tests for these routines predate two signature changes of its own code
(`quantize_f32_to_i8` now fills a caller buffer and returns the inverse scale; `TernaryLinear::new`
gained `provided_scale`); the expected VALUES are what is pinned here.
"""
import numpy as np
import pytest

import oracle as xo

EPS = 1e-5


def tern(n):
    return np.array([(-1.0, 0.0, 1.0)[i % 3] for i in range(n)], np.float32)


# ---- tests/bit1_58_tests.rs ---------------------------------------------------------------------

def test_ternary_pack_unpack_roundtrip():  # bit1_58_tests.rs:10-21
    w = np.array([1, 0, -1, 1, 0, -1, -1, 0, 1, 1], np.float32)
    for pt in (xo.PACK4, xo.PACK5):
        assert np.array_equal(xo.unpack_ternary(xo.pack_ternary(w, 1.0, pt), w.size, pt), w)


def test_absmax_quantization():  # bit1_58_tests.rs:23-35
    q, inv = xo.quantize_f32_to_i8([0.0, -2.5, 5.0, 1.25])
    assert abs(inv - 5.0 / 127.0) < 1e-5
    assert q.tolist() == [0, -64, 127, 32]
    q, inv = xo.quantize_f32_to_i8([0.0, 0.0, 0.0])
    assert q.tolist() == [0, 0, 0] and inv == 1.0


def test_ternary_simd_parity():  # bit1_58_tests.rs:37-66
    for n in (4, 8, 12, 16, 20, 32, 36, 64, 68, 128, 132):
        acts = np.array([(i % 255) - 127 for i in range(n)], np.int32).astype(np.int8)
        w = tern(n)
        want = int(np.dot(acts.astype(np.int64), w.astype(np.int64)))
        assert xo.ternary_dot(acts, xo.pack_ternary(w, 1.0, xo.PACK4), n, xo.PACK4) == want
        assert xo.ternary_dot(acts, xo.pack_ternary(w, 1.0, xo.PACK5), n, xo.PACK5) == want


def test_ternary_linear_layer():  # bit1_58_tests.rs:68-92
    # The expected literals belong to the global abs-mean weight scale 5/8 that the reference
    # computed itself when that test was written; today the caller passes it as provided_scale.
    w = [1, 0, -1, 1, 0, -1, 1, 0]
    x = np.array([[0.5, 1.0, -0.5, 2.0]], np.float32)
    o4 = xo.TernaryLinear(4, 2, w, xo.PACK4, provided_scale=0.625).forward(x)
    o5 = xo.TernaryLinear(4, 2, w, xo.PACK5, provided_scale=0.625).forward(x)
    assert np.array_equal(o4, o5)
    assert abs(o4[0, 0] - 1.879921) < 1e-4 and abs(o4[0, 1] - (-0.944882)) < 1e-4
    # without a scale, exactly-ternary weights keep scale 1 (bit1_58/layers.rs:100-109)
    o1 = xo.TernaryLinear(4, 2, w, xo.PACK4).forward(x)
    assert np.allclose(o1 * 0.625, o4, rtol=1e-6)


def test_pack_unpack_cycle():  # bit1_58_tests.rs:94-101
    w = np.array([-1, 0, 1, -1, 0, 1, 0, -1], np.float32)
    assert np.array_equal(xo.unpack_ternary(xo.pack_ternary(w, 1.0), 8), w)


# ---- tests/quantization_158bit_tests.rs ---------------------------------------------------------

def test_pack4_cases():  # quantization_158bit_tests.rs:15-52
    w = np.array([-1, 0, 1, -1, 1, 1, 0, 0, -1, -1], np.float32)
    assert np.array_equal(xo.unpack_ternary(xo.pack_ternary(w, 1.0), w.size), w)
    for n in (1, 2, 3, 5, 6, 7, 9, 11, 13, 15, 17):
        assert np.array_equal(xo.unpack_ternary(xo.pack_ternary(tern(n), 1.0), n), tern(n))
    for w in (np.zeros(20, np.float32), -np.ones(12, np.float32)):
        assert np.array_equal(xo.unpack_ternary(xo.pack_ternary(w, 1.0), w.size), w)


def test_pack5_cases():  # quantization_158bit_tests.rs:57-77
    w = np.array([-1, 0, 1, -1, 1, 0, 0, -1, 1, -1, 1], np.float32)
    assert np.array_equal(xo.unpack_ternary(xo.pack_ternary(w, 1.0, xo.PACK5), w.size, xo.PACK5), w)
    for n in (1, 2, 3, 4, 6, 7, 8, 9, 11, 14, 16, 21):
        assert np.array_equal(xo.unpack_ternary(xo.pack_ternary(tern(n), 1.0, xo.PACK5), n, xo.PACK5),
                              tern(n))


def test_packed_bytes_literal():
    # layout of one byte: pack4 puts weight i in bits 2i..2i+1 with codes -1->0, 0->1, +1->2;
    # pack5 is the base-3 number with weight i the digit of 3^i (quantization.rs:7-72)
    assert xo.pack_ternary([-1, 0, 1, 1], 1.0, xo.PACK4).tolist() == [0 | 1 << 2 | 2 << 4 | 2 << 6]
    assert xo.pack_ternary([-1, 0, 1, 1, 0], 1.0, xo.PACK5).tolist() == [0 + 1 * 3 + 2 * 9 + 2 * 27 + 1 * 81]
    # scaling before rounding: 0.3/0.5 = 0.6 -> 1; 0.2/0.5 = 0.4 -> 0; -2/0.5 clamps to -1
    assert xo.unpack_ternary(xo.pack_ternary([0.3, 0.2, -2.0], 0.5), 3).tolist() == [1.0, 0.0, -1.0]
    # a non-positive scale maps everything to 0 (quantization.rs:12)
    assert xo.unpack_ternary(xo.pack_ternary([1.0, -1.0], 0.0), 2).tolist() == [0.0, 0.0]


def test_quantize_i8_cases():  # quantization_158bit_tests.rs:81-121
    q, inv = xo.quantize_f32_to_i8(np.zeros(16, np.float32))
    assert inv == 1.0 and not q.any()
    q, inv = xo.quantize_f32_to_i8([0.0, -3.0, 3.0, 1.5])
    assert abs(inv - 3.0 / 127.0) < 1e-6 and q[2] == 127 and q[1] == -127
    acts = ((np.arange(256, dtype=np.float32) - 128.0) * np.float32(0.01)).astype(np.float32)
    q, inv = xo.quantize_f32_to_i8(acts)
    assert np.all(np.abs(acts - q.astype(np.float32) * np.float32(inv)) <= inv + 1e-6)


def test_quantize_rounding_follows_the_selected_body():
    # whole 16-element chunks of the AVX-512 body convert with round-to-nearest-even, its tail and
    # the scalar body with f32::round (quantization.rs:126-139, 181-184): 0.5 -> 0 vs 1
    acts = np.zeros(20, np.float32)
    acts[0] = 127.0     # scale = 1
    acts[1] = 0.5       # tie inside the first whole chunk
    acts[2] = 2.5
    acts[17] = 0.5      # tie inside the tail
    try:
        assert xo.set_quant_body(0) == 0
        q, _ = xo.quantize_f32_to_i8(acts)
        assert (q[1], q[2], q[17]) == (1, 3, 1)
        assert xo.set_quant_body(1) == 0
        q, _ = xo.quantize_f32_to_i8(acts)
        assert (q[1], q[2], q[17]) == (0, 2, 1)
        xo.set_quant_body(-1)
        assert xo.set_isa(xo.ISA_SCALAR) == 0          # the ISA level selects the body too
        q, _ = xo.quantize_f32_to_i8(acts)
        assert (q[1], q[2], q[17]) == (1, 3, 1)
    finally:
        xo.set_quant_body(-1)
        xo.set_isa(xo.ISA_AUTO)


# ---- tests/tensor_rmsnorm_tests.rs, tests/tensor_ops_tests.rs -----------------------------------

def test_rmsnorm_known_answers():  # tensor_rmsnorm_tests.rs:8-84
    out = xo.tensor_rmsnorm(np.full((1, 4), 2.0, np.float32), np.ones(4, np.float32), 1e-6)
    assert np.all(np.abs(out - 1.0) < EPS)
    out = xo.tensor_rmsnorm([[3.0, 4.0]], [1.0, 1.0], 1e-6)
    rms = np.sqrt(np.float32(12.5))
    assert np.all(np.abs(out - np.array([[3.0 / rms, 4.0 / rms]])) < EPS)
    out = xo.tensor_rmsnorm(np.zeros((1, 4), np.float32), [1.0, 2.0, 3.0, 4.0], 1e-6)
    assert np.all(np.abs(out) < EPS)
    out = xo.tensor_rmsnorm([[1.0, 0.0, 3.0], [0.0, 0.0, 4.0]], np.ones(3, np.float32), 1e-6)
    r0, r1 = np.sqrt(10.0 / 3.0), np.sqrt(16.0 / 3.0)
    assert np.all(np.abs(out - np.array([[1 / r0, 0, 3 / r0], [0, 0, 4 / r1]])) < EPS)
    out = xo.tensor_rmsnorm([[1e6, -1e6, 1e6, -1e6]], np.ones(4, np.float32), 1e-6)
    assert np.all(np.isfinite(out))
    o1 = xo.tensor_rmsnorm([[3.0, 4.0]], [1.0, 1.0], 1e-6)
    o2 = xo.tensor_rmsnorm([[3.0, 4.0]], [2.0, 2.0], 1e-6)
    assert np.all(np.abs(o2 - 2.0 * o1) < EPS)
    with pytest.raises(ValueError):
        xo.tensor_rmsnorm([[3.0, 4.0]], [1.0], 1e-6)   # tensor.rs:246-252


def test_fast_tensor_rmsnorm_against_f64():  # tensor_ops_tests.rs:70-110 (candle there, f64 here)
    data = np.array([1.0, 2.0, 3.0, 4.0, -1.0, 0.5, 1.5, -2.0, 0.0, 0.0, 0.0, 1.0,
                     2.0, -2.0, 2.0, -2.0, 1.1, 2.2, 3.3, 4.4, -0.5, -0.5, -0.5, -0.5],
                    np.float32).reshape(2, 3, 4)
    w = np.array([0.5, 1.0, 1.5, 2.0], np.float32)
    got = xo.tensor_rmsnorm(data, w, 1e-6)
    d = data.astype(np.float64)
    want = d / np.sqrt((d * d).mean(-1, keepdims=True) + 1e-6) * w
    assert np.max(np.abs(got - want)) < 1e-5


def test_rmsnorm_matches_naive():  # tensor_ops_tests.rs:318-341
    for n in (1, 3, 7, 8, 9, 15, 16, 17, 31, 32, 33, 64, 100, 128, 256, 3200):
        x = (np.arange(n, dtype=np.float32) * np.float32(0.1) - np.float32(n) / np.float32(2.0)).astype(np.float32)
        w = (np.float32(1.0) + np.arange(n, dtype=np.float32) * np.float32(0.01)).astype(np.float32)
        got = xo.rms_norm(x, w, 1e-6)
        s = np.float32(0.0)
        for v in x:
            s = np.float32(s + np.float32(v * v))
        inv = np.float32(1.0) / np.sqrt(np.float32(s / np.float32(n) + np.float32(1e-6)))
        want = (x * inv).astype(np.float32) * w
        assert np.array_equal(got, want.astype(np.float32)), n   # same order of operations: same bits


# ---- the block as the model runs it (models/llama/attention.rs:103-108) --------------------------

@pytest.mark.parametrize("pack", [xo.PACK4, xo.PACK5])
def test_out_block_equals_its_parts(pack):
    rng = np.random.default_rng(11)
    Hq, S, D, out_dim = 4, 5, 8, 12
    y = rng.standard_normal((1, Hq, S, D)).astype(np.float32)
    nw = (1.0 + 0.1 * rng.standard_normal(Hq * D)).astype(np.float32)
    lin = xo.TernaryLinear(Hq * D, out_dim, rng.standard_normal((out_dim, Hq * D)).astype(np.float32), pack)
    got = xo.attention_out_block(y, nw, 1e-5, lin)
    seq = xo.transpose_heads_to_seq(y)
    want = lin.forward(xo.tensor_rmsnorm(seq, nw, 1e-5))
    assert np.array_equal(got, want)
    # independent arithmetic: dequantised weights times quantised activations in float64
    wq = np.stack([xo.unpack_ternary(lin.packed[o * lin.row_bytes:(o + 1) * lin.row_bytes], Hq * D, pack)
                   for o in range(out_dim)]).astype(np.float64)
    normed = xo.tensor_rmsnorm(seq, nw, 1e-5)[0]
    for t in range(S):
        q, inv = xo.quantize_f32_to_i8(normed[t])
        ref = (wq @ q.astype(np.float64)) * inv * lin.w_scales
        assert np.allclose(got[0, t], ref, rtol=1e-6, atol=1e-7)
    # per-row scale is the mean absolute weight (bit1_58/layers.rs:128-140)
    assert lin.w_scales.shape == (out_dim,) and np.all(lin.w_scales > 0)
    # no sub-norm: projection of the transposed tensor
    assert np.array_equal(xo.attention_out_block(y, None, 1e-5, lin), lin.forward(seq))


# ---- XorSparse rows (src/bit1_58/sparse.rs) -----------------------------------------------------

def test_sparse_row_layout_literal():
    # sparse.rs:9-17: u32 num_blocks, then per 64-element block the u64 mask of the non-zero positions
    # and ceil(nnz/8) bytes of sign bits in scan order (bit set = -1), all little-endian
    vals = np.zeros(70, np.int8)
    vals[[0, 3, 63]] = [1, -1, -1]       # block 0: mask bits 0,3,63; signs (scan order) 0,1,1 -> 0b110
    vals[[64, 69]] = [-1, 1]             # block 1: mask bits 0,5; signs 1,0 -> 0b01
    row = xo.sparse_encode_row(vals, 70)
    want = [2, 0, 0, 0] + list((1 | 1 << 3 | 1 << 63).to_bytes(8, "little")) + [0b110] + \
        list((1 | 1 << 5).to_bytes(8, "little")) + [0b01]
    assert row.tolist() == want
    back, used = xo.sparse_decode_row(row, 70)
    assert used == row.size and np.array_equal(back, vals)


def test_sparse_is_lossless_and_dots_match_dense():
    rng = np.random.default_rng(17)
    for n in (1, 5, 63, 64, 65, 128, 200, 2560):
        vals = rng.integers(-1, 2, n).astype(np.int8)
        row = xo.sparse_encode_row(vals, n)
        back, used = xo.sparse_decode_row(row, n)
        assert used == row.size and np.array_equal(back, vals)
        acts = rng.integers(-127, 128, n).astype(np.int8)
        want = int(np.dot(acts.astype(np.int64), vals.astype(np.int64)))
        assert xo.ternary_dot_sparse(acts, row, n) == want
        assert xo.ternary_dot(acts, xo.pack_ternary(vals.astype(np.float32), 1.0), n) == want
    # all-zero and all-nonzero rows: 12 and 20 bytes per block
    assert xo.sparse_encode_row(np.zeros(64, np.int8), 64).size == 4 + 8
    assert xo.sparse_encode_row(np.ones(64, np.int8), 64).size == 4 + 8 + 8


def test_sparse_linear_equals_dense_linear():
    # TernaryLinear::new_sparse ternarises like ::new (layers.rs:151-181): same scales, same outputs
    rng = np.random.default_rng(18)
    for in_dim, out_dim, scale in ((48, 7, None), (130, 5, 0.4), (64, 3, None)):
        w = rng.standard_normal((out_dim, in_dim)).astype(np.float32)
        sp, de = xo.TernaryLinear(in_dim, out_dim, w, xo.SPARSE, scale), xo.TernaryLinear(in_dim, out_dim, w, xo.PACK4, scale)
        assert np.array_equal(sp.w_scales, de.w_scales)
        x = rng.standard_normal((4, in_dim)).astype(np.float32)
        assert np.array_equal(sp.forward(x), de.forward(x))
