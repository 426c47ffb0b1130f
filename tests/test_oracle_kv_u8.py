"""The oracle's restatement of CpuRingCache::quantize_to_u8 (fast_attention.rs:62-71).

The reference holds no test or golden vector for its u8 shadow, so this restatement is NOT pinned
against reference output ("parity unpinned"); what is checked here is the C code against a
line-by-line numpy/Python transcription of the reference's expressions and against hand-worked
cases.
"""
import numpy as np

import oracle as xo


def quantize_row_py(x):
    """fast_attention.rs:63-70, one expression at a time, in f32."""
    x = np.asarray(x, np.float32)
    max_abs = np.float32(0.0)
    for b in x:                                       # fold(0.0, |a, b| a.max(b.abs()))
        ab = np.abs(b)
        if not np.isnan(ab) and ab > max_abs:
            max_abs = ab
    scale = np.float32(max_abs / np.float32(127.0)) if max_abs > 0 else np.float32(1.0)
    out = np.zeros(len(x), np.uint8)
    with np.errstate(all="ignore"):
        inv = np.float32(np.float32(1.0) / scale)
        for i, b in enumerate(x):
            t = np.float32(np.float32(b * inv) + np.float32(128.0))
            if np.isnan(t):
                out[i] = 0
                continue
            r = np.float32(np.sign(t) * np.floor(np.abs(np.float64(t)) + 0.5))   # round half away
            out[i] = np.uint8(min(max(r, 0.0), 255.0))
    return out, scale


def test_hand_cases():
    q, s = xo.quantize_to_u8(np.array([[1.0, -1.0, 0.5, 0.0]], np.float32))
    assert q.tolist() == [[255, 1, 192, 128]]          # 0.5 * 127 + 128 = 191.5 rounds away to 192
    assert s[0] == np.float32(1.0) / np.float32(127.0)
    q, s = xo.quantize_to_u8(np.zeros((1, 8), np.float32))
    assert (q == 128).all() and s[0] == 1.0           # all-zero row: scale 1.0
    q, s = xo.quantize_to_u8(np.array([[-2.0, 2.0]], np.float32))
    assert q.tolist() == [[1, 255]]


def test_against_python_transcription():
    rng = np.random.default_rng(7)
    rows = [rng.standard_normal(n).astype(np.float32) * sc
            for n in (1, 2, 15, 16, 64, 100, 128) for sc in (1e-30, 1e-3, 1.0, 77.0, 1e30)]
    rows.append(np.array([np.nan, 1.0, -3.0], np.float32))
    rows.append(np.array([np.inf, 1.0, -1.0, 0.0], np.float32))
    rows.append(np.array([1e-41, -1e-41, 0.0], np.float32))          # denormals
    rows.append((np.arange(255) - 127).astype(np.float32))           # every byte value once
    for x in rows:
        q, s = xo.quantize_to_u8(x[None])
        qp, sp = quantize_row_py(x)
        assert np.array_equal(q[0], qp), x
        assert s[0].view(np.uint32) == np.float32(sp).view(np.uint32)


def test_round_trip_error_bound_and_shapes():
    rng = np.random.default_rng(9)
    x = rng.standard_normal((3, 5, 7, 64)).astype(np.float32)
    q, s = xo.quantize_to_u8(x)
    assert q.shape == x.shape and s.shape == x.shape[:-1]
    back = xo.dequantize_u8(q, s)
    assert np.array_equal(back, (q.astype(np.float32) - 128.0) * s[..., None])
    assert np.all(np.abs(back - x) <= 0.5 * s[..., None] * (1 + 1e-6))
    assert np.array_equal(xo.u8_round_trip(x), back)
