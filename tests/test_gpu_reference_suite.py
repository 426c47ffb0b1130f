"""The reference's own tests of this path, run against the GPU library through its C ABI.

Same inputs, same expected values and tolerances as tests/attention_numerics_tests.rs and
tests/fast_attention_tests.rs of the reference; ``DeviceKvCache`` stands where ``CpuRingCache``
stood and ``fast_attention`` keeps its signature.
"""
import math

import numpy as np
import pytest

import oracle as xo
import xor_net_b200 as xn
from xor_net_b200 import DeviceKvCache, FastTensor, fast_attention

pytestmark = pytest.mark.gpu
EPS = 1e-4


def test_attention_single_token_is_identity():
    # attention_numerics_tests.rs:10-30
    num_heads, num_kv_heads, head_dim = 2, 2, 4
    cache = DeviceKvCache.new(1, num_kv_heads, 32, head_dim, False)
    q = FastTensor.new([1.0] * (num_heads * head_dim), [1, num_heads, 1, head_dim])
    k = FastTensor.new([1.0] * (num_kv_heads * head_dim), [1, num_kv_heads, 1, head_dim])
    v_data = [float(i) for i in range(num_kv_heads * head_dim)]
    v = FastTensor.new(v_data, [1, num_kv_heads, 1, head_dim])
    out = fast_attention(q, k, v, 0, 0, cache, num_heads, num_kv_heads, head_dim)
    assert out.shape == [1, num_heads, 1, head_dim]
    for a, e in zip(out.data, v_data):
        assert abs(a - e) < EPS


def test_attention_causal_mask_second_token_no_future():
    # attention_numerics_tests.rs:33-70
    cache = DeviceKvCache.new(1, 1, 32, 2, False)
    fast_attention(FastTensor.new([1.0, 0.0], [1, 1, 1, 2]), FastTensor.new([1.0, 0.0], [1, 1, 1, 2]),
                   FastTensor.new([10.0, 0.0], [1, 1, 1, 2]), 0, 0, cache, 1, 1, 2)
    out = fast_attention(FastTensor.new([1.0, 1.0], [1, 1, 1, 2]), FastTensor.new([0.0, 1.0], [1, 1, 1, 2]),
                         FastTensor.new([0.0, 20.0], [1, 1, 1, 2]), 0, 1, cache, 1, 1, 2)
    for a, e in zip(out.data, [5.0, 10.0]):
        assert abs(a - e) < EPS


def test_attention_output_finite():
    # attention_numerics_tests.rs:73-99
    H, Hkv, D, S = 4, 2, 8, 6
    cache = DeviceKvCache.new(1, Hkv, 64, D, False)
    q = FastTensor.new([math.sin(np.float32(i) * np.float32(0.1)) for i in range(H * S * D)], [1, H, S, D])
    k = FastTensor.new([math.cos(np.float32(i) * np.float32(0.07)) for i in range(Hkv * S * D)], [1, Hkv, S, D])
    v = FastTensor.new([np.float32(i) * np.float32(0.03) - 1.0 for i in range(Hkv * S * D)], [1, Hkv, S, D])
    out = fast_attention(q, k, v, 0, 0, cache, H, Hkv, D)
    assert np.all(np.isfinite(out.data))
    ref = xo.fast_attention(q.array(), k.array(), v.array(), 0, 0, xo.RingCache(1, Hkv, 64, D), H, Hkv, D)
    assert np.max(np.abs(out.array() - ref)) < 1e-5


def test_cache_write_correctness():
    # attention_numerics_tests.rs:102-116 reads the pub field k_buffers[0]
    cache = DeviceKvCache.new(1, 1, 8, 2, False)
    fast_attention(FastTensor.new([1.0, 1.0], [1, 1, 1, 2]), FastTensor.new([5.0, 6.0], [1, 1, 1, 2]),
                   FastTensor.new([0.0, 0.0], [1, 1, 1, 2]), 0, 0, cache, 1, 1, 2)
    assert cache.k_buffers[0][0] == 5.0
    assert cache.k_buffers[0][1] == 6.0


def test_shape_errors_match_reference_messages():
    # fast_attention.rs:86-92
    cache = DeviceKvCache.new(1, 1, 8, 2, False)
    z = FastTensor.new([0.0, 0.0], [1, 1, 1, 2])
    with pytest.raises(ValueError, match="fast_attention: Q shape must be 4D"):
        fast_attention(FastTensor.new([0.0, 0.0], [1, 1, 2]), z, z, 0, 0, cache, 1, 1, 2)
    with pytest.raises(ValueError, match="only supports batch size 1, got 2"):
        fast_attention(FastTensor.new([0.0] * 4, [2, 1, 1, 2]), z, z, 0, 0, cache, 1, 1, 2)


def test_fast_attention_parity_single_token():
    # fast_attention_tests.rs:94-188: prefill of 4 then one decode step, each within 1e-5 of
    # textbook attention (float64 numpy in place of candle); U(-1,1) inputs.
    H, Hkv, D = 4, 2, 8
    for seed in range(4):
        rng = np.random.default_rng(seed)
        cache = DeviceKvCache.new(1, Hkv, 32, D, False)
        qp, kp, vp = (rng.uniform(-1, 1, (1, h, 4, D)).astype(np.float32) for h in (H, Hkv, Hkv))
        out = fast_attention(FastTensor.new(qp, qp.shape), FastTensor.new(kp, kp.shape),
                             FastTensor.new(vp, vp.shape), 0, 0, cache, H, Hkv, D)
        ref = xo.naive_attention_f64(qp[0], kp[0], vp[0], 0, H, Hkv, D)
        assert np.max(np.abs(out.array()[0] - ref)) < 1e-5
        qt, kt, vt = (rng.uniform(-1, 1, (1, h, 1, D)).astype(np.float32) for h in (H, Hkv, Hkv))
        out = fast_attention(FastTensor.new(qt, qt.shape), FastTensor.new(kt, kt.shape),
                             FastTensor.new(vt, vt.shape), 0, 4, cache, H, Hkv, D)
        ref = xo.naive_attention_f64(qt[0], np.concatenate([kp[0], kt[0]], 1),
                                     np.concatenate([vp[0], vt[0]], 1), 4, H, Hkv, D)
        assert np.max(np.abs(out.array()[0] - ref)) < 1e-5
        cache.close()


def test_ring_wrapping_correctness():
    # fast_attention_tests.rs:191-241
    H, Hkv, cap, D = 2, 1, 4, 4
    cache = DeviceKvCache.new(1, Hkv, cap, D, False)
    ones_q = FastTensor.new(np.ones(H * D), [1, H, 1, D])
    ones_kv = FastTensor.new(np.ones(Hkv * D), [1, Hkv, 1, D])
    for pos in range(4):
        fast_attention(ones_q, ones_kv, ones_kv, 0, pos, cache, H, Hkv, D)
    assert np.array_equal(cache.k_buffers[0], np.ones(Hkv * cap * D, np.float32))
    zq = FastTensor.new(np.zeros(H * D), [1, H, 1, D])
    zkv = FastTensor.new(np.zeros(Hkv * D), [1, Hkv, 1, D])
    out = fast_attention(zq, zkv, zkv, 0, 4, cache, H, Hkv, D)
    cache_k = cache.k_buffers[0]
    for d in range(D):
        assert cache_k[0 * D + d] == 0.0
        assert cache_k[1 * D + d] == 1.0
    # folded positions 0..4 visit slots 0,1,2,3,0 (oracle test derives 0.6)
    assert np.allclose(out.data, 0.6, atol=1e-6)
