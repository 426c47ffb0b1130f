"""The BitNet-3B and long-context LLaMA-3-8B workload shapes as parity cases (they are not benchmark lines), through the
C ABI, against the CPU oracle on identical bytes."""
import numpy as np
import pytest

import oracle as xo
import xor_net_b200 as xn
from gpu_util import assert_parity, errs, rand_qkv

pytestmark = pytest.mark.gpu
BASE_SEED = 299792458


def test_config4_mha_head_dim_100_prefill_then_256_decode_steps():
    # BitNet-3B shape: 32 query = 32 KV heads, head_dim 100 (non-power-of-two tail), RoPE theta
    # 10000, scale 1/sqrt(100); 8 sequences: causal prefill of 1024 tokens (tensor-core kernel,
    # TF32 tolerance 5e-3), then 256 decode steps that append to the cache (f32 tolerances).
    # Parity on every step for stream 0 and on every 32nd step for the others.
    H, D, S0, steps, n = 32, 100, 1024, 256, 8
    rng = np.random.default_rng(BASE_SEED + 4000)
    cos, sin = xn.rope_tables(10000.0, D, S0 + steps)
    ctx = xn.Context(1, H, H, D, pool_pages=n * 21, shuffle_seed=4, rope=(cos, sin))
    sts = [ctx.new_stream(S0 + steps) for _ in range(n)]
    refs = [xo.RingCache(1, H, S0 + steps, D) for _ in range(n)]
    # prefill, one call per stream; outputs checked on two streams, caches checked on all
    for i in range(n):
        q, k, v = rand_qkv(rng, H, H, S0, D)
        got = ctx.attention(sts[i], 0, 0, q, k, v, rope=True)
        kr = xo.tensor_rope(k, cos, sin, 0)
        if i < 2:
            want = xo.fast_attention(xo.tensor_rope(q, cos, sin, 0), kr, v, 0, 0, refs[i], H, H, D)
            a, r = errs(got, want)
            assert r <= 5e-3, f"prefill stream {i}: rel {r:.2e}"
        else:
            refs[i].append(0, 0, kr[0], v[0])
    assert ctx.stats()["prefill_launches"] == n
    for i in (0, n - 1):
        kd, vd = sts[i].read_range(0, 0, S0)
        assert np.array_equal(kd, refs[i].k_buffer(0).reshape(H, S0 + steps, D)[:, :S0])
    # decode: all streams in one batched call per step
    worst = (0.0, 0.0)
    for s in range(steps):
        pos = S0 + s
        qkv = [rand_qkv(rng, H, H, 1, D) for _ in range(n)]
        outs = ctx.attention_batch(sts, 0, [pos] * n, [a[0] for a in qkv], [a[1] for a in qkv],
                                   [a[2] for a in qkv], rope=True)
        for i in range(n):
            q, k, v = qkv[i]
            kr = xo.tensor_rope(k, cos, sin, pos)
            if i == 0 or s % 32 == 31:
                want = xo.fast_attention(xo.tensor_rope(q, cos, sin, pos), kr, v, 0, pos, refs[i], H, H, D)
                a, r = assert_parity(outs[i], want, f"stream {i} step {s}")
                worst = (max(worst[0], a), max(worst[1], r))
            else:
                refs[i].append(0, pos, kr[0], v[0])
    print(f"config 4 decode: worst max abs {worst[0]:.2e}, worst rel {worst[1]:.2e}")
    kd, vd = sts[3].read_range(0, 0, S0 + steps)
    assert np.array_equal(kd.ravel(), refs[3].k_buffer(0)) and np.array_equal(vd.ravel(), refs[3].v_buffer(0))
    ctx.close()


def test_config5_long_context_decode_sampled_streams():
    # LLaMA-3-8B shape: 32 query / 8 KV heads, head_dim 128, KV lengths uniform in [2048, 8192],
    # 64-token pages in shuffled order.  One GPU's share at reduced stream and layer count (12
    # streams, 2 layers); the cache is generated on the device, copied back, and the oracle runs on
    # those bytes for the shortest, the longest and two other streams.
    Hq, Hkv, D, n, layers = 32, 8, 128, 12, 2
    rng = np.random.default_rng(BASE_SEED + 5000)
    lens = rng.integers(2048, 8193, n)
    lens[0], lens[1] = 2048, 8192
    ctx = xn.Context(layers, Hq, Hkv, D, pool_pages=int(sum((L + 63) // 64 for L in lens)) + 4,
                     shuffle_seed=5)
    sts = [ctx.new_stream(8192) for _ in range(n)]
    for i, st in enumerate(sts):
        st.fill_normal(-1, 0, int(lens[i]) - 1, BASE_SEED + 5000 + i)
    for layer in range(layers):
        qkv = [rand_qkv(rng, Hq, Hkv, 1, D) for _ in range(n)]
        outs = ctx.attention_batch(sts, layer, [int(L) - 1 for L in lens], [a[0] for a in qkv],
                                   [a[1] for a in qkv], [a[2] for a in qkv])
        for i in (0, 1, 5, 11):
            L = int(lens[i])
            k_all, v_all = sts[i].read_range(layer, 0, L)          # includes the appended token
            ref = xo.RingCache(1, Hkv, L, D)
            ref.append(0, 0, k_all[:, :L - 1], v_all[:, :L - 1])
            want = xo.fast_attention(*qkv[i], 0, L - 1, ref, Hq, Hkv, D)
            a, r = assert_parity(outs[i], want, f"layer {layer} stream {i} len {L}")
            f64 = xo.naive_attention_f64(qkv[i][0][0], k_all, v_all, L - 1, Hq, Hkv, D)
            ga, gr = errs(outs[i][0], f64)
            ra, rr = errs(want[0], f64)
            print(f"len {L}: gpu-vs-oracle rel {r:.2e}; gpu-vs-f64 rel {gr:.2e}; oracle-vs-f64 rel {rr:.2e}")
            assert gr <= 1e-5
    ctx.close()
