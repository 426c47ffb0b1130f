"""The two multi-stream / multi-GPU workload shapes at full width, through the C ABI, against the
CPU oracle on identical bytes.

* Batched decode of the BitNet-2B shape exactly as the benchmark draws it: 64 streams, KV lengths
  uniform in [128, 4096] from the benchmark's seed, shuffled 64-token pages, 30 layers.  The cache
  is generated on the device, copied back, and the oracle (src/nn/fast_attention.rs:138-201) runs on
  those bytes for EVERY stream on the first, a middle and the last layer.
* The long prefill split by KV-head group (LLaMA-3-8B shape, 32 query / 8 KV heads): every one of
  the 8 head groups runs through a context of its own, as it would on its own GPU, the per-group
  output slabs are stitched in head order and the whole [32, S, 128] result is compared with the
  oracle's prefill.  One GPU, no collective: this checks the partitioning, not the transport.
"""
import numpy as np
import pytest

import oracle as xo
import xor_net_b200 as xn
from gpu_util import assert_parity, errs, rand_qkv

pytestmark = pytest.mark.gpu
BASE_SEED = 299792458


def test_config3_every_stream_on_three_layers():
    n, Hq, Hkv, D, layers, lo, hi = 64, 20, 5, 128, 30, 128, 4096
    lens = np.random.default_rng(BASE_SEED + 3000).integers(lo, hi + 1, n).astype(np.int64)
    assert int(lens.sum()) == 138151   # the benchmark's draw for rank 0
    pages = int(sum((int(L) + 63) // 64 for L in lens))
    ctx = xn.Context(layers, Hq, Hkv, D, pool_pages=pages + 8, shuffle_seed=BASE_SEED)
    sts = [ctx.new_stream(hi) for _ in range(n)]
    for i, st in enumerate(sts):
        st.fill_normal(-1, 0, int(lens[i]) - 1, BASE_SEED + 3000 + i)
    rng = np.random.default_rng(BASE_SEED + 3001)
    pos = [int(L) - 1 for L in lens]
    worst = (0.0, 0.0)
    for layer in (0, layers // 2, layers - 1):
        qkv = [rand_qkv(rng, Hq, Hkv, 1, D) for _ in range(n)]
        outs = ctx.attention_batch(sts, layer, pos, [a[0] for a in qkv], [a[1] for a in qkv],
                                   [a[2] for a in qkv])
        caches = []
        for i in range(n):
            L = int(lens[i])
            k_all, v_all = sts[i].read_range(layer, 0, L)   # the appended token included
            assert np.array_equal(k_all[:, L - 1], qkv[i][1][0, :, 0])
            assert np.array_equal(v_all[:, L - 1], qkv[i][2][0, :, 0])
            ref = xo.RingCache(1, Hkv, L, D)
            if L > 1:
                ref.append(0, 0, k_all[:, :L - 1], v_all[:, :L - 1])
            caches.append(ref)
        want = xo.fast_attention_streams([a[0] for a in qkv], [a[1] for a in qkv], [a[2] for a in qkv],
                                         0, pos, caches, Hq, Hkv, D)
        for i in range(n):
            a, r = assert_parity(outs[i], want[i], f"layer {layer} stream {i} len {int(lens[i])}")
            worst = (max(worst[0], a), max(worst[1], r))
        for c in caches:
            c.close()
    print(f"config 3, 64 streams x 3 layers: worst max abs {worst[0]:.2e}, worst rel {worst[1]:.2e}")
    assert ctx.stats()["decode_launches"] == 3
    ctx.close()


def test_config5_head_split_prefill_stitched_on_one_gpu():
    Hq, Hkv, D, theta, world = 32, 8, 128, 500000.0, 8
    S = 4096 + 40                      # reduced from 32768; a ragged last query tile
    G = Hq // Hkv
    cos, sin = xn.rope_tables(theta, D, S)

    def head_tensor(kind, h):          # the problem is defined per global head, whatever the split
        return np.random.default_rng(BASE_SEED + 5000 + 100 * kind + h).standard_normal((S, D)).astype(np.float32)

    full = np.zeros((Hq, S, D), np.float32)
    for rank in range(world):
        kv_heads = xn.sharding.kv_heads_of_rank(Hkv, world, rank)
        q_heads = xn.sharding.query_heads_of_rank(Hq, Hkv, world, rank)
        assert q_heads == [kv * G + j for kv in kv_heads for j in range(G)]
        ctx = xn.Context(1, len(q_heads), len(kv_heads), D, pool_pages=(S + 63) // 64 + 2,
                         shuffle_seed=BASE_SEED + 5000 + rank, rope=(cos, sin))
        st = ctx.new_stream(S)
        q = np.stack([head_tensor(0, h) for h in q_heads])[None]
        k = np.stack([head_tensor(1, kv) for kv in kv_heads])[None]
        v = np.stack([head_tensor(2, kv) for kv in kv_heads])[None]
        slab = ctx.attention(st, 0, 0, q, k, v, rope=True)
        assert ctx.stats()["prefill_launches"] == 1
        full[q_heads[0]:q_heads[-1] + 1] = slab[0]      # contiguous head blocks: already in order
        # the head-sharded cache holds exactly this group's rotated keys
        kd, vd = st.read_range(0, 0, S)
        assert np.array_equal(kd, xo.tensor_rope(k, cos, sin, 0)[0]) and np.array_equal(vd, v[0])
        ctx.close()
    # the oracle on the whole problem, one KV-head group at a time (its loops are per KV head)
    worst = 0.0
    for kv in range(Hkv):
        q = np.stack([head_tensor(0, kv * G + j) for j in range(G)])[None]
        k, v = head_tensor(1, kv)[None, None], head_tensor(2, kv)[None, None]
        ref = xo.RingCache(1, 1, S, D)
        want = xo.fast_attention(xo.tensor_rope(q, cos, sin, 0), xo.tensor_rope(k, cos, sin, 0), v, 0, 0,
                                 ref, G, 1, D)[0]
        got = full[kv * G:(kv + 1) * G]
        assert np.all(np.isfinite(got))
        for t0 in range(0, S, 128):    # every 128-row query tile of every head, first and last included
            for j in range(G):
                _, r = errs(got[j, t0:t0 + 128], want[j, t0:t0 + 128])
                assert r <= 5e-3, f"head {kv * G + j} rows {t0}..: rel {r:.2e} (TF32 bound 5e-3)"
                worst = max(worst, r)
        ref.close()
    print(f"head-split prefill S={S}: worst per-tile rel {worst:.2e}")
