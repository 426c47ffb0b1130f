"""The opt-in u8 cache format (XN_KV_U8) against the CPU oracle, through the C ABI.

Two bars:
  * storage -- the bytes and scales the library keeps equal the reference's u8 shadow
    (CpuRingCache::quantize_to_u8, fast_attention.rs:62-71, applied per (KV head, token) row at
    append, :117-128) BIT FOR BIT, and the dequantised rows read back equal (byte - 128) * scale
    bit for bit;
  * attention -- the output equals the oracle's fast_attention run over those dequantised rows
    within the f32 path's tolerance (max abs <= 1e-4, relative L2 <= 1e-5): only the order of the
    f32 sums and exp2f-vs-expf differ.
The distance to the f32 cache's result is the quantisation error of the format itself and is only
bounded loosely (relative L2 <= 2e-2 on N(0,1) data).
"""
import numpy as np
import pytest

import oracle as xo
import xor_net_b200 as xn
from gpu_util import assert_parity, errs, rand_qkv

pytestmark = pytest.mark.gpu


class PairU8:
    """A device stream of a KV_U8 context and an oracle ring cache fed with the round-tripped rows,
    plus the oracle's shadow arrays (bytes, scales) by slot."""

    def __init__(self, ctx, cap, rope=None):
        self.ctx, self.cap, self.rope = ctx, cap, rope
        self.st = ctx.new_stream(cap)
        self.ref = xo.RingCache(ctx.num_layers, ctx.num_kv_heads, cap, ctx.head_dim)
        H, D = ctx.num_kv_heads, ctx.head_dim
        self.k8 = {l: np.full((H, cap, D), 128, np.uint8) for l in range(ctx.num_layers)}
        self.v8 = {l: np.full((H, cap, D), 128, np.uint8) for l in range(ctx.num_layers)}
        self.ks = {l: np.zeros((H, cap), np.float32) for l in range(ctx.num_layers)}
        self.vs = {l: np.zeros((H, cap), np.float32) for l in range(ctx.num_layers)}

    def oracle_step(self, layer, pos, q, k, v, rope=False):
        if rope:
            cos, sin = self.rope
            q = xo.tensor_rope(q, cos, sin, pos)
            k = xo.tensor_rope(k, cos, sin, pos)
        kq, ksc = xo.quantize_to_u8(k[0])
        vq, vsc = xo.quantize_to_u8(v[0])
        S = k.shape[2]
        for t in range(S):                       # sequential, like the reference's append loop
            slot = (pos + t) % self.cap
            self.k8[layer][:, slot], self.v8[layer][:, slot] = kq[:, t], vq[:, t]
            self.ks[layer][:, slot], self.vs[layer][:, slot] = ksc[:, t], vsc[:, t]
        kd = xo.dequantize_u8(kq, ksc)[None]
        vd = xo.dequantize_u8(vq, vsc)[None]
        return xo.fast_attention(q, kd, vd, layer, pos, self.ref, self.ctx.num_heads,
                                 self.ctx.num_kv_heads, self.ctx.head_dim)

    def step(self, layer, pos, q, k, v, rope=False):
        got = self.ctx.attention(self.st, layer, pos, q, k, v, rope=rope)
        return got, self.oracle_step(layer, pos, q, k, v, rope)

    def check_cache(self, layer):
        k8, v8, ks, vs = self.st.read_u8(layer, 0, self.cap)
        assert np.array_equal(k8, self.k8[layer]), "K bytes differ from the reference's shadow"
        assert np.array_equal(v8, self.v8[layer]), "V bytes differ from the reference's shadow"
        assert np.array_equal(ks.view(np.uint32), self.ks[layer].view(np.uint32)), "K scales differ"
        assert np.array_equal(vs.view(np.uint32), self.vs[layer].view(np.uint32)), "V scales differ"
        k, v = self.st.read_range(layer, 0, self.cap)
        assert np.array_equal(k.ravel(), self.ref.k_buffer(layer))
        assert np.array_equal(v.ravel(), self.ref.v_buffer(layer))


def u8_ctx(L, Hq, Hkv, D, pages, **kw):
    # exact-f32 prefill rows unless a test asks otherwise: this module checks the f32 tolerances
    kw.setdefault("prefill_mode", 1)
    return xn.Context(L, Hq, Hkv, D, pool_pages=pages, kv_format=xn.KV_U8, **kw)


@pytest.mark.parametrize("D", [2, 7, 16, 17, 32, 33, 64, 100, 128, 160, 256])
def test_head_dims(D):
    rng = np.random.default_rng(D)
    for Hq, Hkv in [(4, 2), (3, 3), (8, 2)]:
        ctx = u8_ctx(2, Hq, Hkv, D, 16)
        p = PairU8(ctx, 300)
        q, k, v = rand_qkv(rng, Hq, Hkv, 70, D)
        got, want = p.step(1, 0, q, k, v)                 # prefill rows across a page boundary
        assert_parity(got, want, f"prefill D={D} Hq={Hq} Hkv={Hkv}")
        for pos in (70, 71):
            q, k, v = rand_qkv(rng, Hq, Hkv, 1, D)
            got, want = p.step(1, pos, q, k, v)
            assert_parity(got, want, f"decode D={D} pos={pos}")
        p.check_cache(1)
        p.check_cache(0)                                  # untouched layer: bytes 128, scales 0
        ctx.close()


@pytest.mark.parametrize("Hq,Hkv", [(1, 1), (2, 1), (3, 1), (4, 1), (5, 1), (8, 1), (12, 4), (32, 8), (20, 5)])
def test_group_sizes(Hq, Hkv):
    rng = np.random.default_rng(Hq * 100 + Hkv)
    ctx = u8_ctx(1, Hq, Hkv, 64, 16)
    p = PairU8(ctx, 512)
    q, k, v = rand_qkv(rng, Hq, Hkv, 130, 64)
    got, want = p.step(0, 0, q, k, v)
    assert_parity(got, want, f"G={Hq // Hkv} prefill")
    q, k, v = rand_qkv(rng, Hq, Hkv, 1, 64)
    got, want = p.step(0, 130, q, k, v)
    assert_parity(got, want, f"G={Hq // Hkv} decode")
    p.check_cache(0)
    ctx.close()


def test_decode_lengths_around_boundaries():
    rng = np.random.default_rng(5)
    ctx = u8_ctx(1, 20, 5, 128, 40)
    for L in [1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 191, 192, 193, 1000]:
        p = PairU8(ctx, 2048)
        if L > 1:
            qq, kk, vv = rand_qkv(rng, 20, 5, L - 1, 128)
            p.step(0, 0, qq, kk, vv)
        q, k, v = rand_qkv(rng, 20, 5, 1, 128)
        got, want = p.step(0, L - 1, q, k, v)
        assert_parity(got, want, f"L={L}")
        p.st.destroy()
    ctx.close()


def test_rope_append_and_chunks():
    # fused rotation before the quantiser, chunked prefill, overwrite of existing positions
    rng = np.random.default_rng(17)
    rope = xn.rope_tables(500000.0, 128, 2048)
    ctx = u8_ctx(2, 20, 5, 128, 40, rope=rope)
    p = PairU8(ctx, 1024, rope=rope)
    pos = 0
    for S in (100, 57, 1, 200, 1):
        q, k, v = rand_qkv(rng, 20, 5, S, 128)
        got, want = p.step(1, pos, q, k, v, rope=True)
        assert_parity(got, want, f"rope chunk at {pos}+{S}")
        pos += S
    q, k, v = rand_qkv(rng, 20, 5, 30, 128)
    got, want = p.step(1, 300, q, k, v, rope=True)
    assert_parity(got, want, "overwrite")
    p.check_cache(1)
    ctx.close()


def test_long_stream_cut_units():
    # few streams, long caches: units are cut across thread blocks and merged from partial records
    rng = np.random.default_rng(23)
    ctx = u8_ctx(1, 15, 5, 64, 200)
    pairs = [PairU8(ctx, 4096) for _ in range(2)]
    lens = [3000, 1777]
    for p, L in zip(pairs, lens):
        q, k, v = rand_qkv(rng, 15, 5, L, 64)
        want = p.oracle_step(0, 0, q, k, v)
        got = ctx.attention(p.st, 0, 0, q, k, v)
        assert_parity(got[:, :, -3:], want[:, :, -3:], f"prefill tail L={L}")
    qs, ks, vs = zip(*[rand_qkv(rng, 15, 5, 1, 64) for _ in pairs])
    got = ctx.attention_batch([p.st for p in pairs], 0, lens, qs, ks, vs)
    for i, p in enumerate(pairs):
        want = p.oracle_step(0, lens[i], qs[i], ks[i], vs[i])
        assert_parity(got[i], want, f"decode stream {i}")
        p.check_cache(0)
    ctx.close()


def test_ragged_batch_of_streams():
    rng = np.random.default_rng(31)
    ctx = u8_ctx(2, 20, 5, 64, 300)
    lens = [1, 5, 64, 65, 200, 513, 700, 1023]
    pairs = [PairU8(ctx, 2048) for _ in lens]
    for p, L in zip(pairs, lens):
        q, k, v = rand_qkv(rng, 20, 5, L, 64)
        p.step(1, 0, q, k, v)
    for step in range(3):
        qs, ks, vs = zip(*[rand_qkv(rng, 20, 5, 1, 64) for _ in pairs])
        got = ctx.attention_batch([p.st for p in pairs], 1, [L + step for L in lens], qs, ks, vs)
        for i, p in enumerate(pairs):
            want = p.oracle_step(1, lens[i] + step, qs[i], ks[i], vs[i])
            assert_parity(got[i], want, f"step {step} stream {i}")
    for p in pairs:
        p.check_cache(1)
    ctx.close()


def test_gap_reads_as_never_written():
    # positions skipped over keep byte 128 / scale 0.0 and contribute exact zeros
    rng = np.random.default_rng(41)
    ctx = u8_ctx(1, 4, 2, 64, 16)
    p = PairU8(ctx, 512)
    q, k, v = rand_qkv(rng, 4, 2, 10, 64)
    p.step(0, 0, q, k, v)
    q, k, v = rand_qkv(rng, 4, 2, 3, 64)
    got, want = p.step(0, 100, q, k, v)          # slots 10..99 were never written
    assert_parity(got, want, "gap")
    p.check_cache(0)
    p.st.reset()
    k8, v8, ks, vs = p.st.read_u8(0, 0, 128)
    assert (k8 == 128).all() and (v8 == 128).all() and (ks == 0).all() and (vs == 0).all()
    ctx.close()


def test_ring_wrap():
    # index_pos + seq_len beyond the capacity: positions fold modulo the capacity (generic kernel)
    rng = np.random.default_rng(43)
    ctx = u8_ctx(1, 6, 2, 32, 16)
    p = PairU8(ctx, 96)
    q, k, v = rand_qkv(rng, 6, 2, 90, 32)
    got, want = p.step(0, 0, q, k, v)
    assert_parity(got, want, "fill")
    q, k, v = rand_qkv(rng, 6, 2, 20, 32)
    got, want = p.step(0, 90, q, k, v)           # wraps at 96
    assert_parity(got, want, "wrap")
    q, k, v = rand_qkv(rng, 6, 2, 1, 32)
    got, want = p.step(0, 110, q, k, v)
    assert_parity(got, want, "decode after wrap")
    p.check_cache(0)
    ctx.close()


def test_quantiser_edge_rows():
    # all-zero rows (scale 1.0), a single huge element, values that round to ties, denormals
    ctx = u8_ctx(1, 2, 2, 16, 4)
    p = PairU8(ctx, 64)
    k = np.zeros((1, 2, 4, 16), np.float32)
    v = np.zeros((1, 2, 4, 16), np.float32)
    k[0, 0, 1, 3] = 1e30
    k[0, 1, 1] = np.linspace(-1, 1, 16, dtype=np.float32)
    k[0, 0, 2] = (np.arange(16) - 8).astype(np.float32) * 0.5      # exact halves after scaling
    v[0, 1, 2] = 1e-41                                             # denormals
    v[0, 0, 3] = -np.arange(16, dtype=np.float32)
    q = np.ones((1, 2, 4, 16), np.float32)
    got, want = p.step(0, 0, q, k, v)
    assert_parity(got, want, "edge rows")
    p.check_cache(0)
    ctx.close()


def test_distance_to_f32_cache_is_the_quantisation_error():
    rng = np.random.default_rng(47)
    c8 = u8_ctx(1, 20, 5, 128, 40)
    c32 = xn.Context(1, 20, 5, 128, pool_pages=40, prefill_mode=1)
    s8, s32 = c8.new_stream(1024), c32.new_stream(1024)
    q, k, v = rand_qkv(rng, 20, 5, 600, 128)
    a = c8.attention(s8, 0, 0, q, k, v)
    b = c32.attention(s32, 0, 0, q, k, v)
    ea, er = errs(a, b)
    print(f"u8 cache vs f32 cache: max abs {ea:.3e}, rel L2 {er:.3e}")
    assert 1e-4 < er <= 2e-2
    c8.close()
    c32.close()


def test_device_pointer_batch_and_synthetic_fill():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(53)
    ctx = u8_ctx(2, 15, 5, 64, 600)
    n, L = 6, 900
    streams = [ctx.new_stream(2048) for _ in range(n)]
    for i, s in enumerate(streams):
        s.fill_normal(-1, 0, L, 1234 + i)
    dev = torch.device("cuda:0")
    q = torch.from_numpy(rng.standard_normal((n, 15, 1, 64)).astype(np.float32)).to(dev)
    k = torch.from_numpy(rng.standard_normal((n, 5, 1, 64)).astype(np.float32)).to(dev)
    v = torch.from_numpy(rng.standard_normal((n, 5, 1, 64)).astype(np.float32)).to(dev)
    out = torch.empty_like(q)
    reqs = ctx.make_batch([(s, 1, L, 1, q[i].data_ptr(), k[i].data_ptr(), v[i].data_ptr(), out[i].data_ptr())
                           for i, s in enumerate(streams)], xn.REQ_DEVICE_PTRS)
    torch.cuda.synchronize()
    ctx.submit(reqs)
    ctx.synchronize()
    got = out.cpu().numpy()
    for i, s in enumerate(streams):
        kc, vc = s.read_range(1, 0, L + 1)               # dequantised rows, new token included
        ref = xo.RingCache(1, 5, L + 1, 64)
        ref.append(0, 0, kc[None], vc[None])
        want = xo.fast_attention(q[i:i + 1].cpu().numpy(), kc[None, :, L:], vc[None, :, L:], 0, L, ref, 15, 5, 64)
        assert_parity(got[i:i + 1], want, f"stream {i}")
        # the synthetic fill is the quantised image of the f32 fill (same generator)
        k8, v8, ks, vs = s.read_u8(1, 0, 4)
        assert ks.min() > 0 and vs.min() > 0
        assert ((k8 == 255) | (k8 == 1)).any(axis=-1).all()   # every row's largest element hits +-127
    ctx.close()


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 20, 5), (64, 8, 2), (32, 4, 4)])
def test_tensor_core_prefill_over_u8_cache(D, Hq, Hkv):
    # prefills of >= 128 rows: append (rotate, quantise), dequantise the stream's pages of the layer
    # into the f32 staging area, run the tcgen05 TF32 kernel over it.  Storage stays bit-exact; the
    # output keeps the TF32 kernel's bound (rel L2 <= 5e-3) against the oracle over the dequantised rows.
    rng = np.random.default_rng(800 + D)
    rope = xn.rope_tables(500000.0, D, 4096)
    ctx = u8_ctx(2, Hq, Hkv, D, 80, rope=rope, shuffle_seed=5, prefill_mode=0)
    p = PairU8(ctx, 2048, rope=rope)
    pos = 0
    for S in (300, 1, 130, 700):                  # 1: a decode step between chunks; 700 grows the staging area
        q, k, v = rand_qkv(rng, Hq, Hkv, S, D)
        before = ctx.stats()["prefill_launches"]
        got, want = p.step(1, pos, q, k, v, rope=True)
        assert ctx.stats()["prefill_launches"] - before == (1 if S >= 128 else 0)
        if S >= 128:
            assert errs(got, want)[1] <= 5e-3, f"TF32 chunk at {pos}+{S}: rel {errs(got, want)[1]:.2e}"
        else:
            assert_parity(got, want, f"decode at {pos}")
        pos += S
    p.check_cache(1)
    # a second stream reuses the staging area
    p2 = PairU8(ctx, 2048, rope=rope)
    q, k, v = rand_qkv(rng, Hq, Hkv, 200, D)
    got, want = p2.step(0, 0, q, k, v, rope=True)
    assert errs(got, want)[1] <= 5e-3
    p2.check_cache(0)
    ctx.close()


def test_rejects_bad_format_and_f32_reader():
    with pytest.raises(xn.XnError):
        xn.Context(1, 4, 2, 64, pool_pages=4, kv_format=7)
    c = xn.Context(1, 4, 2, 64, pool_pages=4)
    s = c.new_stream(64)
    with pytest.raises(xn.XnError):
        s.read_u8(0, 0, 4)
    c.close()


def test_pool_bytes_buys_four_times_the_pages():
    a = xn.Context(2, 20, 5, 128, pool_bytes=64 << 20)
    b = u8_ctx(2, 20, 5, 128, 0, pool_bytes=64 << 20)
    pa, pb = a.stats()["pages_total"], b.stats()["pages_total"]
    assert 3.8 * pa < pb <= 4 * pa
    a.close()
    b.close()


def test_whole_block_over_u8_cache():
    # q/k/v projections -> RoPE -> quantised append -> attention -> sub-norm -> o_proj, all on the
    # device: the stored bytes equal the oracle's shadow of the projected, rotated rows bit for
    # bit; the attention rows keep the f32 bounds; the block output keeps the whole-block bound
    # (rel L2 <= 1e-3: an activation may quantise one step apart)
    xo.set_quant_body(1)
    try:
        rng = np.random.default_rng(61)
        Hq, Hkv, D, hidden, layer = 20, 5, 128, 2560, 1
        rope = xn.rope_tables(500000.0, D, 1024)
        ctx = u8_ctx(2, Hq, Hkv, D, 40, rope=rope, shuffle_seed=3)
        mk = lambda o, i: rng.standard_normal((o, i)).astype(np.float32)
        ws = {"q": mk(Hq * D, hidden), "k": mk(Hkv * D, hidden), "v": mk(Hkv * D, hidden), "o": mk(hidden, Hq * D)}
        scale = {n: (float(hidden) ** -0.5 if n != "o" else None) for n in ws}
        dev = {n: xn.TernaryLinear(w.shape[1], w.shape[0], w, xn.PACK4, scale[n]) for n, w in ws.items()}
        ref = {n: xo.TernaryLinear(w.shape[1], w.shape[0], w, xn.PACK4, scale[n]) for n, w in ws.items()}
        nw = (1.0 + 0.2 * rng.standard_normal(Hq * D)).astype(np.float32)
        ctx.set_qkv_proj(layer, dev["q"], dev["k"], dev["v"])
        ctx.set_out_proj(layer, dev["o"], nw, 1e-5)
        lens = [70, 300]
        pairs = [(ctx.new_stream(1024), xo.RingCache(2, Hkv, 1024, D)) for _ in lens]
        oracle = lambda x, pos, cache: xo.causal_self_attention_forward(
            x, pos, layer, cache, rope[0], rope[1], ref["q"], ref["k"], ref["v"], Hq, Hkv, D, nw, 1e-5,
            ref["o"], kv_u8=True)
        for (st, cache), L in zip(pairs, lens):
            x = rng.standard_normal((1, L, hidden)).astype(np.float32)
            attn_dev = ctx.attention_batch([st], layer, [0], [x], qkv_proj=True)[0]
            _, attn_ref = oracle(x, 0, cache)
            assert_parity(attn_dev, xo.transpose_heads_to_seq(attn_ref), f"prefill rows L={L}")
        xs = [rng.standard_normal((1, 1, hidden)).astype(np.float32) for _ in lens]
        y_dev = ctx.attention_batch([p[0] for p in pairs], layer, lens, xs, qkv_proj=True, out_proj=True)
        for i, (st, cache) in enumerate(pairs):
            y_ref, _ = oracle(xs[i], lens[i], cache)
            assert errs(y_dev[i], y_ref)[1] <= 1e-3, f"block output, stream {i}"
            # cache: dequantised rows equal the oracle ring (which holds the round-tripped rows) ...
            k, v = st.read_range(layer, 0, lens[i] + 1)
            kb = cache.k_buffer(layer).reshape(Hkv, 1024, D)[:, :lens[i] + 1]
            vb = cache.v_buffer(layer).reshape(Hkv, 1024, D)[:, :lens[i] + 1]
            assert np.array_equal(k, kb) and np.array_equal(v, vb)
            # ... and they are what the stored bytes and scales say
            k8, v8, ks, vs = st.read_u8(layer, 0, lens[i] + 1)
            assert np.array_equal((k8.astype(np.float32) - 128.0) * ks[..., None], k)
            assert np.array_equal((v8.astype(np.float32) - 128.0) * vs[..., None], v)
        ctx.close()
    finally:
        xo.set_quant_body(-1)


@pytest.mark.parametrize("D", [16, 32, 64, 100, 128, 256])
def test_rotated_decode_steps_all_row_widths(D):
    # decode with pre-RoPE q and k: for power-of-two head dims >= 32 the attention kernel rotates,
    # quantises and stores the new token itself (one launch per call); other dims go through the
    # append kernel.  Either way the stored bytes equal the oracle's shadow of the rotated rows.
    rng = np.random.default_rng(700 + D)
    rope = xn.rope_tables(10000.0, D, 512)
    Hq, Hkv = 8, 2
    ctx = u8_ctx(1, Hq, Hkv, D, 16, rope=rope)
    p = PairU8(ctx, 256, rope=rope)
    q, k, v = rand_qkv(rng, Hq, Hkv, 37, D)
    got, want = p.step(0, 0, q, k, v, rope=True)
    assert_parity(got, want, f"prefill D={D}")
    for pos in range(37, 70):                      # crosses a page boundary at 64
        q, k, v = rand_qkv(rng, Hq, Hkv, 1, D)
        before = ctx.stats()["kernel_launches"]
        got, want = p.step(0, pos, q, k, v, rope=True)
        launches = ctx.stats()["kernel_launches"] - before
        assert_parity(got, want, f"decode D={D} pos={pos}")
        assert launches == (1 if D in (32, 64, 128, 256) else 2), launches
    p.check_cache(0)
    ctx.close()


def test_pinned_host_rows_equal_staged_rows():
    # XN_REQ_HOST_PINNED over the u8 cache: page-locked rows go through the append kernel (not the
    # fused path); the staged path at the same positions (fused append) must leave the same bytes in
    # the cache and return the same result up to the order of the sums (the fused path handles the
    # new token after the cached ones)
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(59)
    ctx = u8_ctx(1, 20, 5, 128, 80)
    lens = [300, 64, 1500, 1]
    pairs = [PairU8(ctx, 2048) for _ in lens]
    for p, L in zip(pairs, lens):
        if L > 1:
            p.step(0, 0, *rand_qkv(rng, 20, 5, L - 1, 128))
    n = len(lens)
    q = torch.from_numpy(rng.standard_normal((n, 20, 128)).astype(np.float32)).pin_memory()
    k = torch.from_numpy(rng.standard_normal((n, 5, 128)).astype(np.float32)).pin_memory()
    v = torch.from_numpy(rng.standard_normal((n, 5, 128)).astype(np.float32)).pin_memory()
    out = torch.zeros(n, 20, 128).pin_memory()
    reqs = ctx.make_batch([(pairs[i].st, 0, lens[i] - 1, 1, q[i].data_ptr(), k[i].data_ptr(),
                            v[i].data_ptr(), out[i].data_ptr()) for i in range(n)], xn.REQ_HOST_PINNED)
    ctx.submit(reqs)
    for i, p in enumerate(pairs):
        want = p.oracle_step(0, lens[i] - 1, q[i].numpy().reshape(1, 20, 1, 128),
                             k[i].numpy().reshape(1, 5, 1, 128), v[i].numpy().reshape(1, 5, 1, 128))
        assert_parity(out[i].numpy().reshape(1, 20, 1, 128), want, f"pinned stream {i}")
        p.check_cache(0)
    before = ctx.stats()["kernel_launches"]
    staged = ctx.attention_batch([p.st for p in pairs], 0, [L - 1 for L in lens],
                                 [q[i].numpy().reshape(1, 20, 1, 128) for i in range(n)],
                                 [k[i].numpy().reshape(1, 5, 1, 128) for i in range(n)],
                                 [v[i].numpy().reshape(1, 5, 1, 128) for i in range(n)])
    assert ctx.stats()["kernel_launches"] - before == 1          # fused: the attention kernel alone
    for i, p in enumerate(pairs):
        assert_parity(staged[i].reshape(20, 128), out[i].numpy(), f"staged vs pinned, stream {i}")
        p.check_cache(0)
    ctx.close()


# ---- the variant with q.k on the integer tensor-core path ---------------------------------------
# Large submissions (>= 524288 attended rows) over 64- and 128-byte rows run
# attn_splitkv_u8_mma_kernel: the K bytes are an MMA operand, the query rows three int8 terms.
# XORNET_ATTN_KV8_MMA_MIN_ROWS=0 forces it for every submission of a context created afterwards.

@pytest.mark.parametrize("case", [
    lambda: test_head_dims(64), lambda: test_head_dims(128),
    lambda: test_group_sizes(1, 1), lambda: test_group_sizes(2, 1), lambda: test_group_sizes(3, 1),
    lambda: test_group_sizes(5, 1), lambda: test_group_sizes(8, 1), lambda: test_group_sizes(32, 8),
    lambda: test_group_sizes(20, 5),
    test_decode_lengths_around_boundaries, test_rope_append_and_chunks, test_long_stream_cut_units,
    test_ragged_batch_of_streams, test_gap_reads_as_never_written, test_whole_block_over_u8_cache,
    test_device_pointer_batch_and_synthetic_fill,
])
def test_tensor_core_variant(monkeypatch, case):
    monkeypatch.setenv("XORNET_ATTN_KV8_MMA_MIN_ROWS", "0")
    case()


def test_large_batch_takes_the_tensor_core_variant_and_agrees():
    # 24 streams x ~700 tokens x 5 KV heads = 84 k attended rows, with the threshold lowered to 65536:
    # the variant is chosen by size; the same batch with the variant disabled must agree within the
    # f32 bounds, and both with the oracle
    import os
    rng = np.random.default_rng(91)
    lens = [int(x) for x in rng.integers(500, 900, 24)]
    outs = {}
    for mode in ("1", "0"):
        os.environ["XORNET_ATTN_KV8_MMA"] = mode
        os.environ["XORNET_ATTN_KV8_MMA_MIN_ROWS"] = "65536"
        try:
            ctx = u8_ctx(1, 20, 5, 128, 400)
        finally:
            del os.environ["XORNET_ATTN_KV8_MMA"]
            del os.environ["XORNET_ATTN_KV8_MMA_MIN_ROWS"]
        streams = [ctx.new_stream(1024) for _ in lens]
        for i, (st, L) in enumerate(zip(streams, lens)):
            st.fill_normal(0, 0, L, 77 + i)
        r2 = np.random.default_rng(92)
        qs, ks, vs = zip(*[rand_qkv(r2, 20, 5, 1, 128) for _ in lens])
        before = ctx.stats()["kernel_launches"]
        outs[mode] = ctx.attention_batch(streams, 0, lens, qs, ks, vs)
        launches = ctx.stats()["kernel_launches"] - before
        assert launches == (2 if mode == "1" else 1)      # append + attention / attention alone
        if mode == "1":
            for i in (0, 7, 23):
                kc, vc = streams[i].read_range(0, 0, lens[i] + 1)
                ref = xo.RingCache(1, 5, lens[i] + 1, 128)
                ref.append(0, 0, kc[None], vc[None])
                want = xo.fast_attention(qs[i], kc[None, :, lens[i]:], vc[None, :, lens[i]:], 0, lens[i], ref, 20, 5, 128)
                assert_parity(outs[mode][i], want, f"stream {i} vs oracle")
        ctx.close()
    for i in range(len(lens)):
        assert_parity(outs["1"][i], outs["0"][i], f"stream {i}: tensor-core variant vs CUDA-core kernel")
