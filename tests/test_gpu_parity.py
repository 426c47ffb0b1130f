"""Parity of the CUDA path with the CPU oracle on identical seeded inputs, through the C ABI.

Tolerance of the f32 path (gpu_util.ABS_TOL / REL_TOL): max abs <= 1e-4 and relative L2 <= 1e-5.
Cache contents (append, fused RoPE) must be bit-identical.
"""
import os

import numpy as np
import pytest

import oracle as xo
import xor_net_b200 as xn
from gpu_util import Pair, assert_parity, errs, rand_qkv

pytestmark = pytest.mark.gpu
F32 = 1  # XN_PREFILL_F32


@pytest.fixture(scope="module")
def ctx2b():
    # exact-f32 prefill: this module checks the f32 tolerances (the TF32 kernel has its own tests)
    c = xn.Context(num_layers=3, num_heads=20, num_kv_heads=5, head_dim=128, pool_pages=600,
                   shuffle_seed=11, rope=xn.rope_tables(500000.0, 128, 8192), prefill_mode=F32)
    yield c
    c.close()


# ---- head dims and group sizes of the reference's primitive tests ------------------------------

@pytest.mark.parametrize("D", [2, 4, 7, 8, 9, 15, 16, 17, 31, 32, 33, 64, 100, 128, 160, 256])
def test_head_dims(D):
    rng = np.random.default_rng(D)
    for Hq, Hkv in [(4, 2), (3, 3), (8, 2)]:
        ctx = xn.Context(2, Hq, Hkv, D, pool_pages=16, prefill_mode=F32)
        p = Pair(ctx, 300)
        q, k, v = rand_qkv(rng, Hq, Hkv, 70, D)
        got, want = p.step(1, 0, q, k, v)                 # prefill across a page boundary
        assert_parity(got, want, f"prefill D={D} Hq={Hq} Hkv={Hkv}")
        for pos in (70, 71):
            q, k, v = rand_qkv(rng, Hq, Hkv, 1, D)
            got, want = p.step(1, pos, q, k, v)
            assert_parity(got, want, f"decode D={D} pos={pos}")
        p.check_cache(1)
        ctx.close()


@pytest.mark.parametrize("Hq,Hkv", [(1, 1), (2, 1), (3, 1), (4, 1), (5, 1), (8, 1), (12, 4), (32, 8), (20, 5)])
def test_group_sizes(Hq, Hkv):
    rng = np.random.default_rng(Hq * 100 + Hkv)
    ctx = xn.Context(1, Hq, Hkv, 64, pool_pages=16, prefill_mode=F32)
    p = Pair(ctx, 512)
    q, k, v = rand_qkv(rng, Hq, Hkv, 130, 64)
    got, want = p.step(0, 0, q, k, v)
    assert_parity(got, want, f"G={Hq // Hkv} prefill")
    q, k, v = rand_qkv(rng, Hq, Hkv, 1, 64)
    got, want = p.step(0, 130, q, k, v)
    assert_parity(got, want, f"G={Hq // Hkv} decode")
    ctx.close()


# ---- lengths around page (64) and tile boundaries, one token at a time ------------------------

def test_decode_lengths_around_boundaries(ctx2b):
    rng = np.random.default_rng(5)
    for L in [1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 191, 192, 193, 1000]:
        p = Pair(ctx2b, 2048)
        if L > 1:
            kk = rng.standard_normal((1, 5, L - 1, 128)).astype(np.float32)
            vv = rng.standard_normal((1, 5, L - 1, 128)).astype(np.float32)
            qq = rng.standard_normal((1, 20, L - 1, 128)).astype(np.float32)
            p.step(0, 0, qq, kk, vv)
        q, k, v = rand_qkv(rng, 20, 5, 1, 128)
        got, want = p.step(0, L - 1, q, k, v)
        assert_parity(got, want, f"L={L}")
        p.st.destroy()


def test_config1_decode_shape(ctx2b):
    # BitNet-2B shape, one query token over 1024 cached tokens (the single-stream decode workload)
    rng = np.random.default_rng(299792458)
    p = Pair(ctx2b, 4096)
    qq, kk, vv = rand_qkv(rng, 20, 5, 1023, 128)
    p.step(2, 0, qq, kk, vv)
    q, k, v = rand_qkv(rng, 20, 5, 1, 128)
    got, want = p.step(2, 1023, q, k, v)
    a, r = assert_parity(got, want, "config 1")
    k_all, v_all = p.st.read_range(2, 0, 1024)
    f64 = xo.naive_attention_f64(q[0], k_all, v_all, 1023, 20, 5, 128)
    ga, gr = errs(got[0], f64)
    ra, rr = errs(want[0], f64)
    print(f"config1: gpu-vs-oracle abs {a:.2e} rel {r:.2e}; gpu-vs-f64 rel {gr:.2e}; oracle-vs-f64 rel {rr:.2e}")
    assert gr <= 1e-5
    p.st.destroy()


# ---- reference quirks ------------------------------------------------------------------------

def test_chunked_prefill_and_overwrite(ctx2b):
    # chunked prefill (index_pos > 0 with seq_len > 1) and re-append at existing positions
    # (speculative decoding replays positions) are legal in the reference
    rng = np.random.default_rng(17)
    p = Pair(ctx2b, 1024)
    pos = 0
    for S in (100, 57, 1, 200):
        q, k, v = rand_qkv(rng, 20, 5, S, 128)
        got, want = p.step(1, pos, q, k, v)
        assert_parity(got, want, f"chunk at {pos}+{S}")
        pos += S
    q, k, v = rand_qkv(rng, 20, 5, 30, 128)       # overwrite positions 300..329
    got, want = p.step(1, 300, q, k, v)
    assert_parity(got, want, "overwrite")
    p.check_cache(1)
    p.st.destroy()


def test_gap_positions_read_as_zeros(ctx2b):
    # starting at index_pos > 0 on an empty cache: skipped positions are zero rows that still
    # take part in the softmax (the reference never masks them)
    rng = np.random.default_rng(23)
    for _ in range(2):  # second round reuses pages that held other data
        p = Pair(ctx2b, 512)
        q, k, v = rand_qkv(rng, 20, 5, 3, 128)
        got, want = p.step(0, 150, q, k, v)
        assert_parity(got, want, "gap")
        p.check_cache(0)
        junk = rand_qkv(rng, 20, 5, 400, 128)
        p.step(0, 0, *junk)
        p.st.destroy()


def test_ring_fold_matches_oracle():
    # positions beyond the capacity fold with % capacity and overwritten slots are visited again
    rng = np.random.default_rng(29)
    ctx = xn.Context(1, 4, 2, 16, pool_pages=8, prefill_mode=F32)
    p = Pair(ctx, 100)
    pos = 0
    for S in (60, 30, 25, 1, 1, 140):
        q, k, v = rand_qkv(rng, 4, 2, S, 16)
        got, want = p.step(0, pos, q, k, v)
        assert_parity(got, want, f"fold at {pos}+{S}")
        pos += S
    p.check_cache(0)
    ctx.close()


# ---- fused RoPE + append: bit-exact cache, parity of the output ---------------------------------

@pytest.mark.parametrize("theta,D,Hq,Hkv", [(500000.0, 128, 20, 5), (10000.0, 100, 8, 8)])
def test_fused_rope_is_bit_exact(theta, D, Hq, Hkv):
    rng = np.random.default_rng(31)
    cos, sin = xn.rope_tables(theta, D, 1024)
    ctx = xn.Context(1, Hq, Hkv, D, pool_pages=16, rope=(cos, sin), prefill_mode=F32)
    st = ctx.new_stream(1024)
    ref = xo.RingCache(1, Hkv, 1024, D)
    pos = 0
    for S in (90, 1, 1, 45):
        q, k, v = rand_qkv(rng, Hq, Hkv, S, D)
        got = ctx.attention(st, 0, pos, q, k, v, rope=True)
        qr, kr = xo.tensor_rope(q, cos, sin, pos), xo.tensor_rope(k, cos, sin, pos)
        want = xo.fast_attention(qr, kr, v, 0, pos, ref, Hq, Hkv, D)
        assert_parity(got, want, f"rope S={S}")
        pos += S
    kd, vd = st.read_range(0, 0, 1024)
    assert np.array_equal(kd.ravel(), ref.k_buffer(0)), "rotated keys differ in some bit"
    assert np.array_equal(vd.ravel(), ref.v_buffer(0))
    with pytest.raises(xn.XnError) as e:  # position beyond the table
        ctx.attention(st, 0, 1024, *rand_qkv(rng, Hq, Hkv, 1, D), rope=True)
    assert e.value.code == 5
    ctx.close()


def test_rope_entry_needs_tables():
    ctx = xn.Context(1, 2, 2, 8, pool_pages=4)
    st = ctx.new_stream(64)
    rng = np.random.default_rng(1)
    with pytest.raises(xn.XnError) as e:
        ctx.attention(st, 0, 0, *rand_qkv(rng, 2, 2, 1, 8), rope=True)
    assert e.value.code == 8
    ctx.close()


# ---- batches of independent streams (the server's shape), ragged lengths ----------------------

def test_batched_ragged_decode(ctx2b):
    # config-3 shape at reduced stream count: per-stream lengths uniform in [128, 4096] would need
    # a larger pool; lengths here span the same page-count range more sparsely
    rng = np.random.default_rng(37)
    lens = [128, 129, 700, 64, 1, 2000, 333, 65, 1023, 1025, 4, 512]
    pairs = [Pair(ctx2b, 4096) for _ in lens]
    for p, L in zip(pairs, lens):
        if L > 1:
            p.step(1, 0, *rand_qkv(rng, 20, 5, L - 1, 128))
    for step in range(2):
        qs, ks, vs = zip(*[tuple(a for a in rand_qkv(rng, 20, 5, 1, 128)) for _ in lens])
        pos = [L - 1 + step for L in lens]
        outs = ctx2b.attention_batch([p.st for p in pairs], 1, pos, qs, ks, vs)
        wants = xo.fast_attention_streams(qs, ks, vs, 1, pos, [p.ref for p in pairs], 20, 5, 128)
        for i, (g, w) in enumerate(zip(outs, wants)):
            assert_parity(g, w, f"stream {i} len {lens[i]} step {step}")
    for p in pairs:
        p.check_cache(1)
        p.st.destroy()


def test_batch_mixes_prefill_and_decode_and_layers(ctx2b):
    rng = np.random.default_rng(41)
    pairs = [Pair(ctx2b, 1024) for _ in range(4)]
    seqs, layers, poss = [50, 1, 200, 1], [0, 1, 2, 0], [0, 0, 0, 0]
    pairs[3].step(0, 0, *rand_qkv(rng, 20, 5, 77, 128))
    poss[3] = 77
    qkv = [rand_qkv(rng, 20, 5, S, 128) for S in seqs]
    outs = ctx2b.attention_batch([p.st for p in pairs], layers, poss, [a[0] for a in qkv],
                                 [a[1] for a in qkv], [a[2] for a in qkv])
    for i, p in enumerate(pairs):
        want = xo.fast_attention(*qkv[i], layers[i], poss[i], p.ref, 20, 5, 128)
        assert_parity(outs[i], want, f"mixed request {i}")
        p.st.destroy()


def test_seq_major_layout(ctx2b):
    # [S, H*D] in and out: the layouts either side of transpose_seq_to_heads / heads_to_seq
    rng = np.random.default_rng(43)
    p = Pair(ctx2b, 512)
    q, k, v = rand_qkv(rng, 20, 5, 37, 128)
    want = xo.fast_attention(q, k, v, 0, 0, p.ref, 20, 5, 128)
    outs = ctx2b.attention_batch([p.st], 0, [0], [xo.transpose_heads_to_seq(q)],
                                 [xo.transpose_heads_to_seq(k)], [xo.transpose_heads_to_seq(v)],
                                 seq_major=True)
    assert_parity(xo.transpose_seq_to_heads(outs[0], 20, 128), want, "seq-major")
    p.st.destroy()


@pytest.mark.parametrize("out_slab", [False, True])
def test_concurrent_blocking_callers_are_coalesced(out_slab):
    # one thread per stream, each blocking in xn_attention per layer, as the reference's server
    # slots and batch_bench do; results must equal the one-by-one oracle.  The context waits up to
    # 50 ms for all of its live streams to show up, which makes the merge deterministic here.
    # out_slab: the group's outputs are collected in one page-locked slab and leave the device in
    # one transfer (the library does that for groups above 128 KB; forced here for eight callers).
    import os
    import threading

    rng = np.random.default_rng(47)
    n, steps = 8, 6
    if out_slab:
        os.environ["XORNET_ATTN_OUT_DMA_MIN_BYTES"] = "0"
    try:
        ctx = xn.Context(num_layers=3, num_heads=20, num_kv_heads=5, head_dim=128, pool_pages=32,
                         prefill_mode=F32, batch_window_us=50000)
    finally:
        os.environ.pop("XORNET_ATTN_OUT_DMA_MIN_BYTES", None)
    pairs = [Pair(ctx, 512) for _ in range(n)]
    data = [[rand_qkv(rng, 20, 5, 1, 128) for _ in range(steps)] for _ in range(n)]
    got = [[None] * steps for _ in range(n)]
    errors = []
    barrier = threading.Barrier(n)

    def worker(i):
        try:
            for s in range(steps):
                barrier.wait()
                got[i][s] = ctx.attention(pairs[i].st, s % 3, s // 3, *data[i][s])
        except Exception as e:  # pragma: no cover
            errors.append(e)
            barrier.abort()

    ts = [threading.Thread(target=worker, args=(i,)) for i in range(n)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errors, errors
    for i in range(n):
        for s in range(steps):
            want = xo.fast_attention(*data[i][s], s % 3, s // 3, pairs[i].ref, 20, 5, 128)
            assert_parity(got[i][s], want, f"thread {i} step {s}")
    stats = ctx.stats()
    assert stats["coalesced_max"] == n, stats
    assert stats["batches"] == steps, stats   # one merged submission per step
    assert stats["out_transfers"] == (steps if out_slab else 0), stats
    ctx.close()


def test_lone_blocking_caller_is_not_delayed():
    # without a batching window a single caller is served at once; with one, it waits at most
    # that long for company that never comes
    import time

    rng = np.random.default_rng(48)
    ctx = xn.Context(num_layers=1, num_heads=4, num_kv_heads=2, head_dim=16, pool_pages=8,
                     prefill_mode=F32, batch_window_us=30000)
    a, b = ctx.new_stream(64), ctx.new_stream(64)   # two live streams, only one calls
    ctx.attention(a, 0, 0, *rand_qkv(rng, 4, 2, 1, 16))
    t0 = time.perf_counter()
    ctx.attention(a, 0, 1, *rand_qkv(rng, 4, 2, 1, 16))
    dt = time.perf_counter() - t0
    assert 0.02 < dt < 0.5, dt
    ctx.close()


# ---- allocator and error behaviour -----------------------------------------------------------

def test_pool_exhaustion_and_reuse():
    ctx = xn.Context(1, 2, 2, 8, pool_pages=3)
    rng = np.random.default_rng(53)
    a, b = ctx.new_stream(1024), ctx.new_stream(1024)
    ctx.attention(a, 0, 0, *rand_qkv(rng, 2, 2, 128, 8))       # 2 pages
    with pytest.raises(xn.XnError) as e:
        ctx.attention(b, 0, 0, *rand_qkv(rng, 2, 2, 128, 8))   # needs 2, 1 left
    assert e.value.code == 4
    assert ctx.stats()["pages_in_use"] == 2 and b.length(0) == 0   # the refused call took nothing
    a.reset()
    b.reset()
    assert ctx.stats()["pages_in_use"] == 0
    ctx.attention(b, 0, 0, *rand_qkv(rng, 2, 2, 128, 8))
    assert len(set(b.pages().tolist())) == 2
    assert b.length(0) == 128
    a.destroy()
    with pytest.raises(xn.XnError) as e:
        ctx.attention_batch([b, b], 0, [128, 128], *[[rand_qkv(rng, 2, 2, 1, 8)[j]] * 2 for j in range(3)])
    assert e.value.code == 1
    ctx.close()


def test_batch_that_does_not_fit_the_pool_touches_no_stream():
    # the page check covers the whole batch before any stream is given pages or its length moves
    ctx = xn.Context(1, 2, 2, 8, pool_pages=3)
    rng = np.random.default_rng(54)
    a, b = ctx.new_stream(1024), ctx.new_stream(1024)
    qs, ks, vs = zip(*[rand_qkv(rng, 2, 2, 128, 8) for _ in range(2)])
    with pytest.raises(xn.XnError) as e:
        ctx.attention_batch([a, b], 0, [0, 0], qs, ks, vs)     # 2 + 2 pages, 3 in the pool
    assert e.value.code == 4
    assert ctx.stats()["pages_in_use"] == 0
    assert a.length(0) == 0 and b.length(0) == 0 and len(a.pages()) == 0
    p = Pair(ctx, 64)
    got, want = p.step(0, 0, *rand_qkv(rng, 2, 2, 3, 8))       # the context is still good
    assert_parity(got, want, "after a refused batch")
    ctx.close()


def test_submission_refused_after_page_assignment_restores_the_streams():
    # A submission can still be refused after its streams were given pages and their lengths were
    # moved (here: more attention rows than one submission may carry).  It must leave no position
    # claimed that was never written: lengths, page tables and the free list as before, and a
    # later read of those positions returns the reference's zeros.
    Hq, Hkv, D = 8, 8, 4
    os.environ["XORNET_ATTN_F32_TILED"] = "0"     # row-wise exact prefill: one unit per row and KV head
    try:
        ctx = xn.Context(1, Hq, Hkv, D, pool_pages=9500, prefill_mode=F32)
    finally:
        del os.environ["XORNET_ATTN_F32_TILED"]
    rng = np.random.default_rng(55)
    st = ctx.new_stream(1 << 20)
    ctx.attention(st, 0, 0, *rand_qkv(rng, Hq, Hkv, 70, D))
    pages_before, used_before = st.pages().tolist(), ctx.stats()["pages_in_use"]
    S = 600000                      # x 8 KV heads = 4.8 M rows, the limit is 2^22
    big = np.zeros((1, Hq, S, D), np.float32)
    with pytest.raises(xn.XnError) as e:
        ctx.attention(st, 0, 70, big, big, big)
    assert e.value.code == 5 and "attention rows" in e.value.text
    assert st.length(0) == 70
    assert st.pages().tolist() == pages_before
    assert ctx.stats()["pages_in_use"] == used_before
    k, _ = st.read_range(0, 64, 200)
    assert np.all(k[:, 6:] == 0.0)                              # beyond position 70: never written
    p = Pair(ctx, 256)
    got, want = p.step(0, 0, *rand_qkv(rng, Hq, Hkv, 5, D))     # the free list is intact
    assert_parity(got, want, "after a rolled-back submission")
    ctx.close()


def test_one_oversized_caller_does_not_fail_the_callers_merged_with_it():
    # two blocking callers are merged into one submission; one of them asks for more pages than
    # the pool has.  In the reference the calls are independent: only the offender fails.
    import threading

    rng = np.random.default_rng(56)
    ctx = xn.Context(1, 4, 2, 16, pool_pages=4, prefill_mode=F32, batch_window_us=200000)
    good, bad = Pair(ctx, 4096), ctx.new_stream(4096)
    qkv_good = rand_qkv(rng, 4, 2, 100, 16)                      # 2 pages
    qkv_bad = rand_qkv(rng, 4, 2, 64 * 4, 16)                    # 4 pages: 2 + 4 > 4
    res = {}

    def call(name, st, qkv):
        try:
            res[name] = ctx.attention(st, 0, 0, *qkv)
        except xn.XnError as e:
            res[name] = e

    ts = [threading.Thread(target=call, args=("good", good.st, qkv_good)),
          threading.Thread(target=call, args=("bad", bad, qkv_bad))]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert ctx.stats()["coalesced_max"] == 2
    # run one by one, whichever goes first fits and the other may or may not: the small one
    # always fits (2 of 4 pages, or 2 of the 4 - 4 = 0 left ... only when the big one went first)
    ok = [n for n in res if not isinstance(res[n], Exception)]
    assert ok, res
    if "good" in ok:
        want = xo.fast_attention(*qkv_good, 0, 0, good.ref, 4, 2, 16)
        assert_parity(res["good"], want, "the caller that fits")
    failed = [n for n in res if isinstance(res[n], Exception)]
    assert len(failed) == 1 and res[failed[0]].code == 4, res
    ctx.close()


def test_shuffled_page_table_is_a_permutation():
    ctx = xn.Context(1, 2, 2, 8, pool_pages=64, shuffle_seed=99)
    st = ctx.new_stream(64 * 64)
    st.fill_normal(0, 0, 64 * 64, 5)
    pages = st.pages()
    assert sorted(pages.tolist()) == list(range(64)) and pages.tolist() != sorted(pages.tolist())
    k, v = st.read_range(0, 0, 64 * 64)
    assert abs(float(k.mean())) < 0.02 and abs(float(k.std()) - 1.0) < 0.02
    assert abs(float(v.mean())) < 0.02 and not np.array_equal(k, v)
    ctx.close()


def test_pinned_host_buffers_skip_the_staging_copies(ctx2b):
    # XN_REQ_HOST_PINNED: the kernels read q,k,v from and write out to page-locked host memory
    # themselves; results must equal the staged host path bit for bit, for decode and prefill
    import torch

    rng = np.random.default_rng(59)
    lens = [300, 64, 1500, 1]
    pairs = [Pair(ctx2b, 2048) for _ in lens]
    for p, L in zip(pairs, lens):
        if L > 1:
            p.step(2, 0, *rand_qkv(rng, 20, 5, L - 1, 128))
    n = len(lens)
    q = torch.from_numpy(rng.standard_normal((n, 20, 128)).astype(np.float32)).pin_memory()
    k = torch.from_numpy(rng.standard_normal((n, 5, 128)).astype(np.float32)).pin_memory()
    v = torch.from_numpy(rng.standard_normal((n, 5, 128)).astype(np.float32)).pin_memory()
    out = torch.zeros(n, 20, 128).pin_memory()
    before = ctx2b.stats()
    reqs = ctx2b.make_batch([(pairs[i].st, 2, lens[i] - 1, 1, q[i].data_ptr(), k[i].data_ptr(),
                              v[i].data_ptr(), out[i].data_ptr()) for i in range(n)], xn.REQ_HOST_PINNED)
    ctx2b.submit(reqs)
    after = ctx2b.stats()
    assert after["h2d_bytes"] - before["h2d_bytes"] >= n * 30 * 128 * 4   # counted as moved by the kernels
    for i, p in enumerate(pairs):
        want = xo.fast_attention(q[i].numpy().reshape(1, 20, 1, 128), k[i].numpy().reshape(1, 5, 1, 128),
                                 v[i].numpy().reshape(1, 5, 1, 128), 2, lens[i] - 1, p.ref, 20, 5, 128)
        assert_parity(out[i].numpy().reshape(1, 20, 1, 128), want, f"pinned stream {i}")
    # same call again through the staged path at the same positions: identical bits
    staged = ctx2b.attention_batch([p.st for p in pairs], 2, [L - 1 for L in lens],
                                   [q[i].numpy().reshape(1, 20, 1, 128) for i in range(n)],
                                   [k[i].numpy().reshape(1, 5, 1, 128) for i in range(n)],
                                   [v[i].numpy().reshape(1, 5, 1, 128) for i in range(n)])
    for i in range(n):
        assert np.array_equal(staged[i].reshape(20, 128), out[i].numpy())
    # mixing pinned and staged requests in one batch is rejected
    reqs[1].flags = 0
    with pytest.raises(xn.XnError) as e:
        ctx2b.submit(reqs)
    assert e.value.code == 1
    for p in pairs:
        p.st.destroy()


def test_expired_device_wait_is_reported_and_the_context_survives():
    # a kernel-side bounded wait that runs out: the kernel records a status and returns, the host
    # reports XN_ERR_DEVICE_WAIT, and the next call works (nothing is trapped, hung or faulted)
    ctx = xn.Context(1, 4, 2, 16, pool_pages=4, prefill_mode=F32)
    rc = ctx.lib.xn_debug_expire_wait(ctx.handle, 20)
    assert rc == 7
    assert b"bounded wait" in ctx.lib.xn_last_error(ctx.handle)
    assert ctx.stats()["device_wait_errors"] == 1
    assert ctx.lib.xn_debug_expire_wait(ctx.handle, 0) == 1        # argument check
    rng = np.random.default_rng(61)
    p = Pair(ctx, 128)
    got, want = p.step(0, 0, *rand_qkv(rng, 4, 2, 40, 16))
    assert_parity(got, want, "after an expired wait")
    ctx.synchronize()                                              # status word was cleared
    ctx.close()


@pytest.mark.parametrize("Hq,Hkv,D,S,pos", [(20, 5, 128, 333, 0), (8, 8, 100, 200, 70), (4, 2, 7, 150, 5),
                                            (6, 2, 160, 130, 0), (3, 1, 256, 90, 33)])
def test_tiled_exact_prefill_equals_the_row_wise_path(Hq, Hkv, D, S, pos):
    # the tiled exact-f32 prefill kernel and the row-wise path (every query row a decode unit) on
    # the same inputs: both within the f32 bounds of the oracle, caches identical
    rng = np.random.default_rng(900 + D)
    outs = {}
    for tiled in ("1", "0"):
        os.environ["XORNET_ATTN_F32_TILED"] = tiled
        try:
            ctx = xn.Context(1, Hq, Hkv, D, pool_pages=16, shuffle_seed=3, prefill_mode=F32)
        finally:
            del os.environ["XORNET_ATTN_F32_TILED"]
        p = Pair(ctx, 512)
        r2 = np.random.default_rng(901 + D)
        if pos:
            p.step(0, 0, *rand_qkv(r2, Hq, Hkv, pos, D))
        before = ctx.stats()
        got, want = p.step(0, pos, *rand_qkv(r2, Hq, Hkv, S, D))
        after = ctx.stats()
        assert_parity(got, want, f"tiled={tiled} D={D}")
        assert (after["prefill_launches"] - before["prefill_launches"]) == (1 if tiled == "1" else 0)
        p.check_cache(0)
        outs[tiled] = got
        ctx.close()
    a, r = errs(outs["1"], outs["0"])
    assert a <= 1e-4 and r <= 1e-5


def test_free_running_callers_through_pipelined_groups_and_output_slabs():
    """Twelve threads, each decoding its own stream layer by layer with no synchronisation between
    them (the reference's slot threads, server/main.rs:176-199): groups form as callers happen to
    arrive, a group is enqueued behind the one still running, and (forced here for small rows) the
    outputs of a group travel through the alternating page-locked slabs.  Every call must still
    return what the oracle computes for that stream alone."""
    import os
    import threading

    rng = np.random.default_rng(4711)
    n, layers, steps, Hq, Hkv, D = 12, 3, 20, 8, 2, 64
    os.environ["XORNET_ATTN_OUT_DMA_MIN_BYTES"] = "0"
    try:
        ctx = xn.Context(num_layers=layers, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, pool_pages=64)
    finally:
        del os.environ["XORNET_ATTN_OUT_DMA_MIN_BYTES"]
    pairs = [Pair(ctx, 256) for _ in range(n)]
    start = [int(x) for x in rng.integers(0, 100, n)]
    for i, p in enumerate(pairs):   # different histories: a prefill of its own length each
        if start[i]:
            for layer in range(layers):
                q, k, v = rand_qkv(rng, Hq, Hkv, start[i], D)
                p.step(layer, 0, q, k, v)
    data = [[[rand_qkv(rng, Hq, Hkv, 1, D) for _ in range(layers)] for _ in range(steps)] for _ in range(n)]
    got = [[[None] * layers for _ in range(steps)] for _ in range(n)]
    errors = []

    def worker(i):
        try:
            for s in range(steps):
                for layer in range(layers):
                    got[i][s][layer] = ctx.attention(pairs[i].st, layer, start[i] + s, *data[i][s][layer])
        except Exception as e:  # pragma: no cover
            errors.append(e)

    ts = [threading.Thread(target=worker, args=(i,)) for i in range(n)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errors, errors
    for i in range(n):
        for s in range(steps):
            for layer in range(layers):
                want = xo.fast_attention(*data[i][s][layer], layer, start[i] + s, pairs[i].ref, Hq, Hkv, D)
                assert_parity(got[i][s][layer], want, f"thread {i} step {s} layer {layer}")
    stats = ctx.stats()
    assert stats["calls"] >= n * steps * layers and stats["device_wait_errors"] == 0
    print(f"free-running callers: {stats['batches']} batches for {n * steps * layers} calls, "
          f"largest group {stats['coalesced_max']}, {stats['out_transfers']} output transfers")
    ctx.close()
