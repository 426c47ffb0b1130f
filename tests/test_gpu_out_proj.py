"""The attention output block on the device (sub-norm + i8 quantiser + ternary o_proj) against the
CPU oracle, through the C ABI.

Bars: given the same input rows the block is BIT-EXACT (integer dot products; the float steps keep
the reference's order of operations, AVX-512 quantiser body).  Fused behind attention the input
rows themselves carry the f32 attention tolerance, so one quantisation step of one activation may
flip; the fused result is therefore checked (a) bit-exactly against the oracle block applied to
the device's own attention output and (b) against the all-oracle chain with a relative L2 bound of
1e-3 per output tensor (measured: 1.1e-4).
"""
import numpy as np
import pytest

import oracle as xo
import xor_net_b200 as xn
from gpu_util import Pair, errs, rand_qkv

pytestmark = pytest.mark.gpu
CHAIN_REL = 1e-3


@pytest.fixture(autouse=True)
def avx512_quantiser():
    xo.set_quant_body(1)   # the body the device restates, whatever this host's CPU is
    yield
    xo.set_quant_body(-1)


def make_block(rng, Hq, D, out_dim, pack, norm=True, scale=None):
    in_dim = Hq * D
    w = rng.standard_normal((out_dim, in_dim)).astype(np.float32)
    dev = xn.TernaryLinear(in_dim, out_dim, w, pack, scale)
    ref = xo.TernaryLinear(in_dim, out_dim, w, pack, scale)
    assert np.array_equal(dev.packed[:ref.packed.size], ref.packed) and np.array_equal(dev.w_scales, ref.w_scales)
    nw = (1.0 + 0.2 * rng.standard_normal(in_dim)).astype(np.float32) if norm else None
    return dev, ref, nw


def ref_block(ref, nw, eps, y):
    x = xo.tensor_rmsnorm(y, nw, eps) if nw is not None else np.asarray(y, np.float32)
    return ref.forward(x)


@pytest.mark.parametrize("Hq,D,out_dim,pack,norm,rows", [
    (20, 128, 2560, xn.PACK4, True, 64),    # the 2B shape, one decode batch
    (20, 128, 2560, xn.PACK5, True, 3),
    (32, 128, 96, xn.PACK4, True, 70),      # in_dim 4096: four activation chunks, two row tiles
    (4, 8, 12, xn.PACK5, False, 5),
    (3, 10, 7, xn.PACK4, True, 9),          # in_dim 30: a 14-element tail that rounds half away
    (1, 3, 1, xn.PACK5, True, 1),
])
def test_block_alone_is_bit_exact(Hq, D, out_dim, pack, norm, rows):
    rng = np.random.default_rng(Hq * 1000 + D + out_dim)
    ctx = xn.Context(2, Hq, 1, D, pool_pages=2)
    dev, ref, nw = make_block(rng, Hq, D, out_dim, pack, norm)
    ctx.set_out_proj(1, dev, nw, 1e-5)
    y = (rng.standard_normal((rows, Hq * D)) * rng.uniform(0.1, 3.0, (rows, 1))).astype(np.float32)
    got = ctx.out_proj(1, y)
    want = ref_block(ref, nw, 1e-5, y)
    assert np.array_equal(got, want), f"max diff {np.max(np.abs(got - want))}"
    assert ctx.stats()["out_proj_rows"] == rows
    ctx.close()


@pytest.mark.parametrize("rows", [1, 64, 65, 128, 129, 300, 700])
def test_tensor_core_and_cuda_core_projections_agree(rows, monkeypatch):
    # the tcgen05 (kind::i8) kernel and the dp4a kernel compute the same integers; token tiles of
    # 64 / 128 / 256 rows, ragged last tile, output rows that do not fill the last 128-row block
    rng = np.random.default_rng(rows)
    Hq, D, out_dim = 6, 64, 200
    dev, ref, nw = make_block(rng, Hq, D, out_dim, xn.PACK4)
    y = rng.standard_normal((rows, Hq * D)).astype(np.float32)
    outs = []
    for tc in ("1", "0"):
        monkeypatch.setenv("XORNET_ATTN_OUTPROJ_TC", tc)
        ctx = xn.Context(1, Hq, 1, D, pool_pages=1)
        ctx.set_out_proj(0, dev, nw, 1e-5)
        outs.append(ctx.out_proj(0, y))
        ctx.close()
    assert np.array_equal(outs[0], outs[1])
    assert np.array_equal(outs[0], ref_block(ref, nw, 1e-5, y))


def test_sparse_representation_gives_the_dense_results():
    # XN_SPARSE: the XorSparse blob of TernaryRep::Sparse is decoded on upload; lossless, so the
    # projected rows equal the pack4 layer's bit for bit (and the oracle's)
    rng = np.random.default_rng(77)
    Hq, D, out_dim, rows = 20, 128, 200, 70
    w = rng.standard_normal((out_dim, Hq * D)).astype(np.float32)
    nw = (1.0 + 0.2 * rng.standard_normal(Hq * D)).astype(np.float32)
    y = rng.standard_normal((rows, Hq * D)).astype(np.float32)
    outs = []
    for pack in (xn.SPARSE, xn.PACK4):
        ctx = xn.Context(1, Hq, 1, D, pool_pages=1)
        ctx.set_out_proj(0, xn.TernaryLinear(Hq * D, out_dim, w, pack), nw, 1e-5)
        outs.append(ctx.out_proj(0, y))
        ctx.close()
    assert np.array_equal(outs[0], outs[1])
    ref = xo.TernaryLinear(Hq * D, out_dim, w, xo.SPARSE)
    assert np.array_equal(outs[0], ref.forward(xo.tensor_rmsnorm(y, nw, 1e-5)))
    # a blob whose rows describe another width is refused
    ctx = xn.Context(1, Hq, 1, D, pool_pages=1)
    bad = xn.TernaryLinear(Hq * D, out_dim, w, xn.SPARSE)
    bad.packed = xn.TernaryLinear(64, out_dim, w[:, :64].copy(), xn.SPARSE).packed
    with pytest.raises(xn.XnError) as e:
        ctx.set_out_proj(0, bad, nw, 1e-5)
    assert e.value.code == 2
    ctx.close()


def test_rounding_ties_follow_the_avx512_body():
    # rows whose scale is exactly 1 (max |x| = 127) with values on .5: whole chunks round to even,
    # the tail rounds half away from zero; an all-zero row has scale 1 and gives zeros
    ctx = xn.Context(1, 1, 1, 40, pool_pages=1)
    w = np.zeros((40, 40), np.float32)
    np.fill_diagonal(w, 1.0)                      # identity: output o = quantised activation o
    lin = xn.TernaryLinear(40, 40, w, xn.PACK4)
    ctx.set_out_proj(0, lin, None, 0.0)
    y = np.zeros((3, 40), np.float32)
    y[0, 0] = 127.0
    y[0, 1:6] = [0.5, 1.5, 2.5, -0.5, -1.5]       # inside whole 16-element chunks
    y[0, 33:38] = [0.5, 1.5, 2.5, -0.5, -1.5]     # tail (40 = 2*16 + 8)
    y[1, :] = 0.0
    y[2, 5] = -3.0
    got = ctx.out_proj(0, y)
    assert got[0, 0] == 127.0
    assert got[0, 1:6].tolist() == [0.0, 2.0, 2.0, -0.0, -2.0]
    assert got[0, 33:38].tolist() == [1.0, 2.0, 3.0, -1.0, -2.0]
    assert not got[1].any()
    assert got[2, 5] == np.float32(-127.0) * (np.float32(3.0) / np.float32(127.0))
    want = xo.TernaryLinear(40, 40, w, xo.PACK4).forward(y)
    assert np.array_equal(got, want)
    ctx.close()


def test_device_pointers_and_replacing_a_block():
    import torch

    rng = np.random.default_rng(9)
    ctx = xn.Context(1, 4, 2, 16, pool_pages=2)
    dev, ref, nw = make_block(rng, 4, 16, 24, xn.PACK4)
    ctx.set_out_proj(0, dev, nw, 1e-6)
    y = rng.standard_normal((10, 64)).astype(np.float32)
    yd = torch.from_numpy(y).cuda()
    od = torch.zeros(10, 24, device="cuda")
    torch.cuda.synchronize()
    ctx._check(ctx.lib.xn_out_proj(ctx.handle, 0, 10, yd.data_ptr(), od.data_ptr(), xn.REQ_DEVICE_PTRS))
    ctx.synchronize()
    assert np.array_equal(od.cpu().numpy(), ref_block(ref, nw, 1e-6, y))
    dev2, ref2, _ = make_block(rng, 4, 16, 8, xn.PACK5, norm=False)
    ctx.set_out_proj(0, dev2, None, 0.0)            # replace: other width, other packing, no norm
    assert np.array_equal(ctx.out_proj(0, y), ref2.forward(y))
    ctx.close()


def test_errors():
    ctx = xn.Context(2, 4, 2, 16, pool_pages=2)
    st = ctx.new_stream(64)
    rng = np.random.default_rng(1)
    q, k, v = rand_qkv(rng, 4, 2, 1, 16)
    ctx._out_dims = {0: 8}
    with pytest.raises(xn.XnError) as e:                         # no block on that layer
        ctx.attention_batch([st], 0, [0], [q], [k], [v], out_proj=True)
    assert e.value.code == 1
    with pytest.raises(xn.XnError) as e:
        ctx.out_proj(0, np.zeros((1, 64), np.float32))
    assert e.value.code == 1
    bad = xn.TernaryLinear(48, 8, np.zeros((8, 48), np.float32))
    with pytest.raises(xn.XnError) as e:                         # in_dim must be heads * head_dim
        ctx.set_out_proj(0, bad)
    assert e.value.code == 2 and "Input dimension mismatch" in str(e.value)
    assert st.length(0) == 0
    ctx.close()


@pytest.mark.parametrize("pack", [xn.PACK4, xn.PACK5])
def test_fused_behind_decode_and_prefill(pack):
    rng = np.random.default_rng(21 + pack)
    Hq, Hkv, D, out_dim = 20, 5, 128, 2560
    ctx = xn.Context(2, Hq, Hkv, D, pool_pages=40, shuffle_seed=5, prefill_mode=1)  # exact-f32 prefill
    dev, ref, nw = make_block(rng, Hq, D, out_dim, pack)
    ctx.set_out_proj(1, dev, nw, 1e-5)
    lens = [1, 70, 300, 513]
    pairs = [Pair(ctx, 1024) for _ in lens]
    worst = 0.0
    # prefill (S rows) through the fused path, then one decode step each, batched
    for p, L in zip(pairs, lens):
        q, k, v = rand_qkv(rng, Hq, Hkv, L, D)
        fused = ctx.attention_batch([p.st], 1, [0], [q], [k], [v], out_proj=True)[0]
        plain, want_attn = p.step(1, 0, q, k, v)                 # same position again: same cache, same output
        assert np.array_equal(fused, xo.attention_out_block(plain, nw, 1e-5, ref)), f"prefill L={L}"
        chain = xo.attention_out_block(want_attn, nw, 1e-5, ref)
        if L == 1:
            assert np.array_equal(fused, chain)                  # one key: softmax weight is exactly 1
        worst = max(worst, errs(fused, chain)[1])
    qs, ks, vs = zip(*[rand_qkv(rng, Hq, Hkv, 1, D) for _ in lens])
    fused = ctx.attention_batch([p.st for p in pairs], 1, lens, qs, ks, vs, out_proj=True)
    assert ctx.stats()["decode_launches"] >= 1
    for i, p in enumerate(pairs):
        plain, want_attn = p.step(1, lens[i], qs[i], ks[i], vs[i])
        assert np.array_equal(fused[i], xo.attention_out_block(plain, nw, 1e-5, ref)), f"decode {i}"
        worst = max(worst, errs(fused[i], xo.attention_out_block(want_attn, nw, 1e-5, ref))[1])
        p.check_cache(1)
    print(f"fused vs all-oracle chain: worst rel {worst:.2e}")
    assert worst <= CHAIN_REL
    ctx.close()


def test_fused_behind_tf32_prefill_rope_seq_major_and_mixed_batch():
    rng = np.random.default_rng(33)
    Hq, Hkv, D, out_dim = 8, 2, 64, 40
    cos, sin = xn.rope_tables(10000.0, D, 512)
    ctx = xn.Context(3, Hq, Hkv, D, pool_pages=30, rope=(cos, sin), prefill_mode=2)  # TF32 prefill
    blocks = {}
    for layer, pack in ((0, xn.PACK4), (2, xn.PACK5)):
        dev, ref, nw = make_block(rng, Hq, D, out_dim + layer, pack)
        ctx.set_out_proj(layer, dev, nw, 1e-5)
        blocks[layer] = (ref, nw)
    a, b, c3 = ctx.new_stream(512), ctx.new_stream(512), ctx.new_stream(512)
    S = 200
    mk = lambda s: (rng.standard_normal((1, s, Hq * D)).astype(np.float32),
                    rng.standard_normal((1, s, Hkv * D)).astype(np.float32),
                    rng.standard_normal((1, s, Hkv * D)).astype(np.float32))
    ins = [mk(S), mk(1), mk(S)]
    outs = [np.empty((1, S, out_dim), np.float32), np.empty((1, 1, Hq * D), np.float32),
            np.empty((1, S, out_dim + 2), np.float32)]
    f = xn.REQ_ROPE | xn.REQ_SEQ_MAJOR
    ptr = lambda x: x.ctypes.data
    reqs = ctx.make_batch([(a, 0, 0, S, ptr(ins[0][0]), ptr(ins[0][1]), ptr(ins[0][2]), ptr(outs[0])),
                           (b, 1, 0, 1, ptr(ins[1][0]), ptr(ins[1][1]), ptr(ins[1][2]), ptr(outs[1])),
                           (c3, 2, 0, S, ptr(ins[2][0]), ptr(ins[2][1]), ptr(ins[2][2]), ptr(outs[2]))], f)
    reqs[0].flags |= xn.REQ_OUT_PROJ
    reqs[2].flags |= xn.REQ_OUT_PROJ
    ctx.submit(reqs)
    assert ctx.stats()["prefill_launches"] == 1 and ctx.stats()["out_proj_rows"] == 2 * S   # both prompts in one launch
    for i, layer, st in ((0, 0, a), (2, 2, c3)):
        ref, nw = blocks[layer]
        plain = ctx.attention_batch([st], layer, [0], [ins[i][0]], [ins[i][1]], [ins[i][2]], rope=True,
                                    seq_major=True)[0]                       # [1, S, Hq*D]
        want = ref.forward(xo.tensor_rmsnorm(plain, nw, 1e-5))
        assert np.array_equal(outs[i], want), f"request {i}"
    # the unflagged request of the batch got plain attention output
    q = xo.tensor_rope(xo.transpose_seq_to_heads(ins[1][0], Hq, D), cos, sin, 0)
    assert np.allclose(outs[1], xo.transpose_heads_to_seq(
        xo.transpose_seq_to_heads(ins[1][2], Hkv, D).repeat(Hq // Hkv, axis=1)), atol=1e-6)
    assert q.shape == (1, Hq, 1, D)
    ctx.close()


def test_fused_with_pinned_host_tensors():
    import torch

    rng = np.random.default_rng(44)
    Hq, Hkv, D, out_dim = 20, 5, 128, 2560
    ctx = xn.Context(1, Hq, Hkv, D, pool_pages=20)
    dev, ref, nw = make_block(rng, Hq, D, out_dim, xn.PACK4)
    ctx.set_out_proj(0, dev, nw, 1e-5)
    lens = [130, 1, 64]
    pairs = [Pair(ctx, 512) for _ in lens]
    for p, L in zip(pairs, lens):
        p.step(0, 0, *rand_qkv(rng, Hq, Hkv, L, D))
    n = len(lens)
    q = torch.from_numpy(rng.standard_normal((n, Hq, D)).astype(np.float32)).pin_memory()
    k = torch.from_numpy(rng.standard_normal((n, Hkv, D)).astype(np.float32)).pin_memory()
    v = torch.from_numpy(rng.standard_normal((n, Hkv, D)).astype(np.float32)).pin_memory()
    out = torch.zeros(n, out_dim).pin_memory()
    reqs = ctx.make_batch([(pairs[i].st, 0, lens[i], 1, q[i].data_ptr(), k[i].data_ptr(), v[i].data_ptr(),
                            out[i].data_ptr()) for i in range(n)], xn.REQ_HOST_PINNED | xn.REQ_OUT_PROJ)
    ctx.submit(reqs)
    for i, p in enumerate(pairs):
        plain, _ = p.step(0, lens[i], q[i].numpy().reshape(1, Hq, 1, D), k[i].numpy().reshape(1, Hkv, 1, D),
                          v[i].numpy().reshape(1, Hkv, 1, D))
        assert np.array_equal(out[i].numpy().reshape(1, 1, out_dim), xo.attention_out_block(plain, nw, 1e-5, ref))
    ctx.close()
