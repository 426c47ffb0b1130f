"""The tensor-core (tcgen05, TF32) causal prefill kernel against the CPU oracle, through the C ABI.

Tolerance of the TF32 path: relative L2 error <= 5e-3 per output tensor (inputs are truncated to
TF32 by the tensor cores; accumulation is f32).  The cache written by a TF32 prefill is still
exact, so a decode step that follows meets the f32 tolerances.
"""
import numpy as np
import pytest

import oracle as xo
import xor_net_b200 as xn
from gpu_util import Pair, assert_parity, errs, rand_qkv

pytestmark = pytest.mark.gpu
TF32 = 2         # XN_PREFILL_TF32: use the tensor-core kernel for every multi-row call
TF32_REL = 5e-3  # north-star bound for the TF32 prefill path


def check_tf32(got, want, what):
    a, r = errs(got, want)
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    assert r <= TF32_REL, f"{what}: rel {r:.3e} > {TF32_REL}"
    return a, r


@pytest.mark.parametrize("S", [2, 64, 127, 128, 129, 200, 257, 1000])
def test_prefill_lengths_2b_shape(S):
    rng = np.random.default_rng(S)
    ctx = xn.Context(1, 20, 5, 128, pool_pages=40, shuffle_seed=3, prefill_mode=TF32)
    p = Pair(ctx, 2048)
    got, want = p.step(0, 0, *rand_qkv(rng, 20, 5, S, 128))
    a, r = check_tf32(got, want, f"S={S}")
    print(f"S={S}: max abs {a:.2e} rel {r:.2e}")
    assert ctx.stats()["prefill_launches"] == 1
    p.check_cache(0)                        # appended K/V are exact
    q, k, v = rand_qkv(rng, 20, 5, 1, 128)  # decode over the prefilled cache: f32 tolerances
    got, want = p.step(0, S, q, k, v)
    assert_parity(got, want, f"decode after TF32 prefill S={S}")
    ctx.close()


def test_chunked_prefill_with_offset():
    # index_pos > 0 with many rows: the causal diagonal moves by index_pos
    rng = np.random.default_rng(77)
    ctx = xn.Context(2, 20, 5, 128, pool_pages=40, prefill_mode=TF32)
    p = Pair(ctx, 2048)
    pos = 0
    for S in (300, 512, 70, 129):
        got, want = p.step(1, pos, *rand_qkv(rng, 20, 5, S, 128))
        check_tf32(got, want, f"chunk at {pos}+{S}")
        pos += S
    p.check_cache(1)
    ctx.close()


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 32, 100), (8, 2, 64), (4, 4, 32), (6, 2, 96), (3, 1, 16)])
def test_head_dims_and_groups(Hq, Hkv, D):
    rng = np.random.default_rng(D)
    ctx = xn.Context(1, Hq, Hkv, D, pool_pages=24, prefill_mode=TF32)
    p = Pair(ctx, 1024)
    got, want = p.step(0, 0, *rand_qkv(rng, Hq, Hkv, 333, D))
    check_tf32(got, want, f"D={D}")
    got, want = p.step(0, 333, *rand_qkv(rng, Hq, Hkv, 150, D))
    check_tf32(got, want, f"D={D} second chunk")
    ctx.close()


def test_fused_rope_prefill_config2_shape():
    # the 2048-token prefill workload: 2048 tokens, 20/5 heads, head_dim 128, fused RoPE (theta 500000) and
    # append into 64-token pages, causal; output 2048 x 20 x 128
    rng = np.random.default_rng(299792458 + 2000)
    cos, sin = xn.rope_tables(500000.0, 128, 4096)
    ctx = xn.Context(1, 20, 5, 128, pool_pages=40, shuffle_seed=5, rope=(cos, sin))  # AUTO mode
    st = ctx.new_stream(4096)
    ref = xo.RingCache(1, 5, 4096, 128)
    q, k, v = rand_qkv(rng, 20, 5, 2048, 128)
    got = ctx.attention(st, 0, 0, q, k, v, rope=True)
    assert ctx.stats()["prefill_launches"] == 1
    want = xo.fast_attention(xo.tensor_rope(q, cos, sin, 0), xo.tensor_rope(k, cos, sin, 0), v, 0, 0,
                             ref, 20, 5, 128)
    a, r = check_tf32(got, want, "config 2")
    print(f"config2 TF32 prefill: max abs {a:.2e} rel {r:.2e}")
    kd, vd = st.read_range(0, 0, 2048)
    assert np.array_equal(kd.ravel(), ref.k_buffer(0)[: 5 * 4096 * 128].reshape(5, 4096, 128)[:, :2048].ravel())
    ctx.close()


def test_seq_major_prefill():
    rng = np.random.default_rng(5)
    ctx = xn.Context(1, 20, 5, 128, pool_pages=16, prefill_mode=TF32)
    p = Pair(ctx, 512)
    q, k, v = rand_qkv(rng, 20, 5, 300, 128)
    want = xo.fast_attention(q, k, v, 0, 0, p.ref, 20, 5, 128)
    outs = ctx.attention_batch([p.st], 0, [0], [xo.transpose_heads_to_seq(q)],
                               [xo.transpose_heads_to_seq(k)], [xo.transpose_heads_to_seq(v)],
                               seq_major=True)
    check_tf32(xo.transpose_seq_to_heads(outs[0], 20, 128), want, "seq-major TF32")
    ctx.close()


def test_large_scores_trigger_the_lazy_rescale():
    # scores that keep growing along the sequence force accumulator rescales (max jumps > 2^8)
    rng = np.random.default_rng(9)
    Hq, Hkv, D, S = 4, 2, 64, 400
    ctx = xn.Context(1, Hq, Hkv, D, pool_pages=16, prefill_mode=TF32)
    p = Pair(ctx, 512)
    q, k, v = rand_qkv(rng, Hq, Hkv, S, D)
    ramp = np.linspace(0.2, 6.0, S, dtype=np.float32)[None, None, :, None]
    k = (np.abs(k) * ramp).astype(np.float32)
    q = (np.abs(q) * 2.0).astype(np.float32)
    got, want = p.step(0, 0, q, k, v)
    check_tf32(got, want, "rescale")
    ctx.close()


def test_unaligned_device_tensors_fall_back_to_the_exact_path():
    # the tensor-core kernel moves whole 16-byte pieces of q and out; tensors that start off that
    # grid are served by the exact-f32 path instead of being refused
    import torch

    rng = np.random.default_rng(5)
    ctx = xn.Context(1, 4, 2, 64, pool_pages=8, prefill_mode=TF32)
    p = Pair(ctx, 256)
    S = 130
    q, k, v = rand_qkv(rng, 4, 2, S, 64)
    dev = torch.device("cuda:0")
    qd = torch.zeros(q.size + 1, device=dev)
    od = torch.zeros(q.size + 1, device=dev)
    qd[1:] = torch.from_numpy(q.ravel()).to(dev)
    kd, vd = torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev)
    torch.cuda.synchronize()
    assert (qd.data_ptr() + 4) % 16 != 0
    reqs = ctx.make_batch([(p.st, 0, 0, S, qd.data_ptr() + 4, kd.data_ptr(), vd.data_ptr(),
                            od.data_ptr() + 4)], xn.REQ_DEVICE_PTRS)
    ctx.submit(reqs)
    ctx.synchronize()
    assert ctx.stats()["prefill_launches"] == 1      # the tiled exact-f32 kernel: the f32 bounds below hold
    want = xo.fast_attention(q, k, v, 0, 0, p.ref, 4, 2, 64)
    assert_parity(od[1:].cpu().numpy().reshape(q.shape), want, "unaligned device tensors")
    ctx.close()


@pytest.mark.parametrize("Hq,Hkv,D,S,pos", [(20, 5, 128, 700, 0), (8, 2, 64, 333, 130), (4, 4, 128, 129, 64)])
def test_query_rotation_inside_the_kernel_equals_the_rotation_scratch(Hq, Hkv, D, S, pos):
    """For head_dim 64 / 128 the prefill kernel rotates the query rows itself (the append kernel
    then moves K and V only).  Same arithmetic as the append kernel's rotation, so the result must
    equal, bit for bit, the one computed from the rotated scratch copy (rotation in the kernel
    switched off), for head-major and sequence-major rows, and stay within the TF32 bound of the
    oracle (src/tensor.rs:295-316 applied before src/nn/fast_attention.rs:75)."""
    import os
    rng = np.random.default_rng(D + S)
    cos, sin = xn.rope_tables(10000.0, D, 1024)
    q, k, v = rand_qkv(rng, Hq, Hkv, S, D)
    k0, v0 = rand_qkv(rng, Hq, Hkv, pos, D)[1:] if pos else (None, None)
    outs, caches, launches = [], [], []
    for flag in ("1", "0"):
        os.environ["XORNET_ATTN_PREFILL_ROPE_Q"] = flag
        try:
            ctx = xn.Context(1, Hq, Hkv, D, pool_pages=24, shuffle_seed=9, rope=(cos, sin), prefill_mode=TF32)
        finally:
            del os.environ["XORNET_ATTN_PREFILL_ROPE_Q"]
        for seq_major in (False, True):
            st = ctx.new_stream(1024)
            if pos:   # an earlier chunk, so that the rotation uses positions pos..pos+S-1
                ctx.attention(st, 0, 0, rng.standard_normal((1, Hq, pos, D)).astype(np.float32), k0, v0, rope=True)
            before = ctx.stats()["kernel_launches"]
            if seq_major:
                o = ctx.attention_batch([st], 0, [pos], [xo.transpose_heads_to_seq(q)],
                                        [xo.transpose_heads_to_seq(k)], [xo.transpose_heads_to_seq(v)],
                                        seq_major=True, rope=True)[0]
                o = xo.transpose_seq_to_heads(o, Hq, D)
            else:
                o = ctx.attention(st, 0, pos, q, k, v, rope=True)
            launches.append(ctx.stats()["kernel_launches"] - before)
            outs.append(np.asarray(o).reshape(Hq, S, D))
            caches.append(st.read_range(0, 0, pos + S))
        ctx.close()
    assert launches == [2, 2, 2, 2]           # append + prefill either way
    assert np.array_equal(outs[0], outs[2]) and np.array_equal(outs[1], outs[3])
    assert np.array_equal(outs[0], outs[1])
    for kd, vd in caches[1:]:
        assert np.array_equal(kd, caches[0][0]) and np.array_equal(vd, caches[0][1])
    ref = xo.RingCache(1, Hkv, 1024, D)
    if pos:
        ref.append(0, 0, xo.tensor_rope(k0, cos, sin, 0)[0], v0[0])
    want = xo.fast_attention(xo.tensor_rope(q, cos, sin, pos), xo.tensor_rope(k, cos, sin, pos), v, 0, pos,
                             ref, Hq, Hkv, D)
    check_tf32(outs[0], want[0], f"D={D} S={S} pos={pos}")
    ref.close()


def test_several_prompts_share_one_launch():
    """A submission with several tensor-core prefills (a batch of prompts of different lengths, one
    of them a later chunk, on different layers) runs as ONE launch whose blocks are ordered by
    weight across all requests.  Results equal, bit for bit, the ones of one launch per request,
    and match the oracle (src/nn/fast_attention.rs:138-201 per request)."""
    import os
    Hq, Hkv, D = 8, 2, 128
    shapes = [(700, 0, 0), (129, 0, 1), (300, 256, 1), (128, 0, 0)]   # (rows, index_pos, layer)
    rng = np.random.default_rng(4242)
    cos, sin = xn.rope_tables(10000.0, D, 1024)
    qkv = [rand_qkv(rng, Hq, Hkv, S, D) for S, _, _ in shapes]
    first = rand_qkv(rng, Hq, Hkv, 256, D)        # the earlier chunk of the third stream
    outs = {}
    for flag in ("1", "0"):
        os.environ["XORNET_ATTN_PREFILL_MULTI"] = flag
        try:
            ctx = xn.Context(2, Hq, Hkv, D, pool_pages=64, shuffle_seed=11, rope=(cos, sin), prefill_mode=TF32)
        finally:
            del os.environ["XORNET_ATTN_PREFILL_MULTI"]
        sts = [ctx.new_stream(1024) for _ in shapes]
        ctx.attention(sts[2], 1, 0, *first, rope=True)
        before = ctx.stats()["prefill_launches"]
        res = ctx.attention_batch(sts, [l for _, _, l in shapes], [p for _, p, _ in shapes],
                                  [a[0] for a in qkv], [a[1] for a in qkv], [a[2] for a in qkv], rope=True)
        assert ctx.stats()["prefill_launches"] - before == (1 if flag == "1" else len(shapes))
        outs[flag] = res
        if flag == "1":
            for i, (S, pos, layer) in enumerate(shapes):
                ref = xo.RingCache(1, Hkv, 1024, D)
                if pos:
                    ref.append(0, 0, xo.tensor_rope(first[1], cos, sin, 0)[0], first[2][0])
                want = xo.fast_attention(xo.tensor_rope(qkv[i][0], cos, sin, pos), xo.tensor_rope(qkv[i][1], cos, sin, pos),
                                         qkv[i][2], 0, pos, ref, Hq, Hkv, D)
                check_tf32(res[i], want, f"request {i}")
                kd, vd = sts[i].read_range(layer, 0, pos + S)
                assert np.array_equal(kd.ravel(), ref.k_buffer(0).reshape(Hkv, 1024, D)[:, :pos + S].ravel())
                ref.close()
        ctx.close()
    for a, b in zip(outs["1"], outs["0"]):
        assert np.array_equal(a, b)
