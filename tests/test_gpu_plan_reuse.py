"""A decode step submits the same streams at the same positions once per layer.  The library keeps
the plan of such a submission on the device and reuses it for the next one when only the tensors'
addresses and the layer differ.  These tests pin down that a reused plan gives the oracle's result
(src/nn/fast_attention.rs:138-201) and that everything which changes the geometry (a new position,
a reset stream, a layer that needs zero-filling, another set of streams) plans afresh."""
import os

import numpy as np
import pytest
import torch

import oracle as xo
import xor_net_b200 as xn
from gpu_util import assert_parity

pytestmark = pytest.mark.gpu
Hq, Hkv, D, LAYERS = 8, 2, 64, 4


def _oracle_step(sts, layer, pos, q, k, v):
    """The oracle over the bytes the device cache holds for `layer` (new rows included)."""
    want = []
    for i, st in enumerate(sts):
        L = pos[i] + 1
        k_all, v_all = st.read_range(layer, 0, L)
        assert np.array_equal(k_all[:, L - 1], k[i][:, 0]) and np.array_equal(v_all[:, L - 1], v[i][:, 0])
        ref = xo.RingCache(1, Hkv, L, D)
        if L > 1:
            ref.append(0, 0, k_all[:, :L - 1], v_all[:, :L - 1])
        want.append(xo.fast_attention(q[i][None], k[i][None], v[i][None], 0, pos[i], ref, Hq, Hkv, D)[0])
        ref.close()
    return want


def _submit_layer(ctx, sts, layer, pos, gen, pinned=False):
    n = len(sts)
    mk = (lambda *s: torch.randn(*s, generator=gen).pin_memory()) if pinned else \
         (lambda *s: torch.randn(*s, generator=gen).cuda())
    q, k, v = mk(n, Hq, 1, D), mk(n, Hkv, 1, D), mk(n, Hkv, 1, D)
    o = torch.empty(n, Hq, 1, D).pin_memory() if pinned else torch.empty(n, Hq, 1, D, device="cuda")
    b = ctx.make_batch([(sts[i], layer, pos[i], 1, q[i].data_ptr(), k[i].data_ptr(), v[i].data_ptr(),
                         o[i].data_ptr()) for i in range(n)],
                       xn.REQ_HOST_PINNED if pinned else xn.REQ_DEVICE_PTRS)
    ctx.submit(b)
    ctx.synchronize()
    return q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), o.cpu().numpy()


@pytest.mark.parametrize("pinned", [False, True])
def test_layers_of_a_step_reuse_the_plan_and_match_the_oracle(pinned):
    lens = [130, 64, 1, 257, 700, 65]
    ctx = xn.Context(LAYERS, Hq, Hkv, D, pool_pages=64)
    sts = [ctx.new_stream(1024) for _ in lens]
    for i, st in enumerate(sts):
        if lens[i] > 1:
            st.fill_normal(-1, 0, lens[i] - 1, 1234 + i)
    gen = torch.Generator().manual_seed(7)
    reuses = 0
    for step in range(2):
        pos = [L - 1 + step for L in lens]
        for layer in range(LAYERS):
            q, k, v, o = _submit_layer(ctx, sts, layer, pos, gen, pinned)
            for i, w in enumerate(_oracle_step(sts, layer, pos, q, k, v)):
                assert_parity(o[i], w, f"step {step} layer {layer} stream {i}")
            if layer > 0:
                reuses += 1
            assert ctx.stats()["plan_reuses"] == reuses, (step, layer)
    # one launch per layer, reused plan or not (the append is inside the attention kernel)
    assert ctx.stats()["decode_launches"] == 2 * LAYERS
    assert [st.length(l) for st in sts for l in range(LAYERS)] == [L + 1 for L in lens for _ in range(LAYERS)]
    ctx.close()


def test_what_changes_the_geometry_plans_afresh():
    lens = [200, 90, 333]
    ctx = xn.Context(LAYERS, Hq, Hkv, D, pool_pages=64)
    sts = [ctx.new_stream(1024) for _ in lens]
    for i, st in enumerate(sts):
        for layer in range(LAYERS - 1):          # the last layer stays empty: its rows read as zeros
            st.fill_normal(layer, 0, lens[i] - 1, 99 + i)
    gen = torch.Generator().manual_seed(11)
    pos = [L - 1 for L in lens]

    def check(layer, sts_, pos_, expect_reuse):
        before = ctx.stats()["plan_reuses"]
        q, k, v, o = _submit_layer(ctx, sts_, layer, pos_, gen)
        for i, w in enumerate(_oracle_step(sts_, layer, pos_, q, k, v)):
            assert_parity(o[i], w, f"layer {layer} stream {i}")
        assert ctx.stats()["plan_reuses"] - before == (1 if expect_reuse else 0), (layer, expect_reuse)

    check(0, sts, pos, False)
    check(1, sts, pos, True)
    check(3, sts, pos, False)            # never written below `pos`: zero-fill first, so no reuse
    check(2, sts, pos, False)            # the zero-filling submission was not kept
    check(2, sts, pos, True)             # the same layer again (an overwrite at the same position)
    check(1, sts[:2], pos[:2], False)    # fewer streams
    check(2, sts[:2], pos[:2], True)
    ctx.drop_plan()
    check(1, sts[:2], pos[:2], False)    # dropped by hand (xn_debug_drop_plan)
    check(2, sts[:2], pos[:2], True)
    check(0, [sts[1], sts[0]], [pos[1], pos[0]], False)   # another order
    sts[0].reset()
    sts[0].fill_normal(-1, 0, 5, 5)
    check(1, [sts[1], sts[0]], [pos[1], 5], False)        # a reset stream
    check(2, [sts[1], sts[0]], [pos[1], 5], True)
    check(3, [sts[1], sts[0]], [pos[1] + 1, 6], False)    # the next token
    ctx.close()


def test_reuse_can_be_switched_off_and_changes_no_bit():
    outs = []
    for flag in ("1", "0"):
        os.environ["XORNET_ATTN_PLAN_REUSE"] = flag
        try:
            ctx = xn.Context(LAYERS, Hq, Hkv, D, pool_pages=64)
        finally:
            del os.environ["XORNET_ATTN_PLAN_REUSE"]
        sts = [ctx.new_stream(512) for _ in range(5)]
        for i, st in enumerate(sts):
            st.fill_normal(-1, 0, 100 + 37 * i, 4321 + i)
        gen = torch.Generator().manual_seed(3)
        res = [_submit_layer(ctx, sts, layer, [100 + 37 * i for i in range(5)], gen)[3] for layer in range(LAYERS)]
        assert ctx.stats()["plan_reuses"] == (LAYERS - 1 if flag == "1" else 0)
        outs.append(np.stack(res))
        ctx.close()
    assert np.array_equal(outs[0], outs[1])


def test_page_locked_outputs_back_to_back_or_scattered_give_the_same_bits():
    """Outputs of page-locked callers that form one run of host memory are produced in a device
    buffer and copied home in one transfer; scattered outputs are stored by the kernel directly.
    Same bits either way, with and without plan reuse, and the oracle's result."""
    lens = [100, 65, 400, 31, 257]
    n = len(lens)
    pos = [L - 1 for L in lens]
    results = []
    for scattered in (False, True):
        os.environ["XORNET_ATTN_OUT_DMA_MIN_BYTES"] = "0"     # small rows here: take the transfer at any size
        try:
            ctx = xn.Context(LAYERS, Hq, Hkv, D, pool_pages=64)
        finally:
            del os.environ["XORNET_ATTN_OUT_DMA_MIN_BYTES"]
        sts = [ctx.new_stream(512) for _ in lens]
        for i, st in enumerate(sts):
            st.fill_normal(-1, 0, lens[i] - 1, 600 + i)
        gen = torch.Generator().manual_seed(21)
        outs = []
        for layer in range(LAYERS):
            q = torch.randn(n, Hq, 1, D, generator=gen).pin_memory()
            k = torch.randn(n, Hkv, 1, D, generator=gen).pin_memory()
            v = torch.randn(n, Hkv, 1, D, generator=gen).pin_memory()
            width = Hq * D + (48 if scattered else 0)          # a gap between two requests' outputs
            o = torch.full((n, width), 7.0).pin_memory()
            b = ctx.make_batch([(sts[i], layer, pos[i], 1, q[i].data_ptr(), k[i].data_ptr(), v[i].data_ptr(),
                                 o[i].data_ptr()) for i in range(n)], xn.REQ_HOST_PINNED)
            ctx.submit(b)
            got = o[:, :Hq * D].numpy().reshape(n, Hq, 1, D).copy()
            assert scattered is False or bool((o[:, Hq * D:] == 7.0).all())    # the gaps stay untouched
            for i, w in enumerate(_oracle_step(sts, layer, pos, q.numpy(), k.numpy(), v.numpy())):
                assert_parity(got[i], w, f"scattered={scattered} layer {layer} stream {i}")
            outs.append(got)
        assert ctx.stats()["plan_reuses"] == LAYERS - 1
        assert ctx.stats()["out_transfers"] == (0 if scattered else LAYERS)
        results.append(np.stack(outs))
        ctx.close()
    assert np.array_equal(results[0], results[1])
