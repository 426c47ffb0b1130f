"""Device groups: one context per GPU behind one handle, streams placed by load, blocking callers
of different devices served in parallel.  The placement and bookkeeping run on any number of GPUs;
the cross-device cases skip below two."""
import threading

import numpy as np
import pytest

import oracle as xo
import xor_net_b200 as xn
from gpu_util import assert_parity, rand_qkv

pytestmark = pytest.mark.gpu


def n_devices():
    import torch

    return torch.cuda.device_count()


def test_group_on_one_device_places_and_attends():
    g = xn.Group(2, 4, 2, 16, devices=[0], pool_pages=16, prefill_mode=1)
    assert len(g) == 1
    rng = np.random.default_rng(3)
    sts = [g.new_stream(128, expected_tokens=10 * (i + 1)) for i in range(3)]
    assert all(st.ctx is g.contexts[0] for st in sts)
    ref = xo.RingCache(2, 2, 128, 16)
    q, k, v = rand_qkv(rng, 4, 2, 9, 16)
    got = sts[1].ctx.attention(sts[1], 1, 0, q, k, v)
    assert_parity(got, xo.fast_attention(q, k, v, 1, 0, ref, 4, 2, 16), "group stream")
    assert g.contexts[0].stats()["streams_live"] == 3
    g.close()


def test_default_group_backs_the_reference_style_cache():
    xn.close_default_contexts()
    cache = xn.DeviceKvCache.new(1, 2, 64, 8)
    rng = np.random.default_rng(4)
    q, k, v = rand_qkv(rng, 2, 2, 5, 8)
    out = xn.fast_attention(xn.FastTensor(q, q.shape), xn.FastTensor(k, k.shape), xn.FastTensor(v, v.shape), 0, 0,
                            cache, 2, 2, 8)
    ref = xo.RingCache(1, 2, 64, 8)
    assert_parity(out.array(), xo.fast_attention(q, k, v, 0, 0, ref, 2, 2, 8), "default group")
    assert cache.device is not None
    cache.close()
    xn.close_default_contexts()


@pytest.mark.skipif("n_devices() < 2")
def test_streams_spread_over_devices_and_callers_run_in_parallel():
    nd = min(n_devices(), 4)
    g = xn.Group(1, 4, 2, 16, devices=list(range(nd)), pool_pages=32, prefill_mode=1)
    lens = [300, 40, 200, 150, 90, 260, 30, 120]
    sts = [g.new_stream(512, expected_tokens=L) for L in lens]
    by_dev = {}
    for st, L in zip(sts, lens):
        by_dev.setdefault(st.ctx.device, []).append(L)
    assert len(by_dev) == nd                                  # every device got streams
    loads = [sum(v) for v in by_dev.values()]
    assert max(loads) - min(loads) <= max(lens)               # least-loaded placement
    rr = [g.new_stream(64, policy=xn.PLACE_ROUND_ROBIN) for _ in range(nd)]
    assert sorted(st.ctx.device for st in rr) == list(range(nd))
    # one blocking caller per stream, all at once: each device's queue serves its own callers
    rng = np.random.default_rng(5)
    data = [rand_qkv(rng, 4, 2, L, 16) for L in lens]
    got, errors = [None] * len(sts), []

    def worker(i):
        try:
            got[i] = sts[i].ctx.attention(sts[i], 0, 0, *data[i])
        except Exception as e:  # pragma: no cover
            errors.append(e)

    ts = [threading.Thread(target=worker, args=(i,)) for i in range(len(sts))]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errors, errors
    for i, L in enumerate(lens):
        ref = xo.RingCache(1, 2, 512, 16)
        assert_parity(got[i], xo.fast_attention(*data[i], 0, 0, ref, 4, 2, 16), f"stream {i} on device {sts[i].ctx.device}")
    assert sum(c.stats()["calls"] for c in g.contexts) == len(sts)
    g.close()
