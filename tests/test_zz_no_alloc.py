"""The allocation-free decode entry point against the regular one, through the C ABI.

Why the entry point exists: a caller may be barred from cudaMalloc -- its serving loop gave all
device memory to its own arena, or it sits on a latency-critical thread where an allocation's
implicit device-wide synchronisation is not acceptable.  ``xn_decode_attention_static`` keeps its
split-KV scratch in a fixed array inside the library image and takes caller-owned device buffers.

This file sorts last on purpose so a run that stops at the first failure has already run every
other test.  It passes alone in a fresh process and after the rest of the suite: it builds its
own context, and the static scratch needs no particular starting contents.
"""
import ctypes as C

import numpy as np
import pytest

import oracle as xo
import xor_net_b200 as xn
from gpu_util import ABS_TOL, REL_TOL, assert_parity, rand_qkv

pytestmark = pytest.mark.gpu


def static_decode(lib, torch, q, k_all, v_all, Hq, Hkv, D, kv_len, pad):
    """Runs the entry point on caller-owned device tensors; caches are [Hkv, kv_len + pad, D]."""
    cap = kv_len + pad
    kc = torch.zeros(Hkv, cap, D, device="cuda")
    vc = torch.zeros(Hkv, cap, D, device="cuda")
    kc[:, :kv_len] = torch.from_numpy(k_all).cuda()
    vc[:, :kv_len] = torch.from_numpy(v_all).cuda()
    qd = torch.from_numpy(np.ascontiguousarray(q.reshape(Hq, D))).cuda()
    out = torch.empty(Hq, D, device="cuda")
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    rc = lib.xn_decode_attention_static(qd.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(),
                                        Hq, Hkv, D, kv_len, cap,
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.xn_last_error(None)
    torch.cuda.synchronize()
    return out.cpu().numpy().reshape(1, Hq, 1, D), free0 - torch.cuda.mem_get_info()[0]


@pytest.mark.parametrize("Hq,Hkv,D,L0", [(20, 5, 128, 1023), (8, 8, 100, 300), (4, 2, 8, 5)])
def test_static_entry_matches_regular_entry_twice(Hq, Hkv, D, L0):
    import torch

    lib = xn.load()
    rng = np.random.default_rng(1000 + D)
    ctx = xn.Context(1, Hq, Hkv, D, pool_pages=40, prefill_mode=1)
    st = ctx.new_stream(2048)
    ctx.attention(st, 0, 0, *rand_qkv(rng, Hq, Hkv, L0, D))  # fill the cache
    grown = []
    for call in range(2):  # two calls in a row, different inputs and lengths
        pos = L0 + call
        q, k, v = rand_qkv(rng, Hq, Hkv, 1, D)
        want = ctx.attention(st, 0, pos, q, k, v)            # the existing entry point
        k_all, v_all = st.read_range(0, 0, pos + 1)           # cache including the new token
        got, used = static_decode(lib, torch, q, k_all, v_all, Hq, Hkv, D, pos + 1, pad=37 * call)
        assert_parity(got, want, f"static call {call}", ABS_TOL, REL_TOL)
        # ... and against the CPU oracle run over the same cached bytes
        ref = xo.RingCache(1, Hkv, pos + 1, D)
        ref.append(0, 0, k_all[:, :pos], v_all[:, :pos])
        cpu = xo.fast_attention(q, k, v, 0, pos, ref, Hq, Hkv, D)
        assert_parity(got, cpu, f"static call {call} vs oracle", ABS_TOL, REL_TOL)
        ref.close()
        grown.append(used)
    assert grown[1] == 0, "the second call changed the amount of free device memory"
    ctx.close()


@pytest.mark.parametrize("Hq,Hkv,D,L", [
    (1, 1, 8, 177601),     # 592 splits of 301 tokens: the last split starts past kv_len (empty record)
    (8, 2, 256, 3000),     # the widest row the scratch takes
    (600, 300, 16, 700),   # so many heads that the record budget leaves one split per head
])
def test_static_entry_split_limits_against_the_oracle(Hq, Hkv, D, L):
    """The split-count caps (records per call, blocks per launch), an empty trailing split and
    head_dim 256, on dense caller-owned caches, two calls in a row; the checker is the CPU oracle."""
    import torch

    lib = xn.load()
    rng = np.random.default_rng(7 * D + Hq)
    k_all = rng.standard_normal((Hkv, L, D)).astype(np.float32)
    v_all = rng.standard_normal((Hkv, L, D)).astype(np.float32)
    ref = xo.RingCache(1, Hkv, L, D)
    ref.append(0, 0, k_all[:, :L - 1], v_all[:, :L - 1])
    for call in range(2):
        q = rng.standard_normal((1, Hq, 1, D)).astype(np.float32)
        want = xo.fast_attention(q, k_all[None, :, L - 1:L], v_all[None, :, L - 1:L], 0, L - 1, ref, Hq, Hkv, D)
        got, used = static_decode(lib, torch, q, k_all, v_all, Hq, Hkv, D, L, pad=5 * call)
        assert_parity(got, want, f"static call {call}", ABS_TOL, REL_TOL)
        if call:
            assert used == 0, "the second call changed the amount of free device memory"
    ref.close()


def test_static_entry_rejects_sizes_beyond_its_scratch():
    import torch

    lib = xn.load()
    buf = torch.zeros(4096, device="cuda")
    p = buf.data_ptr()
    assert lib.xn_decode_attention_static(p, p, p, p, 4, 2, 257, 4, 4, None) == 5
    assert b"head_dim 257" in lib.xn_last_error(None)
    assert lib.xn_decode_attention_static(p, p, p, p, 2048, 2048, 1, 1, 1, None) == 5
    assert b"partial records" in lib.xn_last_error(None)
    assert lib.xn_decode_attention_static(p, p, p, p, 4, 2, 8, 9, 8, None) == 1   # kv_len > capacity
    assert lib.xn_decode_attention_static(None, p, p, p, 4, 2, 8, 4, 8, None) == 1
    assert lib.xn_decode_attention_static(p, p, p, p, 5, 2, 8, 4, 8, None) == 2
