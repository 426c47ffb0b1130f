"""CPU-only checks: the C-ABI library loads, exports every declared symbol, refuses to compute
without a GPU, and the split-KV planner deals tiles correctly."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import xor_net_b200 as xn


def header_symbols(repo_root):
    text = open(os.path.join(repo_root, "include", "xn_attn.h")).read()
    return sorted(set(re.findall(r"XN_API\s+[\w\s\*]+?\b(xn_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(repo_root):
    xn.build_library()
    lib = C.CDLL(xn.LIB_PATH)
    names = header_symbols(repo_root)
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/xn_attn.h but not exported"
    # the ctypes table covers the same set, so a binding cannot silently lag the header
    assert sorted(xn.SIGNATURES) == names


def test_version_string():
    assert xn.load().xn_version() == b"xn_attn 0.1 sm_100a"


def test_no_cpu_fallback_without_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(xn.XnError) as e:
        xn.Context(1, 2, 2, 4, pool_pages=4)
    assert e.value.code == 10 and "no CPU fallback" in str(e.value)


def test_ctx_create_argument_errors():
    lib = xn.load()
    from xor_net_b200._ffi import CtxDesc

    h = C.c_void_p()
    d = CtxDesc()
    d.num_layers, d.num_heads, d.num_kv_heads, d.head_dim, d.pool_pages = 1, 5, 2, 8, 4
    assert lib.xn_ctx_create(C.byref(d), C.byref(h)) == 2  # heads not a multiple of kv heads
    d.num_heads, d.head_dim = 4, 300
    assert lib.xn_ctx_create(C.byref(d), C.byref(h)) == 2
    assert b"head_dim" in lib.xn_last_error(None)
    assert lib.xn_ctx_create(None, C.byref(h)) == 1
    assert lib.xn_ctx_destroy(None) == 3
    assert lib.xn_attention(None, None, 0, 0, 1, None, None, None, None) == 3


def test_rope_tables_match_oracle_bitwise():
    import oracle as xo

    for theta, D, scaling in [(500000.0, 128, None), (10000.0, 100, None),
                              (500000.0, 128, (8.0, 1.0, 4.0, 8192))]:
        c1, s1 = xn.rope_tables(theta, D, 300, scaling)
        c2, s2 = xo.rope_tables(theta, D, 300, scaling)
        assert np.array_equal(c1, c2) and np.array_equal(s1, s2)


def run_plan(kv_len, tile, max_ctas):
    lib = xn.load()
    kv = np.asarray(kv_len, dtype=np.int32)
    cap = len(kv) + max_ctas + 8
    arrs = [np.zeros(cap, np.int32) for _ in range(4)]
    cta = np.zeros(max_ctas + 1, np.int32)
    n_items, n_parts = C.c_int32(), C.c_int32()
    P = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))
    ctas = lib.xn_plan_split(len(kv), P(kv), tile, max_ctas, cap, P(arrs[0]), P(arrs[1]),
                             P(arrs[2]), P(arrs[3]), P(cta), C.byref(n_items), C.byref(n_parts))
    assert ctas >= 0
    n = n_items.value
    return ctas, [a[:n] for a in arrs], cta[:ctas + 1], n_parts.value


@pytest.mark.parametrize("seed", range(6))
def test_plan_split_covers_every_tile_once_and_balances(seed):
    rng = np.random.default_rng(seed)
    n_units = int(rng.integers(1, 400))
    kv = rng.integers(1, 4097, n_units)
    tile, max_ctas = 64, 148
    ctas, (unit, tb, te, part), cta, n_parts = run_plan(kv, tile, max_ctas)
    tiles = (kv + tile - 1) // tile
    assert ctas == min(max_ctas, tiles.sum())
    cover = [np.zeros(t, np.int32) for t in tiles]
    for u, b, e in zip(unit, tb, te):
        assert 0 <= b < e <= tiles[u]
        cover[u][b:e] += 1
    assert all(np.all(c == 1) for c in cover)
    per_cta = [int(sum(te[i] - tb[i] for i in range(cta[b], cta[b + 1]))) for b in range(ctas)]
    assert max(per_cta) - min(per_cta) <= 1
    # units cut across blocks get consecutive partial slots; whole units are written directly
    counts = np.bincount(unit, minlength=n_units)
    assert n_parts == int(counts[counts > 1].sum())
    for u in range(n_units):
        p = part[unit == u]
        if counts[u] == 1:
            assert p[0] == -1
        else:
            assert np.array_equal(np.sort(p), np.arange(p.min(), p.min() + counts[u]))
    used = part[part >= 0]
    assert np.array_equal(np.sort(used), np.arange(n_parts))


def test_plan_split_edge_cases():
    ctas, (unit, tb, te, part), cta, n_parts = run_plan([1], 64, 148)
    assert ctas == 1 and list(unit) == [0] and list(part) == [-1] and n_parts == 0
    ctas, (unit, tb, te, part), cta, n_parts = run_plan([64 * 300], 64, 148)
    assert ctas == 148 and n_parts == 148 and np.all(unit == 0)
    ctas, items, cta, n_parts = run_plan([], 64, 148)
    assert ctas == 0
    assert xn.load().xn_plan_split(1, None, 64, 148, 8, None, None, None, None, None, None, None) < 0


def test_ternary_pack_matches_the_oracle_packer():
    # xn_ternary_pack is host-only (TernaryLinear::new, dense representation): no GPU needed
    import oracle as xo
    from xor_net_b200.api import TernaryLinear

    rng = np.random.default_rng(3)
    for pack in (xo.PACK4, xo.PACK5):
        for in_dim, out_dim in ((1, 1), (7, 3), (64, 5), (33, 2), (2560, 3)):
            w = rng.standard_normal((out_dim, in_dim)).astype(np.float32)
            tern = rng.integers(-1, 2, (out_dim, in_dim)).astype(np.float32)
            for weights, scale in ((w, None), (w, 0.7), (tern, None), (tern, 0.25)):
                a = xo.TernaryLinear(in_dim, out_dim, weights, pack, scale)
                b = TernaryLinear(in_dim, out_dim, weights, pack, scale)
                assert np.array_equal(a.packed, b.packed[:a.packed.size]), (pack, in_dim, out_dim, scale)
                assert np.array_equal(a.w_scales, b.w_scales)
    with pytest.raises(ValueError):
        TernaryLinear(4, 2, np.zeros(7, np.float32))


def test_sparse_pack_matches_the_oracle_encoder():
    # xn_ternary_pack_sparse is host-only (TernaryLinear::new_sparse): no GPU needed
    import oracle as xo
    from xor_net_b200.api import TernaryLinear

    rng = np.random.default_rng(4)
    for in_dim, out_dim in ((1, 1), (7, 3), (64, 5), (65, 2), (2560, 3)):
        w = rng.standard_normal((out_dim, in_dim)).astype(np.float32)
        tern = rng.integers(-1, 2, (out_dim, in_dim)).astype(np.float32)
        for weights, scale in ((w, None), (w, 0.7), (tern, None)):
            a = xo.TernaryLinear(in_dim, out_dim, weights, xo.SPARSE, scale)
            b = TernaryLinear(in_dim, out_dim, weights, xn.SPARSE, scale)
            assert np.array_equal(a.packed, b.packed) and np.array_equal(a.w_scales, b.w_scales)


def test_static_decode_entry_names_no_allocating_call(repo_root):
    """The allocation-free entry point and its two kernels must not name any allocating or freeing
    CUDA routine: read its definition and the kernels' header as text."""
    src = open(os.path.join(repo_root, "xor-net_b200", "csrc", "xn_attn.cu")).read()
    start = src.index('extern "C" int32_t xn_decode_attention_static')
    body = src[start:]
    body = body[:body.index("\n}\n") + 3]
    kernels = open(os.path.join(repo_root, "xor-net_b200", "csrc", "xn_static_decode.cuh")).read()
    for text in (body, kernels):
        for word in ("cudaMalloc", "cudaFree", "cudaHostAlloc", "cudaMallocHost", "cudaMallocAsync", "operator new",
                     "std::vector", "malloc("):
            assert word not in text, f"{word!r} appears in the allocation-free entry point"
    assert "cudaGetSymbolAddress" in body and "g_static_scratch" in body


def test_stream_placement_policy():
    """xn_place_stream: least-loaded by tokens, ties by live streams, then round-robin; and the
    plain round-robin rule (stream number mod devices)."""
    least, rr = xn.PLACE_LEAST_LOADED, xn.PLACE_ROUND_ROBIN
    assert xn.place_stream([5, 3, 9], [1, 1, 1], 0, least) == 1
    assert xn.place_stream([4, 4, 4], [2, 1, 2], 0, least) == 1          # tie on tokens: fewest streams
    assert [xn.place_stream([0, 0, 0, 0], [0, 0, 0, 0], t, least) for t in range(6)] == [0, 1, 2, 3, 0, 1]
    assert [xn.place_stream([7, 1, 1], [0, 0, 0], t, rr) for t in range(5)] == [0, 1, 2, 0, 1]
    with pytest.raises(xn.XnError):
        xn.place_stream([1, 2], [0, 0], 0, 7)
    # placing a seeded draw of lengths one by one keeps the GPUs within one stream of each other
    rng = np.random.default_rng(299792458 + 3000)
    lens = rng.integers(128, 4097, 512)
    tokens, live = [0] * 8, [0] * 8
    for i, L in enumerate(lens):
        w = xn.place_stream(tokens, live, i, least)
        tokens[w] += int(L)
        live[w] += 1
    assert max(tokens) - min(tokens) <= 4096
    rr_tokens = [int(lens[r::8].sum()) for r in range(8)]
    assert (max(tokens) / (sum(tokens) / 8)) < (max(rr_tokens) / (sum(rr_tokens) / 8))


def test_bounds_checking_build_compiles(repo_root, tmp_path):
    """The opt-in -DXN_BOUNDS build (copy producers range-check page ids and report kDevBadIndex
    instead of issuing the copy) compiles for sm_100a and exports the same symbols."""
    import subprocess

    from xor_net_b200 import _build

    out = str(tmp_path / "libxn_attn_bounds.so")
    cmd = [_build._nvcc(), *_build.NVCC_FLAGS, "-DXN_BOUNDS", "-I", _build.INCLUDE, "-o", out, *_build.sources()]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    lib = C.CDLL(out)
    for name in header_symbols(repo_root):
        assert hasattr(lib, name)


def test_rust_binding_source_agrees_with_the_header(repo_root):
    """The Rust crate cannot be compiled where no Rust toolchain exists, so its declarations are
    checked as text: every extern it names is declared in the header, the counters struct lists
    the header's fields in the header's order, and the binding goes through the device group (no
    fixed device ordinal, no pool sized from a sequence length)."""
    src = open(os.path.join(repo_root, "xor-net_b200", "rust", "xor-net-attn", "src", "lib.rs")).read()
    hdr = open(os.path.join(repo_root, "include", "xn_attn.h")).read()
    declared = set(re.findall(r"XN_API\s+[\w\s\*]+?\b(xn_\w+)\s*\(", hdr))
    named = set(re.findall(r"\bfn (xn_\w+)\s*\(", src))
    assert named and named <= declared, sorted(named - declared)
    for must in ("xn_attention_rope", "xn_stream_reset", "xn_stats_get", "xn_ctx_synchronize",
                 "xn_group_create", "xn_group_stream_create", "xn_debug_check_guards"):
        assert must in named, must
    h_fields = re.findall(r"uint64_t (\w+);", hdr[hdr.index("typedef struct xn_stats {"):hdr.index("} xn_stats;")])
    r_fields = re.findall(r"pub (\w+): u64", src[src.index("pub struct XnStats {"):])[:len(h_fields)]
    assert r_fields == h_fields
    assert "impl Clone for DeviceKvCache" not in src and "NOT `Clone`" in src
    assert "shared_context(0" not in src and "max_seq_len + 63" not in src
