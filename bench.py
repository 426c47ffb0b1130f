#!/usr/bin/env python
"""Benchmark of the attention path: batched multi-stream decode over the paged KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3|c1|c5] [--impl reference]

Workload (default ``c3``, BitNet-2B shape): 64 independent streams per GPU, one new token each,
20 query heads, 5 KV heads, head_dim 128, per-stream cached lengths drawn uniformly from
[128, 4096] with a fixed seed, f32 KV in 64-token pages handed out in a shuffled order, 30
layers each with its own N(0,1) cache contents.  One *step* = one decode step of every stream
through all layers = one batched submission per layer.  Data is synthetic: generated on the
device by the library's counter-based generator (the cache) and seeded N(0,1) inputs.

Printed JSON (one line, rank 0):
  value    algorithmic HBM GB/s of the whole job, inputs resident in HBM (device pointers);
           algorithmic bytes per layer = sum over streams of
           2*Hkv*L*D*4 (K and V read once) + 4*Hkv*D*4 (new K,V read + append) + 2*Hq*D*4 (q, out)
  e2e      the same metric through the blocking C-ABI call with HOST buffers: every layer call
           copies q,k,v host->device and the output device->host inside the timed region
  roofline the split-KV attention kernel alone: CUDA events around each of its launches
  cpu_baseline / --impl reference: the CPU oracle (a C port of the reference's AVX-512 path,
           all host threads) on a bounded sample of the same workload
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BASE_SEED = 299792458  # the reference's habitual seed (examples/batch_bench.rs:189)

WORKLOADS = {
    "c2": (1, 20, 5, 128, 1, 2048, 2048, "causal GQA prefill, BitNet-2B shape, 2048 tokens"),
    "c5p": (1, 32, 8, 128, 1, 32768, 32768, "one long causal prefill split by KV head over the GPUs"),
    # name: (streams per GPU, Hq, Hkv, D, layers, L_lo, L_hi, description)
    "c3": (64, 20, 5, 128, 30, 128, 4096,
           "batched decode, BitNet-2B shape: 64 streams/GPU x 30 layers, KV len U[128,4096]"),
    "c3o": (64, 20, 5, 128, 30, 128, 4096,
            "batched decode + output block (sub-norm, ternary o_proj 2560x2560) on the device, "
            "BitNet-2B shape: 64 streams/GPU x 30 layers, KV len U[128,4096]"),
    "c3b": (64, 20, 5, 128, 30, 128, 4096,
            "batched decode, whole attention block on the device (ternary q/k/v projections, RoPE, "
            "attention, sub-norm, ternary o_proj; hidden 2560), BitNet-2B shape: 64 streams/GPU x 30 "
            "layers, KV len U[128,4096]"),
    "c1": (1, 20, 5, 128, 1, 1024, 1024,
           "single-stream decode, BitNet-2B shape: 1 stream, 1 layer, KV len 1024"),
    "c5": (32, 32, 8, 128, 32, 2048, 8192,
           "long-context batched decode, LLaMA-3-8B shape: 32 streams/GPU x 32 layers, KV len U[2048,8192]"),
}


def host_threads():
    """Threads the CPU legs use: every core this process may run on.  (The launcher of multi-rank
    runs exports OMP_NUM_THREADS=1, which must not shrink the CPU baseline to one thread.)"""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def algorithmic_bytes_per_layer(lens, Hq, Hkv, D, u8=False):
    """Bytes one layer's decode step must move: every cached K and V row once, the new token's rows
    in and into the cache, q in and the output out.  In the u8 cache format a cached row is D bytes
    plus one f32 scale."""
    row = (D + 4) if u8 else D * 4
    return int(sum(2 * Hkv * int(L) * row + 2 * Hkv * D * 4 + 2 * Hkv * row + 2 * Hq * D * 4 for L in lens))


def stream_lengths(n, lo, hi, seed):
    rng = np.random.default_rng(seed)
    return rng.integers(lo, hi + 1, n).astype(np.int64)


def place_streams(xn, lens_global, world, policy):
    """Owner GPU of every stream of one global list, decided in creation order like the library's
    device group does (xn_place_stream): "least" = the GPU with the fewest announced tokens (ties:
    fewest streams, then round-robin), "rr" = stream number mod number of GPUs."""
    tokens, live, owner = [0] * world, [0] * world, []
    for i, L in enumerate(lens_global):
        w = i % world if policy == "rr" else xn.place_stream(tokens, live, i, xn.PLACE_LEAST_LOADED)
        owner.append(w)
        tokens[w] += int(L)
        live[w] += 1
    return owner


def load_traffic(name):
    """DRAM bytes per launch of a kernel from the tracked summary of its ncu capture
    (profiles/<name>.json: dram__bytes_read.sum + dram__bytes_write.sum, the commit it was taken at)."""
    path = os.path.join(ROOT, "profiles", name + ".json")
    if not os.path.exists(path):
        return None, None
    with open(path) as f:
        d = json.load(f)
    return float(d["dram_bytes_read"]) + float(d["dram_bytes_written"]), \
        f"ncu capture at commit {d.get('commit', '?')}: {d.get('workload', '')}"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.lines = []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(gpu_index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            inside = t0 - 0.05 <= ts <= t1 + 0.15
            try:
                if inside:
                    sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            if inside:
                for nm, val in zip(names, parts[3:7]):
                    if val.lower().startswith("active"):
                        reasons.add(nm)
        if not sm:  # region shorter than the sampling period: use every sample taken
            for ts, line in self.lines:
                try:
                    sm.append(float(line.split(",")[0]))
                except ValueError:
                    pass
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# =================================================================================================
# CPU baseline (the oracle: C port of the reference's path), bounded sample
# =================================================================================================

def cpu_sample(lens, Hq, Hkv, D, kv_by_stream, q, k, v, layer, budget_s=12.0, max_reps=50):
    """Times the oracle on the given streams of one layer with every host thread.

    kv_by_stream[i] = (K, V) each [Hkv, L_i - 1, D] already cached; q/k/v per stream are the new
    token's tensors.  Returns (GB/s, seconds per pass, outputs of the last pass, threads).
    """
    import oracle as xo

    n = len(lens)
    threads = host_threads()
    cap = int(max(lens))
    caches = []
    for i in range(n):
        c = xo.RingCache(layer + 1, Hkv, cap, D)
        if lens[i] > 1:
            c.append(layer, 0, kv_by_stream[i][0], kv_by_stream[i][1])
        caches.append(c)
    pos = [int(L) - 1 for L in lens]
    nbytes = algorithmic_bytes_per_layer(lens, Hq, Hkv, D)
    xo.fast_attention_streams(q, k, v, layer, pos, caches, Hq, Hkv, D, threads)  # warm-up
    t_total, reps, outs = 0.0, 0, None
    while reps < max_reps and (reps < 3 or t_total < budget_s):
        t0 = time.perf_counter()
        outs = xo.fast_attention_streams(q, k, v, layer, pos, caches, Hq, Hkv, D, threads)
        t_total += time.perf_counter() - t0
        reps += 1
    per_pass = t_total / reps
    return nbytes / per_pass / 1e9, per_pass, outs, threads, reps


def run_reference_arm(args):
    """--impl reference: the reference's CPU algorithm (oracle port; the reference itself is
    Rust and no Rust toolchain exists here) on the host cores, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import oracle as xo

    n_streams, Hq, Hkv, D, layers, lo, hi, desc = WORKLOADS[args.workload]
    lens_all = stream_lengths(n_streams, lo, hi, BASE_SEED + 3000)
    sample = min(args.cpu_streams, n_streams)
    lens = lens_all[:sample]
    rng = np.random.default_rng(BASE_SEED + 3000 + 1)
    threads = host_threads()
    cap = int(max(lens))
    caches, qs, ks, vs = [], [], [], []
    for L in lens:
        c = xo.RingCache(1, Hkv, cap, D)
        if L > 1:
            c.append(0, 0, rng.standard_normal((Hkv, int(L) - 1, D)).astype(np.float32),
                     rng.standard_normal((Hkv, int(L) - 1, D)).astype(np.float32))
        caches.append(c)
        qs.append(rng.standard_normal((1, Hq, 1, D)).astype(np.float32))
        ks.append(rng.standard_normal((1, Hkv, 1, D)).astype(np.float32))
        vs.append(rng.standard_normal((1, Hkv, 1, D)).astype(np.float32))
    pos = [int(L) - 1 for L in lens]
    nbytes = algorithmic_bytes_per_layer(lens, Hq, Hkv, D)
    for _ in range(args.warmup):
        xo.fast_attention_streams(qs, ks, vs, 0, pos, caches, Hq, Hkv, D, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        xo.fast_attention_streams(qs, ks, vs, 0, pos, caches, Hq, Hkv, D, threads)
    dt = time.perf_counter() - t0
    gbs = nbytes * args.steps / dt / 1e9
    sample_txt = (f"{sample} of {n_streams} streams x 1 of {layers} layers per step "
                  f"({nbytes / 1e6:.1f} MB algorithmic), isa level {xo.active_isa()}")
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {desc}", "sample": sample_txt},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": sample_txt},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tokens_per_s": sample * args.steps / dt,
    }
    print(json.dumps(line))
    return 0


# =================================================================================================
# Prefill (tensor-core TF32 kernel)
# =================================================================================================

def prefill_flops(Hq, D, S, P=0):
    """Algorithmic flops of causal attention: QK^T and PV over unmasked pairs only."""
    return 4 * Hq * D * (S * P + S * (S + 1) // 2)


def load_tf32_peak():
    """A PROXY for the TF32 dense peak: half of the measured bf16 cuBLAS burst figure (the two kinds
    differ by exactly 2x in nominal tensor-core rate); no TF32 peak is measured on this pool."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]) / 2.0, "proxy (measured bf16 burst / 2)"
    return 1590.0 / 2.0, "proxy (fallback bf16 / 2)"


def tf32_matmul_tflops(torch, n=8192, reps=5):
    """Context for the proxy peak: one library TF32 GEMM (torch.matmul, n^3) timed in this run."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(n, n, device="cuda")
        b = torch.randn(n, n, device="cuda")
        for _ in range(2):
            a @ b
        best = float("inf")
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            a @ b
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


L2_BYTES = 126 << 20


def measure_prefill(xn, torch, tstream, device, S, Hq, Hkv, D, theta, steps, warmup, e2e=True, u8=False,
                    min_seconds=0.25, index_pos=0, chunk=0, n_seqs=1, prefill_mode=0):
    """One causal prefill of S tokens (fused RoPE + append + attention) per step, one layer.

    ``ms`` is the device time of one call (append + attention) behind an L2 flush, median over the
    steps.  ``pipelined_ms`` is the device time per call in a long stream of back-to-back calls (CUDA
    events around runs of calls, median over the runs) that walk round-robin over enough independent
    input sets (own q, k, v, out and cache pages each) that a set has left L2 before it is used
    again; the GPU settles at its power-capped clocks there.  ``kernel_ms`` is the tensor-core
    kernel alone (events around each launch).

    With ``chunk`` > 0 the S tokens arrive as chunks of that many rows at growing positions (the
    chunked prefill of examples/chat.rs:297-306); ``index_pos`` > 0 puts a filled prefix before them.
    ``n_seqs`` > 1 submits that many independent sequences of S tokens in one call.
    """
    P = int(index_pos)
    cos, sin = xn.rope_tables(theta, D, P + S)
    set_bytes = ((Hq + 2 * Hkv) + Hq + 2 * Hkv) * S * D * 4 * n_seqs
    n_sets = int(min(8, max(2, -(-2 * L2_BYTES // set_bytes) + 1)))
    ctx = xn.Context(num_layers=1, num_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                     pool_pages=(n_sets + 1) * n_seqs * ((P + S + 63) // 64 + 2), device=device,
                     shuffle_seed=BASE_SEED + 2000, rope=(cos, sin), cuda_stream=tstream.cuda_stream,
                     kv_format=xn.KV_U8 if u8 else xn.KV_F32, prefill_mode=prefill_mode)
    gen = torch.Generator(device="cpu").manual_seed(BASE_SEED + 2000)
    q_h = torch.randn(Hq, S, D, generator=gen).pin_memory()
    k_h = torch.randn(Hkv, S, D, generator=gen).pin_memory()
    v_h = torch.randn(Hkv, S, D, generator=gen).pin_memory()
    o_h = torch.empty(Hq, S, D).pin_memory()
    pieces = [(0, S)] if not chunk else [(a, min(chunk, S - a)) for a in range(0, S, chunk)]
    sets, keep = [], []
    for i in range(n_sets):
        st = ctx.new_stream(P + S)
        if P:
            st.fill_normal(0, 0, P, BASE_SEED + 2000 + i)
        q_d, k_d, v_d = q_h.cuda(), k_h.cuda(), v_h.cuda()
        o_d = torch.empty(Hq, S, D, device="cuda")
        keep.append((q_d, k_d, v_d, o_d))
        if n_seqs > 1:   # further sequences of the same call: own streams, own tensors
            entries = [(st, 0, P, S, q_d.data_ptr(), k_d.data_ptr(), v_d.data_ptr(), o_d.data_ptr())]
            for _ in range(n_seqs - 1):
                st2 = ctx.new_stream(P + S)
                t4 = (q_h.cuda(), k_h.cuda(), v_h.cuda(), torch.empty(Hq, S, D, device="cuda"))
                keep.append(t4)
                entries.append((st2, 0, P, S, t4[0].data_ptr(), t4[1].data_ptr(), t4[2].data_ptr(), t4[3].data_ptr()))
            sets.append([ctx.make_batch(entries, xn.REQ_DEVICE_PTRS | xn.REQ_ROPE)])
            continue
        if chunk:   # chunks are row ranges of the sequence-major tensors
            qs, ks, vs = (x.transpose(0, 1).contiguous() for x in (q_d, k_d, v_d))
            os_ = torch.empty(S, Hq, D, device="cuda")
            keep.append((qs, ks, vs, os_))
            sets.append([ctx.make_batch([(st, 0, P + a, n, qs[a].data_ptr(), ks[a].data_ptr(), vs[a].data_ptr(),
                                          os_[a].data_ptr())], xn.REQ_DEVICE_PTRS | xn.REQ_ROPE | xn.REQ_SEQ_MAJOR)
                         for a, n in pieces])
        else:
            sets.append([ctx.make_batch([(st, 0, P, S, q_d.data_ptr(), k_d.data_ptr(), v_d.data_ptr(),
                                          o_d.data_ptr())], xn.REQ_DEVICE_PTRS | xn.REQ_ROPE)])
    host_st = ctx.new_stream(P + S) if e2e else None

    def call(i):
        for b in sets[i % n_sets]:
            ctx.submit(b)

    for i in range(max(warmup, 3) + n_sets):
        call(i)
    torch.cuda.synchronize()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # > L2 (126 MB)
    # -- one call at a time behind an L2 flush (the flush keeps the GPU busy while the host
    #    enqueues, so the events bracket device time only)
    iso = []
    for j in range(max(steps, 5)):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(tstream)
        call(j)
        e1.record(tstream)
        torch.cuda.synchronize()
        iso.append(e0.elapsed_time(e1))
    ms = float(np.median(iso))
    # -- the tensor-core kernel alone (events around each launch; they sit between the append and
    #    the prefill kernel, so this loop runs without their overlap)
    ctx.profile_enable(True)
    ctx.profile_read()
    n_prof = max(3, min(steps, 10))
    launched0 = ctx.stats()["kernel_launches"]
    for j in range(n_prof):
        flush.zero_()
        call(j)
    torch.cuda.synchronize()
    kern_ms, kern_n = ctx.profile_read("prefill")
    ctx.profile_enable(False)
    launches_per_call = (ctx.stats()["kernel_launches"] - launched0) / n_prof
    kern_per_call = kern_ms / n_prof   # all prefill launches of one call (chunks, sequences)
    # -- back-to-back calls, timed in runs: sustained (power-capped) clocks
    run = max(4, min(64, steps))
    runs, total, i = [], 0.0, 0
    while len(runs) < 3 or (total < min_seconds * 1e3 and len(runs) < 400):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(tstream)
        for _ in range(run):
            call(i)
            i += 1
        e1.record(tstream)
        torch.cuda.synchronize()
        runs.append(e0.elapsed_time(e1) / run)
        total += runs[-1] * run
    pipe_ms = float(np.median(runs))
    flops = prefill_flops(Hq, D, S, P) * n_seqs
    res = {"seq_len": S, "index_pos": P, "chunk": chunk or S, "sequences": n_seqs, "flops": flops, "ms": ms,
           "tflops": flops / (ms * 1e-3) / 1e12,
           "timing": f"median of {len(iso)} calls, each behind a 256 MB write that flushes L2",
           "pipelined_ms": pipe_ms, "pipelined_tflops": flops / (pipe_ms * 1e-3) / 1e12,
           "pipelined_timing": f"median of {len(runs)} runs of {run} back-to-back calls over {n_sets} rotating "
                               f"input sets ({n_sets * set_bytes / 1e6:.0f} MB, larger than L2); sustained clocks",
           "kernel_ms": kern_per_call,
           "kernel_tflops": flops / (kern_per_call * 1e-3) / 1e12 if kern_n else None,
           "launches_per_step": launches_per_call}
    if e2e and not chunk and n_seqs == 1:
        host = ctx.make_batch([(host_st, 0, P, S, q_h.data_ptr(), k_h.data_ptr(), v_h.data_ptr(), o_h.data_ptr())],
                              xn.REQ_ROPE | xn.REQ_HOST_PINNED)  # page-locked host buffers
        if P:
            host_st.fill_normal(0, 0, P, BASE_SEED + 2999)
        ctx.submit(host)
        t0 = time.perf_counter()
        n = max(1, min(steps, 5))
        for _ in range(n):
            ctx.submit(host)
        dt = (time.perf_counter() - t0) / n
        res["e2e_ms"] = dt * 1e3
        res["e2e_tflops"] = flops / dt / 1e12
        res["e2e_h2d_bytes"] = (Hq + 2 * Hkv) * S * D * 4
        res["e2e_d2h_bytes"] = Hq * S * D * 4
    ctx.close()
    return res


def run_prefill_arm(args):
    """--workload c2: causal GQA prefill, BitNet-2B shape, 2048 tokens (--seq overrides the length)."""
    import torch

    import xor_net_b200 as xn

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    tstream = torch.cuda.Stream(device=local_rank)
    torch.cuda.set_stream(tstream)
    S = args.seq or 2048
    sampler = ClockSampler(local_rank) if rank == 0 else None
    wall0 = time.time()
    u8 = args.kv == "u8"
    r = measure_prefill(xn, torch, tstream, local_rank, S, 20, 5, 128, 500000.0, args.steps, args.warmup, u8=u8,
                        index_pos=args.pos, chunk=args.chunk, min_seconds=args.min_seconds,
                        prefill_mode=1 if args.f32 else 0)
    wall1 = time.time()
    clocks = sampler.stop(wall0, wall1) if sampler else None
    if rank != 0:
        return 0
    peak, peak_kind = load_tf32_peak()
    line = {
        "metric": "prefill_attn_tflops", "value": r["tflops"] * world, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": r["ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32",
        "data": "synthetic",
        "config": {"workload": f"c2: causal GQA prefill, BitNet-2B shape, {S} tokens, 20/5 heads, "
                               "head_dim 128, fused RoPE theta 5e5 + append into 64-token pages" +
                               (" [exact-f32 path: tiled CUDA-core kernel]" if args.f32 else "") +
                               (f", behind {args.pos} cached tokens" if args.pos else "") +
                               (f", in chunks of {args.chunk} rows" if args.chunk else "") +
                               (" [opt-in u8 cache format: quantised append, pages dequantised into an f32 "
                                "staging area for the tensor-core kernel]" if u8 else ""),
                   "l2": r["timing"],
                   "parallelism": f"{world} independent replica(s)"},
        "e2e": {"value": r.get("e2e_tflops"), "unit": "TFLOP/s",
                "h2d_bytes_per_step": r.get("e2e_h2d_bytes"), "d2h_bytes_per_step": r.get("e2e_d2h_bytes"),
                "ms_per_step": r.get("e2e_ms")},
        "gpu_launches": r["launches_per_step"] * args.steps,
        "roofline": {"bound": "tensor", "kernel": "prefill_f32_kernel (CUDA cores)" if args.f32 else "prefill_tf32_kernel",
                     "achieved": r["kernel_tflops"],
                     "peak": peak, "unit": "TFLOP/s", "frac": r["kernel_tflops"] / peak,
                     "peak_source": peak_kind, "traffic": None, "avg_launch_ms": r["kernel_ms"],
                     "algorithmic_flops_per_launch": r["flops"],
                     "call_frac": r["tflops"] / peak, "pipelined_call_ms": r["pipelined_ms"],
                     "library_tf32_matmul_tflops": tf32_matmul_tflops(torch)},
        "clocks": clocks, "cpu_baseline": None,
    }
    print(json.dumps(line))
    return 0


# =================================================================================================
# Long prefill split by KV-head group across GPUs, outputs gathered over NVLink (config 5)
# =================================================================================================

def run_split_prefill_arm(args):
    """--workload c5p: one causal prefill (LLaMA-3-8B shape: 32 query / 8 KV heads, head_dim 128,
    RoPE theta 5e5) of --seq tokens (default 32768), KV heads dealt to the GPUs in contiguous
    blocks; every rank computes its heads with the tensor-core kernel.  Two ways to bring the
    per-rank outputs [heads/N, S, D] together on rank 0 are timed:
      gather  each rank writes a local slab, then one NCCL gather;
      fused   the kernel's epilogue stores go straight into rank 0's slab (peer-mapped symmetric
              memory, plain st.global over NVLink), so the transfer overlaps the compute.
    Total work is fixed as N grows: "scaling": "strong"."""
    import torch
    import torch.distributed as dist

    import oracle as xo
    import xor_net_b200 as xn

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer stores only
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    tstream = torch.cuda.Stream(device=local_rank)
    torch.cuda.set_stream(tstream)
    Hq, Hkv, D, theta = 32, 8, 128, 500000.0
    S = args.seq or 32768
    kv_heads = xn.sharding.kv_heads_of_rank(Hkv, world, rank)
    G = Hq // Hkv
    hq_l, hkv_l = len(kv_heads) * G, len(kv_heads)
    cos, sin = xn.rope_tables(theta, D, S)
    ctx = xn.Context(num_layers=1, num_heads=hq_l, num_kv_heads=hkv_l, head_dim=D,
                     pool_pages=(S + 63) // 64 + 2, device=local_rank, shuffle_seed=BASE_SEED + 5000,
                     rope=(cos, sin), cuda_stream=tstream.cuda_stream)
    st = ctx.new_stream(S)

    def head_tensor(kind, h, rows):  # the full problem is defined per global head, whatever N is
        g = torch.Generator(device="cpu").manual_seed(BASE_SEED + 5000 + 100 * kind + h)
        return torch.randn(rows, D, generator=g)

    q_l = torch.stack([head_tensor(0, kv * G + j, S) for kv in kv_heads for j in range(G)]).cuda()
    k_l = torch.stack([head_tensor(1, kv, S) for kv in kv_heads]).cuda()
    v_l = torch.stack([head_tensor(2, kv, S) for kv in kv_heads]).cuda()
    out_l = torch.zeros(hq_l, S, D, device="cuda")
    full = torch.zeros(world, hq_l, S, D, device="cuda") if rank == 0 else None
    flops = prefill_flops(Hq, D, S)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(tstream)
        for _ in range(steps):
            fn()
        e1.record(tstream)
        barrier()
        (ms,), _ = xn.sharding.aggregate([e0.elapsed_time(e1) / steps], [0.0], device="cuda")
        return ms

    local_batch = ctx.make_batch([(st, 0, 0, S, q_l.data_ptr(), k_l.data_ptr(), v_l.data_ptr(),
                                   out_l.data_ptr())], xn.REQ_DEVICE_PTRS | xn.REQ_ROPE)

    def step_gather():
        ctx.submit(local_batch)
        if world > 1:
            dist.gather(out_l, list(full.unbind(0)) if rank == 0 else None, dst=0)
        else:
            full[0].copy_(out_l)

    steps, warmup = max(1, args.steps), max(3, args.warmup)
    gather_ms = timed(step_gather, steps, warmup)
    compute_ms = timed(lambda: ctx.submit(local_batch), steps, warmup)

    fused_ms, fused_note, root_view = None, None, None
    if world > 1:
        try:
            import torch.distributed._symmetric_memory as symm_mem

            slab = symm_mem.empty(world * hq_l * S * D, dtype=torch.float32, device=torch.device("cuda", local_rank))
            hdl = symm_mem.rendezvous(slab, dist.group.WORLD)
            root_view = hdl.get_buffer(0, (world, hq_l, S, D), torch.float32)  # rank 0's slab, peer-mapped
            fused_batch = ctx.make_batch([(st, 0, 0, S, q_l.data_ptr(), k_l.data_ptr(), v_l.data_ptr(),
                                           root_view[rank].data_ptr())], xn.REQ_DEVICE_PTRS | xn.REQ_ROPE)
            fused_ms = timed(lambda: ctx.submit(fused_batch), steps, warmup)
            if rank == 0:
                torch.cuda.synchronize()
                same = bool(torch.equal(slab.view(world, hq_l, S, D), full))
                fused_note = f"fused output equals gathered output: {same}"
        except Exception as e:  # symmetric memory not available on this box
            fused_note = f"fused path unavailable: {type(e).__name__}: {e}"

    line = None
    if rank == 0:
        # parity on sampled rows: row t of head h equals a decode step at position t over that
        # head's keys 0..t, which the oracle computes directly
        torch.cuda.synchronize()
        got = full.view(Hq, S, D).cpu().numpy()
        worst = 0.0
        for h in (0, Hq - 1):
            kv = h // G
            kh = xo.tensor_rope(head_tensor(1, kv, S).numpy()[None, None], cos, sin, 0)[0]
            vh = head_tensor(2, kv, S).numpy()[None]
            qh = xo.tensor_rope(head_tensor(0, h, S).numpy()[None, None], cos, sin, 0)[0, 0]
            for t in (0, 127, 128, S // 2 + 5, S - 129, S - 1):
                ref = xo.RingCache(1, 1, t + 1, D)
                ref.append(0, 0, kh[:, :t + 1], vh[:, :t + 1])
                want = xo.fast_attention(qh[t].reshape(1, 1, 1, D), kh[:, t:t + 1][None], vh[:, t:t + 1][None],
                                         0, t, ref, 1, 1, D)
                rel = float(np.linalg.norm(got[h, t] - want.ravel()) / np.linalg.norm(want))
                worst = max(worst, rel)
        peak, peak_kind = load_tf32_peak()
        best_ms = min(x for x in (gather_ms, fused_ms) if x)
        line = {
            "metric": "prefill_attn_tflops", "value": flops / (best_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": best_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "tf32",
            "data": "synthetic",
            "config": {"workload": f"c5p: one causal prefill of {S} tokens, 32/8 heads, head_dim 128, "
                                   f"KV heads split over {world} GPU(s), outputs gathered on rank 0",
                       "parallelism": f"{hkv_l} KV head(s) + {hq_l} query heads per GPU"},
            "split_prefill": {"compute_only_ms": compute_ms, "with_nccl_gather_ms": gather_ms,
                              "fused_peer_store_ms": fused_ms, "note": fused_note,
                              "tflops_compute_only": flops / (compute_ms * 1e-3) / 1e12,
                              "gather_bytes_to_root": (world - 1) * hq_l * S * D * 4},
            "roofline": {"bound": "tensor", "kernel": "prefill_tf32_kernel",
                         "achieved": flops / (compute_ms * 1e-3) / 1e12 / world, "peak": peak, "unit": "TFLOP/s",
                         "frac": flops / (compute_ms * 1e-3) / 1e12 / world / peak, "peak_source": peak_kind,
                         "traffic": None},
            "parity_sampled_rows_rel_l2": worst, "parity_tolerance": "rel_l2 <= 5e-3 (TF32 prefill)",
            "gpu_launches": 2 * steps, "cpu_baseline": None, "e2e": None,
        }
        print(json.dumps(line))
    ctx.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


# =================================================================================================
# Short summaries of the other workload shapes (extras of the default line)
# =================================================================================================

def measure_decode(xn, torch, tstream, device, lens, Hq, Hkv, D, layers, steps, grow=False, theta=None,
                   min_seconds=0.15):
    """Batched decode over device-resident inputs: one submission per layer and step.  With ``grow``
    every step appends at the next position (one layer), else the positions stay put.  Returns the
    per-step device time, the split-KV kernel's own time per launch and algorithmic GB/s."""
    n = len(lens)
    rope = xn.rope_tables(theta, D, int(max(lens)) + steps + 2) if theta else None
    pages = int(sum((int(L) + steps + 64) // 64 + 1 for L in lens))
    ctx = xn.Context(num_layers=layers, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, pool_pages=pages + 8,
                     device=device, shuffle_seed=BASE_SEED + 77, cuda_stream=tstream.cuda_stream, rope=rope)
    sts = [ctx.new_stream(int(max(lens)) + steps + 2) for _ in range(n)]
    for i, st in enumerate(sts):
        if lens[i] > 1:
            st.fill_normal(-1, 0, int(lens[i]) - 1, BASE_SEED + 7000 + i)
    gen = torch.Generator(device="cpu").manual_seed(BASE_SEED + 7000)
    q = torch.randn(layers, n, Hq, D, generator=gen).cuda()
    k = torch.randn(layers, n, Hkv, D, generator=gen).cuda()
    v = torch.randn(layers, n, Hkv, D, generator=gen).cuda()
    o = torch.zeros(layers, n, Hq, D, device="cuda")
    flags = xn.REQ_DEVICE_PTRS | (xn.REQ_ROPE if theta else 0)

    def batch(l, s):
        return ctx.make_batch([(sts[i], l, int(lens[i]) - 1 + s, 1, q[l, i].data_ptr(), k[l, i].data_ptr(),
                                v[l, i].data_ptr(), o[l, i].data_ptr()) for i in range(n)], flags)

    if grow:
        plan = [[batch(0, s)] for s in range(steps)]           # every step at the next position
        per_step_bytes = [algorithmic_bytes_per_layer([int(L) + s for L in lens], Hq, Hkv, D) for s in range(steps)]
    else:
        plan = [[batch(l, 0) for l in range(layers)]] * steps
        per_step_bytes = [algorithmic_bytes_per_layer(lens, Hq, Hkv, D) * layers] * steps
    for b in plan[0] * 3:
        ctx.submit(b)
    torch.cuda.synchronize()
    brackets = []
    while len(brackets) < 1 or (sum(brackets) < min_seconds * 1e3 and len(brackets) < 100 and not grow):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(tstream)
        for step in plan:
            ctx.drop_plan()   # a step of a real decode loop is at a new position: its first layer plans afresh
            for b in step:
                ctx.submit(b)
        e1.record(tstream)
        torch.cuda.synchronize()
        brackets.append(e0.elapsed_time(e1))
    ms = float(np.median(brackets))
    ctx.profile_enable(True)
    ctx.profile_read()
    for b in plan[-1]:
        ctx.submit(b)
    kern_ms, kern_n = ctx.profile_read("splitkv")
    ctx.profile_enable(False)
    ctx.close()
    peak, peak_kind = load_peaks()
    kern = kern_ms / max(kern_n, 1)
    launch_bytes = per_step_bytes[-1] / (1 if grow else layers)
    return {"streams": n, "layers": layers, "steps": steps, "kv_tokens": int(sum(int(L) for L in lens)),
            "ms_per_step": ms / steps, "gbs": sum(per_step_bytes) / (ms * 1e-3) / 1e9,
            "tokens_per_s": n * steps / (ms * 1e-3),
            "kernel_us": kern * 1e3, "kernel_gbs": launch_bytes / (kern * 1e-3) / 1e9 if kern else None,
            "roofline": {"bound": "hbm", "achieved": launch_bytes / (kern * 1e-3) / 1e9 if kern else None, "peak": peak,
                         "unit": "GB/s", "frac": launch_bytes / (kern * 1e-3) / 1e9 / peak if kern else None,
                         "peak_source": peak_kind, "algorithmic_bytes_per_launch": launch_bytes}}


def run_dropin_leg(xn, n_streams, layers, Hq, Hkv, D, lo, hi, steps, warmup, device, pool_mb):
    """The call xor-net's front-ends make: one OS thread per stream blocking in fast_attention with
    pageable buffers, one call per layer (server/main.rs:126, examples/batch_bench.rs:194-199),
    driven by the compiled C++ harness over the C++ host mirror.  Returns its JSON."""
    exe = xn.build_host_tool("dropin_bench")
    env = dict(os.environ)
    env.setdefault("XORNET_ATTN_DEVICES", str(device))
    env.setdefault("XORNET_ATTN_POOL_MB", str(pool_mb))
    res = subprocess.run([exe, str(n_streams), str(layers), str(Hq), str(Hkv), str(D), str(lo), str(hi), str(steps),
                          str(warmup), str(BASE_SEED)], env=env, capture_output=True, text=True, timeout=600)
    if res.returncode != 0:
        return {"error": (res.stderr or res.stdout)[-400:]}
    out = json.loads(res.stdout.strip().splitlines()[-1])
    out["api"] = ("fast_attention of the C++ host mirror -> xn_attention: one OS thread per stream, pageable "
                  "std::vector<float> tensors, one blocking call per layer; the library merges concurrent callers")
    return out


# =================================================================================================
# GPU arm
# =================================================================================================

def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    import xor_net_b200 as xn

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention library has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    n_streams, Hq, Hkv, D, layers, lo, hi, desc = WORKLOADS[args.workload]
    if args.layers:   # reduced-size run for profiler captures; named in config.workload
        layers = args.layers
        desc += f" [reduced to {layers} layers]"
    if args.streams:
        n_streams = args.streams
        desc += f" [reduced to {n_streams} streams]"
    # ONE global list of world x n_streams lengths (weak scaling: the work per GPU is fixed on
    # average); every stream lives on one GPU for good, no data-path collective
    lens_global = stream_lengths(world * n_streams, lo, hi, BASE_SEED + 3000)
    owner = place_streams(xn, lens_global, world, args.placement)
    mine = [i for i in range(len(lens_global)) if owner[i] == rank]
    lens = lens_global[mine]
    n_total_streams = len(lens_global)
    n_streams = len(mine)
    tokens_by_rank = [int(sum(int(lens_global[i]) for i in range(n_total_streams) if owner[i] == r))
                      for r in range(world)]
    pages_needed = int(sum((int(L) + 63) // 64 for L in lens))
    # a real (non-default) stream shared by torch and the library, so that CUDA events recorded
    # here bracket the library's launches
    tstream = torch.cuda.Stream(device=local_rank)
    torch.cuda.set_stream(tstream)
    whole_block = args.workload.endswith("b")   # x in, y out: projections on the device too
    rope = xn.rope_tables(500000.0, D, int(hi) + 1) if whole_block else None
    u8 = args.kv == "u8"
    if u8:
        desc += " [opt-in u8 cache format: results differ from the f32 cache by the quantisation error]"
    ctx = xn.Context(num_layers=layers, num_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                     pool_pages=pages_needed + 8, device=local_rank,
                     shuffle_seed=BASE_SEED + rank, cuda_stream=tstream.cuda_stream, rope=rope,
                     kv_format=xn.KV_U8 if u8 else xn.KV_F32)
    streams = [ctx.new_stream(int(hi)) for _ in range(n_streams)]
    for i, st in enumerate(streams):
        if lens[i] > 1:
            st.fill_normal(-1, 0, int(lens[i]) - 1, BASE_SEED + 3000 + 1000003 + mine[i])
    ctx.synchronize()

    # per-layer inputs, resident on the device and mirrored in pinned host memory
    q_elems, kv_elems = n_streams * Hq * D, n_streams * Hkv * D
    gen = torch.Generator(device="cpu").manual_seed(BASE_SEED + 3000 + rank)
    q_h = torch.randn(layers, n_streams, Hq, D, generator=gen).pin_memory()
    k_h = torch.randn(layers, n_streams, Hkv, D, generator=gen).pin_memory()
    v_h = torch.randn(layers, n_streams, Hkv, D, generator=gen).pin_memory()
    o_h = torch.empty(layers, n_streams, Hq, D).pin_memory()
    q_d, k_d, v_d = q_h.cuda(non_blocking=True), k_h.cuda(non_blocking=True), v_h.cuda(non_blocking=True)
    o_d = torch.zeros(layers, n_streams, Hq, D, device="cuda")
    torch.cuda.synchronize()

    # the "o" workloads run the layer's output block behind the attention, on the device: out is
    # then [streams, hidden] per layer (hidden = Hq*D, as in the 2B model's square o_proj)
    out_block = args.workload.endswith("o") or whole_block
    extra_flags = 0
    if out_block:
        rng = np.random.default_rng(BASE_SEED + 4000 + rank)
        hidden = Hq * D
        lin = xn.TernaryLinear(hidden, hidden, rng.integers(-1, 2, (hidden, hidden)).astype(np.float32),
                               xn.PACK4, provided_scale=0.02)
        norm_w = (1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
        for l in range(layers):   # same synthetic weights on every layer; each layer has its own copy
            ctx.set_out_proj(l, lin, norm_w, 1e-5)
        extra_flags = xn.REQ_OUT_PROJ
    if whole_block:
        # q/k/v projections with a global weight scale that keeps the projected rows O(1)
        qkv_lin = [xn.TernaryLinear(hidden, rows, rng.integers(-1, 2, (rows, hidden)).astype(np.float32),
                                    xn.PACK4, provided_scale=float(hidden) ** -0.5)
                   for rows in (Hq * D, Hkv * D, Hkv * D)]
        for l in range(layers):
            ctx.set_qkv_proj(l, *qkv_lin)
        extra_flags |= xn.REQ_QKV_PROJ
        # x replaces q (one hidden-state row per stream and layer); k and v are not passed
        x_h = torch.randn(layers, n_streams, hidden, generator=gen).pin_memory()
        x_d = x_h.cuda(non_blocking=True)
        torch.cuda.synchronize()

    def batches(q, k, v, o, flags):
        out = []
        for l in range(layers):
            if whole_block:
                x = x_d if (flags & xn.REQ_DEVICE_PTRS) else x_h
                entries = [(streams[i], l, int(lens[i]) - 1, 1, x[l, i].data_ptr(), None, None,
                            o[l, i].data_ptr()) for i in range(n_streams)]
            else:
                entries = [(streams[i], l, int(lens[i]) - 1, 1, q[l, i].data_ptr(), k[l, i].data_ptr(),
                            v[l, i].data_ptr(), o[l, i].data_ptr()) for i in range(n_streams)]
            out.append(ctx.make_batch(entries, flags))
        return out

    dev_batches = batches(q_d, k_d, v_d, o_d, xn.REQ_DEVICE_PTRS | extra_flags)
    # host buffers are page-locked: the kernels move them over PCIe themselves
    host_batches = batches(q_h, k_h, v_h, o_h, xn.REQ_HOST_PINNED | extra_flags)
    staged_batches = batches(q_h, k_h, v_h, o_h, extra_flags)  # same buffers treated as pageable

    # Every step of a real decode loop moves to a new position, so its first layer plans afresh and
    # the other layers reuse that plan.  The bench re-submits the same positions step after step:
    # it drops the kept plan at the start of every step to measure the same thing.
    def step_device():
        ctx.drop_plan()
        for b in dev_batches:
            ctx.submit(b)

    def step_host():
        ctx.drop_plan()
        for b in host_batches:
            ctx.submit(b)

    def step_staged():
        for b in staged_batches:
            ctx.submit(b)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    bytes_per_layer = algorithmic_bytes_per_layer(lens, Hq, Hkv, D, u8)
    bytes_per_step = bytes_per_layer * layers

    # ---- device-resident timing (value) + live kernel timing (roofline) -------------------------
    for _ in range(max(args.warmup, 3)):
        step_device()
    barrier()
    # K steps between two events, a barrier and a synchronize on both sides; the bracket is repeated
    # until the timed regions add up to --min-seconds, and the median bracket is reported
    sampler = ClockSampler(local_rank) if rank == 0 else None
    wall0 = time.time()
    brackets, launches_per_bracket = [], 0
    while len(brackets) < 1 or (sum(brackets) < args.min_seconds * 1e3 and len(brackets) < 200):
        s0 = ctx.stats()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record(tstream)
        for _ in range(args.steps):
            step_device()
        ev1.record(tstream)
        barrier()
        t_bracket = ev0.elapsed_time(ev1)
        if world > 1:   # every rank must take the same number of brackets: agree on the slowest time
            (t_bracket,), _ = xn.sharding.aggregate([t_bracket], [0.0], device="cuda")
        brackets.append(t_bracket)
        launches_per_bracket = ctx.stats()["kernel_launches"] - s0["kernel_launches"]
    wall1 = time.time()
    ms = float(np.median(brackets))
    clocks = sampler.stop(wall0, wall1) if sampler else None
    # the attention kernel alone: CUDA events around each of its launches, in a pass of its own
    # (the events would sit between kernels that otherwise overlap head to tail)
    ctx.profile_enable(True)
    ctx.profile_read()
    for _ in range(max(1, min(args.steps, 5))):
        step_device()
    (kern_ms, kern_n), _, (ob_ms, ob_n), (qb_ms, qb_n) = ctx.profile_read_all()
    ctx.profile_enable(False)
    ctx.synchronize()

    # ---- end to end through the blocking C-ABI call with host buffers ----------------------------
    e2e_steps = 0 if args.no_e2e else args.steps
    for _ in range(0 if args.no_e2e else max(1, min(args.warmup, 3))):
        step_host()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reuses0 = ctx.stats()["plan_reuses"]
    t0 = time.perf_counter()
    e0.record(tstream)
    for _ in range(e2e_steps):
        step_host()
    e1.record(tstream)
    barrier()
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_reuses = ctx.stats()["plan_reuses"] - reuses0
    e2e_ms = max(e0.elapsed_time(e1), 0.0)
    # the host side of the call is part of it: the wall clock is the honest end-to-end time
    e2e_ms = max(e2e_ms, e2e_wall_ms)
    # the same through the library's own staging copies (what a caller with pageable memory gets)
    staged_ms = 0.0
    if e2e_steps:
        step_staged()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            step_staged()
        barrier()
        staged_ms = (time.perf_counter() - t0) * 1e3

    # job-wide figures: slowest rank's time, all ranks' bytes (no-op in a single process); the
    # kernel's roofline figure is per rank: its own bytes over its own launch time
    my_kern_ms = kern_ms / max(kern_n, 1)
    my_achieved = bytes_per_layer / (my_kern_ms * 1e-3) / 1e9 if my_kern_ms > 0 else 0.0
    (ms, e2e_ms), (total_bytes_per_step,) = xn.sharding.aggregate(
        [ms, e2e_ms], [float(bytes_per_step)], device="cuda")
    per_rank = [{"rank": rank, "streams": n_streams, "kv_tokens": int(lens.sum()), "kernel_ms": my_kern_ms,
                 "kernel_gbs": my_achieved}]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, per_rank[0])
        per_rank = gathered
    kern_avg_ms = max(p["kernel_ms"] for p in per_rank)

    # outputs of both paths agree (same kernels, same inputs)
    same = bool(torch.equal(o_d.cpu(), o_h)) if e2e_steps > 0 else None

    line = None
    if rank == 0:
        peak, peak_kind = load_peaks()
        achieved = min(p["kernel_gbs"] for p in per_rank)   # the slowest rank's own bytes / own time
        value = total_bytes_per_step * args.steps / (ms * 1e-3) / 1e9
        e2e_value = total_bytes_per_step * e2e_steps / (e2e_ms * 1e-3) / 1e9
        launches = launches_per_bracket
        # DRAM bytes per launch of the split-KV kernel from an ncu capture of this same workload
        # (dram__bytes_read.sum + dram__bytes_write.sum; the summary is kept under profiles/);
        # only valid for the unmodified c3 workload, whose per-launch work is fixed by its seed
        traffic, traffic_src = None, None
        if args.workload == "c3" and not args.streams and not args.layers and world == 1:
            traffic, traffic_src = load_traffic("attn_splitkv_u8_c3_traffic" if u8 else "attn_splitkv_c3_traffic")
        line = {
            "metric": "decode_attn_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: {desc}", "streams": n_total_streams,
                       "streams_per_gpu": [p["streams"] for p in per_rank],
                       "layers": layers, "num_heads": Hq, "num_kv_heads": Hkv, "head_dim": D,
                       "kv_tokens_per_gpu": tokens_by_rank, "page_tokens": 64,
                       "kv_format": "u8 bytes + one f32 scale per row" if u8 else "f32",
                       "placement": ("least-loaded GPU by announced tokens (xn_place_stream)" if args.placement == "least"
                                     else "round-robin: stream id mod GPUs"),
                       "parallelism": f"streams sharded over {world} GPU(s), no collective",
                       "timing": f"median of {len(brackets)} brackets of {args.steps} steps "
                                 f"({sum(brackets) / 1e3:.2f} s timed)",
                       "l2": "inputs larger than L2: %.1f GB of KV per GPU read per step" %
                             (bytes_per_step / 1e9)},
            "tokens_per_s": n_total_streams * args.steps / (ms * 1e-3),
            "e2e": {"value": e2e_value, "unit": "GB/s",
                    "h2d_bytes_per_step": layers * (n_streams * Hq * D if whole_block else q_elems + 2 * kv_elems) * 4,
                    "d2h_bytes_per_step": layers * q_elems * 4,
                    "ms_per_step": e2e_ms / max(e2e_steps, 1),
                    "tokens_per_s": n_total_streams * e2e_steps / (e2e_ms * 1e-3),
                    "api": "xn_attention_batch, page-locked host pointers (XN_REQ_HOST_PINNED), one "
                           "blocking call per layer",
                    "plans_reused_per_step": e2e_reuses / max(e2e_steps, 1),
                    "staged_ms_per_step": staged_ms / max(e2e_steps, 1),
                    "staged_value": (bytes_per_step * e2e_steps / (staged_ms * 1e-3) / 1e9) if staged_ms else None},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm",
                         "kernel": ("attn_splitkv_u8_mma_kernel (large batches) / attn_splitkv_u8_kernel" if u8
                                    else "attn_splitkv_kernel<32,4>"),
                         "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak if peak else None, "peak_source": peak_kind,
                         "traffic": traffic, "traffic_source": traffic_src, "avg_launch_ms": kern_avg_ms,
                         "launches_timed": int(kern_n),
                         "algorithmic_bytes_per_launch": bytes_per_layer,
                         "per_rank": per_rank,
                         "note": "achieved = the slowest rank's own algorithmic bytes over its own launch time"},
            "clocks": clocks,
            "host_and_device_paths_agree": same,
        }
        if whole_block:
            line["qkv_block"] = {
                "kernels": "subnorm_quant_kernel (quantiser only) + ternary_gemm_tc_kernel, one pair per layer",
                "avg_pair_ms": qb_ms / max(qb_n, 1), "pairs_timed": int(qb_n),
                "rows_per_pair": n_streams, "in_dim": Hq * D, "out_dim": (Hq + 2 * Hkv) * D}
        if out_block:
            line["out_block"] = {
                "kernels": "subnorm_quant_kernel + ternary_gemm_tc_kernel (tcgen05 kind::i8), one pair per layer",
                "avg_pair_ms": ob_ms / max(ob_n, 1), "pairs_timed": int(ob_n),
                "rows_per_pair": n_streams, "in_dim": Hq * D, "out_dim": Hq * D,
                "weight_bytes_per_layer": Hq * D * (Hq * D // 4)}

    # ---- CPU baseline on a bounded sample (rank 0, N=1 only) -------------------------------------
    if rank == 0 and world == 1 and not args.no_cpu and e2e_steps > 0 and not whole_block:
        sample = min(args.cpu_streams, n_streams)
        layer = layers // 2
        kv = []
        for i in range(sample):
            kk, vv = streams[i].read_range(layer, 0, int(lens[i]) - 1) if lens[i] > 1 else (
                np.zeros((Hkv, 0, D), np.float32), np.zeros((Hkv, 0, D), np.float32))
            kv.append((kk, vv))
        qs = [q_h[layer, i].numpy().reshape(1, Hq, 1, D) for i in range(sample)]
        ks = [k_h[layer, i].numpy().reshape(1, Hkv, 1, D) for i in range(sample)]
        vs = [v_h[layer, i].numpy().reshape(1, Hkv, 1, D) for i in range(sample)]
        if u8:   # the checker attends over what the u8 cache holds: the new rows round-tripped too
            import oracle as xo
            ks, vs = [xo.u8_round_trip(a) for a in ks], [xo.u8_round_trip(a) for a in vs]
        gbs, per_pass, outs, threads, reps = cpu_sample(lens[:sample], Hq, Hkv, D, kv, qs, ks, vs,
                                                        layer, budget_s=args.cpu_seconds)
        got = o_h[layer, :sample].numpy()
        want = np.stack([o.reshape(Hq, D) for o in outs])
        tol = "max_abs<=1e-4, rel_l2<=1e-5"
        if out_block:   # the checker runs the block too (not timed): oracle chain vs device chain
            import oracle as xo
            xo.set_quant_body(1)
            ref_lin = xo.TernaryLinear(Hq * D, Hq * D, xo.unpack_ternary(lin.packed, Hq * D * Hq * D),
                                       xo.PACK4, provided_scale=0.02)
            want = np.stack([xo.attention_out_block(o, norm_w, 1e-5, ref_lin).reshape(Hq, D) for o in outs])
            tol = "rel_l2<=1e-3 (an activation may quantise one step apart: the attention rows differ in the last bits)"
        max_abs = float(np.max(np.abs(got - want)))
        rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        line["cpu_baseline"] = {
            "value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{sample} of {n_streams} streams x 1 of {layers} layers (layer {layer}), "
                      f"{reps} passes of {per_pass * 1e3:.1f} ms, host nproc {os.cpu_count()}",
            "tokens_per_s": sample / per_pass}
        line["parity_vs_cpu_sample"] = {"max_abs": max_abs, "rel_l2": rel, "tolerance": tol}
    elif rank == 0:
        line["cpu_baseline"] = None
    if rank == 0 and world == 1 and whole_block and e2e_steps > 0 and not args.no_cpu:
        # the checker runs the whole block on a few streams (not timed): oracle chain vs device chain
        import oracle as xo
        xo.set_quant_body(1)
        layer, hidden = layers // 2, Hq * D
        mk = lambda l_, rows: xo.TernaryLinear(hidden, rows, xo.unpack_ternary(l_.packed, rows * hidden), xo.PACK4,
                                               provided_scale=float(l_.w_scales[0]))
        ref_q, ref_k, ref_v = (mk(l_, rows) for l_, rows in zip(qkv_lin, (Hq * D, Hkv * D, Hkv * D)))
        ref_o = mk(lin, hidden)
        worst = 0.0
        for i in range(min(4, n_streams)):
            L = int(lens[i])
            cache = xo.RingCache(1, Hkv, L, D)
            if L > 1:
                kk, vv = streams[i].read_range(layer, 0, L - 1)
                cache.append(0, 0, kk, vv)
            y_ref, _ = xo.causal_self_attention_forward(
                x_h[layer, i].numpy().reshape(1, 1, hidden), L - 1, 0, cache, rope[0], rope[1], ref_q, ref_k, ref_v,
                Hq, Hkv, D, norm_w, 1e-5, ref_o, kv_u8=u8)
            got = o_h[layer, i].numpy().reshape(1, 1, hidden)
            worst = max(worst, float(np.linalg.norm(got - y_ref) / np.linalg.norm(y_ref)))
        line["parity_vs_cpu_sample"] = {"rel_l2": worst, "streams": min(4, n_streams), "layer": layer,
                                        "tolerance": "rel_l2<=1e-3 (whole block; an activation may quantise one "
                                                     "step apart where the attention rows differ in the last bits)"}

    ctx.close()
    if rank == 0 and not args.no_prefill:
        # the other half of the metric: causal prefill TFLOP/s on the tensor-core kernel
        peak, peak_kind = load_tf32_peak()
        pre = {}
        for S in (2048, 8192):
            r = measure_prefill(xn, torch, tstream, local_rank, S, 20, 5, 128, 500000.0,
                                steps=10, warmup=3, e2e=(S == 2048), min_seconds=0.1)
            r["frac_of_tf32_peak"] = r["tflops"] / peak                 # the whole call: append + attention
            r["kernel_frac_of_tf32_peak"] = r["kernel_tflops"] / peak   # the tensor-core kernel alone
            pre[f"S{S}"] = r
        # chunked prefill (examples/chat.rs:297-306): 512-row chunks behind a long prefix
        r = measure_prefill(xn, torch, tstream, local_rank, 2048, 20, 5, 128, 500000.0, steps=10, warmup=3,
                            e2e=False, min_seconds=0.1, index_pos=6144, chunk=512)
        r["frac_of_tf32_peak"] = r["tflops"] / peak
        pre["S2048_chunks512_at6144"] = r
        # the exact-f32 path (XN_PREFILL_F32): the tiled CUDA-core kernel, and beside it the row-wise
        # stand-in it replaced (every query row served as a decode unit by the split-KV kernel)
        f32 = {}
        for name, env in (("tiled_kernel", "1"), ("row_wise", "0")):
            os.environ["XORNET_ATTN_F32_TILED"] = env
            r = measure_prefill(xn, torch, tstream, local_rank, 2048, 20, 5, 128, 500000.0, steps=5, warmup=3,
                                e2e=False, min_seconds=0.05, prefill_mode=1)
            f32[name] = {"ms": r["ms"], "tflops": r["tflops"], "kernel_ms": r["kernel_ms"]}
        os.environ.pop("XORNET_ATTN_F32_TILED", None)
        f32["note"] = "f32 CUDA-core math: against the 2 x 74 TFLOP/s an SM's FMA pipes allow, not the tensor peak"
        pre["S2048_exact_f32"] = f32
        line["prefill"] = {"kernel": "prefill_tf32_kernel (tcgen05 TF32, TMEM accumulators)",
                           "shape": "1 sequence, 20/5 heads, head_dim 128, fused RoPE + append",
                           "tf32_peak_tflops": peak, "peak_source": peak_kind,
                           "library_tf32_matmul_tflops": tf32_matmul_tflops(torch), **pre}
    if rank == 0 and world == 1 and not args.no_extras and args.workload == "c3":
        # the other workload shapes, one short summary each
        c1 = measure_decode(xn, torch, tstream, local_rank, [1024], 20, 5, 128, 1, steps=200)
        c1["workload"] = WORKLOADS["c1"][-1]
        c1["note"] = "5.3 MB per launch: bound by launch and hand-over latency, not by HBM"
        lens5 = stream_lengths(8 * 32, 2048, 8192, BASE_SEED + 5000)
        own5 = place_streams(xn, lens5, 8, args.placement)
        c5 = measure_decode(xn, torch, tstream, local_rank, [int(L) for i, L in enumerate(lens5) if own5[i] == 0],
                            32, 8, 128, 32, steps=3)
        c5["workload"] = WORKLOADS["c5"][-1] + " (one GPU's share of 256 streams placed over 8 GPUs)"
        c4p = measure_prefill(xn, torch, tstream, local_rank, 1024, 32, 32, 100, 10000.0, steps=10, warmup=3,
                              e2e=False, min_seconds=0.1, n_seqs=8)
        c4p["frac_of_tf32_peak"] = c4p["tflops"] / peak
        c4p["kernel_frac_of_tf32_peak"] = c4p["kernel_tflops"] / peak
        c4p["roofline"] = {"bound": "tensor", "achieved": c4p["kernel_tflops"], "peak": peak, "unit": "TFLOP/s",
                           "frac": c4p["kernel_tflops"] / peak, "peak_source": peak_kind,
                           "note": "flops counted with head_dim 100; the kernel pads rows to 104 / 112 columns"}
        c4d = measure_decode(xn, torch, tstream, local_rank, [1025] * 8, 32, 32, 100, 1, steps=256, grow=True,
                             theta=10000.0)
        line["configs"] = {"c1": c1, "c5": c5,
                           "c4": {"workload": "BitNet-3B shape: 32/32 heads, head_dim 100, RoPE theta 1e4, 8 sequences: "
                                              "1024-token prefill, then 256 decode steps that append",
                                  "prefill": c4p, "decode": c4d}}
        line["e2e"]["dropin"] = run_dropin_leg(xn, 64, 30, 20, 5, 128, 128, 4096, steps=10, warmup=2,
                                               device=local_rank, pool_mb=28000)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-streams", type=int, default=16, help="streams in the CPU sample")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="time budget of the CPU sample")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill summary")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the summaries of the other workload shapes and the drop-in leg")
    ap.add_argument("--seq", type=int, default=0, help="prefill length for --workload c2")
    ap.add_argument("--min-seconds", type=float, default=0.5,
                    help="keep repeating the timed bracket until it has covered this much device time")
    ap.add_argument("--f32", action="store_true", help="c2: the exact-f32 prefill path (XN_PREFILL_F32)")
    ap.add_argument("--pos", type=int, default=0, help="c2: cached tokens in front of the prefill (index_pos)")
    ap.add_argument("--chunk", type=int, default=0, help="c2: feed the prefill in chunks of this many rows")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiling)")
    ap.add_argument("--streams", type=int, default=0, help="override streams per GPU (profiling)")
    ap.add_argument("--placement", default="least", choices=["least", "rr"],
                    help="which GPU a stream lives on: least-loaded by announced tokens, or stream id mod GPUs")
    ap.add_argument("--kv", default="f32", choices=["f32", "u8"],
                    help="KV cache format of the decode workloads (u8: the opt-in compressed pages)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.workload == "c2":
        return run_prefill_arm(args)
    if args.workload == "c5p":
        return run_split_prefill_arm(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
