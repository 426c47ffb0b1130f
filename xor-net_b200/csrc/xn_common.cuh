// Shared device helpers and host/device plan structures for the sm_100a attention kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace xn {

constexpr int kPageTokens = 64;  // tokens per KV page

// Device error word values written by kernels whose bounded waits ran out.
enum : int { kDevOk = 0, kDevWaitFull = 1, kDevWaitEmpty = 2, kDevBadIndex = 3, kDevWaitMma = 4 };

// The status word lives in page-locked host memory mapped into the device: a plain store, made
// visible to the host, is all a kernel needs when one of its bounded waits ran out.
__device__ __forceinline__ void report_status(int* status, int code) {
    *reinterpret_cast<volatile int*>(status) = code;
    __threadfence_system();
}

// Opt-in build (-DXN_BOUNDS) in which the copy producers range-check every page id they take
// from a host-built table: a bad one is reported through the status word (kDevBadIndex) and its
// copy is not issued -- the kernel gives up and returns, it never traps.  The default build trusts
// the planner.
#ifdef XN_BOUNDS
#define XN_PAGE_OK(page, pool_pages) ((page) >= 0 && (long long)(page) < (long long)(pool_pages))
#else
#define XN_PAGE_OK(page, pool_pages) true
#endif

// ---- plan structures (built on the host per batch, copied once to the device) ---------------

// One attention request as the kernels see it.  Strides are in floats.
struct ReqDev {
    const float* q;    // rotated query rows (user memory, staged copy, or the rotation scratch)
    const float* k;    // new keys   (input to the append kernel)
    const float* v;    // new values
    const float* q_in; // query rows as supplied (input to the append kernel when rotating)
    float* out;
    long long q_hs, q_ts;     // query head / token strides of `q`
    long long qi_hs, qi_ts;   // strides of `q_in`
    long long kv_hs, kv_ts;   // strides of k and v
    long long o_hs, o_ts;     // output strides
    int page_off;             // offset of this stream's page ids inside the plan's page array
    int layer;
    int seq_len;
    int index_pos;
    int cap;                  // ring capacity (positions fold modulo cap)
    int n_pages;
    unsigned flags;           // bit 0: rotate q and k with the context tables; bit 1: copy q
                              // (unrotated) into the scratch `q` points at; bit 3: one new
                              // token, appended (and rotated) by the attention kernel itself;
                              // bit 4: the prefill kernel rotates the query rows (the append
                              // kernel leaves them alone)
    int pad;
};

// What differs between two decode submissions of the same geometry (the same streams at the same
// positions, e.g. the layers of one decode step): the tensors' addresses and the layer.  Passed as
// a kernel parameter, it lets a launch reuse the plan the previous submission left on the device.
constexpr int kPatchReqs = 128;
struct ReqPatch {
    const float* q;
    const float* k;
    const float* v;
    float* out;
};
struct ReqPatchTable {
    int n;        // 0: the request descriptors are used as they are
    int layer;
    long long pad;
    ReqPatch e[kPatchReqs];
};

// A (request, KV head, query-head subgroup, query row) to attend over kv_len cached tokens.
struct UnitDev {
    int req;
    int kv_head;
    int head0;      // first query head of the subgroup
    int nheads;     // query heads in the subgroup (<= template GT)
    int t_q;        // query row within the request
    int kv_len;     // cached tokens to attend (index_pos + t_q + 1)
    int part_begin; // first partial slot, or -1 when the unit is written directly
    int part_count;
    int merge_slot; // arrival counter of a cut unit
    int store_new;  // fused append: this unit writes the new token's K/V rows into the cache
};

// A contiguous tile range of one unit given to one thread block.
struct ItemDev {
    int unit;
    int tile_begin;
    int tile_end;
    int part;  // partial slot or -1 (direct)
};

// ---- PTX wrappers: mbarrier + bulk async copy (TMA engine, no tensor map, no multicast) ------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// try_wait with a suspend-time hint: the thread may sleep in hardware, for up to about `hint_ns`,
// until the phase completes.  A polling loop without the hint re-issues the instruction back to
// back, and a handful of polling warps then crowd the copy producer's and the MMA issuer's own
// barrier and copy instructions out of the SM's memory-instruction queue.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}

// Waits for the given phase parity at most `limit_ns` (default ~2 s).  Returns false when it
// gave up; the caller records an error code and leaves its loop, so a lost copy can never hang
// the GPU.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  unsigned long long limit_ns = 2000000000ull) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = 0;
    for (uint32_t spins = 1;; ++spins) {
        if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
        if ((spins & 0x3fu) == 0) {
            unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) return false;
        }
    }
}

// Non-blocking test of the phase, and a bounded wait built on it: the thread keeps polling, so it
// notices the completion within a few cycles (try_wait may park the thread and wake it late),
// at the price of occupying the shared-memory pipe.  For waits on a kernel's critical hand-offs.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool mbar_spin_bounded(uint64_t* bar, uint32_t parity,
                                                  unsigned long long limit_ns = 2000000000ull) {
    unsigned long long t0 = 0;
    for (uint32_t spins = 1;; ++spins) {
        if (mbar_test_wait(bar, parity)) return true;
        if ((spins & 0xfffu) == 0) {
            unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) return false;
        }
    }
}

// The same poll with a short sleep between two tests, for waits that usually last long (a whole
// work item): the thread stays off the shared-memory pipe most of the time and still notices the
// completion within about `sleep_ns` (a parked try_wait was seen to wake tens of microseconds late).
__device__ __forceinline__ bool mbar_poll_sleep_bounded(uint64_t* bar, uint32_t parity, unsigned sleep_ns,
                                                        unsigned long long limit_ns = 2000000000ull) {
    unsigned long long t0 = 0;
    for (uint32_t spins = 1;; ++spins) {
        if (mbar_test_wait(bar, parity)) return true;
        __nanosleep(sleep_ns);
        if ((spins & 0xffu) == 0) {
            unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) return false;
        }
    }
}

// One lane polls for the warp and the result is broadcast.  The __syncwarp() behind the broadcast
// is needed: it reconverges the warp (without it, warp shuffles that followed such a wait were
// seen to exchange wrong lanes' values) and orders the other lanes' later reads behind the
// poller's acquire.
__device__ __forceinline__ bool warp_spin_bounded(uint64_t* bar, uint32_t parity, int lane) {
    int ok = 1;
    if (lane == 0) ok = mbar_spin_bounded(bar, parity) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    return ok != 0;
}
__device__ __forceinline__ bool warp_poll_sleep_bounded(uint64_t* bar, uint32_t parity, int lane,
                                                        unsigned sleep_ns) {
    int ok = 1;
    if (lane == 0) ok = mbar_poll_sleep_bounded(bar, parity, sleep_ns) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    return ok != 0;
}

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.  Both addresses
// must be 16-byte aligned and bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- programmatic dependent launch ------------------------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may start while its
// predecessor in the stream still runs, once every block of the predecessor has called
// pdl_launch_dependents() (or exited); it must call pdl_wait() before it touches anything the
// predecessor writes (the wait returns when the predecessor has completed and flushed).
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- counter-based N(0,1) generator ---------------------------------------------------------

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float normal_from(uint64_t seed, uint64_t idx) {
    uint64_t r = mix64(seed * 0xD1342543DE82EF95ull + idx);
    uint32_t a = static_cast<uint32_t>(r), b = static_cast<uint32_t>(r >> 32);
    float u1 = (static_cast<float>(a >> 8) + 1.0f) * (1.0f / 16777217.0f);  // (0,1)
    float u2 = static_cast<float>(b >> 8) * (1.0f / 16777216.0f);           // [0,1)
    return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}

}  // namespace xn
