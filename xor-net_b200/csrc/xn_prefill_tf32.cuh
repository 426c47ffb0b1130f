// Causal prefill attention on the 5th-generation tensor cores (tcgen05, TF32 inputs, f32
// accumulators in tensor memory), sm_100a only.
//
// Replaces, for long prompts, the per-row loop of the reference (src/nn/fast_attention.rs:
// 157-198): S = Q K^T and O = P V become tcgen05.mma.kind::tf32 instructions; the causal loop
// bound `limit = index_pos + t_q` (:162) becomes "key tiles above the diagonal are never issued,
// the diagonal tile is masked element-wise".
//
// One thread block = one (query head, 128-row query tile).  A score tile spans 128 keys = two of
// the cache's 64-token pages (a tcgen05.mma of this kind costs the same for N = 64 and N = 128).
// Tensor memory (512 columns): Q [0,128) | two S/P buffers [128,384) | O [384,512).
// Roles (320 threads):
//   warp 0      TMA producer: tensor-map loads of K tiles (2 stages of 2 pages, 128-byte swizzle)
//               and V pages (3 stages, 128-byte swizzle of 32-byte chunks), mbarrier byte counts;
//   warp 1      MMA issuer (one lane): S_j = Q K_j^T with Q read from tensor memory, issued one
//               tile ahead of O += P_j V_j, which reads P from tensor memory (P overwrites S_j
//               in place) and V MN-major straight from its [token][dim] page; tcgen05.commit
//               signals the mbarriers;
//   warps 2..9  two softmax warpgroups; thread r of each owns query row r, warpgroup 0 the first
//               page of every score tile, warpgroup 1 the second.  Prologue: Q goes global ->
//               shared memory (whole rows per warp instruction) -> registers -> tensor memory
//               (rounded to TF32); for head_dim 64 / 128 the rotary
//               embedding of the query rows (src/tensor.rs:295-316, call site
//               src/models/llama/attention.rs:88) is applied on the way, with the append
//               kernel's unfused arithmetic, so the append kernel handles K and V only and the
//               prologue does not wait for it.  Per tile: tcgen05.ld of the S
//               row, causal mask, row maximum exchanged between the two warpgroups through
//               shared memory, exp2 with the softmax scale folded into one FMA, P written back
//               with tcgen05.st.  The accumulator is rescaled lazily: only when a row's maximum
//               grows by more than 2^8.  Epilogue: O / l to global.
// The kernel may be launched as a programmatic dependent of the append kernel: its blocks set up
// (barriers, tensor memory) while that kernel drains and wait for it before their first read.
// Every wait is bounded; on expiry the kernel records a status code, drains and returns.
#pragma once
#include <cuda.h>

#include "xn_common.cuh"

namespace xn {

struct PrefillArgs {
    const float* q;       // queries: rotated already (rope_q == 0) or as supplied (rope_q == 1)
    long long q_hs, q_ts; // query head / token strides in floats
    const float* cos_t;   // rotary tables [position][head_dim / 2], read when rope_q
    const float* sin_t;
    int rope_q;           // rotate the query rows in the prologue (head_dim 64 or 128 only)
    const int* pages;     // page ids of the stream (device)
    float* out;           // output base
    long long o_hs, o_ts; // output head / token strides in floats
    long long layer_page_base;  // layer * pool_pages
    long long pool_pages;       // pages per layer (the bounds-checking build checks page ids against it)
    int num_kv_heads;
    int group;            // query heads per KV head
    int seq_len;          // S
    int index_pos;        // P
    int head_dim;         // D (multiple of 4, 16..128)
    float scale_log2;     // (1/sqrt(D)) * log2(e)
    int* status;
};

// One thread block of a launch that serves several requests: which request, which query tile,
// which head.  The host orders the blocks by score tiles, heaviest first, across all requests.
struct PrefillBlock {
    int req;
    int qt;
    int head;
    int pad;
};

namespace pf {

constexpr int kBM = 128;          // query rows per block
constexpr int kPage = 64;         // tokens per cache page
constexpr int kBN = 128;          // keys per score tile (= 2 pages): N of the S = Q K^T MMA
constexpr int kKB = 4;            // 32-float (128-byte) column blocks per row, at most
constexpr int kKSub = kBN * 128;  // bytes of one K column block   [128 rows x 128 B]
constexpr int kVSub = kPage * 128;// bytes of one V column block   [64 rows x 128 B]
constexpr int kKBytes = kKB * kKSub;     // 64 KB per K tile
constexpr int kVBytes = kKB * kVSub;     // 32 KB per V page
constexpr int kKStages = 2;       // K tiles in flight
constexpr int kVStages = 3;       // V pages in flight
constexpr int kSBufs = 2;         // score / probability buffers in tensor memory
constexpr int kSmemData = kKStages * kKBytes + kVStages * kVBytes;  // 224 KB
constexpr int kSmemBytes = kSmemData + 1024 /* alignment slack */ + 2048 /* barriers, exchange */;
constexpr int kThreads = 320;     // TMA warp, MMA warp, two softmax warpgroups
constexpr int kTmemCols = 512;
constexpr int kTmemQ = 0;         // 128 columns
constexpr int kTmemS = 128;       // kSBufs x 128 columns
constexpr int kTmemO = 384;       // 128 columns
constexpr float kRescaleThreshold = 8.0f;  // log2 units

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma.
//   bits [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte
//   offset >> 4, [46,48) descriptor version (1 on sm_100), [61,64) layout:
//   2 = 128-byte swizzle of 16-byte chunks (K-major operands, TMA SWIZZLE_128B);
//   1 = 128-byte swizzle of 32-byte chunks, the only layout the tensor cores accept for an
//       MN-major TF32 operand (TMA SWIZZLE_128B_ATOM_32B; the pattern repeats every 4 rows).
constexpr uint32_t kLayoutSw128 = 2, kLayoutSw128Base32 = 1;
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout) {
    uint64_t d = 0;
    d |= uint64_t((saddr >> 4) & 0x3fff);
    d |= uint64_t((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= uint64_t((sbo_bytes >> 4) & 0x3fff) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(layout) << 61;
    return d;
}

// Instruction descriptor, kind::tf32, f32 accumulate: [4,6) D format 1 = f32, [7,10) A format
// 2 = tf32, [10,13) B format 2 = tf32, bit 15 A major, bit 16 B major (1 = MN-major),
// [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(b_mn_major) << 16) |
           (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, "
        "%12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, "
        "%30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, "
        "%12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, "
        "%30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
        : "memory");
}

// A 16-byte read-only load the compiler keeps where it is written: the prologue issues the loads of
// eight rows back to back and only then starts to consume them.
__device__ __forceinline__ float4 ldg_keep(const float* p) {
    float4 v;
    asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Round an f32 to the nearest TF32 (ties away from zero): the tensor core drops the low 13
// mantissa bits, so adding half an ulp of the kept part to the bit pattern rounds the magnitude.
__device__ __forceinline__ uint32_t round_tf32(uint32_t bits) { return bits + 0x1000u; }

}  // namespace pf

// MULTI: one launch for several requests (a batch of prompts): the block reads its request's
// arguments and its (query tile, head) from tables the host placed in the plan.
template <bool MULTI>
__global__ void __launch_bounds__(pf::kThreads, 1)
prefill_tf32_kernel(const __grid_constant__ CUtensorMap k_map,
                    const __grid_constant__ CUtensorMap v_map, const PrefillArgs a_one,
                    const PrefillArgs* __restrict__ table, const PrefillBlock* __restrict__ blocks) {
    using namespace pf;
    PrefillBlock pb = {0, 0, 0, 0};
    if (MULTI) pb = blocks[blockIdx.x];
    const PrefillArgs a = MULTI ? table[pb.req] : a_one;
    extern __shared__ unsigned char smem_dyn[];
    // 128-byte swizzled tiles want 1024-byte alignment
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    unsigned char* k_s = smem;
    unsigned char* v_s = k_s + kKStages * kKBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemData);
    uint64_t* q_ready = bars + 0;
    uint64_t* k_full = bars + 1;                 // [kKStages]
    uint64_t* k_empty = k_full + kKStages;       // [kKStages]
    uint64_t* v_full = k_empty + kKStages;       // [kVStages]
    uint64_t* v_empty = v_full + kVStages;       // [kVStages]
    uint64_t* s_full = v_empty + kVStages;       // [kSBufs]
    uint64_t* p_full = s_full + kSBufs;          // [kSBufs]
    uint64_t* pv_done = p_full + kSBufs;         // [kSBufs]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + kSBufs);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);
    volatile int* sm_dead = abort_flag + 1;  // written and read by the softmax warps only
    float* xchg = reinterpret_cast<float*>(bars + 32);  // [2 warpgroups][128 rows]
    static_assert((1 + 2 * kKStages + 2 * kVStages + 3 * kSBufs) * 8 + 16 <= 256, "barrier area");

    pdl_launch_dependents();   // see attn_splitkv_kernel
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // 1-D grid, longest query tiles first across ALL heads (blocks are handed to SMs in index
    // order, so the causal triangle is packed heaviest-first); neighbouring blocks are the heads
    // of one KV group on the same rows, which keeps their shared K/V pages hot in L2.
    const int n_qtiles = (a.seq_len + kBM - 1) / kBM;
    const int n_heads = a.num_kv_heads * a.group;
    const int qt = MULTI ? pb.qt : n_qtiles - 1 - int(blockIdx.x) / n_heads;
    const int h = MULTI ? pb.head : int(blockIdx.x) % n_heads;
    const int h_kv = h / a.group;
    const int t0 = qt * kBM;
    const int last_row = min(t0 + kBM, a.seq_len) - 1;
    const int n_pages = (a.index_pos + last_row) / kPage + 1;  // cache pages this block reads
    const int n_tiles = (n_pages + 1) / 2;                     // 128-key score tiles
    const int D = a.head_dim;
    const int n_kb = (D + 31) / 32;        // column blocks actually loaded
    const int k_steps = (D + 7) / 8;       // K=8 MMA steps over head_dim
    const int n_pv = (D + 15) / 16 * 16;   // N of the PV MMA

    if (tid == 0) {
        mbar_init(q_ready, 256);
        for (int s = 0; s < kKStages; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
        }
        for (int s = 0; s < kVStages; ++s) {
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int s = 0; s < kSBufs; ++s) {
            mbar_init(&s_full[s], 1);
            mbar_init(&p_full[s], 256);
            mbar_init(&pv_done[s], 1);
        }
        *abort_flag = 0;
        *sm_dead = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(uint32_t(kTmemCols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_q = tmem_base + kTmemQ;
    const uint32_t tmem_s = tmem_base + kTmemS;
    const uint32_t tmem_o = tmem_base + kTmemO;

    if (warp == 0) {
        // =============================== TMA producer ===============================
        // Order of issue = order of consumption by the MMA warp: K tile j+1 is wanted before the
        // V pages of tile j.
        if (lane == 0) {
            pdl_wait();   // the pages (and the page table) are written before this kernel: wait for the append
            bool bad_page = false;   // bounds-checking build only
            auto page_row = [&](int pg) -> int {
                if (!XN_PAGE_OK(a.pages[pg], a.pool_pages)) { bad_page = true; return -1; }
                return int(((a.layer_page_base + a.pages[pg]) * a.num_kv_heads + h_kv) * kPage);
            };
            auto load_k_tile = [&](int j) -> bool {
                const int st = j % kKStages;
                if (j >= kKStages && !mbar_poll_sleep_bounded(&k_empty[st], uint32_t((j / kKStages - 1) & 1), 64u)) return false;
                const int np = min(2, n_pages - 2 * j);
                int rows[2] = {0, 0};
                for (int p = 0; p < np; ++p) rows[p] = page_row(2 * j + p);
                if (bad_page) return false;   // before any byte count is armed: nothing is in flight
                mbar_arrive_expect_tx(&k_full[st], uint32_t(np * n_kb) * kVSub);
                for (int p = 0; p < np; ++p) {
                    const int row = rows[p];
                    for (int kb = 0; kb < n_kb; ++kb)
                        tma_load_2d(k_s + st * kKBytes + kb * kKSub + p * kVSub, &k_map, kb * 32, row, &k_full[st]);
                }
                return true;
            };
            auto load_v_page = [&](int pg) -> bool {
                const int st = pg % kVStages;
                // stages 1 and 2 stage the query tile first: page 1 is the first to go there
                if (pg == 1 && !mbar_poll_sleep_bounded(q_ready, 0, 64u)) return false;
                if (pg >= kVStages && !mbar_poll_sleep_bounded(&v_empty[st], uint32_t((pg / kVStages - 1) & 1), 64u)) return false;
                const int row = page_row(pg);
                if (bad_page) return false;
                mbar_arrive_expect_tx(&v_full[st], uint32_t(n_kb) * kVSub);
                for (int kb = 0; kb < n_kb; ++kb)
                    tma_load_2d(v_s + st * kVBytes + kb * kVSub, &v_map, kb * 32, row, &v_full[st]);
                return true;
            };
            bool ok = load_k_tile(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) ok = load_k_tile(j + 1);
                for (int p = 2 * j; p < min(2 * j + 2, n_pages) && ok; ++p) ok = load_v_page(p);
                if (*abort_flag) break;
            }
            if (!ok) { report_status(a.status, bad_page ? kDevBadIndex : kDevWaitEmpty); *abort_flag = 1; }
        }
    } else if (warp == 1) {
        // =============================== MMA issuer ===============================
        // One lane issues every tcgen05.mma of the block, so its instruction stream is kept
        // short: descriptors are a constant plus a small offset, ring positions and mbarrier
        // parities are carried as counters, and the head_dim = 128 loops are fully unrolled.
        // A tcgen05.mma of this kind costs about the same for N = 64 and N = 128, which is why
        // the score tile spans two pages.
        if (lane == 0) {
            const uint32_t idesc_qk = make_idesc(kBM, kBN, 0);
            const uint32_t idesc_pv = make_idesc(kBM, n_pv, 1);
            // descriptors of stage 0; offsets are in 16-byte units
            const uint64_t kdesc0 = smem_desc(smem_u32(k_s), 0, 1024, kLayoutSw128);
            const uint64_t vdesc0 = smem_desc(smem_u32(v_s), kVSub, 512, kLayoutSw128Base32);
            constexpr uint64_t kKStageStep = uint64_t(kKBytes) >> 4;
            constexpr uint64_t kVStageStep = uint64_t(kVBytes) >> 4;
            constexpr uint64_t kKBlockStep = uint64_t(kKSub) >> 4;  // next 32-float column block
            bool ok = mbar_spin_bounded(q_ready, 0);
            if (!ok) { report_status(a.status, kDevWaitFull); *abort_flag = 1; }
            fence_after_sync();

            int k_st = 0, k_ph = 0;     // K ring position / parity of the next S = Q K^T
            int v_st = 0, v_ph = 0;     // V ring position / parity of the next page of O += P V
            int pv_issued = 0;          // tiles whose O += P V has been issued

            auto issue_qk = [&](int j) -> bool {
                if (!mbar_spin_bounded(&k_full[k_st], uint32_t(k_ph))) return false;
                fence_after_sync();
                const uint64_t kd = kdesc0 + uint64_t(k_st) * kKStageStep;
                const uint32_t d_addr = tmem_s + (j & 1) * kBN;
                if (k_steps == 16) {
#pragma unroll
                    for (int ks = 0; ks < 16; ++ks)
                        mma_ts(d_addr, tmem_q + ks * 8, kd + (ks >> 2) * kKBlockStep + (ks & 3) * 2, idesc_qk,
                               ks > 0 ? 1u : 0u);
                } else {
                    for (int ks = 0; ks < k_steps; ++ks)
                        mma_ts(d_addr, tmem_q + ks * 8, kd + (ks >> 2) * kKBlockStep + (ks & 3) * 2, idesc_qk,
                               ks > 0 ? 1u : 0u);
                }
                mma_commit(&k_empty[k_st]);
                mma_commit(&s_full[j & 1]);
                if (++k_st == kKStages) { k_st = 0; k_ph ^= 1; }
                return true;
            };
            // O += P_j V_j, one page (64 keys, 8 MMAs) at a time.  V is [token][dim]: MN-major B;
            // 8 tokens = 1024 B inside each column block, column blocks kVSub apart (leading
            // offset), 4-token swizzle groups 512 B apart (stride offset).
            auto issue_pv = [&](int j) -> bool {
                if (!mbar_spin_bounded(&p_full[j & 1], uint32_t((j >> 1) & 1))) return false;
                const int np = min(2, n_pages - 2 * j);
                for (int p = 0; p < np; ++p) {
                    if (!mbar_spin_bounded(&v_full[v_st], uint32_t(v_ph))) return false;
                    fence_after_sync();
                    const uint64_t vd = vdesc0 + uint64_t(v_st) * kVStageStep;
                    const uint32_t p_addr = tmem_s + (j & 1) * kBN + p * kPage;
                    const uint32_t first = (j > 0 || p > 0) ? 1u : 0u;
#pragma unroll
                    for (int ks = 0; ks < kPage / 8; ++ks)
                        mma_ts(tmem_o, p_addr + ks * 8, vd + ks * 64, idesc_pv, ks > 0 ? 1u : first);
                    mma_commit(&v_empty[v_st]);
                    if (++v_st == kVStages) { v_st = 0; v_ph ^= 1; }
                }
                mma_commit(&pv_done[j & 1]);
                ++pv_issued;
                return true;
            };
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (!issue_qk(j)) { ok = false; break; }
                if (j >= 1 && !issue_pv(j - 1)) { ok = false; break; }
            }
            if (ok && !issue_pv(n_tiles - 1)) ok = false;
            if (!ok) { report_status(a.status, kDevWaitMma); *abort_flag = 1; }
        }
    } else {
        // =============================== softmax + epilogue ===============================
        // Two warpgroups; both own all 128 rows (thread r of each = query row r).  Warpgroup 0
        // handles the first page (columns 0..63) of every score tile, warpgroup 1 the second;
        // they exchange their row maxima through shared memory so that both scale with the same
        // reference, and each keeps its own partial row sum.
        constexpr unsigned kFull = 0xffffffffu;
        const int wg = (warp - 2) >> 2;          // 0 or 1
        const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
        const int r = quarter * 32 + lane;       // query row inside the tile
        const uint32_t lane_base = uint32_t(quarter * 32) << 16;
        const int t = t0 + r;                    // query row inside the request
        const int pq = a.index_pos + t;          // its absolute position
        const int col0 = wg * kPage;             // this warpgroup's columns of a score tile
        auto wg_barrier = [&]() { named_bar_sync(1, 256); };

        // ---- prologue: Q -> tensor memory (rounded to TF32)
        // Global -> shared memory with whole rows per warp instruction (a thread reading its own
        // row would touch 32 cache lines per instruction), optionally rotating on the way, then
        // shared -> registers -> tensor memory with thread r owning row r.  The staging tile sits
        // in V stages 1 and 2, which the TMA warp leaves alone until q_ready completes.
        // 16-byte chunk c of row r sits at chunk position c ^ (r & 31): conflict-free both ways.
        {
            float4* qs = reinterpret_cast<float4*>(v_s + kVBytes);   // [128 rows][32 chunks]
            const int w8 = warp - 2;        // 0..7: rows [16 w8, 16 w8 + 16) of the tile
            const int n_ch = D >> 2;        // 16-byte chunks per row
            const bool rope = a.rope_q != 0;
            const int half_ch = n_ch >> 1;  // rope: 8 or 16; pair i of a row is (x[i], x[i + D/2])
            // rotated rows come out of the append kernel's scratch: wait for it; rows rotated here
            // are the caller's own and need no wait
            if (!rope) pdl_wait();
            const float* qbase = a.q + size_t(h) * a.q_hs;
            if (!rope) {
                // sixteen rows, one 16-byte chunk per lane and row, all loads issued before the first use
                float4 x[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int tt = t0 + w8 * 16 + i;
                    x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (tt < a.seq_len && lane < n_ch) x[i] = ldg_keep(qbase + size_t(tt) * a.q_ts + lane * 4);
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int rr = w8 * 16 + i;
                    uint4 xr;   // rows past the end and chunks past head_dim were loaded as zeros
                    xr.x = round_tf32(__float_as_uint(x[i].x));
                    xr.y = round_tf32(__float_as_uint(x[i].y));
                    xr.z = round_tf32(__float_as_uint(x[i].z));
                    xr.w = round_tf32(__float_as_uint(x[i].w));
                    reinterpret_cast<uint4*>(qs)[rr * 32 + (lane ^ (rr & 31))] = xr;
                }
            } else {
                // Rotating: a lane owns pair-chunk p of a row: it loads x[4p..4p+3], x[D/2 + 4p..], and
                // the cos and sin chunks of the row's position, and produces both rotated chunks.
                // half_ch lanes cover a row, so one instruction serves 32 / half_ch rows (2 for
                // head_dim 128, 4 for 64); the 16 rows of the warp take 8 (4) such steps, whose loads
                // are all issued before the first is used.
                const int pch = lane & (half_ch - 1);
                const int rsub = lane / half_ch;
                const int rows_per_step = 32 / half_ch;
                const int n_steps = 16 / rows_per_step;
                const int half = D >> 1;
                float4 lo[8], hi[8], cv[8], sv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int tt = t0 + w8 * 16 + i * rows_per_step + rsub;
                    lo[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    hi[i] = lo[i];
                    cv[i] = lo[i];
                    sv[i] = lo[i];
                    if (i < n_steps && tt < a.seq_len) {
                        const float* qrow = qbase + size_t(tt) * a.q_ts + pch * 4;
                        const size_t trow = size_t(a.index_pos + tt) * size_t(half) + size_t(pch) * 4;
                        lo[i] = ldg_keep(qrow);
                        hi[i] = ldg_keep(qrow + half);
                        cv[i] = ldg_keep(a.cos_t + trow);
                        sv[i] = ldg_keep(a.sin_t + trow);
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (i >= n_steps) break;
                    const int rr = w8 * 16 + i * rows_per_step + rsub;
                    // the append kernel's arithmetic (unfused): lo' = lo c - hi s, hi' = lo s + hi c
                    uint4 l4, h4;
                    l4.x = round_tf32(__float_as_uint(__fsub_rn(__fmul_rn(lo[i].x, cv[i].x), __fmul_rn(hi[i].x, sv[i].x))));
                    l4.y = round_tf32(__float_as_uint(__fsub_rn(__fmul_rn(lo[i].y, cv[i].y), __fmul_rn(hi[i].y, sv[i].y))));
                    l4.z = round_tf32(__float_as_uint(__fsub_rn(__fmul_rn(lo[i].z, cv[i].z), __fmul_rn(hi[i].z, sv[i].z))));
                    l4.w = round_tf32(__float_as_uint(__fsub_rn(__fmul_rn(lo[i].w, cv[i].w), __fmul_rn(hi[i].w, sv[i].w))));
                    h4.x = round_tf32(__float_as_uint(__fadd_rn(__fmul_rn(lo[i].x, sv[i].x), __fmul_rn(hi[i].x, cv[i].x))));
                    h4.y = round_tf32(__float_as_uint(__fadd_rn(__fmul_rn(lo[i].y, sv[i].y), __fmul_rn(hi[i].y, cv[i].y))));
                    h4.z = round_tf32(__float_as_uint(__fadd_rn(__fmul_rn(lo[i].z, sv[i].z), __fmul_rn(hi[i].z, cv[i].z))));
                    h4.w = round_tf32(__float_as_uint(__fadd_rn(__fmul_rn(lo[i].w, sv[i].w), __fmul_rn(hi[i].w, cv[i].w))));
                    uint4* row = reinterpret_cast<uint4*>(qs) + rr * 32;
                    row[pch ^ (rr & 31)] = l4;
                    row[(pch + half_ch) ^ (rr & 31)] = h4;
                    // chunks past head_dim (head_dim 64: chunks 16..31) must read as zeros
                    if (n_ch < 32) {
                        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                        row[(pch + 2 * half_ch) ^ (rr & 31)] = z;
                        row[(pch + 3 * half_ch) ^ (rr & 31)] = z;
                    }
                }
            }
            wg_barrier();
            for (int c0 = col0; c0 < min(col0 + kPage, k_steps * 8); c0 += 32) {
                uint32_t qv[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v4 = reinterpret_cast<const uint4*>(qs)[r * 32 + (((c0 >> 2) + c) ^ (r & 31))];
                    qv[4 * c] = v4.x;
                    qv[4 * c + 1] = v4.y;
                    qv[4 * c + 2] = v4.z;
                    qv[4 * c + 3] = v4.w;
                }
                tmem_st32(tmem_q + lane_base + c0, qv);
            }
            tmem_wait_st();
            fence_before_sync();
            mbar_arrive(q_ready);
        }

        float m_ref = -INFINITY, l_sum = 0.f;
        bool dead = false;
        for (int j = 0; j < n_tiles; ++j) {
            const int sb = j & 1;
            if (!warp_spin_bounded(&s_full[sb], uint32_t((j >> 1) & 1), lane)) dead = true;
            // all eight warps must take the same exit: agree through a flag only they write
            if (lane == 0 && dead) { *sm_dead = 1; *abort_flag = 1; }
            fence_after_sync();
            uint32_t x0[32], x1[32];
            const uint32_t s_addr = tmem_s + lane_base + sb * kBN + col0;
            const int key0 = j * kBN + col0;                  // first key of this warpgroup's page
            const bool have_page = 2 * j + wg < n_pages;      // the tile's second page may not exist
            float mx = -INFINITY;
            if (!dead && have_page) {
                tmem_ld32(s_addr, x0);
                tmem_ld32(s_addr + 32, x1);
                tmem_wait_ld();
                if (key0 + kPage - 1 > a.index_pos + t0) {    // some row masks some key here
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        if (key0 + c > pq) x0[c] = 0xff800000u;  // -inf
                        if (key0 + 32 + c > pq) x1[c] = 0xff800000u;
                    }
                }
                // raw scores stay unscaled: max commutes with the positive scale, and the scale
                // is folded into the exponent's fused multiply-add below
#pragma unroll
                for (int c = 0; c < 32; ++c)
                    mx = fmaxf(mx, fmaxf(__uint_as_float(x0[c]), __uint_as_float(x1[c])));
                mx *= a.scale_log2;
            }
            xchg[wg * 128 + r] = mx;
            wg_barrier();
            dead = __any_sync(kFull, *sm_dead != 0);
            if (dead) break;  // taken by all eight warps: the flag was set before the barrier
            mx = fmaxf(mx, xchg[(wg ^ 1) * 128 + r]);
            float alpha = 1.f;
            bool need = false;
            if (j == 0) {
                m_ref = mx;  // key 0 is visible to every row, so mx is finite
            } else if (mx > m_ref + kRescaleThreshold) {
                alpha = ex2(m_ref - mx);
                m_ref = mx;
                need = true;
            }
            if (__any_sync(kFull, need)) {
                // the accumulator must be quiet: wait for O += P_{j-1} V_{j-1}; each warpgroup
                // rescales its half of the columns
                if (!warp_spin_bounded(&pv_done[(j - 1) & 1], uint32_t(((j - 1) >> 1) & 1), lane)) {
                    // cannot bail out alone (the other warpgroup may not rescale): record and go on
                    report_status(a.status, kDevWaitMma);
                }
                fence_after_sync();
                for (int c0 = col0; c0 < min(col0 + kPage, n_pv); c0 += 32) {
                    uint32_t o[32];
                    tmem_ld32(tmem_o + lane_base + c0, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                    tmem_st32(tmem_o + lane_base + c0, o);
                }
                tmem_wait_st();
            }
            l_sum *= alpha;
            if (have_page) {
                float psum0 = 0.f, psum1 = 0.f;
                const float neg_m = -m_ref;
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const float p0 = ex2(fmaf(__uint_as_float(x0[c]), a.scale_log2, neg_m));
                    const float p1 = ex2(fmaf(__uint_as_float(x1[c]), a.scale_log2, neg_m));
                    psum0 += p0;
                    psum1 += p1;
                    x0[c] = round_tf32(__float_as_uint(p0));
                    x1[c] = round_tf32(__float_as_uint(p1));
                }
                l_sum += psum0 + psum1;
                tmem_st32(s_addr, x0);
                tmem_st32(s_addr + 32, x1);
                tmem_wait_st();
            }
            fence_before_sync();
            mbar_arrive(&p_full[sb]);
            wg_barrier();  // the exchange area is rewritten by the next tile
        }
        if (dead && lane == 0) report_status(a.status, kDevWaitFull);

        // ---- epilogue: O / l -> global; each warpgroup its half of the columns
        if (!dead) {
            xchg[wg * 128 + r] = l_sum;
            wg_barrier();
            const float l_tot = l_sum + xchg[(wg ^ 1) * 128 + r];
            const int jl = n_tiles - 1;
            if (warp_spin_bounded(&pv_done[jl & 1], uint32_t((jl >> 1) & 1), lane)) {
                fence_after_sync();
                const float inv = 1.0f / l_tot;
                // Stage the tile in shared memory (the K stages are idle by now) so that the
                // global stores are whole 512-byte rows per warp instead of 16 bytes per thread:
                // matters most when `out` is a peer GPU's memory.  16-byte chunk c of row r sits
                // at chunk position c ^ (r & 31): conflict-free both ways.
                float4* tile = reinterpret_cast<float4*>(k_s);  // [128 rows][32 chunks]
                for (int c0 = col0; c0 < min(col0 + kPage, n_pv); c0 += 32) {
                    uint32_t o[32];
                    tmem_ld32(tmem_o + lane_base + c0, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        const int chunk = (c0 + c) >> 2;
                        tile[r * 32 + (chunk ^ (r & 31))] =
                            make_float4(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv,
                                        __uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
                    }
                }
                wg_barrier();
                const int w8 = warp - 2;  // 0..7: 16 rows each
                for (int rr = w8 * 16; rr < w8 * 16 + 16; ++rr) {
                    const int tt = t0 + rr;
                    if (tt < a.seq_len && lane * 4 + 3 < D) {
                        float* orow = a.out + size_t(h) * a.o_hs + size_t(tt) * a.o_ts;
                        *reinterpret_cast<float4*>(orow + lane * 4) = tile[rr * 32 + (lane ^ (rr & 31))];
                    }
                }
            } else {
                report_status(a.status, kDevWaitMma);
                *abort_flag = 1;
            }
        }
    }

    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(uint32_t(kTmemCols))
                     : "memory");
    }
}

}  // namespace xn
