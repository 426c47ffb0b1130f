// Causal prefill attention on the 5th-generation tensor cores (tcgen05, TF32 inputs, f32
// accumulators in tensor memory), sm_100a only.
//
// Replaces, for long prompts, the per-row loop of the reference (src/nn/fast_attention.rs:
// 157-198): S = Q K^T and O = P V become tcgen05.mma.kind::tf32 instructions; the causal loop
// bound `limit = index_pos + t_q` (:162) becomes "key tiles above the diagonal are never issued,
// the diagonal tile is masked element-wise".
//
// One thread block = one (query head, 128-row query tile).  Key/value tiles are the cache's
// 64-token pages.  Tensor memory (512 columns): Q [0,128) | four S/P buffers [128,384) |
// O [384,512).  Roles (192 threads):
//   warp 0      TMA producer: tensor-map loads of K pages (4 stages, 128-byte swizzle) and V
//               pages (3 stages, 128-byte swizzle of 32-byte chunks) with mbarrier byte counts;
//               K runs two tiles ahead of V, the order in which the MMA warp consumes them;
//   warp 1      MMA issuer (one lane): S_j = Q K_j^T with Q read from tensor memory, issued two
//               tiles ahead of O += P_j V_j, which reads P from tensor memory (P overwrites S_j
//               in place) and V MN-major straight from its [token][dim] page; tcgen05.commit
//               signals the mbarriers;
//   warps 2..5  thread r owns query row r.  Prologue: the row of Q goes global -> registers ->
//               tensor memory (rounded to TF32).  Per tile: tcgen05.ld of the S row (the next
//               tile's load is issued before this tile's arithmetic), causal mask, running
//               max / sum, exp2 with the softmax scale folded into one FMA, P written back with
//               tcgen05.st and published one tile later.  The accumulator is rescaled lazily:
//               only when a row's maximum grows by more than 2^8.  Epilogue: O / l to global.
// Every wait is bounded; on expiry the kernel records a status code, drains and returns.
#pragma once
#include <cuda.h>

#include "xn_common.cuh"

namespace xn {

struct PrefillArgs {
    const float* q;       // rotated queries (device)
    long long q_hs, q_ts; // query head / token strides in floats
    const int* pages;     // page ids of the stream (device)
    float* out;           // output base
    long long o_hs, o_ts; // output head / token strides in floats
    long long layer_page_base;  // layer * pool_pages
    int num_kv_heads;
    int group;            // query heads per KV head
    int seq_len;          // S
    int index_pos;        // P
    int head_dim;         // D (multiple of 4, 16..128)
    float scale_log2;     // (1/sqrt(D)) * log2(e)
    int* status;
#ifdef XN_PF_TIMING
    long long* timing;    // instrumentation build only: cycle counters of one softmax thread
#endif
};

namespace pf {

constexpr int kBM = 128;          // query rows per block
constexpr int kBN = 64;           // keys per tile (= page)
constexpr int kKB = 4;            // 32-float (128-byte) column blocks per row, at most
constexpr int kKVSub = kBN * 128; // bytes of one K/V column block [64 rows x 128 B]
constexpr int kKVBytes = kKB * kKVSub;   // 32 KB
constexpr int kKStages = 4;       // K pages in flight
constexpr int kVStages = 3;       // V pages in flight
constexpr int kSBufs = 4;         // score / probability buffers in tensor memory
constexpr int kLookahead = 2;     // S_j is issued this many tiles before O += P V of tile j
constexpr int kSmemData = (kKStages + kVStages) * kKVBytes;  // 224 KB
constexpr int kSmemBytes = kSmemData + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kTmemQ = 0;         // 128 columns
constexpr int kTmemS = 128;       // kSBufs x 64 columns
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

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Same wait, written so that the compiler sees the 64 registers of an earlier, still in-flight
// pair of loads as produced here: nothing may read or copy them before this point.
__device__ __forceinline__ void tmem_wait_ld_into(uint32_t (&x)[32], uint32_t (&y)[32]) {
    asm volatile(
        "tcgen05.wait::ld.sync.aligned;"
        : "+r"(x[0]), "+r"(x[1]), "+r"(x[2]), "+r"(x[3]), "+r"(x[4]), "+r"(x[5]), "+r"(x[6]), "+r"(x[7]),
          "+r"(x[8]), "+r"(x[9]), "+r"(x[10]), "+r"(x[11]), "+r"(x[12]), "+r"(x[13]), "+r"(x[14]),
          "+r"(x[15]), "+r"(x[16]), "+r"(x[17]), "+r"(x[18]), "+r"(x[19]), "+r"(x[20]), "+r"(x[21]),
          "+r"(x[22]), "+r"(x[23]), "+r"(x[24]), "+r"(x[25]), "+r"(x[26]), "+r"(x[27]), "+r"(x[28]),
          "+r"(x[29]), "+r"(x[30]), "+r"(x[31]), "+r"(y[0]), "+r"(y[1]), "+r"(y[2]), "+r"(y[3]),
          "+r"(y[4]), "+r"(y[5]), "+r"(y[6]), "+r"(y[7]), "+r"(y[8]), "+r"(y[9]), "+r"(y[10]),
          "+r"(y[11]), "+r"(y[12]), "+r"(y[13]), "+r"(y[14]), "+r"(y[15]), "+r"(y[16]), "+r"(y[17]),
          "+r"(y[18]), "+r"(y[19]), "+r"(y[20]), "+r"(y[21]), "+r"(y[22]), "+r"(y[23]), "+r"(y[24]),
          "+r"(y[25]), "+r"(y[26]), "+r"(y[27]), "+r"(y[28]), "+r"(y[29]), "+r"(y[30]), "+r"(y[31])
        :
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Round an f32 to the nearest TF32 (ties away from zero): the tensor core drops the low 13
// mantissa bits, so adding half an ulp of the kept part to the bit pattern rounds the magnitude.
__device__ __forceinline__ uint32_t round_tf32(uint32_t bits) { return bits + 0x1000u; }

// State one softmax thread carries across tiles.
struct RowState {
    float m_ref;   // reference maximum (scaled, log2 domain) the stored probabilities use
    float l_sum;   // running sum of probabilities
};

}  // namespace pf

__global__ void __launch_bounds__(pf::kThreads, 1)
prefill_tf32_kernel(const __grid_constant__ CUtensorMap k_map,
                    const __grid_constant__ CUtensorMap v_map, const PrefillArgs a) {
    using namespace pf;
    extern __shared__ unsigned char smem_dyn[];
    // 128-byte swizzled tiles want 1024-byte alignment
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    unsigned char* k_s = smem;
    unsigned char* v_s = k_s + kKStages * kKVBytes;
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
    static_assert((1 + 2 * kKStages + 2 * kVStages + 3 * kSBufs) * 8 + 16 <= 256, "barrier area");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_qtiles = (a.seq_len + kBM - 1) / kBM;
    const int qt = n_qtiles - 1 - blockIdx.x;  // longest rows first
    const int h = blockIdx.y;
    const int h_kv = h / a.group;
    const int t0 = qt * kBM;
    const int last_row = min(t0 + kBM, a.seq_len) - 1;
    const int n_tiles = (a.index_pos + last_row) / kBN + 1;
    const int D = a.head_dim;
    const int n_kb = (D + 31) / 32;        // column blocks actually loaded
    const int k_steps = (D + 7) / 8;       // K=8 MMA steps over head_dim
    const int n_pv = (D + 15) / 16 * 16;   // N of the PV MMA

    if (tid == 0) {
        mbar_init(q_ready, 128);
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
            mbar_init(&p_full[s], 128);
            mbar_init(&pv_done[s], 1);
        }
        *abort_flag = 0;
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
        if (lane == 0) {
            for (int t = 0; t < n_tiles + kLookahead; ++t) {
                if (t < n_tiles) {
                    const int st = t % kKStages;
                    const long long row = ((a.layer_page_base + a.pages[t]) * a.num_kv_heads + h_kv) * kBN;
                    if (t >= kKStages && !mbar_wait_bounded(&k_empty[st], uint32_t((t / kKStages - 1) & 1))) {
                        atomicExch(a.status, kDevWaitEmpty); *abort_flag = 1; break;
                    }
                    mbar_arrive_expect_tx(&k_full[st], uint32_t(n_kb) * kKVSub);
                    for (int kb = 0; kb < n_kb; ++kb)
                        tma_load_2d(k_s + st * kKVBytes + kb * kKVSub, &k_map, kb * 32, int(row), &k_full[st]);
                }
                const int jv = t - kLookahead;
                if (jv >= 0) {
                    const int st = jv % kVStages;
                    const long long row = ((a.layer_page_base + a.pages[jv]) * a.num_kv_heads + h_kv) * kBN;
                    if (jv >= kVStages && !mbar_wait_bounded(&v_empty[st], uint32_t((jv / kVStages - 1) & 1))) {
                        atomicExch(a.status, kDevWaitEmpty); *abort_flag = 1; break;
                    }
                    mbar_arrive_expect_tx(&v_full[st], uint32_t(n_kb) * kKVSub);
                    for (int kb = 0; kb < n_kb; ++kb)
                        tma_load_2d(v_s + st * kKVBytes + kb * kKVSub, &v_map, kb * 32, int(row), &v_full[st]);
                }
                if (*abort_flag) break;
            }
        }
    } else if (warp == 1) {
        // =============================== MMA issuer ===============================
        // One lane issues every tcgen05.mma of the block, so its instruction stream is kept
        // short: descriptors are a constant plus a small offset, ring positions and mbarrier
        // parities are carried as counters, and the head_dim = 128 loops are fully unrolled.
        if (lane == 0) {
            const uint32_t idesc_qk = make_idesc(kBM, kBN, 0);
            const uint32_t idesc_pv = make_idesc(kBM, n_pv, 1);
            // descriptor of stage 0; a stage is kKVBytes further, offsets are in 16-byte units
            const uint64_t kdesc0 = smem_desc(smem_u32(k_s), 0, 1024, kLayoutSw128);
            const uint64_t vdesc0 = smem_desc(smem_u32(v_s), kKVSub, 512, kLayoutSw128Base32);
            constexpr uint64_t kStageStep = uint64_t(kKVBytes) >> 4;
            constexpr uint64_t kBlockStep = uint64_t(kKVSub) >> 4;  // next 32-float column block
            bool ok = mbar_wait_bounded(q_ready, 0);
            if (!ok) { atomicExch(a.status, kDevWaitFull); *abort_flag = 1; }
            fence_after_sync();

            int k_st = 0, k_ph = 0;     // K ring position / parity of the next S = Q K^T
            int s_qk = 0;               // score buffer of the next S = Q K^T
            int v_st = 0, v_ph = 0;     // V ring position / parity of the next O += P V
            int s_pv = 0, p_ph = 0;     // score buffer / parity of the next O += P V
            int pv_issued = 0;

            auto issue_qk = [&]() -> bool {
                if (!mbar_wait_bounded(&k_full[k_st], uint32_t(k_ph))) return false;
                fence_after_sync();
                const uint64_t kd = kdesc0 + uint64_t(k_st) * kStageStep;
                const uint32_t d_addr = tmem_s + s_qk * kBN;
                if (k_steps == 16) {
#pragma unroll
                    for (int ks = 0; ks < 16; ++ks)
                        mma_ts(d_addr, tmem_q + ks * 8, kd + (ks >> 2) * kBlockStep + (ks & 3) * 2, idesc_qk,
                               ks > 0 ? 1u : 0u);
                } else {
                    for (int ks = 0; ks < k_steps; ++ks)
                        mma_ts(d_addr, tmem_q + ks * 8, kd + (ks >> 2) * kBlockStep + (ks & 3) * 2, idesc_qk,
                               ks > 0 ? 1u : 0u);
                }
                mma_commit(&k_empty[k_st]);
                mma_commit(&s_full[s_qk]);
                if (++k_st == kKStages) { k_st = 0; k_ph ^= 1; }
                s_qk = (s_qk + 1) & (kSBufs - 1);
                return true;
            };
            // O += P_j V_j.  V is [token][dim]: MN-major B; 8 tokens = 1024 B inside each column
            // block, column blocks kKVSub apart (leading offset), 4-token swizzle groups 512 B apart
            auto issue_pv = [&]() -> bool {
                if (!mbar_wait_bounded(&p_full[s_pv], uint32_t(p_ph)) ||
                    !mbar_wait_bounded(&v_full[v_st], uint32_t(v_ph)))
                    return false;
                fence_after_sync();
                const uint64_t vd = vdesc0 + uint64_t(v_st) * kStageStep;
                const uint32_t p_addr = tmem_s + s_pv * kBN;
                const uint32_t first = pv_issued > 0 ? 1u : 0u;
#pragma unroll
                for (int ks = 0; ks < kBN / 8; ++ks)
                    mma_ts(tmem_o, p_addr + ks * 8, vd + ks * 64, idesc_pv, ks > 0 ? 1u : first);
                mma_commit(&v_empty[v_st]);
                mma_commit(&pv_done[s_pv]);
                if (++v_st == kVStages) { v_st = 0; v_ph ^= 1; }
                if (++s_pv == kSBufs) { s_pv = 0; p_ph ^= 1; }
                ++pv_issued;
                return true;
            };
            static_assert((kSBufs & (kSBufs - 1)) == 0, "score buffers: power of two");
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (!issue_qk()) { ok = false; break; }
                if (j >= kLookahead && !issue_pv()) { ok = false; break; }
            }
            while (ok && pv_issued < n_tiles)
                if (!issue_pv()) ok = false;
            if (!ok) { atomicExch(a.status, kDevWaitMma); *abort_flag = 1; }
        }
    } else {
        // =============================== softmax + epilogue ===============================
        constexpr unsigned kFull = 0xffffffffu;
        const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
        const int r = quarter * 32 + lane;       // query row inside the tile
        const uint32_t lane_base = uint32_t(quarter * 32) << 16;
        const int t = t0 + r;                    // query row inside the request
        const int pq = a.index_pos + t;          // its absolute position

        // ---- prologue: this thread's row of Q -> tensor memory (rounded to TF32) ----
        {
            const float* qrow = a.q + size_t(h) * a.q_hs + size_t(t) * a.q_ts;
            const bool valid = t < a.seq_len;
            for (int c0 = 0; c0 < k_steps * 8; c0 += 32) {
                uint32_t qv[32];
#pragma unroll
                for (int c = 0; c < 32; c += 4) {
                    float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (valid && c0 + c < D) v4 = *reinterpret_cast<const float4*>(qrow + c0 + c);
                    qv[c] = round_tf32(__float_as_uint(v4.x));
                    qv[c + 1] = round_tf32(__float_as_uint(v4.y));
                    qv[c + 2] = round_tf32(__float_as_uint(v4.z));
                    qv[c + 3] = round_tf32(__float_as_uint(v4.w));
                }
                tmem_st32(tmem_q + lane_base + c0, qv);
            }
            tmem_wait_st();
            fence_before_sync();
            mbar_arrive(q_ready);
        }

        RowState st{-INFINITY, 0.f};
        bool dead = false;
        int pending = -1;  // tile whose P is stored but not yet published
#ifdef XN_PF_TIMING
        long long tm_pub = 0;
#endif

        // waits for S_j and starts loading this thread's row of it
        auto fetch = [&](int j, uint32_t (&x0)[32], uint32_t (&x1)[32]) -> bool {
            const int sb = j % kSBufs;
            if (!__all_sync(kFull, mbar_wait_bounded(&s_full[sb], uint32_t((j / kSBufs) & 1)))) return false;
            fence_after_sync();
            const uint32_t s_addr = tmem_s + lane_base + sb * kBN;
            tmem_ld32(s_addr, x0);
            tmem_ld32(s_addr + 32, x1);
            return true;
        };
        // makes the P of tile `pending` visible to the MMA warp
        auto publish = [&]() {
            if (pending >= 0) {
#ifdef XN_PF_TIMING
                long long t_p = clock64();
#endif
                tmem_wait_st();
                fence_before_sync();
                mbar_arrive(&p_full[pending % kSBufs]);
                pending = -1;
#ifdef XN_PF_TIMING
                tm_pub += clock64() - t_p;
#endif
            }
        };
        // mask, max, (rare) accumulator rescale, probabilities; stores P_j
        auto process = [&](int j, uint32_t (&x0)[32], uint32_t (&x1)[32]) -> bool {
            const bool diag = j * kBN + kBN - 1 > a.index_pos + t0;  // some row masks some key here
            if (diag) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    if (j * kBN + c > pq) x0[c] = 0xff800000u;  // -inf
                    if (j * kBN + 32 + c > pq) x1[c] = 0xff800000u;
                }
            }
            // raw scores stay unscaled: max commutes with the positive scale, and the scale is
            // folded into the exponent's fused multiply-add below
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 32; ++c)
                mx = fmaxf(mx, fmaxf(__uint_as_float(x0[c]), __uint_as_float(x1[c])));
            mx *= a.scale_log2;
            float alpha = 1.f;
            bool need = false;
            if (j == 0) {
                st.m_ref = mx;  // key 0 is visible to every row, so mx is finite
            } else if (mx > st.m_ref + kRescaleThreshold) {
                alpha = ex2(st.m_ref - mx);
                st.m_ref = mx;
                need = true;
            }
            if (__any_sync(kFull, need)) {
                // the accumulator must be quiet: publish what is pending, then wait for
                // O += P_{j-1} V_{j-1}
                publish();
                const int sp = (j - 1) % kSBufs;
                if (!__all_sync(kFull, mbar_wait_bounded(&pv_done[sp], uint32_t(((j - 1) / kSBufs) & 1))))
                    return false;
                fence_after_sync();
                st.l_sum *= alpha;
                for (int c0 = 0; c0 < n_pv; c0 += 32) {
                    uint32_t o[32];
                    tmem_ld32(tmem_o + lane_base + c0, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                    tmem_st32(tmem_o + lane_base + c0, o);
                }
                tmem_wait_st();
            }
            float psum0 = 0.f, psum1 = 0.f;
            const float neg_m = -st.m_ref;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const float p0 = ex2(fmaf(__uint_as_float(x0[c]), a.scale_log2, neg_m));
                const float p1 = ex2(fmaf(__uint_as_float(x1[c]), a.scale_log2, neg_m));
                psum0 += p0;
                psum1 += p1;
                x0[c] = round_tf32(__float_as_uint(p0));
                x1[c] = round_tf32(__float_as_uint(p1));
            }
            st.l_sum += psum0 + psum1;
            publish();  // the previous tile's P: its stores have long completed
            const uint32_t s_addr = tmem_s + lane_base + (j % kSBufs) * kBN;
            tmem_st32(s_addr, x0);
            tmem_st32(s_addr + 32, x1);
            pending = j;
            return true;
        };

#ifdef XN_PF_TIMING
        long long tm_wait_s = 0, tm_wait_ld = 0, tm_proc = 0, tm_total = clock64();
#define PF_T0 long long t_0 = clock64();
#define PF_ACC(var) var += clock64() - t_0;
#else
#define PF_T0
#define PF_ACC(var)
#endif
        uint32_t a0[32], a1[32], b0[32], b1[32];
        if (!fetch(0, a0, a1)) dead = true;
        for (int j = 0; j < n_tiles && !dead; j += 2) {
            // tile j lives in (a0,a1); tile j+1 is fetched into (b0,b1) while j is processed
            { PF_T0 tmem_wait_ld_into(a0, a1); PF_ACC(tm_wait_ld) }
            { PF_T0 if (j + 1 < n_tiles && !fetch(j + 1, b0, b1)) { dead = true; break; } PF_ACC(tm_wait_s) }
            { PF_T0 if (!process(j, a0, a1)) { dead = true; break; } PF_ACC(tm_proc) }
            if (j + 1 >= n_tiles) break;
            { PF_T0 tmem_wait_ld_into(b0, b1); PF_ACC(tm_wait_ld) }
            { PF_T0 if (j + 2 < n_tiles && !fetch(j + 2, a0, a1)) { dead = true; break; } PF_ACC(tm_wait_s) }
            { PF_T0 if (!process(j + 1, b0, b1)) { dead = true; break; } PF_ACC(tm_proc) }
            if (__any_sync(kFull, *abort_flag != 0)) { dead = true; break; }
        }
        if (dead) {
            atomicExch(a.status, kDevWaitFull);
            *abort_flag = 1;
        } else {
            publish();
        }
#ifdef XN_PF_TIMING
        if (a.timing && blockIdx.x == 0 && blockIdx.y == 0 && tid == 64) {
            a.timing[0] = n_tiles; a.timing[1] = clock64() - tm_total; a.timing[2] = tm_wait_s;
            a.timing[3] = tm_wait_ld; a.timing[4] = tm_proc; a.timing[5] = tm_pub;
        }
#endif

        // ---- epilogue: O / l -> global
        const bool aborted = __any_sync(kFull, *abort_flag != 0);  // warp-uniform
        if (!dead && !aborted) {
            const int jl = n_tiles - 1;
            if (__all_sync(kFull, mbar_wait_bounded(&pv_done[jl % kSBufs], uint32_t((jl / kSBufs) & 1)))) {
                fence_after_sync();
                const float inv = 1.0f / st.l_sum;
                float* orow = a.out + size_t(h) * a.o_hs + size_t(t) * a.o_ts;
                for (int c0 = 0; c0 < n_pv; c0 += 32) {
                    uint32_t o[32];
                    tmem_ld32(tmem_o + lane_base + c0, o);
                    tmem_wait_ld();
                    if (t < a.seq_len) {
#pragma unroll
                        for (int c = 0; c < 32; c += 4) {
                            if (c0 + c + 3 < D) {
                                float4 v4 = make_float4(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv,
                                                        __uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
                                *reinterpret_cast<float4*>(orow + c0 + c) = v4;
                            }
                        }
                    }
                }
            } else {
                atomicExch(a.status, kDevWaitMma);
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
