// Split-KV attention over the paged f32 KV cache ("flash decoding"), sm_100a.
//
// Replaces the per-row loop of the reference: batched q.k dots, softmax over the whole row,
// weighted V sum (src/nn/fast_attention.rs:157-198 with src/nn/fast_attention_simd.rs:594-630,
// :272-339, :132-163).  One launch serves a whole batch of streams; prefill rows are served as
// rows of different cached length over the same pages.
//
// Shape of the computation (bandwidth bound: every cached K and V element is read once from
// HBM and shared by the query heads of its KV group):
//   * work unit  = (request, KV head, <=GT query heads, query row), kv_len cached tokens;
//   * tile       = TPS consecutive tokens of one unit: a K block and a V block, each a
//                  contiguous run inside one 64-token page;
//   * the host cuts the flattened tile list into equal chunks, several per SM; thread blocks
//     (one per SM) take chunks dynamically, so neither ragged lengths nor uneven per-SM memory
//     throughput leave an SM idle; a unit cut across chunks yields partial records, combined
//     with the usual log-sum-exp weights by the block that delivers the last one;
//   * inside a block one producer lane streams tiles into a ring of shared-memory stages with
//     1-D bulk async copies (TMA engine, mbarrier byte counting, no tensor map, no multicast);
//     WARPS consumer warps each own a fixed subset of a tile's tokens and keep an independent
//     online-softmax state (running max, sum, accumulator) merged once per unit.
#pragma once
// Barrier waits on the kernel's hand-offs poll (non-blocking test in a loop): measured a little
// faster here than the parking try_wait (116.9 vs 117.7 us per launch on the config-3 batch).
#ifndef XN_DECODE_WAIT
#define XN_DECODE_WAIT mbar_spin_bounded
#endif
#include <cstdio>

#include "xn_common.cuh"

namespace xn {

// Tokens per stage and ring depth for head dims up to 128 (build-time knobs for tuning).
#ifndef XN_DECODE_TPS
#define XN_DECODE_TPS 64
#endif
#ifndef XN_DECODE_STAGES
#define XN_DECODE_STAGES 3
#endif
#ifndef XN_DECODE_WARPS
#define XN_DECODE_WARPS 8
#endif

template <int NV>
struct DecodeCfg {
    static constexpr int kWarps = (NV <= 32) ? XN_DECODE_WARPS : 8;  // consumer warps
    static constexpr int kRedWarps = 8;                   // warp states merged per round
    static constexpr int kThreads = (kWarps + 1) * 32;    // + 1 producer warp
    static constexpr int kLPK = (NV <= 32) ? 8 : 16;      // lanes sharing one key in q.k
    static constexpr int kKPI = 32 / kLPK;                // keys per warp iteration
    static constexpr int kTPS = (NV <= 32) ? XN_DECODE_TPS : 32;  // tokens per stage
    static constexpr int kKPW = kTPS / kWarps;            // keys per warp per stage
    static constexpr int kIters = kKPW / kKPI;
    static constexpr int kSlotsQ = (NV + kLPK - 1) / kLPK;  // float4 of q per lane per head
    static constexpr int kSlotsV = (NV + 31) / 32;          // float4 of output per lane per head
    static constexpr int kStages = (NV <= 32) ? XN_DECODE_STAGES : 3;
    static constexpr int kStageFloats = 2 * kTPS * NV * 4;  // K block then V block
    static_assert(kIters >= 1, "tile too small for the warp layout");
};

// Sum GT per-lane partial dots over the LPK lanes that share a key.  On return every lane holds
// the full sum for head owned_head<GT>(sub), using GT-1 + log2(LPK/GT)... shuffles instead of
// GT*log2(LPK): the halves of the value set are exchanged while the lane set is halved.
template <int GT, int LPK>
__device__ __forceinline__ float group_reduce(const float (&s)[GT], int sub) {
    constexpr unsigned kFull = 0xffffffffu;
    float keep;
    int first_add = 1;
    if constexpr (GT == 4) {
        const bool b0 = sub & 1, b1 = sub & 2;
        float ka = b0 ? s[2] : s[0], kb = b0 ? s[3] : s[1];
        float sa = b0 ? s[0] : s[2], sb = b0 ? s[1] : s[3];
        ka += __shfl_xor_sync(kFull, sa, 1);
        kb += __shfl_xor_sync(kFull, sb, 1);
        keep = b1 ? kb : ka;
        float send = b1 ? ka : kb;
        keep += __shfl_xor_sync(kFull, send, 2);
        first_add = 4;
    } else if constexpr (GT == 2) {
        const bool b0 = sub & 1;
        keep = b0 ? s[1] : s[0];
        float send = b0 ? s[0] : s[1];
        keep += __shfl_xor_sync(kFull, send, 1);
        first_add = 2;
    } else {
        keep = s[0];
    }
#pragma unroll
    for (int o = first_add; o < LPK; o <<= 1) keep += __shfl_xor_sync(kFull, keep, o);
    return keep;
}

// acc += p * v on four lanes with two packed f32x2 FMAs (sm_100 issues two fused
// multiply-adds per instruction this way; each component is the same correctly rounded fma).
__device__ __forceinline__ void fma4_scalar(float4& acc, float p, const float4& v) {
    const float2 pp = make_float2(p, p);
    const float2 lo = __ffma2_rn(pp, make_float2(v.x, v.y), make_float2(acc.x, acc.y));
    const float2 hi = __ffma2_rn(pp, make_float2(v.z, v.w), make_float2(acc.z, acc.w));
    acc = make_float4(lo.x, lo.y, hi.x, hi.y);
}

// two running partial dots (even / odd components) of q . k, again with packed FMAs
__device__ __forceinline__ void dot4_acc(float2& part, const float4& q, const float4& k) {
    part = __ffma2_rn(make_float2(q.x, q.y), make_float2(k.x, k.y), part);
    part = __ffma2_rn(make_float2(q.z, q.w), make_float2(k.z, k.w), part);
}

template <int GT>
__device__ __forceinline__ int owned_head(int sub) {
    if constexpr (GT == 4) return ((sub & 1) << 1) | ((sub >> 1) & 1);
    if constexpr (GT == 2) return sub & 1;
    return 0;
}

// Partial record of one (item, head): [m, l, 0, 0, acc[Dp]] floats.
__host__ __device__ __forceinline__ size_t part_stride_floats(int nv) { return size_t(nv) * 4 + 4; }

// What the producer tells the consumers about the tile in a stage.
struct StageHdr {
    const float* q;   // row of the unit's first query head (global)
    float* out;       // output row of the unit's first query head
    long long q_hs;   // query head stride (floats)
    long long o_hs;   // output head stride (floats)
    int flags;        // kHdr* bits
    int ntok;         // valid tokens in this tile
    int nheads;       // query heads of the unit (<= GT)
    int part;         // partial slot of the item, or -1: the block writes the output itself
    int part_begin;   // first partial slot of the unit
    int part_count;   // items the unit was cut into
    int merge_slot;   // arrival counter of the unit (cut units only)
    int new_key;      // row of this tile that holds the request's new token (fused append), or -1
    float* k_dst;     // cache rows the new token's K / V must be written to (nullptr: another
    float* v_dst;     //   unit of the same KV head does it)
};
enum : int { kHdrFirst = 1, kHdrLast = 2, kHdrQStaged = 4, kHdrEnd = 8, kHdrRope = 16 };

// Words of the per-context synchronisation array used by the kernel.
enum : int { kSyncChunk = 0, kSyncDone = 1, kSyncMerge0 = 2 };

template <int NV, int GT>
struct DecodeSmem {
    using Cfg = DecodeCfg<NV>;
    static constexpr bool kStageQ = NV <= 32;  // query rows travel with the first tile of an item
    // extra area of a stage: GT query rows, then one cos row and one sin row (fused RoPE)
    static constexpr size_t kQFloats = kStageQ ? size_t(GT + 1) * NV * 4 : 0;
    static constexpr size_t kStageBytes = (size_t(Cfg::kStageFloats) + kQFloats) * 4;
    static constexpr size_t kRedFloats = size_t(Cfg::kRedWarps) * GT * NV * 4;
    static constexpr size_t kScratchFloats = size_t(Cfg::kWarps) * (Cfg::kKPW + 1) * 4;  // GT<=4
    static constexpr size_t kBytes = Cfg::kStages * kStageBytes + kRedFloats * 4 +
                                     kScratchFloats * 4 + Cfg::kWarps * 4 * 2 * 4 /* m,l */ +
                                     Cfg::kStages * sizeof(StageHdr) + 2 * Cfg::kStages * 8 /* barriers */ +
                                     32 /* flags */;
};

// Launch: one block per SM (at most `n_chunks` blocks).  The host cut the flattened tile list of
// the batch into `n_chunks` chunks (several per block); a block takes chunk blockIdx.x first and
// then whatever `sync[kSyncChunk]` hands out next, so a block that runs on a slower path to
// memory simply takes fewer chunks.
//
//   producer warp  all 32 lanes resolve the descriptors of up to 32 items of a chunk at once
//                  (item -> unit -> request, page ids), lane 0 then writes a StageHdr and issues
//                  the bulk copies tile by tile: no dependent global load sits between two tiles;
//                  When the request carries one new token and asks for it (ReqDev flag 8), the
//                  tile that ends the unit takes its last row from the request's k / v instead of
//                  the cache, and the consumer warp that owns that row rotates it (RoPE, if asked),
//                  and stores it into the cache: the append of src/nn/fast_attention.rs:104-116
//                  without a separate kernel;
//   consumer warps follow the headers: load q (from the stage when it was staged) at the first
//                  tile of an item, accumulate, merge their states at its last tile and write
//                  either the output row (unit in one piece) or a partial record.  The block
//                  that writes a unit's last missing partial combines all of them (arrival
//                  counter in `sync`), so no second kernel is needed.
// EXACT: rows are exactly NV float4 long (nv_arg == NV), which turns every bound check on the
// row length into a compile-time constant.
template <int NV, int GT, bool EXACT>
__global__ void __launch_bounds__(DecodeCfg<NV>::kThreads, 1)
attn_splitkv_kernel(const ReqDev* __restrict__ reqs, const UnitDev* __restrict__ units,
                    const ItemDev* __restrict__ items, const int* __restrict__ chunk_item_begin,
                    int n_chunks, const int* __restrict__ page_ids,
                    const float* __restrict__ k_pool, const float* __restrict__ v_pool,
                    float* __restrict__ partials, int* __restrict__ sync, long long pool_pages,
                    int num_kv_heads, int head_dim, int nv_arg, float scale,
                    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                    int* __restrict__ status, const __grid_constant__ ReqPatchTable patch) {
    const int nv = EXACT ? NV : nv_arg;
    using Cfg = DecodeCfg<NV>;
    using Sm = DecodeSmem<NV, GT>;
    constexpr int W = Cfg::kWarps, LPK = Cfg::kLPK, KPI = Cfg::kKPI, TPS = Cfg::kTPS;
    constexpr int KPW = Cfg::kKPW, ITERS = Cfg::kIters, ST = Cfg::kStages;
    constexpr int SQ = Cfg::kSlotsQ, SV = Cfg::kSlotsV;
    constexpr unsigned kFull = 0xffffffffu;

    // a kernel launched behind this one as a programmatic dependent (the output block's quantiser)
    // may be set up now; it waits for this kernel's completion before it reads the rows
    pdl_launch_dependents();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* red = reinterpret_cast<float*>(smem_raw + ST * Sm::kStageBytes);
    float* scratch = red + Sm::kRedFloats;
    float* sm_m = scratch + Sm::kScratchFloats;  // [W][4]
    float* sm_l = sm_m + W * 4;                  // [W][4]
    StageHdr* hdr = reinterpret_cast<StageHdr*>(sm_l + W * 4);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(hdr + ST);
    uint64_t* empty_bar = full_bar + ST;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + ST);
    volatile int* last_flag = abort_flag + 1;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int dp = nv * 4;  // padded row length in floats
    const size_t page_floats = size_t(kPageTokens) * dp;
    auto stage_ptr = [&](int s) { return reinterpret_cast<float*>(smem_raw + size_t(s) * Sm::kStageBytes); };

    if (tid == 0) {
        for (int s = 0; s < ST; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], W);
        }
        *abort_flag = 0;
        *last_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == 0) {
        // =============================== producer ===============================
        int fill = 0;
        bool ok = true;
        int chunk = blockIdx.x;
        while (ok && chunk < n_chunks) {
            const int it_lo = chunk_item_begin[chunk], it_hi = chunk_item_begin[chunk + 1];
            for (int base = it_lo; base < it_hi && ok; base += 32) {
                // ---- every lane resolves one item of this batch of 32 ----
                const int my_it = base + lane;
                ItemDev item = {0, 0, 0, -1};
                UnitDev u = {};
                const float* q_ptr = nullptr;
                float* o_ptr = nullptr;
                long long q_hs = 0, o_hs = 0;
                const int* pages = page_ids;
                size_t layer_base = 0;
                const float* k_new = nullptr;  // fused append: the new token's rows of this KV head
                const float* v_new = nullptr;
                int fused = 0;                 // bit 0 fused append, bit 1 rotate, bit 2 this unit stores
                int pos = 0;
                if (my_it < it_hi) {
                    item = items[my_it];
                    u = units[item.unit];
                    const ReqDev& r = reqs[u.req];
                    // a reused plan: addresses and layer come with the launch
                    const bool patched = patch.n != 0;
                    const float* rq = patched ? patch.e[u.req].q : r.q;
                    const float* rk = patched ? patch.e[u.req].k : r.k;
                    const float* rv = patched ? patch.e[u.req].v : r.v;
                    float* ro = patched ? patch.e[u.req].out : r.out;
                    const int rlayer = patched ? patch.layer : r.layer;
                    q_ptr = rq + size_t(u.head0) * r.q_hs + size_t(u.t_q) * r.q_ts;
                    o_ptr = ro + size_t(u.head0) * r.o_hs + size_t(u.t_q) * r.o_ts;
                    q_hs = r.q_hs;
                    o_hs = r.o_hs;
                    pages = page_ids + r.page_off;
                    layer_base = size_t(rlayer) * size_t(pool_pages);
                    if (r.flags & 8u) {
                        k_new = rk + size_t(u.kv_head) * r.kv_hs;
                        v_new = rv + size_t(u.kv_head) * r.kv_hs;
                        fused = 1 | ((r.flags & 1u) ? 2 : 0) | (u.store_new ? 4 : 0);
                        pos = r.index_pos;
                    }
                }
                const int n_here = min(32, it_hi - base);
                for (int k = 0; k < n_here && ok; ++k) {
                    __syncwarp();
                    const int tile_begin = __shfl_sync(kFull, item.tile_begin, k);
                    const int tile_end = __shfl_sync(kFull, item.tile_end, k);
                    const int kv_len = __shfl_sync(kFull, u.kv_len, k);
                    const int kv_head = __shfl_sync(kFull, u.kv_head, k);
                    const unsigned long long pages_k =
                        __shfl_sync(kFull, reinterpret_cast<unsigned long long>(pages), k);
                    const unsigned long long lbase_k = __shfl_sync(kFull, (unsigned long long)layer_base, k);
                    StageHdr h;
                    h.q = reinterpret_cast<const float*>(__shfl_sync(kFull, reinterpret_cast<unsigned long long>(q_ptr), k));
                    h.out = reinterpret_cast<float*>(__shfl_sync(kFull, reinterpret_cast<unsigned long long>(o_ptr), k));
                    h.q_hs = __shfl_sync(kFull, q_hs, k);
                    h.o_hs = __shfl_sync(kFull, o_hs, k);
                    h.nheads = __shfl_sync(kFull, u.nheads, k);
                    h.part = __shfl_sync(kFull, item.part, k);
                    h.part_begin = __shfl_sync(kFull, u.part_begin, k);
                    h.part_count = __shfl_sync(kFull, u.part_count, k);
                    h.merge_slot = __shfl_sync(kFull, u.merge_slot, k);
                    h.new_key = -1;
                    h.k_dst = nullptr;
                    h.v_dst = nullptr;
                    const int fused_k = __shfl_sync(kFull, fused, k);
                    const int pos_k = __shfl_sync(kFull, pos, k);
                    const float* k_new_k = reinterpret_cast<const float*>(
                        __shfl_sync(kFull, reinterpret_cast<unsigned long long>(k_new), k));
                    const float* v_new_k = reinterpret_cast<const float*>(
                        __shfl_sync(kFull, reinterpret_cast<unsigned long long>(v_new), k));
                    const bool stage_q = Sm::kStageQ && (head_dim % 4 == 0) &&
                                         ((reinterpret_cast<uintptr_t>(h.q) | uintptr_t(h.q_hs * 4)) & 15) == 0;
                    const int* pages_ptr = reinterpret_cast<const int*>(pages_k);
                    for (int tb = tile_begin; tb < tile_end && ok; tb += 32) {
                        // page ids of the next 32 tiles, one per lane
                        const int my_tile = tb + lane;
                        int my_page = 0;
                        if (my_tile < tile_end) my_page = pages_ptr[(my_tile * TPS) / kPageTokens];
                        const int n_t = min(32, tile_end - tb);
                        for (int tt = 0; tt < n_t; ++tt, ++fill) {
                            __syncwarp();
                            const int page = __shfl_sync(kFull, my_page, tt);
                            if (lane == 0) {
                                const int tile = tb + tt;
                                const int s = fill % ST;
                                if (fill >= ST && !XN_DECODE_WAIT(&empty_bar[s], ((fill / ST) - 1) & 1)) {
                                    report_status(status, kDevWaitEmpty);
                                    *abort_flag = 1;
                                    ok = false;
                                } else if (!XN_PAGE_OK(page, pool_pages)) {
                                    report_status(status, kDevBadIndex);
                                    *abort_flag = 1;
                                    ok = false;
                                } else {
                                    const int tok0 = tile * TPS;
                                    const int ntok = min(TPS, kv_len - tok0);
                                    const size_t src = ((size_t(lbase_k) + size_t(page)) * num_kv_heads + kv_head) *
                                                           page_floats +
                                                       size_t(tok0 % kPageTokens) * dp;
                                    const bool first = tile == tile_begin;
                                    // fused append: the tile that ends the unit takes its last
                                    // row from the request instead of the cache
                                    const bool has_new = (fused_k & 1) && tok0 + ntok == kv_len;
                                    const int n_cache = has_new ? ntok - 1 : ntok;
                                    const uint32_t bytes = uint32_t(n_cache) * dp * 4;
                                    const uint32_t row_bytes = uint32_t(dp) * 4;
                                    const bool rope_here = (fused_k & 2) && (first || has_new);
                                    h.flags = (first ? kHdrFirst : 0) | (tile == tile_end - 1 ? kHdrLast : 0) |
                                              (first && stage_q ? kHdrQStaged : 0) | ((fused_k & 2) ? kHdrRope : 0);
                                    h.ntok = ntok;
                                    h.new_key = has_new ? ntok - 1 : -1;
                                    h.k_dst = (has_new && (fused_k & 4)) ? const_cast<float*>(k_pool) + src + size_t(ntok - 1) * dp : nullptr;
                                    h.v_dst = (has_new && (fused_k & 4)) ? const_cast<float*>(v_pool) + src + size_t(ntok - 1) * dp : nullptr;
                                    hdr[s] = h;
                                    float* dst = stage_ptr(s);
                                    const uint32_t q_bytes = (first && stage_q) ? uint32_t(h.nheads) * row_bytes : 0u;
                                    mbar_arrive_expect_tx(&full_bar[s], 2 * bytes + q_bytes + (has_new ? 2 * row_bytes : 0u) +
                                                                            (rope_here ? row_bytes : 0u));
                                    if (bytes) {
                                        bulk_g2s(dst, k_pool + src, bytes, &full_bar[s]);
                                        bulk_g2s(dst + TPS * NV * 4, v_pool + src, bytes, &full_bar[s]);
                                    }
                                    if (has_new) {
                                        bulk_g2s(dst + size_t(n_cache) * dp, k_new_k, row_bytes, &full_bar[s]);
                                        bulk_g2s(dst + TPS * NV * 4 + size_t(n_cache) * dp, v_new_k, row_bytes, &full_bar[s]);
                                    }
                                    if (q_bytes)
                                        for (int hh = 0; hh < h.nheads; ++hh)
                                            bulk_g2s(dst + Cfg::kStageFloats + hh * dp, h.q + size_t(hh) * h.q_hs,
                                                     row_bytes, &full_bar[s]);
                                    if (rope_here) {  // cos row then sin row of the token's position
                                        const int half = head_dim / 2;
                                        float* cs = dst + Cfg::kStageFloats + GT * NV * 4;
                                        bulk_g2s(cs, cos_t + size_t(pos_k) * half, row_bytes / 2, &full_bar[s]);
                                        bulk_g2s(cs + half, sin_t + size_t(pos_k) * half, row_bytes / 2, &full_bar[s]);
                                    }
                                }
                            }
                            ok = __shfl_sync(kFull, ok ? 1 : 0, 0) != 0;
                            if (!ok) break;
                        }
                    }
                }
            }
            // next chunk: dynamic
            int next = 0;
            if (lane == 0) next = atomicAdd(&sync[kSyncChunk], 1) + int(gridDim.x);
            chunk = __shfl_sync(kFull, next, 0);
        }
        if (lane == 0) {
            if (ok) {
                // end-of-work marker
                const int s = fill % ST;
                if (fill >= ST && !XN_DECODE_WAIT(&empty_bar[s], ((fill / ST) - 1) & 1)) {
                    report_status(status, kDevWaitEmpty);
                    *abort_flag = 1;
                } else {
                    StageHdr h = {};
                    h.flags = kHdrEnd;
                    hdr[s] = h;
                    mbar_arrive(&full_bar[s]);
                }
            } else {
                // Do not retire the block with copies still landing in its shared memory.
                for (int f = max(0, fill - ST); f < fill; ++f)
                    mbar_wait_bounded(&full_bar[f % ST], (f / ST) & 1);
            }
            // the last block to finish re-arms the chunk counter for the next launch
            __threadfence();
            if (atomicAdd(&sync[kSyncDone], 1) == int(gridDim.x) - 1) {
                sync[kSyncChunk] = 0;
                sync[kSyncDone] = 0;
            }
        }
        return;
    }

    // =============================== consumers ===============================
    const int cw = warp - 1;
    const int sub = lane % LPK, grp = lane / LPK;
    const int hown = owned_head<GT>(sub);
    const bool canon = sub < GT;  // one lane per (key group, head) publishes p
    float* my_scr = scratch + cw * (KPW + 1) * 4;
    const int ctid = tid - 32;  // 0 .. W*32-1

    float4 qreg[GT][SQ];
    float4 acc[GT][SV];
    float m_run = -INFINITY, l_run = 0.f;

    for (int fill = 0;; ++fill) {
        const int s = fill % ST;
        const bool got = __all_sync(kFull, XN_DECODE_WAIT(&full_bar[s], (fill / ST) & 1));
        if (!got) {
            report_status(status, kDevWaitFull);
            *abort_flag = 1;
            break;  // the producer notices the flag or runs into its own bounded wait
        }
        // (the abort flag is deliberately not polled here: every consumer warp must leave at the
        // same tile, or the block-wide barriers of the merge below would lose a participant)
        const StageHdr h = hdr[s];
        if (h.flags & kHdrEnd) break;
        const float4* Ks = reinterpret_cast<const float4*>(stage_ptr(s));
        const float4* Vs = Ks + TPS * NV;

        if (h.flags & kHdrFirst) {
            // query rows of the unit's heads, the float4 slots this lane multiplies
#pragma unroll
            for (int hh = 0; hh < GT; ++hh) {
#pragma unroll
                for (int j = 0; j < SQ; ++j) {
                    const int idx = j * LPK + sub;
                    float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (hh < h.nheads && idx < nv) {
                        if (h.flags & kHdrQStaged) {
                            val = reinterpret_cast<const float4*>(stage_ptr(s) + Cfg::kStageFloats)[hh * nv + idx];
                        } else {
                            const float* qrow = h.q + size_t(hh) * h.q_hs;
                            const int d = idx * 4;
                            if (d + 0 < head_dim) val.x = qrow[d + 0];
                            if (d + 1 < head_dim) val.y = qrow[d + 1];
                            if (d + 2 < head_dim) val.z = qrow[d + 2];
                            if (d + 3 < head_dim) val.w = qrow[d + 3];
                        }
                    }
                    qreg[hh][j] = val;
                }
            }
            if (h.flags & kHdrRope) {
                // rotate-half RoPE of the staged q rows (src/nn/fast_attention_simd.rs:380-387):
                // dims (i, i + D/2) sit in slots (j, j + SQ/2) of the same lane; unfused
                // multiplies so that the values equal the reference's
                const float4* cs4 = reinterpret_cast<const float4*>(stage_ptr(s) + Cfg::kStageFloats + GT * NV * 4);
                const float4* sn4 = cs4 + nv / 2;
#pragma unroll
                for (int j = 0; j < SQ / 2; ++j) {
                    const int idx = j * LPK + sub;
                    const float4 c = cs4[idx], sn = sn4[idx];
#pragma unroll
                    for (int hh = 0; hh < GT; ++hh) {
                        const float4 a = qreg[hh][j], b = qreg[hh][j + SQ / 2];
                        qreg[hh][j] = make_float4(__fsub_rn(__fmul_rn(a.x, c.x), __fmul_rn(b.x, sn.x)),
                                                  __fsub_rn(__fmul_rn(a.y, c.y), __fmul_rn(b.y, sn.y)),
                                                  __fsub_rn(__fmul_rn(a.z, c.z), __fmul_rn(b.z, sn.z)),
                                                  __fsub_rn(__fmul_rn(a.w, c.w), __fmul_rn(b.w, sn.w)));
                        qreg[hh][j + SQ / 2] = make_float4(__fadd_rn(__fmul_rn(a.x, sn.x), __fmul_rn(b.x, c.x)),
                                                           __fadd_rn(__fmul_rn(a.y, sn.y), __fmul_rn(b.y, c.y)),
                                                           __fadd_rn(__fmul_rn(a.z, sn.z), __fmul_rn(b.z, c.z)),
                                                           __fadd_rn(__fmul_rn(a.w, sn.w), __fmul_rn(b.w, c.w)));
                    }
                }
            }
            m_run = -INFINITY;
            l_run = 0.f;
#pragma unroll
            for (int hh = 0; hh < GT; ++hh)
#pragma unroll
                for (int sv = 0; sv < SV; ++sv) acc[hh][sv] = make_float4(0.f, 0.f, 0.f, 0.f);
        }

        if (h.new_key >= 0 && ((h.new_key / KPI) % W) == cw) {
            // This warp owns the new token's row: rotate K in place if asked (lanes l and
            // l ^ nv/2 hold the two halves of a pair), then store K and V into the cache.
            float4* k4 = reinterpret_cast<float4*>(stage_ptr(s)) + size_t(h.new_key) * nv;
            const float4* v4 = reinterpret_cast<const float4*>(stage_ptr(s)) + TPS * NV + size_t(h.new_key) * nv;
            if (lane < nv) {  // nv is 16 or 32 on this path
                float4 kv = k4[lane];
                if (h.flags & kHdrRope) {
                    const int half4 = nv / 2;
                    const float4* cs4 = reinterpret_cast<const float4*>(stage_ptr(s) + Cfg::kStageFloats + GT * NV * 4);
                    const float4* sn4 = cs4 + half4;
                    float4 other;
                    other.x = __shfl_xor_sync(nv == 32 ? kFull : 0x0000ffffu, kv.x, half4);
                    other.y = __shfl_xor_sync(nv == 32 ? kFull : 0x0000ffffu, kv.y, half4);
                    other.z = __shfl_xor_sync(nv == 32 ? kFull : 0x0000ffffu, kv.z, half4);
                    other.w = __shfl_xor_sync(nv == 32 ? kFull : 0x0000ffffu, kv.w, half4);
                    const bool lo = lane < half4;
                    const float4 c = cs4[lo ? lane : lane - half4], sn = sn4[lo ? lane : lane - half4];
                    if (lo) {  // x1*cos - x2*sin
                        kv = make_float4(__fsub_rn(__fmul_rn(kv.x, c.x), __fmul_rn(other.x, sn.x)),
                                         __fsub_rn(__fmul_rn(kv.y, c.y), __fmul_rn(other.y, sn.y)),
                                         __fsub_rn(__fmul_rn(kv.z, c.z), __fmul_rn(other.z, sn.z)),
                                         __fsub_rn(__fmul_rn(kv.w, c.w), __fmul_rn(other.w, sn.w)));
                    } else {   // x1*sin + x2*cos
                        kv = make_float4(__fadd_rn(__fmul_rn(other.x, sn.x), __fmul_rn(kv.x, c.x)),
                                         __fadd_rn(__fmul_rn(other.y, sn.y), __fmul_rn(kv.y, c.y)),
                                         __fadd_rn(__fmul_rn(other.z, sn.z), __fmul_rn(kv.z, c.z)),
                                         __fadd_rn(__fmul_rn(other.w, sn.w), __fmul_rn(kv.w, c.w)));
                    }
                    k4[lane] = kv;
                }
                if (h.k_dst) {
                    reinterpret_cast<float4*>(h.k_dst)[lane] = kv;
                    reinterpret_cast<float4*>(h.v_dst)[lane] = v4[lane];
                }
            }
            __syncwarp();
        }

        {
            const int ntok = h.ntok;
            // ---- scores for this warp's keys ----
            float sc[ITERS];
            float bm = -INFINITY;
#pragma unroll
            for (int i = 0; i < ITERS; ++i) {
                const int key = i * (W * KPI) + cw * KPI + grp;
                const float4* krow = Ks + size_t(key) * nv;
                float2 part2[GT];
#pragma unroll
                for (int hh = 0; hh < GT; ++hh) part2[hh] = make_float2(0.f, 0.f);
#pragma unroll
                for (int j = 0; j < SQ; ++j) {
                    const int idx = j * LPK + sub;
                    if (idx < nv) {
                        const float4 kv = krow[idx];
#pragma unroll
                        for (int hh = 0; hh < GT; ++hh) dot4_acc(part2[hh], qreg[hh][j], kv);
                    }
                }
                float part[GT];
#pragma unroll
                for (int hh = 0; hh < GT; ++hh) part[hh] = part2[hh].x + part2[hh].y;
                float dot = group_reduce<GT, LPK>(part, sub);
                // invalid keys hold stale shared memory: discard whatever came out
                sc[i] = (key < ntok) ? dot * scale : -INFINITY;
                bm = fmaxf(bm, sc[i]);
            }
#pragma unroll
            for (int o = LPK; o < 32; o <<= 1) bm = fmaxf(bm, __shfl_xor_sync(kFull, bm, o));

            const float m_new = fmaxf(m_run, bm);
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = expf(m_run - m_safe);  // exp(-inf) = 0 on the first tile
            float psum = 0.f;
#pragma unroll
            for (int i = 0; i < ITERS; ++i) {
                const float p = (sc[i] == -INFINITY) ? 0.f : expf(sc[i] - m_safe);
                psum += p;
                if (canon) my_scr[(i * KPI + grp) * GT + hown] = p;
            }
            l_run = l_run * alpha + psum;
            if (canon && grp == 0) my_scr[KPW * 4 + hown] = alpha;
            const bool moved = __any_sync(kFull, m_new > m_run);
            m_run = m_new;
            __syncwarp();

            if (moved) {
                float al[GT];
#pragma unroll
                for (int hh = 0; hh < GT; ++hh) al[hh] = my_scr[KPW * 4 + hh];
#pragma unroll
                for (int hh = 0; hh < GT; ++hh)
#pragma unroll
                    for (int sv = 0; sv < SV; ++sv) {
                        acc[hh][sv].x *= al[hh];
                        acc[hh][sv].y *= al[hh];
                        acc[hh][sv].z *= al[hh];
                        acc[hh][sv].w *= al[hh];
                    }
            }

            // ---- weighted V rows of the same keys ----
            // No branch per key: a key beyond the tile's end has p = 0 and is pointed at the
            // tile's first row (always valid data of this unit), never at stale shared memory.
#pragma unroll
            for (int kk = 0; kk < KPW; ++kk) {
                const int key = (kk / KPI) * (W * KPI) + cw * KPI + (kk % KPI);
                const int key_c = key < ntok ? key : 0;
                float pv[GT];
#pragma unroll
                for (int hh = 0; hh < GT; ++hh) pv[hh] = my_scr[kk * GT + hh];
                const float4* vrow = Vs + size_t(key_c) * nv;
#pragma unroll
                for (int sv = 0; sv < SV; ++sv) {
                    const int idx = lane + 32 * sv;
                    if (idx < nv) {
                        const float4 vv = vrow[idx];
#pragma unroll
                        for (int hh = 0; hh < GT; ++hh) fma4_scalar(acc[hh][sv], pv[hh], vv);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[s]);
        if (!(h.flags & kHdrLast)) continue;

        // ---- last tile of the item: merge the W warp states ----
        float l_tot = l_run;
#pragma unroll
        for (int o = LPK; o < 32; o <<= 1) l_tot += __shfl_xor_sync(kFull, l_tot, o);
        if (canon && grp == 0) {
            sm_m[cw * 4 + hown] = m_run;
            sm_l[cw * 4 + hown] = l_tot;
        }
        named_bar_sync(1, W * 32);
        float f[GT];
#pragma unroll
        for (int hh = 0; hh < GT; ++hh) {
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < W; ++w) M = fmaxf(M, sm_m[w * 4 + hh]);
            const float mw = sm_m[cw * 4 + hh];
            f[hh] = (mw == -INFINITY) ? 0.f : expf(mw - M);
        }
        // The W warp states go through the reduction buffer RW warps at a time; thread e of the
        // first GT*nv consumer threads owns output element e and adds up each round.
        constexpr int RW = Cfg::kRedWarps;
        float4 esum[(GT * NV + W * 32 - 1) / (W * 32)];
#pragma unroll
        for (int i = 0; i < int(sizeof(esum) / sizeof(esum[0])); ++i) esum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int round = 0; round < W / RW; ++round) {
            if (cw / RW == round) {
#pragma unroll
                for (int hh = 0; hh < GT; ++hh)
#pragma unroll
                    for (int sv = 0; sv < SV; ++sv) {
                        const int idx = lane + 32 * sv;
                        if (idx < nv) {
                            float4 a = acc[hh][sv];
                            a.x *= f[hh]; a.y *= f[hh]; a.z *= f[hh]; a.w *= f[hh];
                            reinterpret_cast<float4*>(red)[(size_t(cw % RW) * GT + hh) * nv + idx] = a;
                        }
                    }
            }
            named_bar_sync(1, W * 32);
            int slot = 0;
            for (int e = ctid; e < GT * nv; e += W * 32, ++slot) {
                const int hh = e / nv, idx = e % nv;
                float4 sum = esum[slot];
#pragma unroll
                for (int w = 0; w < RW; ++w) {
                    const float4 a = reinterpret_cast<const float4*>(red)[(size_t(w) * GT + hh) * nv + idx];
                    sum.x += a.x; sum.y += a.y; sum.z += a.z; sum.w += a.w;
                }
                esum[slot] = sum;
            }
            if (round + 1 < W / RW) named_bar_sync(1, W * 32);
        }
        {
            int slot = 0;
            for (int e = ctid; e < GT * nv; e += W * 32, ++slot) {
                const int hh = e / nv, idx = e % nv;
                if (hh >= h.nheads) continue;
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < W; ++w) M = fmaxf(M, sm_m[w * 4 + hh]);
                float L = 0.f;
#pragma unroll
                for (int w = 0; w < W; ++w) {
                    const float mw = sm_m[w * 4 + hh];
                    L += sm_l[w * 4 + hh] * ((mw == -INFINITY) ? 0.f : expf(mw - M));
                }
                const float4 sum = esum[slot];
                if (h.part < 0) {
                    float* orow = h.out + size_t(hh) * h.o_hs;
                    const float inv = 1.0f / L;
                    const int d = idx * 4;
                    if (d + 3 < head_dim && ((reinterpret_cast<uintptr_t>(orow + d) & 15) == 0)) {
                        *reinterpret_cast<float4*>(orow + d) =
                            make_float4(sum.x * inv, sum.y * inv, sum.z * inv, sum.w * inv);
                    } else {
                        if (d + 0 < head_dim) orow[d + 0] = sum.x * inv;
                        if (d + 1 < head_dim) orow[d + 1] = sum.y * inv;
                        if (d + 2 < head_dim) orow[d + 2] = sum.z * inv;
                        if (d + 3 < head_dim) orow[d + 3] = sum.w * inv;
                    }
                } else {
                    float* rec = partials + (size_t(h.part) * GT + hh) * part_stride_floats(nv);
                    if (idx == 0) *reinterpret_cast<float4*>(rec) = make_float4(M, L, 0.f, 0.f);
                    reinterpret_cast<float4*>(rec + 4)[idx] = sum;
                }
            }
        }
        if (h.part < 0) continue;

        // ---- the unit was cut: whoever delivers its last partial combines them all ----
        // (block barrier, then one thread fences and counts: the fence is cumulative over the
        // writes the barrier ordered before it, so the other threads need none of their own)
        named_bar_sync(1, W * 32);
        if (ctid == 0) {
            __threadfence();
            const int old = atomicAdd(&sync[kSyncMerge0 + h.merge_slot], 1);
            const int last = old == h.part_count - 1;
            if (last) {
                sync[kSyncMerge0 + h.merge_slot] = 0;  // re-armed for the next launch
                __threadfence();                       // the other partials are read after this
            }
            *last_flag = last;
        }
        named_bar_sync(1, W * 32);
        if (*last_flag) {
            const size_t ps = part_stride_floats(nv);
            for (int e = ctid; e < GT * nv; e += W * 32) {
                const int hh = e / nv, idx = e % nv;
                if (hh >= h.nheads) continue;
                float M = -INFINITY;
                for (int i = 0; i < h.part_count; ++i)
                    M = fmaxf(M, __ldcg(partials + (size_t(h.part_begin + i) * GT + hh) * ps));
                float L = 0.f;
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int i = 0; i < h.part_count; ++i) {
                    const float* rec = partials + (size_t(h.part_begin + i) * GT + hh) * ps;
                    const float mi = __ldcg(rec);
                    const float wgt = (mi == -INFINITY) ? 0.f : expf(mi - M);
                    L += __ldcg(rec + 1) * wgt;
                    const float4 a = __ldcg(reinterpret_cast<const float4*>(rec + 4) + idx);
                    sum.x = fmaf(wgt, a.x, sum.x);
                    sum.y = fmaf(wgt, a.y, sum.y);
                    sum.z = fmaf(wgt, a.z, sum.z);
                    sum.w = fmaf(wgt, a.w, sum.w);
                }
                const float inv = 1.0f / L;
                float* orow = h.out + size_t(hh) * h.o_hs;
                const int d = idx * 4;
                if (d + 0 < head_dim) orow[d + 0] = sum.x * inv;
                if (d + 1 < head_dim) orow[d + 1] = sum.y * inv;
                if (d + 2 < head_dim) orow[d + 2] = sum.z * inv;
                if (d + 3 < head_dim) orow[d + 3] = sum.w * inv;
            }
        }
        // (no barrier here: `red` and `last_flag` are next written behind the next item's barriers,
        // which no thread passes before every thread has left this point)
    }
}

// Generic attention for requests whose positions fold around the ring (index_pos + seq_len >
// capacity): logical positions 0..=limit are visited in order and mapped with % cap exactly as
// the reference does (fast_attention_simd.rs:608, :145), so a slot that was overwritten is
// counted once per visit.  One block per (request row, query head); plain loads, chunked online
// softmax.  Never on the fast path.  With pool8 != nullptr the cache is the u8 format (rows of dq
// bytes with one scale each, blocks of K bytes | V bytes | K scales | V scales) and the values
// are (byte - 128) * scale.
__global__ void __launch_bounds__(256, 1)
attn_ring_kernel(const ReqDev* __restrict__ reqs, const int* __restrict__ ring_rows, int n_rows,
                 const int* __restrict__ page_ids, const float* __restrict__ k_pool,
                 const float* __restrict__ v_pool, long long pool_pages, int num_heads,
                 int num_kv_heads, int head_dim, int nv, float scale,
                 const unsigned char* __restrict__ pool8, int dq) {
    constexpr int kChunk = 1024;
    __shared__ float s_q[256];
    __shared__ float s_p[kChunk];
    __shared__ float s_red[256];
    const int row = blockIdx.x / num_heads, h = blockIdx.x % num_heads;
    if (row >= n_rows) return;
    const int req = ring_rows[2 * row], t_q = ring_rows[2 * row + 1];
    const ReqDev& r = reqs[req];
    const int* pages = page_ids + r.page_off;
    const int h_kv = h / (num_heads / num_kv_heads);
    const int tid = threadIdx.x;
    const int dp = nv * 4;
    const size_t page_floats = size_t(kPageTokens) * dp;
    const size_t layer_base = size_t(r.layer) * size_t(pool_pages);
    const int limit = r.index_pos + t_q;  // inclusive
    const float* qrow = r.q + size_t(h) * r.q_hs + size_t(t_q) * r.q_ts;
    if (tid < head_dim) s_q[tid] = qrow[tid];
    __syncthreads();

    float m_run = -INFINITY, l_run = 0.f, acc = 0.f;
    for (int c0 = 0; c0 <= limit; c0 += kChunk) {
        const int cn = min(kChunk, limit + 1 - c0);
        float lmax = -INFINITY;
        for (int i = tid; i < cn; i += 256) {
            const int slot = (c0 + i) % r.cap;
            float dot = 0.f;
            if (pool8) {
                const unsigned char* blk = pool8 + ((layer_base + size_t(pages[slot / kPageTokens])) * num_kv_heads + h_kv) *
                                                       (size_t(kPageTokens) * (2 * size_t(dq) + 8));
                const unsigned char* krow = blk + size_t(slot % kPageTokens) * dq;
                const float ks = reinterpret_cast<const float*>(blk + 2 * size_t(kPageTokens) * dq)[slot % kPageTokens];
                for (int d = 0; d < head_dim; ++d) dot = fmaf(s_q[d], (float(krow[d]) - 128.0f) * ks, dot);
            } else {
                const float* krow = k_pool +
                                    ((layer_base + size_t(pages[slot / kPageTokens])) * num_kv_heads + h_kv) * page_floats +
                                    size_t(slot % kPageTokens) * dp;
                for (int d = 0; d < head_dim; ++d) dot = fmaf(s_q[d], krow[d], dot);
            }
            dot *= scale;
            s_p[i] = dot;
            lmax = fmaxf(lmax, dot);
        }
        s_red[tid] = lmax;
        __syncthreads();
        for (int o = 128; o > 0; o >>= 1) {
            if (tid < o) s_red[tid] = fmaxf(s_red[tid], s_red[tid + o]);
            __syncthreads();
        }
        const float m_new = fmaxf(m_run, s_red[0]);
        __syncthreads();
        float lsum = 0.f;
        for (int i = tid; i < cn; i += 256) {
            const float p = expf(s_p[i] - m_new);
            s_p[i] = p;
            lsum += p;
        }
        s_red[tid] = lsum;
        __syncthreads();
        for (int o = 128; o > 0; o >>= 1) {
            if (tid < o) s_red[tid] += s_red[tid + o];
            __syncthreads();
        }
        const float alpha = expf(m_run - m_new);
        l_run = l_run * alpha + s_red[0];
        m_run = m_new;
        if (tid < head_dim) {
            acc *= alpha;
            for (int i = 0; i < cn; ++i) {
                const int slot = (c0 + i) % r.cap;
                if (pool8) {
                    const unsigned char* blk = pool8 + ((layer_base + size_t(pages[slot / kPageTokens])) * num_kv_heads + h_kv) *
                                                           (size_t(kPageTokens) * (2 * size_t(dq) + 8));
                    const float vs = reinterpret_cast<const float*>(blk + 2 * size_t(kPageTokens) * dq)[kPageTokens + slot % kPageTokens];
                    const float vv = (float(blk[size_t(kPageTokens + slot % kPageTokens) * dq + tid]) - 128.0f) * vs;
                    acc = fmaf(s_p[i], vv, acc);
                } else {
                    const float* vrow = v_pool +
                                        ((layer_base + size_t(pages[slot / kPageTokens])) * num_kv_heads + h_kv) * page_floats +
                                        size_t(slot % kPageTokens) * dp;
                    acc = fmaf(s_p[i], vrow[tid], acc);
                }
            }
        }
        __syncthreads();
    }
    if (tid < head_dim) r.out[size_t(h) * r.o_hs + size_t(t_q) * r.o_ts + tid] = acc / l_run;
}

}  // namespace xn
