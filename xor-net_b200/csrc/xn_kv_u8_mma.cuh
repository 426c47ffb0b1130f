// Split-KV attention over u8 pages with the q.k products on the integer tensor-core path
// (mma.sync m16n8k32, u8 x s8 -> s32), sm_100a.
//
// The cached K bytes ARE an MMA operand: a tile of 16 keys x 32 dims is four 32-bit words per lane
// straight out of the page, no dequantisation.  The query rows become three int8 terms per head,
// q = sq * (q1 + q2 / 128 + q3 / 16384) with |residual| <= max|q| * 2.4e-7, so three exact integer
// MMAs per 32 dims give the dot products to f32 accuracy; the -128 of the byte format enters as
// the accumulators' initial value (-128 * sum of the term's int8 values).  P.V stays on the CUDA
// cores (V is stored key-major, which no MMA operand layout takes without a transpose): the
// weights travel from the accumulator layout to the lanes that hold the V rows through a
// 256-byte shared-memory tile.
//
// Work decomposition, plan, partial records and merge protocol are those of attn_splitkv_u8_kernel
// (xn_kv_u8.cuh); one-warp blocks; a warp iteration covers 16 keys, whose K rows, V rows and scales
// are contiguous in the page: one lane fetches them with four 1-D bulk copies (TMA engine, byte
// counting on an mbarrier private to the warp; no tensor map, no multicast) a few tiles ahead.  The softmax keeps one running
// reference per head for the whole warp.  Shapes: row widths of 64 and 128 bytes (head_dim 64 or
// 128 exactly), up to 4 query heads per unit.  The append is not fused into this kernel.
#pragma once
#include "xn_kv_u8.cuh"

namespace xn {
namespace kv8m {

using kv8::block_bytes;
using kv8::exp2_weight;
using kv8::kLazy;
using kv8::part_stride;

constexpr int kThreads = 32;
constexpr int kTileKeys = 16;   // keys per warp iteration (the M of the MMA)
#ifndef XN_KV8M_PREFETCH
#define XN_KV8M_PREFETCH 3
#endif
#ifndef XN_KV8M_BLOCKS
#define XN_KV8M_BLOCKS 12
#endif
constexpr int kPrefetch = XN_KV8M_PREFETCH;
constexpr int kBlocksPerSm = XN_KV8M_BLOCKS;

// per stage: K rows [16][DQ], V rows [16][DQ], then 16 K scales and 16 V scales
__host__ __device__ constexpr size_t stage_bytes(int dq) { return size_t(2) * kTileKeys * dq + 128; }
__host__ __device__ constexpr size_t red_bytes(int gt, int dq) { return size_t(512 / dq) * 2 * gt * dq * 4; }
__host__ __device__ constexpr size_t smem_bytes(int gt, int dq) {
    return kPrefetch * stage_bytes(dq) > red_bytes(gt, dq) ? kPrefetch * stage_bytes(dq) : red_bytes(gt, dq);
}

__device__ __forceinline__ void imma_u8s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// LPK = DQ / 16 lanes share a key in the P.V phase (4 or 8); GT query heads per unit (<= 4).
template <int LPK, int GT>
__global__ void __launch_bounds__(kThreads, kBlocksPerSm)
attn_splitkv_u8_mma_kernel(const ReqDev* __restrict__ reqs, const UnitDev* __restrict__ units,
                           const ItemDev* __restrict__ items, const int* __restrict__ chunk_item_begin,
                           int n_chunks, const int* __restrict__ page_ids,
                           const uint8_t* __restrict__ pool, float* __restrict__ partials,
                           int* __restrict__ sync, long long pool_pages, int num_kv_heads, int head_dim,
                           float scale_log2, const float* __restrict__ cos_t,
                           const float* __restrict__ sin_t, int* __restrict__ status) {
    constexpr int DQ = LPK * 16;           // bytes per stored row
    constexpr int BPL = DQ / 4;            // bytes of a K row per lane in the MMA layout
    constexpr int KS = DQ / 32;            // MMA k-steps per row
    constexpr int KW = BPL / 4;            // 32-bit words of a K row per lane (= 2 * KS)
    constexpr int KPI = 32 / LPK;          // keys per P.V sub-iteration
    constexpr int SUBS = kTileKeys / KPI;  // P.V sub-iterations per tile
    constexpr int PF = kPrefetch;
    constexpr unsigned kFull = 0xffffffffu;
    (void)cos_t;
    (void)sin_t;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* red = reinterpret_cast<float*>(smem_raw);   // [KPI groups][GT][DQ], while the ring is idle
    __shared__ __align__(16) float sm_p[kTileKeys][4];  // weights (times the V scale) of a tile: [key][head]
    __shared__ __align__(16) float sm_alpha[4];
    __shared__ int sm_next, sm_last;
    __shared__ __align__(8) uint64_t full_bar[PF];

    pdl_launch_dependents();
    const int lane = threadIdx.x;
    if (lane == 0) {
        for (int s = 0; s < PF; ++s) mbar_init(&full_bar[s], 1);
        mbar_fence_init();
    }
    __syncwarp();
    int fill = 0, use = 0;   // tiles requested / consumed by this warp so far (ring position, parity)
    bool ok = true;
    const int g = lane >> 2, t = lane & 3;             // MMA layout: rows g and g + 8, column group t
    const int sub = lane % LPK, grp = lane / LPK;      // P.V layout: key group, 16-byte slice of a row
    const size_t blk_bytes = block_bytes(DQ);
    const size_t page_stride = size_t(num_kv_heads) * blk_bytes;
    const size_t pstride = part_stride(DQ);
    auto stage_k = [&](int s) { return smem_raw + size_t(s) * kv8m::stage_bytes(DQ); };
    auto stage_v = [&](int s) { return stage_k(s) + kTileKeys * DQ; };
    auto stage_sc = [&](int s) { return reinterpret_cast<float*>(stage_v(s) + kTileKeys * DQ); };

    int chunk = blockIdx.x;
    while (ok && chunk < n_chunks) {
        const int it_lo = chunk_item_begin[chunk], it_hi = chunk_item_begin[chunk + 1];
        for (int it = it_lo; ok && it < it_hi; ++it) {
            const ItemDev item = items[it];
            const UnitDev u = units[item.unit];
            const ReqDev& r = reqs[u.req];
            const float* qrow = r.q + size_t(u.head0) * r.q_hs + size_t(u.t_q) * r.q_ts;
            float* orow = r.out + size_t(u.head0) * r.o_hs + size_t(u.t_q) * r.o_ts;
            const long long q_hs = r.q_hs, o_hs = r.o_hs;
            const int* pages = page_ids + r.page_off;
            const uint8_t* base = pool + (size_t(r.layer) * size_t(pool_pages) * num_kv_heads + u.kv_head) * blk_bytes;
            const int tok_begin = item.tile_begin * kPageTokens;
            const int tok_end = min(item.tile_end * kPageTokens, u.kv_len);

            // ---- query head g of the unit as three int8 terms, in the B-operand layout ----
            // lane (g, t) holds dims BPL * t .. BPL * t + BPL - 1 of head g; word j of the K rows
            // (k-step j / 2, half j % 2) pairs with bq[term][j]
            uint32_t bq[3][KW];
            float sq_own;        // scale of head g's first term
            int corr_own[3];     // 128 * sum over all dims of the term's values, head g
            {
                float x[BPL];
                float amax = 0.f;
#pragma unroll
                for (int j = 0; j < BPL; ++j) {
                    x[j] = g < u.nheads ? qrow[size_t(g) * q_hs + BPL * t + j] : 0.f;
                    amax = fmaxf(amax, fabsf(x[j]));
                }
                amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 2));
                sq_own = amax > 0.f ? amax * (1.0f / 127.0f) : 1.0f;
                float sc = sq_own;
#pragma unroll
                for (int term = 0; term < 3; ++term) {
                    const float inv = 1.0f / sc;
                    int sum = 0;
#pragma unroll
                    for (int j = 0; j < KW; ++j) bq[term][j] = 0u;
#pragma unroll
                    for (int j = 0; j < BPL; ++j) {
                        const float qv = rintf(x[j] * inv);
                        x[j] = fmaf(-qv, sc, x[j]);              // residual, exact enough: |x| <= sc / 2
                        const int qi = int(qv);
                        sum += qi;
                        bq[term][j / 4] |= (uint32_t(qi) & 0xffu) << (8 * (j % 4));
                    }
                    sum += __shfl_xor_sync(kFull, sum, 1);
                    sum += __shfl_xor_sync(kFull, sum, 2);
                    corr_own[term] = 128 * sum;
                    sc *= (1.0f / 128.0f);
                }
            }
            // the accumulator layout wants heads 2t and 2t + 1: their scales and corrections
            float sqh[2];
            int cinit[3][2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int src = (2 * t + e) * 4;   // lane (g = 2t + e, t = 0)
                sqh[e] = __shfl_sync(kFull, sq_own, src) * scale_log2;
#pragma unroll
                for (int term = 0; term < 3; ++term) cinit[term][e] = -__shfl_sync(kFull, corr_own[term], src);
            }

            float m_ref[2] = {-INFINITY, -INFINITY};   // running reference of heads 2t, 2t + 1 (lanes t < 2)
            float l_part[2] = {0.f, 0.f};              // this lane's share of the weight sums
            float2 acc[GT][8];
#pragma unroll
            for (int hh = 0; hh < GT; ++hh)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[hh][e] = make_float2(0.f, 0.f);

            // ---- copies: one commit group per tile of 16 keys ----
            // (an item starts on a page boundary; the id of the page after the current one is fetched
            // a page ahead, so that its latency is not paid when the boundary is reached)
            const uint8_t* page_blk = nullptr;
            int next_page = pages[tok_begin / kPageTokens];
            // a tile of 16 keys is always fetched whole (it lies inside one page; rows past the
            // item's end hold finite bytes and are masked below)
            auto issue = [&](int k0) {
                if (k0 < tok_end) {
                    if (k0 % kPageTokens == 0) {
                        page_blk = base + size_t(next_page) * page_stride;
                        if (k0 + kPageTokens < tok_end) next_page = pages[k0 / kPageTokens + 1];
                    }
                    if (lane == 0) {
                        const int s = fill % PF;
                        const int tk0 = k0 % kPageTokens;
                        const uint8_t* sc = page_blk + 2 * size_t(kPageTokens) * DQ;
                        mbar_arrive_expect_tx(&full_bar[s], uint32_t(2 * kTileKeys * DQ + 128));
                        bulk_g2s(stage_k(s), page_blk + size_t(tk0) * DQ, kTileKeys * DQ, &full_bar[s]);
                        bulk_g2s(stage_v(s), page_blk + size_t(kPageTokens + tk0) * DQ, kTileKeys * DQ, &full_bar[s]);
                        bulk_g2s(stage_sc(s), sc + 4 * size_t(tk0), 64, &full_bar[s]);
                        bulk_g2s(stage_sc(s) + 16, sc + 4 * size_t(kPageTokens + tk0), 64, &full_bar[s]);
                    }
                    ++fill;
                }
            };

#pragma unroll
            for (int p = 0; p < PF; ++p) issue(tok_begin + p * kTileKeys);
            for (int kt = tok_begin; ok && kt < tok_end; kt += kTileKeys) {
                {
                    const int p = use % PF;
                    int got = 1;
                    if (lane == 0) got = mbar_spin_bounded(&full_bar[p], (use / PF) & 1) ? 1 : 0;
                    got = __shfl_sync(kFull, got, 0);
                    if (!got) {   // a copy was lost: report it and leave (nothing else is waited for)
                        if (lane == 0) report_status(status, kDevWaitFull);
                        ok = false;
                        break;
                    }
                    ++use;
                    // ---- q.k on the tensor cores ----
                    uint32_t kw[2][KW];
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr)
#pragma unroll
                        for (int c = 0; c < BPL / 16; ++c) {
                            const uint4 w = *reinterpret_cast<const uint4*>(stage_k(p) + size_t(g + 8 * rr) * DQ + BPL * t + 16 * c);
                            kw[rr][4 * c + 0] = w.x; kw[rr][4 * c + 1] = w.y;
                            kw[rr][4 * c + 2] = w.z; kw[rr][4 * c + 3] = w.w;
                        }
                    int ci[3][4];
#pragma unroll
                    for (int term = 0; term < 3; ++term) {
                        ci[term][0] = ci[term][2] = cinit[term][0];
                        ci[term][1] = ci[term][3] = cinit[term][1];
                    }
#pragma unroll
                    for (int s = 0; s < KS; ++s) {
                        const uint32_t a[4] = {kw[0][2 * s], kw[1][2 * s], kw[0][2 * s + 1], kw[1][2 * s + 1]};
#pragma unroll
                        for (int term = 0; term < 3; ++term) imma_u8s8(ci[term], a, bq[term][2 * s], bq[term][2 * s + 1]);
                    }
                    // ---- scores of keys g and g + 8 for heads 2t, 2t + 1 (log2 domain) ----
                    const float* scp = stage_sc(p);
                    float sv[2][2];
                    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        const bool valid = kt + g + 8 * rr < tok_end;
                        const float ks = scp[g + 8 * rr];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float dot = fmaf(float(ci[2][2 * rr + e]), 1.0f / 16384.0f,
                                                   fmaf(float(ci[1][2 * rr + e]), 1.0f / 128.0f,
                                                        float(ci[0][2 * rr + e])));
                            sv[rr][e] = valid ? dot * (ks * sqh[e]) : -INFINITY;
                            tmax[e] = fmaxf(tmax[e], sv[rr][e]);
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        tmax[e] = fmaxf(tmax[e], __shfl_xor_sync(kFull, tmax[e], 4));
                        tmax[e] = fmaxf(tmax[e], __shfl_xor_sync(kFull, tmax[e], 8));
                        tmax[e] = fmaxf(tmax[e], __shfl_xor_sync(kFull, tmax[e], 16));
                    }
                    // ---- running reference per head; rescale only on a jump of more than kLazy ----
                    const bool moved0 = tmax[0] > m_ref[0] + kLazy, moved1 = tmax[1] > m_ref[1] + kLazy;
                    if (__any_sync(kFull, (moved0 || moved1) && t < 2)) {
                        float al[2];
                        al[0] = moved0 ? exp2_weight(m_ref[0] - tmax[0]) : 1.f;
                        al[1] = moved1 ? exp2_weight(m_ref[1] - tmax[1]) : 1.f;
                        if (moved0) m_ref[0] = tmax[0];
                        if (moved1) m_ref[1] = tmax[1];
                        l_part[0] *= al[0];
                        l_part[1] *= al[1];
                        if (g == 0 && t < 2) {
                            sm_alpha[2 * t] = al[0];
                            sm_alpha[2 * t + 1] = al[1];
                        }
                        __syncwarp();
                        const float4 a4 = *reinterpret_cast<const float4*>(sm_alpha);
                        const float av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                        for (int hh = 0; hh < GT; ++hh) {
                            const float2 a2 = make_float2(av[hh], av[hh]);
#pragma unroll
                            for (int e = 0; e < 8; ++e) acc[hh][e] = __fmul2_rn(acc[hh][e], a2);
                        }
                        __syncwarp();
                    }
                    // ---- weights, times the V scale, into the exchange tile ----
                    if (t < 2) {
#pragma unroll
                        for (int rr = 0; rr < 2; ++rr) {
                            const bool valid = kt + g + 8 * rr < tok_end;
                            const float vs = scp[16 + g + 8 * rr];
                            float pw[2];
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                pw[e] = valid ? exp2_weight(sv[rr][e] - m_ref[e]) : 0.f;
                                l_part[e] += pw[e];
                                pw[e] = valid ? pw[e] * vs : 0.f;
                            }
                            *reinterpret_cast<float2*>(&sm_p[g + 8 * rr][2 * t]) = make_float2(pw[0], pw[1]);
                        }
                    }
                    __syncwarp();
                    // ---- weighted V rows on the CUDA cores ----
#pragma unroll
                    for (int i = 0; i < SUBS; ++i) {
                        const int kk = KPI * i + grp;
                        const float4 p4 = *reinterpret_cast<const float4*>(sm_p[kk]);
                        const float pv[4] = {p4.x, p4.y, p4.z, p4.w};
                        const uint4 w = *reinterpret_cast<const uint4*>(stage_v(p) + size_t(kk) * DQ + 16 * sub);
                        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
                        float2 vf[8];
                        kv8::dequant<4>(ws, vf);
#pragma unroll
                        for (int hh = 0; hh < GT; ++hh) {
                            const float2 p2 = make_float2(pv[hh], pv[hh]);
#pragma unroll
                            for (int e = 0; e < 8; ++e) acc[hh][e] = __ffma2_rn(p2, vf[e], acc[hh][e]);
                        }
                    }
                    __syncwarp();   // sm_p is rewritten by the next tile
                    issue(kt + PF * kTileKeys);
                }
            }
            if (!ok) break;
            __syncwarp();

            // ---- the item's result: sum the key groups' accumulators through shared memory ----
            float* mine = red + (size_t(grp) * GT) * DQ + sub * 16;
#pragma unroll
            for (int hh = 0; hh < GT; ++hh)
#pragma unroll
                for (int e = 0; e < 8; e += 2)
                    *reinterpret_cast<float4*>(mine + size_t(hh) * DQ + 2 * e) =
                        make_float4(acc[hh][e].x, acc[hh][e].y, acc[hh][e + 1].x, acc[hh][e + 1].y);
            // weight sums and references of the 4 heads, on every lane
            float Lh[4], Mh[4];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float lv = t < 2 ? l_part[e] : 0.f;
                lv += __shfl_xor_sync(kFull, lv, 4);
                lv += __shfl_xor_sync(kFull, lv, 8);
                lv += __shfl_xor_sync(kFull, lv, 16);
                // lanes (g, t) with t < 2 now hold the sum for head 2t + e
                Lh[e] = __shfl_sync(kFull, lv, 0);       // head e       (t = 0)
                Lh[2 + e] = __shfl_sync(kFull, lv, 1);   // head 2 + e   (t = 1)
                Mh[e] = __shfl_sync(kFull, m_ref[e], 0);
                Mh[2 + e] = __shfl_sync(kFull, m_ref[e], 1);
            }
            __syncwarp();
            for (int e = lane; e < GT * DQ; e += kThreads) {
                const int hh = e / DQ, d = e % DQ;
                if (hh >= u.nheads) continue;
                float sum = 0.f;
#pragma unroll
                for (int gg = 0; gg < KPI; ++gg) sum += red[(size_t(gg) * GT + hh) * DQ + d];
                const float L = hh == 0 ? Lh[0] : (hh == 1 ? Lh[1] : (hh == 2 ? Lh[2] : Lh[3]));
                const float M = hh == 0 ? Mh[0] : (hh == 1 ? Mh[1] : (hh == 2 ? Mh[2] : Mh[3]));
                if (item.part < 0) {
                    if (d < head_dim) orow[size_t(hh) * o_hs + d] = sum * (1.0f / L);
                } else {
                    float* rec = partials + (size_t(item.part) * GT + hh) * pstride;
                    if (d == 0) {
                        rec[0] = M;
                        rec[1] = L;
                    }
                    rec[4 + d] = sum;
                }
            }
            if (item.part >= 0) {
                __syncwarp();
                if (lane == 0) {
                    __threadfence();
                    const int old = atomicAdd(&sync[kSyncMerge0 + u.merge_slot], 1);
                    const int last = old == u.part_count - 1;
                    if (last) {
                        sync[kSyncMerge0 + u.merge_slot] = 0;
                        __threadfence();
                    }
                    sm_last = last;
                }
                __syncwarp();
                if (sm_last) {
                    // combine the unit's partial records, all heads at once (as in attn_splitkv_u8_kernel)
                    constexpr int J = (DQ + 31) / 32;
                    const size_t rstride = size_t(GT) * pstride;
                    const float* rec0 = partials + size_t(u.part_begin) * rstride;
                    float Mrun[GT], L[GT], sum[GT][J];
#pragma unroll
                    for (int hh = 0; hh < GT; ++hh) {
                        Mrun[hh] = -INFINITY;
                        L[hh] = 0.f;
#pragma unroll
                        for (int j = 0; j < J; ++j) sum[hh][j] = 0.f;
                    }
                    for (int i0 = 0; i0 < u.part_count; i0 += 32) {
                        const int cnt = min(32, u.part_count - i0);
                        float mi[GT], li[GT], wgt[GT];
#pragma unroll
                        for (int hh = 0; hh < GT; ++hh) {
                            const float* rec = rec0 + size_t(i0 + lane) * rstride + size_t(hh) * pstride;
                            mi[hh] = lane < cnt ? __ldcg(rec) : -INFINITY;
                            li[hh] = lane < cnt ? __ldcg(rec + 1) : 0.f;
                        }
#pragma unroll
                        for (int hh = 0; hh < GT; ++hh) {
                            float mb = mi[hh];
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) mb = fmaxf(mb, __shfl_xor_sync(kFull, mb, o));
                            const float mn = fmaxf(Mrun[hh], mb);
                            const float alpha = (Mrun[hh] == -INFINITY) ? 0.f : exp2f(Mrun[hh] - mn);
                            wgt[hh] = (mi[hh] == -INFINITY) ? 0.f : exp2f(mi[hh] - mn);
                            float lw = li[hh] * wgt[hh];
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) lw += __shfl_xor_sync(kFull, lw, o);
                            L[hh] = L[hh] * alpha + lw;
#pragma unroll
                            for (int j = 0; j < J; ++j) sum[hh][j] *= alpha;
                            Mrun[hh] = mn;
                        }
#pragma unroll 4
                        for (int i = 0; i < cnt; ++i) {
                            const float* rec = rec0 + size_t(i0 + i) * rstride + 4;
#pragma unroll
                            for (int hh = 0; hh < GT; ++hh) {
                                const float wi = __shfl_sync(kFull, wgt[hh], i);
#pragma unroll
                                for (int j = 0; j < J; ++j) {
                                    const int d = lane + 32 * j;
                                    if (d < DQ) sum[hh][j] = fmaf(wi, __ldcg(rec + size_t(hh) * pstride + d), sum[hh][j]);
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int hh = 0; hh < GT; ++hh) {
                        if (hh >= u.nheads) break;
                        const float inv = 1.0f / L[hh];
#pragma unroll
                        for (int j = 0; j < J; ++j) {
                            const int d = lane + 32 * j;
                            if (d < head_dim) orow[size_t(hh) * o_hs + d] = sum[hh][j] * inv;
                        }
                    }
                }
            }
            __syncwarp();   // red / the ring, sm_p and sm_last are rewritten by the next item
        }
        if (lane == 0) sm_next = atomicAdd(&sync[kSyncChunk], 1) + int(gridDim.x);
        __syncwarp();
        chunk = sm_next;
        __syncwarp();
    }
    if (lane == 0) {
        __threadfence();
        if (atomicAdd(&sync[kSyncDone], 1) == int(gridDim.x) - 1) {
            sync[kSyncChunk] = 0;
            sync[kSyncDone] = 0;
        }
    }
}

}  // namespace kv8m
}  // namespace xn
