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
//   * the host deals the flattened tile list evenly to the thread blocks (one per SM), so
//     ragged lengths cost nothing; a unit cut across blocks yields partials that
//     `attn_merge_kernel` combines with the usual log-sum-exp weights;
//   * inside a block one producer lane streams tiles into a ring of shared-memory stages with
//     1-D bulk async copies (TMA engine, mbarrier byte counting, no tensor map, no multicast);
//     WARPS consumer warps each own a fixed subset of a tile's tokens and keep an independent
//     online-softmax state (running max, sum, accumulator) merged once per unit.
#pragma once
#include "xn_common.cuh"

namespace xn {

template <int NV>
struct DecodeCfg {
    static constexpr int kWarps = 8;                      // consumer warps
    static constexpr int kThreads = (kWarps + 1) * 32;    // + 1 producer warp
    static constexpr int kLPK = (NV <= 32) ? 8 : 16;      // lanes sharing one key in q.k
    static constexpr int kKPI = 32 / kLPK;                // keys per warp iteration
    static constexpr int kTPS = (NV <= 32) ? 64 : 32;     // tokens per stage
    static constexpr int kKPW = kTPS / kWarps;            // keys per warp per stage
    static constexpr int kIters = kKPW / kKPI;
    static constexpr int kSlotsQ = (NV + kLPK - 1) / kLPK;  // float4 of q per lane per head
    static constexpr int kSlotsV = (NV + 31) / 32;          // float4 of output per lane per head
    static constexpr int kStages = 3;
    static constexpr int kStageFloats = 2 * kTPS * NV * 4;  // K block then V block
    static_assert(kIters >= 1, "tile too small for the warp layout");
};

template <int NV, int GT>
struct DecodeSmem {
    using Cfg = DecodeCfg<NV>;
    static constexpr size_t kStageBytes = size_t(Cfg::kStageFloats) * 4;
    static constexpr size_t kRedFloats = size_t(Cfg::kWarps) * GT * NV * 4;
    static constexpr size_t kScratchFloats = size_t(Cfg::kWarps) * (Cfg::kKPW + 1) * 4;  // GT<=4
    static constexpr size_t kBytes = Cfg::kStages * kStageBytes + kRedFloats * 4 +
                                     kScratchFloats * 4 + Cfg::kWarps * 4 * 2 * 4 /* m,l */ +
                                     2 * Cfg::kStages * 8 /* barriers */ + 16 /* flags */;
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

template <int GT>
__device__ __forceinline__ int owned_head(int sub) {
    if constexpr (GT == 4) return ((sub & 1) << 1) | ((sub >> 1) & 1);
    if constexpr (GT == 2) return sub & 1;
    return 0;
}

// Partial record of one (item, head): [m, l, 0, 0, acc[Dp]] floats.
__host__ __device__ __forceinline__ size_t part_stride_floats(int nv) { return size_t(nv) * 4 + 4; }

template <int NV, int GT>
__global__ void __launch_bounds__(DecodeCfg<NV>::kThreads, 1)
attn_splitkv_kernel(const ReqDev* __restrict__ reqs, const UnitDev* __restrict__ units,
                    const ItemDev* __restrict__ items, const int* __restrict__ cta_item_begin,
                    const int* __restrict__ page_ids, const float* __restrict__ k_pool,
                    const float* __restrict__ v_pool, float* __restrict__ partials,
                    long long pool_pages, int num_kv_heads, int head_dim, int nv, float scale,
                    int* __restrict__ status) {
    using Cfg = DecodeCfg<NV>;
    using Sm = DecodeSmem<NV, GT>;
    constexpr int W = Cfg::kWarps, LPK = Cfg::kLPK, KPI = Cfg::kKPI, TPS = Cfg::kTPS;
    constexpr int KPW = Cfg::kKPW, ITERS = Cfg::kIters, ST = Cfg::kStages;
    constexpr int SQ = Cfg::kSlotsQ, SV = Cfg::kSlotsV;
    constexpr unsigned kFull = 0xffffffffu;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* stage_base = reinterpret_cast<float*>(smem_raw);
    float* red = reinterpret_cast<float*>(smem_raw + ST * Sm::kStageBytes);
    float* scratch = red + Sm::kRedFloats;
    float* sm_m = scratch + Sm::kScratchFloats;  // [W][4]
    float* sm_l = sm_m + W * 4;                  // [W][4]
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(sm_l + W * 4);
    uint64_t* empty_bar = full_bar + ST;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + ST);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int item_lo = cta_item_begin[blockIdx.x], item_hi = cta_item_begin[blockIdx.x + 1];
    const int dp = nv * 4;  // padded row length in floats
    const size_t page_floats = size_t(kPageTokens) * dp;

    if (tid == 0) {
        for (int s = 0; s < ST; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], W);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == 0) {
        // ---------------- producer: one lane feeds the stage ring ----------------
        if (lane == 0) {
            int fill = 0;
            bool ok = true;
            for (int it = item_lo; it < item_hi && ok; ++it) {
                const ItemDev item = items[it];
                const UnitDev u = units[item.unit];
                const ReqDev& r = reqs[u.req];
                const int* pages = page_ids + r.page_off;
                const size_t layer_base = size_t(r.layer) * size_t(pool_pages);
                for (int tile = item.tile_begin; tile < item.tile_end; ++tile, ++fill) {
                    const int s = fill % ST;
                    if (fill >= ST) {
                        if (!mbar_wait_bounded(&empty_bar[s], ((fill / ST) - 1) & 1)) {
                            atomicExch(status, kDevWaitEmpty);
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                    }
                    const int tok0 = tile * TPS;
                    const int ntok = min(TPS, u.kv_len - tok0);
                    const int page = pages[tok0 / kPageTokens];
                    const size_t src = ((layer_base + size_t(page)) * num_kv_heads + u.kv_head) *
                                           page_floats +
                                       size_t(tok0 % kPageTokens) * dp;
                    const uint32_t bytes = uint32_t(ntok) * dp * 4;
                    float* dst = stage_base + size_t(s) * Cfg::kStageFloats;
                    mbar_arrive_expect_tx(&full_bar[s], 2 * bytes);
                    bulk_g2s(dst, k_pool + src, bytes, &full_bar[s]);
                    bulk_g2s(dst + TPS * NV * 4, v_pool + src, bytes, &full_bar[s]);
                }
            }
            if (!ok) {
                // Do not retire the block with copies still landing in its shared memory.
                for (int f = max(0, fill - ST); f < fill; ++f)
                    mbar_wait_bounded(&full_bar[f % ST], (f / ST) & 1);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int cw = warp - 1;
    const int sub = lane % LPK, grp = lane / LPK;
    const int hown = owned_head<GT>(sub);
    const bool canon = sub < GT;  // one lane per (key group, head) publishes p
    float* my_scr = scratch + cw * (KPW + 1) * 4;
    const int ctid = tid - 32;  // 0 .. W*32-1

    int fill = 0;
    bool dead = false;  // set when a wait gave up: keep the barrier protocol, skip the math

    for (int it = item_lo; it < item_hi; ++it) {
        const ItemDev item = items[it];
        const UnitDev u = units[item.unit];
        const ReqDev& r = reqs[u.req];

        // query rows of the unit's heads, the float4 slots this lane multiplies
        float4 qreg[GT][SQ];
#pragma unroll
        for (int h = 0; h < GT; ++h) {
            const float* qrow = r.q + size_t(u.head0 + h) * r.q_hs + size_t(u.t_q) * r.q_ts;
#pragma unroll
            for (int j = 0; j < SQ; ++j) {
                const int idx = j * LPK + sub;
                float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
                if (h < u.nheads && idx < nv) {
                    const int d = idx * 4;
                    if (d + 3 < head_dim && ((reinterpret_cast<uintptr_t>(qrow + d) & 15) == 0)) {
                        val = *reinterpret_cast<const float4*>(qrow + d);
                    } else {
                        if (d + 0 < head_dim) val.x = qrow[d + 0];
                        if (d + 1 < head_dim) val.y = qrow[d + 1];
                        if (d + 2 < head_dim) val.z = qrow[d + 2];
                        if (d + 3 < head_dim) val.w = qrow[d + 3];
                    }
                }
                qreg[h][j] = val;
            }
        }

        float m_run = -INFINITY, l_run = 0.f;
        float4 acc[GT][SV];
#pragma unroll
        for (int h = 0; h < GT; ++h)
#pragma unroll
            for (int s = 0; s < SV; ++s) acc[h][s] = make_float4(0.f, 0.f, 0.f, 0.f);

        for (int tile = item.tile_begin; tile < item.tile_end; ++tile, ++fill) {
            const int s = fill % ST;
            if (!dead) {
                if (!mbar_wait_bounded(&full_bar[s], (fill / ST) & 1)) {
                    atomicExch(status, kDevWaitFull);
                    *abort_flag = 1;
                    dead = true;
                }
            }
            if (!dead && *abort_flag) dead = true;
            if (!dead) {
                const int ntok = min(TPS, u.kv_len - tile * TPS);
                const float4* Ks =
                    reinterpret_cast<const float4*>(stage_base + size_t(s) * Cfg::kStageFloats);
                const float4* Vs = Ks + TPS * NV;

                // ---- scores for this warp's keys ----
                float sc[ITERS];
                float bm = -INFINITY;
#pragma unroll
                for (int i = 0; i < ITERS; ++i) {
                    const int key = i * (W * KPI) + cw * KPI + grp;
                    const float4* krow = Ks + size_t(key) * nv;
                    float part[GT];
#pragma unroll
                    for (int h = 0; h < GT; ++h) part[h] = 0.f;
#pragma unroll
                    for (int j = 0; j < SQ; ++j) {
                        const int idx = j * LPK + sub;
                        if (NV % LPK == 0 && nv == NV ? true : idx < nv) {
                            const float4 kv = krow[idx];
#pragma unroll
                            for (int h = 0; h < GT; ++h) {
                                part[h] = fmaf(qreg[h][j].x, kv.x, part[h]);
                                part[h] = fmaf(qreg[h][j].y, kv.y, part[h]);
                                part[h] = fmaf(qreg[h][j].z, kv.z, part[h]);
                                part[h] = fmaf(qreg[h][j].w, kv.w, part[h]);
                            }
                        }
                    }
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
                    for (int h = 0; h < GT; ++h) al[h] = my_scr[KPW * 4 + h];
#pragma unroll
                    for (int h = 0; h < GT; ++h)
#pragma unroll
                        for (int sv = 0; sv < SV; ++sv) {
                            acc[h][sv].x *= al[h];
                            acc[h][sv].y *= al[h];
                            acc[h][sv].z *= al[h];
                            acc[h][sv].w *= al[h];
                        }
                }

                // ---- weighted V rows of the same keys ----
#pragma unroll
                for (int kk = 0; kk < KPW; ++kk) {
                    const int key = (kk / KPI) * (W * KPI) + cw * KPI + (kk % KPI);
                    if (key < ntok) {
                        float pv[GT];
#pragma unroll
                        for (int h = 0; h < GT; ++h) pv[h] = my_scr[kk * GT + h];
                        const float4* vrow = Vs + size_t(key) * nv;
#pragma unroll
                        for (int sv = 0; sv < SV; ++sv) {
                            const int idx = lane + 32 * sv;
                            if (idx < nv) {
                                const float4 vv = vrow[idx];
#pragma unroll
                                for (int h = 0; h < GT; ++h) {
                                    acc[h][sv].x = fmaf(pv[h], vv.x, acc[h][sv].x);
                                    acc[h][sv].y = fmaf(pv[h], vv.y, acc[h][sv].y);
                                    acc[h][sv].z = fmaf(pv[h], vv.z, acc[h][sv].z);
                                    acc[h][sv].w = fmaf(pv[h], vv.w, acc[h][sv].w);
                                }
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
        }

        // ---- merge the W warp states of this item ----
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
        for (int h = 0; h < GT; ++h) {
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < W; ++w) M = fmaxf(M, sm_m[w * 4 + h]);
            const float mw = sm_m[cw * 4 + h];
            f[h] = (mw == -INFINITY) ? 0.f : expf(mw - M);
        }
#pragma unroll
        for (int h = 0; h < GT; ++h)
#pragma unroll
            for (int sv = 0; sv < SV; ++sv) {
                const int idx = lane + 32 * sv;
                if (idx < nv) {
                    float4 a = acc[h][sv];
                    a.x *= f[h]; a.y *= f[h]; a.z *= f[h]; a.w *= f[h];
                    reinterpret_cast<float4*>(red)[(size_t(cw) * GT + h) * nv + idx] = a;
                }
            }
        named_bar_sync(1, W * 32);
        if (!dead) {
            for (int e = ctid; e < GT * nv; e += W * 32) {
                const int h = e / nv, idx = e % nv;
                if (h >= u.nheads) continue;
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < W; ++w) M = fmaxf(M, sm_m[w * 4 + h]);
                float L = 0.f;
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int w = 0; w < W; ++w) {
                    const float mw = sm_m[w * 4 + h];
                    const float fw = (mw == -INFINITY) ? 0.f : expf(mw - M);
                    L += sm_l[w * 4 + h] * fw;
                    const float4 a = reinterpret_cast<const float4*>(red)[(size_t(w) * GT + h) * nv + idx];
                    sum.x += a.x; sum.y += a.y; sum.z += a.z; sum.w += a.w;
                }
                if (item.part < 0) {
                    float* orow = r.out + size_t(u.head0 + h) * r.o_hs + size_t(u.t_q) * r.o_ts;
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
                    float* rec = partials + (size_t(item.part) * GT + h) * part_stride_floats(nv);
                    if (idx == 0) *reinterpret_cast<float4*>(rec) = make_float4(M, L, 0.f, 0.f);
                    reinterpret_cast<float4*>(rec + 4)[idx] = sum;
                }
            }
        }
    }
}

// Combines the partials of every unit that was cut across thread blocks.  One warp per
// (unit, head): out = sum_i exp(m_i - M) acc_i / sum_i exp(m_i - M) l_i.
template <int GT>
__global__ void attn_merge_kernel(const ReqDev* __restrict__ reqs, const UnitDev* __restrict__ units,
                                  const int* __restrict__ merge_units, int n_merge,
                                  const float* __restrict__ partials, int nv, int head_dim) {
    const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (gw >= n_merge * GT) return;
    const UnitDev u = units[merge_units[gw / GT]];
    const int h = gw % GT;
    if (h >= u.nheads) return;
    const ReqDev& r = reqs[u.req];
    const size_t ps = part_stride_floats(nv);
    float M = -INFINITY;
    for (int i = 0; i < u.part_count; ++i)
        M = fmaxf(M, partials[(size_t(u.part_begin + i) * GT + h) * ps]);
    float L = 0.f;
    for (int i = 0; i < u.part_count; ++i) {
        const float* rec = partials + (size_t(u.part_begin + i) * GT + h) * ps;
        const float mi = rec[0];
        L += (mi == -INFINITY) ? 0.f : rec[1] * expf(mi - M);
    }
    const float inv = 1.0f / L;
    float* orow = r.out + size_t(u.head0 + h) * r.o_hs + size_t(u.t_q) * r.o_ts;
    for (int idx = lane; idx < nv; idx += 32) {
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int i = 0; i < u.part_count; ++i) {
            const float* rec = partials + (size_t(u.part_begin + i) * GT + h) * ps;
            const float mi = rec[0];
            const float w = (mi == -INFINITY) ? 0.f : expf(mi - M);
            const float4 a = reinterpret_cast<const float4*>(rec + 4)[idx];
            sum.x = fmaf(w, a.x, sum.x);
            sum.y = fmaf(w, a.y, sum.y);
            sum.z = fmaf(w, a.z, sum.z);
            sum.w = fmaf(w, a.w, sum.w);
        }
        const int d = idx * 4;
        if (d + 0 < head_dim) orow[d + 0] = sum.x * inv;
        if (d + 1 < head_dim) orow[d + 1] = sum.y * inv;
        if (d + 2 < head_dim) orow[d + 2] = sum.z * inv;
        if (d + 3 < head_dim) orow[d + 3] = sum.w * inv;
    }
}

// Generic attention for requests whose positions fold around the ring (index_pos + seq_len >
// capacity): logical positions 0..=limit are visited in order and mapped with % cap exactly as
// the reference does (fast_attention_simd.rs:608, :145), so a slot that was overwritten is
// counted once per visit.  One block per (request row, query head); plain loads, chunked online
// softmax.  Never on the fast path.
__global__ void __launch_bounds__(256, 1)
attn_ring_kernel(const ReqDev* __restrict__ reqs, const int* __restrict__ ring_rows, int n_rows,
                 const int* __restrict__ page_ids, const float* __restrict__ k_pool,
                 const float* __restrict__ v_pool, long long pool_pages, int num_heads,
                 int num_kv_heads, int head_dim, int nv, float scale) {
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
            const float* krow = k_pool +
                                ((layer_base + size_t(pages[slot / kPageTokens])) * num_kv_heads + h_kv) * page_floats +
                                size_t(slot % kPageTokens) * dp;
            float dot = 0.f;
            for (int d = 0; d < head_dim; ++d) dot = fmaf(s_q[d], krow[d], dot);
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
                const float* vrow = v_pool +
                                    ((layer_base + size_t(pages[slot / kPageTokens])) * num_kv_heads + h_kv) * page_floats +
                                    size_t(slot % kPageTokens) * dp;
                acc = fmaf(s_p[i], vrow[tid], acc);
            }
        }
        __syncthreads();
    }
    if (tid < head_dim) r.out[size_t(h) * r.o_hs + size_t(t_q) * r.o_ts + tid] = acc / l_run;
}

}  // namespace xn
