// Causal prefill attention in exact f32 on the CUDA cores, tiled: the per-row loop of the
// reference (src/nn/fast_attention.rs:157-198 -- scores by batched_dot_product, softmax_inplace,
// weighted_sum) for many query rows at once, for the cases the tensor-core kernel does not take
// (head dims that are not a multiple of 4 or above 128, short chunks, contexts created with
// XN_PREFILL_F32).
//
// One thread block = one (request, query head, 64-row query tile).  It walks the cache pages the
// tile may see, one tile of TK keys at a time (a whole 64-token page, or half a page for rows
// longer than 128 floats): K and V tiles are contiguous inside a page and arrive by 1-D bulk
// async copies (TMA engine, mbarrier byte counts, two stages, no tensor map, no multicast).
// 256 threads form a 16 x 16 grid; thread (ty, tx) owns query rows 4ty..4ty+3 and
//   * of the score tile S = Q K^T the keys tx*KPT .. tx*KPT+KPT-1 (KPT = TK / 16), with the walk over
//     the row dimension rotated by tx so that the sixteen threads of a row group read different
//     shared-memory banks of the K tile;
//   * of the output tile the columns 4tx + 64j .. +3.
// The softmax is the online form (running maximum and sum per row, shared by the sixteen threads
// of a row through shuffles), with expf and an f32 accumulator: the result differs from the
// reference's full-row softmax by rounding only.  Keys above the causal limit
// `index_pos + t` (:162) are masked in the tiles that straddle it; tiles wholly above are skipped.
// Every mbarrier wait is bounded; on expiry the block records a status code and returns.
#pragma once
#include "xn_common.cuh"

namespace xn {

// One (request, query head, 64-row query tile).
struct F32Item {
    int req;
    int head;
    int qt;
    int pad;
};

namespace pf32 {

constexpr int kTQ = 64;        // query rows per block
constexpr int kThreads = 256;  // 16 x 16

// bytes of dynamic shared memory for rows of `dp` floats and key tiles of `tk` keys
__host__ __device__ constexpr size_t smem_bytes(int dp, int tk) {
    return size_t(kTQ) * dp * 4          // Q tile
           + size_t(kTQ) * (tk + 4) * 4  // P tile (padded rows)
           + size_t(2) * 2 * tk * dp * 4 // two stages of K and V
           + 64;                         // barriers
}

}  // namespace pf32

template <int TK, int NJ>  // keys per tile (64 or 32); float4 output columns per thread (1, 2 or 4)
__global__ void __launch_bounds__(pf32::kThreads, 1)
prefill_f32_kernel(const ReqDev* __restrict__ reqs, const F32Item* __restrict__ items,
                   const int* __restrict__ page_ids, const float* __restrict__ k_pool,
                   const float* __restrict__ v_pool, long long pool_pages, int num_kv_heads, int group,
                   int head_dim, int nv, float scale, int* __restrict__ status) {
    using namespace pf32;
    constexpr int KPT = TK / 16;           // keys per thread in the score tile
    constexpr int kTilesPerPage = kPageTokens / TK;
    extern __shared__ __align__(128) unsigned char smem_f32[];
    const int dp = nv * 4;                 // floats per cached row
    const int nd4 = nv;                    // float4 per row
    float* q_s = reinterpret_cast<float*>(smem_f32);                 // [kTQ][dp]
    float* p_s = q_s + size_t(kTQ) * dp;                             // [kTQ][TK + 4]
    float* kv_s = p_s + size_t(kTQ) * (TK + 4);                      // [2 stages][K | V][TK][dp]
    uint64_t* full = reinterpret_cast<uint64_t*>(kv_s + size_t(4) * TK * dp);
    __shared__ int abort_s;

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const F32Item it = items[blockIdx.x];
    const ReqDev& r = reqs[it.req];
    const int h = it.head, h_kv = h / group;
    const int t0 = it.qt * kTQ;
    const int n_rows = min(kTQ, r.seq_len - t0);
    const int last_pos = r.index_pos + t0 + n_rows - 1;               // highest position a row of the tile sees
    const int n_tiles = last_pos / TK + 1;
    const int* pages = page_ids + r.page_off;
    const size_t page_floats = size_t(kPageTokens) * dp;

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        abort_s = 0;
        mbar_fence_init();
    }
    __syncthreads();
    auto issue = [&](int j) {   // K and V tile j -> stage j & 1 (thread 0)
        const int page = pages[j / kTilesPerPage];
        if (!XN_PAGE_OK(page, pool_pages)) {   // bounds-checking build: report, skip the copy, give up
            report_status(status, kDevBadIndex);
            abort_s = 1;
            mbar_arrive(&full[j & 1]);         // nothing will fill the stage: let the waiters through
            return;
        }
        const size_t off = ((size_t(r.layer) * size_t(pool_pages) + size_t(page)) * num_kv_heads + h_kv) * page_floats +
                           size_t(j % kTilesPerPage) * TK * dp;
        float* dst = kv_s + size_t(j & 1) * 2 * TK * dp;
        const uint32_t bytes = uint32_t(TK) * dp * 4;
        mbar_arrive_expect_tx(&full[j & 1], 2 * bytes);
        bulk_g2s(dst, k_pool + off, bytes, &full[j & 1]);
        bulk_g2s(dst + size_t(TK) * dp, v_pool + off, bytes, &full[j & 1]);
    };
    if (tid == 0) {
        issue(0);
        if (n_tiles > 1) issue(1);
    }
    // Q tile -> shared memory (rows past the request and columns past head_dim are zeros)
    for (int e = tid; e < kTQ * dp; e += kThreads) {
        const int row = e / dp, d = e - row * dp;
        float v = 0.f;
        if (row < n_rows && d < head_dim) v = r.q[size_t(h) * r.q_hs + size_t(t0 + row) * r.q_ts + d];
        q_s[e] = v;
    }
    __syncthreads();

    float m_run[4], l_run[4];
    float4 acc[4][NJ];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m_run[i] = -INFINITY;
        l_run[i] = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) acc[i][j] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int row0 = ty * 4;                  // this thread's query rows inside the tile
    const int pos0 = r.index_pos + t0 + row0; // position of its first row

    for (int j = 0; j < n_tiles; ++j) {
        if (!mbar_wait_bounded(&full[j & 1], uint32_t((j >> 1) & 1))) {
            abort_s = 1;
            report_status(status, kDevWaitFull);
        }
        __syncthreads();
        if (abort_s) break;
        const float* k_t = kv_s + size_t(j & 1) * 2 * TK * dp;
        const float* v_t = k_t + size_t(TK) * dp;
        // ---- scores of 4 rows x KPT keys
        float s[4][KPT];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int kk = 0; kk < KPT; ++kk) s[i][kk] = 0.f;
        int d4 = tx % nd4;                    // rotated walk: the 16 threads of a row group read different banks
        for (int step = 0; step < nd4; ++step, d4 = d4 + 1 == nd4 ? 0 : d4 + 1) {
            float4 qv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) qv[i] = *reinterpret_cast<const float4*>(q_s + size_t(row0 + i) * dp + d4 * 4);
#pragma unroll
            for (int kk = 0; kk < KPT; ++kk) {
                const float4 kv = *reinterpret_cast<const float4*>(k_t + size_t(tx * KPT + kk) * dp + d4 * 4);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    s[i][kk] = fmaf(qv[i].x, kv.x, s[i][kk]);
                    s[i][kk] = fmaf(qv[i].y, kv.y, s[i][kk]);
                    s[i][kk] = fmaf(qv[i].z, kv.z, s[i][kk]);
                    s[i][kk] = fmaf(qv[i].w, kv.w, s[i][kk]);
                }
            }
        }
        // ---- scale, causal mask, online softmax (row state shared by the 16 threads of a row group)
        const int key0 = j * TK + tx * KPT;
        const bool straddles = j * TK + TK - 1 > r.index_pos + t0;   // some row of the tile masks some key
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float mx = -INFINITY;
#pragma unroll
            for (int kk = 0; kk < KPT; ++kk) {
                float x = s[i][kk] * scale;
                if (straddles && key0 + kk > pos0 + i) x = -INFINITY;
                s[i][kk] = x;
                mx = fmaxf(mx, x);
            }
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float m_new = fmaxf(m_run[i], mx);
            const float m_safe = m_new == -INFINITY ? 0.f : m_new;   // a row beyond the request sees nothing
            const float alpha = expf(m_run[i] - m_safe);             // exp(-inf) = 0 on the first tile
            float sum = 0.f;
#pragma unroll
            for (int kk = 0; kk < KPT; ++kk) {
                const float p = expf(s[i][kk] - m_safe);
                s[i][kk] = p;
                sum += p;
            }
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            l_run[i] = l_run[i] * alpha + sum;
            m_run[i] = m_new;
#pragma unroll
            for (int jj = 0; jj < NJ; ++jj) {
                acc[i][jj].x *= alpha;
                acc[i][jj].y *= alpha;
                acc[i][jj].z *= alpha;
                acc[i][jj].w *= alpha;
            }
#pragma unroll
            for (int kk = 0; kk < KPT; ++kk) p_s[size_t(row0 + i) * (TK + 4) + tx * KPT + kk] = s[i][kk];
        }
        __syncthreads();
        // ---- O += P V: 4 rows x (4 NJ) columns per thread
        for (int k4 = 0; k4 < TK; k4 += 4) {
            float4 pv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) pv[i] = *reinterpret_cast<const float4*>(p_s + size_t(row0 + i) * (TK + 4) + k4);
#pragma unroll
            for (int jj = 0; jj < NJ; ++jj) {
                const int col = tx * 4 + 64 * jj;
                if (col >= dp) break;
                const float4 v0 = *reinterpret_cast<const float4*>(v_t + size_t(k4) * dp + col);
                const float4 v1 = *reinterpret_cast<const float4*>(v_t + size_t(k4 + 1) * dp + col);
                const float4 v2 = *reinterpret_cast<const float4*>(v_t + size_t(k4 + 2) * dp + col);
                const float4 v3 = *reinterpret_cast<const float4*>(v_t + size_t(k4 + 3) * dp + col);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float4& a = acc[i][jj];
                    a.x = fmaf(pv[i].x, v0.x, a.x); a.y = fmaf(pv[i].x, v0.y, a.y); a.z = fmaf(pv[i].x, v0.z, a.z); a.w = fmaf(pv[i].x, v0.w, a.w);
                    a.x = fmaf(pv[i].y, v1.x, a.x); a.y = fmaf(pv[i].y, v1.y, a.y); a.z = fmaf(pv[i].y, v1.z, a.z); a.w = fmaf(pv[i].y, v1.w, a.w);
                    a.x = fmaf(pv[i].z, v2.x, a.x); a.y = fmaf(pv[i].z, v2.y, a.y); a.z = fmaf(pv[i].z, v2.z, a.z); a.w = fmaf(pv[i].z, v2.w, a.w);
                    a.x = fmaf(pv[i].w, v3.x, a.x); a.y = fmaf(pv[i].w, v3.y, a.y); a.z = fmaf(pv[i].w, v3.z, a.z); a.w = fmaf(pv[i].w, v3.w, a.w);
                }
            }
        }
        __syncthreads();   // every thread is done with this stage and with the P tile
        if (tid == 0 && j + 2 < n_tiles) issue(j + 2);
    }
    if (abort_s) return;   // the cause is in the status word already
    // ---- O / l -> out
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row0 + i;
        if (row >= n_rows) continue;
        const float inv = 1.0f / l_run[i];
        float* orow = r.out + size_t(h) * r.o_hs + size_t(t0 + row) * r.o_ts;
#pragma unroll
        for (int jj = 0; jj < NJ; ++jj) {
            const int col = tx * 4 + 64 * jj;
            const float vals[4] = {acc[i][jj].x * inv, acc[i][jj].y * inv, acc[i][jj].z * inv, acc[i][jj].w * inv};
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (col + c < head_dim) orow[col + c] = vals[c];
        }
    }
}

}  // namespace xn
