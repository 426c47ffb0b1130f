// Fused RoPE + KV-append into the paged cache, plus the small cache maintenance kernels.
#pragma once
#include "xn_common.cuh"

namespace xn {

__device__ __forceinline__ size_t slot_offset(const int* pages, long long pool_pages, int layer,
                                              int num_kv_heads, int kv_head, int slot, int dp) {
    const size_t page_floats = size_t(kPageTokens) * dp;
    return ((size_t(layer) * size_t(pool_pages) + size_t(pages[slot / kPageTokens])) * num_kv_heads +
            kv_head) * page_floats +
           size_t(slot % kPageTokens) * dp;
}

// One half-warp per (new token, row), rows = [q heads (only when rotating)] + [k heads] +
// [v heads].
//   * K rows: the append loop of src/nn/fast_attention.rs:104-116 (slot = position % capacity),
//     preceded, when the request asks for it, by the rotation of src/nn/fast_attention_simd.rs:
//     380-387 with table row index_pos + t (src/tensor.rs:302-309).  The rotation is written
//     with explicitly unfused multiplies and add/sub so that the stored bits equal the
//     reference's.
//   * V rows: plain copy.
//   * Q rows: rotated into a dense [Hq, S, D] scratch read by the attention kernels (also used,
//     without rotation, to bring queries that live in mapped host memory next to the kernels).
// When one call carries more new tokens than the ring holds, only the last writer of a slot
// stores (the reference's sequential loop leaves exactly that value).
// Rows move as float4 when head_dim is a multiple of 8 and both pointers are 16-byte aligned,
// element by element otherwise.
__device__ __forceinline__ void rotate4(float4& lo, float4& hi, const float4& c, const float4& s) {
    const float4 a = lo, b = hi;
    lo.x = __fsub_rn(__fmul_rn(a.x, c.x), __fmul_rn(b.x, s.x));
    lo.y = __fsub_rn(__fmul_rn(a.y, c.y), __fmul_rn(b.y, s.y));
    lo.z = __fsub_rn(__fmul_rn(a.z, c.z), __fmul_rn(b.z, s.z));
    lo.w = __fsub_rn(__fmul_rn(a.w, c.w), __fmul_rn(b.w, s.w));
    hi.x = __fadd_rn(__fmul_rn(a.x, s.x), __fmul_rn(b.x, c.x));
    hi.y = __fadd_rn(__fmul_rn(a.y, s.y), __fmul_rn(b.y, c.y));
    hi.z = __fadd_rn(__fmul_rn(a.z, s.z), __fmul_rn(b.z, c.z));
    hi.w = __fadd_rn(__fmul_rn(a.w, s.w), __fmul_rn(b.w, c.w));
}

__device__ __forceinline__ void row_rotate(const float* __restrict__ src, float* __restrict__ dst,
                                           const float* __restrict__ c, const float* __restrict__ s,
                                           int head_dim, int hl, bool vec) {
    const int half = head_dim / 2;
    if (vec) {
        for (int i = hl * 4; i < half; i += 64) {
            float4 lo = *reinterpret_cast<const float4*>(src + i);
            float4 hi = *reinterpret_cast<const float4*>(src + i + half);
            const float4 cv = *reinterpret_cast<const float4*>(c + i);
            const float4 sv = *reinterpret_cast<const float4*>(s + i);
            rotate4(lo, hi, cv, sv);
            *reinterpret_cast<float4*>(dst + i) = lo;
            *reinterpret_cast<float4*>(dst + i + half) = hi;
        }
    } else {
        for (int i = hl; i < half; i += 16) {
            const float x1 = src[i], x2 = src[i + half], cv = c[i], sv = s[i];
            dst[i] = __fsub_rn(__fmul_rn(x1, cv), __fmul_rn(x2, sv));
            dst[i + half] = __fadd_rn(__fmul_rn(x1, sv), __fmul_rn(x2, cv));
        }
        if ((head_dim & 1) && hl == 0) dst[head_dim - 1] = src[head_dim - 1];
    }
}

__device__ __forceinline__ void row_copy(const float* __restrict__ src, float* __restrict__ dst,
                                         int head_dim, int hl, bool vec) {
    if (vec) {
        for (int i = hl * 4; i < head_dim; i += 64)
            *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(src + i);
    } else {
        for (int i = hl; i < head_dim; i += 16) dst[i] = src[i];
    }
}

// F2: instantiation for head dims that are a multiple of 4 but not of 8 (100: the second half of a
// row starts 8 bytes off a 16-byte boundary): rows move as float2, two per lane and half, with the
// four rows of a pass in flight together.  A separate instantiation so that the float4 variant
// keeps its register budget (two blocks per SM).
template <bool F2>
__global__ void __launch_bounds__(256)
rope_append_kernel(const ReqDev* __restrict__ reqs, const int* __restrict__ page_ids,
                   float* __restrict__ k_pool, float* __restrict__ v_pool,
                   const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                   long long pool_pages, int num_heads, int num_kv_heads, int head_dim, int nv) {
    pdl_launch_dependents();   // a prefill kernel launched as a programmatic dependent may set up now
    const ReqDev& r = reqs[blockIdx.y];
    const bool rope = r.flags & 1u;
    // q is rotated, or just moved next to the kernels -- unless the prefill kernel rotates the
    // query rows itself (bit 4)
    const bool q_rows = (r.flags & 3u) && !(r.flags & 16u);
    if (r.flags & 16u) {
        // The prefill kernel behind this one reads the query rows itself.  Ask for them now, so
        // that they travel from DRAM to L2 while this kernel moves K and V (nothing waits here).
        const long long lines_per_row = ((long long)head_dim * 4 + 127) / 128;
        const long long n_lines = (long long)r.seq_len * num_heads * lines_per_row;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_lines;
             i += (long long)gridDim.x * blockDim.x) {
            const long long row = i / lines_per_row, line = i % lines_per_row;
            const long long t = row / num_heads, hh = row % num_heads;
            const float* p = r.q_in + size_t(hh) * r.qi_hs + size_t(t) * r.qi_ts + line * 32;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
        }
    }
    const int rows_per_tok = (q_rows ? num_heads : 0) + 2 * num_kv_heads;
    const long long n_rows = (long long)r.seq_len * rows_per_tok;
    const int hl = threadIdx.x & 15;         // lane inside the half-warp
    const int hw = threadIdx.x >> 4;         // half-warp inside the block (16 per block)
    const int half = head_dim / 2;
    const int dp = nv * 4;
    const int* pages = page_ids + r.page_off;
    const bool dim_vec = (head_dim % 8) == 0;
    // Four rows per half-warp and pass: their page-table reads, then their row loads, are in
    // flight together (one row at a time is a chain of three dependent memory round trips).
    constexpr int U = 4;
    const long long stride = (long long)gridDim.x * 16;
    for (long long row0 = (long long)blockIdx.x * 16 + hw; row0 < n_rows; row0 += stride * U) {
        const float* src[U];
        float* dst[U];
        const float* c[U];
        const float* s[U];
        int kind[U];   // 0 skip, 1 copy, 2 rotate
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long row = row0 + u * stride;
            kind[u] = 0;
            src[u] = nullptr;
            dst[u] = nullptr;
            c[u] = s[u] = nullptr;
            if (row >= n_rows) continue;
            const int t = int(row / rows_per_tok);
            int rr = int(row % rows_per_tok);
            const int pos = r.index_pos + t;
            c[u] = cos_t + size_t(pos) * half;
            s[u] = sin_t + size_t(pos) * half;
            if (q_rows && rr < num_heads) {
                // query row -> scratch (ReqDev::q points at it), rotated when the request asks for it
                src[u] = r.q_in + size_t(rr) * r.qi_hs + size_t(t) * r.qi_ts;
                dst[u] = const_cast<float*>(r.q) + size_t(rr) * r.q_hs + size_t(t) * r.q_ts;
                kind[u] = rope ? 2 : 1;
            } else {
                if (q_rows) rr -= num_heads;
                if ((long long)t + r.cap < (long long)r.seq_len) continue;  // overwritten later in this call
                const int slot = pos % r.cap;
                if (rr < num_kv_heads) {
                    src[u] = r.k + size_t(rr) * r.kv_hs + size_t(t) * r.kv_ts;
                    dst[u] = k_pool + slot_offset(pages, pool_pages, r.layer, num_kv_heads, rr, slot, dp);
                    kind[u] = rope ? 2 : 1;
                } else {
                    rr -= num_kv_heads;
                    src[u] = r.v + size_t(rr) * r.kv_hs + size_t(t) * r.kv_ts;
                    dst[u] = v_pool + slot_offset(pages, pool_pages, r.layer, num_kv_heads, rr, slot, dp);
                    kind[u] = 1;
                }
            }
        }
        bool fast = dim_vec && head_dim <= 128;   // whole rows as one float4 per lane and half
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (kind[u] && ((reinterpret_cast<uintptr_t>(src[u]) | reinterpret_cast<uintptr_t>(dst[u])) & 15)) fast = false;
        bool fast2 = F2 && !dim_vec && (head_dim % 4) == 0 && head_dim <= 128;
        if (F2) {
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (kind[u] && ((reinterpret_cast<uintptr_t>(src[u]) | reinterpret_cast<uintptr_t>(dst[u])) & 7)) fast2 = false;
        }
        if (fast) {
            const int i = hl * 4;
            const bool in = i < half;
            float4 lo[U], hi[U], cv[U], sv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (!kind[u] || !in) continue;
                lo[u] = *reinterpret_cast<const float4*>(src[u] + i);
                hi[u] = *reinterpret_cast<const float4*>(src[u] + i + half);
                if (kind[u] == 2) {
                    cv[u] = *reinterpret_cast<const float4*>(c[u] + i);
                    sv[u] = *reinterpret_cast<const float4*>(s[u] + i);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (!kind[u] || !in) continue;
                if (kind[u] == 2) rotate4(lo[u], hi[u], cv[u], sv[u]);
                *reinterpret_cast<float4*>(dst[u] + i) = lo[u];
                *reinterpret_cast<float4*>(dst[u] + i + half) = hi[u];
            }
        } else if (F2 && fast2) {
#pragma unroll 1
            for (int k = 0; k < 2; ++k) {
                const int i = (hl + 16 * k) * 2;
                if (i >= half) break;
                float2 lo[U], hi[U], cv[U], sv[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (!kind[u]) continue;
                    lo[u] = *reinterpret_cast<const float2*>(src[u] + i);
                    hi[u] = *reinterpret_cast<const float2*>(src[u] + i + half);
                    if (kind[u] == 2) {
                        cv[u] = *reinterpret_cast<const float2*>(c[u] + i);
                        sv[u] = *reinterpret_cast<const float2*>(s[u] + i);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (!kind[u]) continue;
                    float2 a = lo[u], b = hi[u];
                    if (kind[u] == 2) {   // unfused, as everywhere: x1 c - x2 s, x1 s + x2 c
                        a.x = __fsub_rn(__fmul_rn(lo[u].x, cv[u].x), __fmul_rn(hi[u].x, sv[u].x));
                        a.y = __fsub_rn(__fmul_rn(lo[u].y, cv[u].y), __fmul_rn(hi[u].y, sv[u].y));
                        b.x = __fadd_rn(__fmul_rn(lo[u].x, sv[u].x), __fmul_rn(hi[u].x, cv[u].x));
                        b.y = __fadd_rn(__fmul_rn(lo[u].y, sv[u].y), __fmul_rn(hi[u].y, cv[u].y));
                    }
                    *reinterpret_cast<float2*>(dst[u] + i) = a;
                    *reinterpret_cast<float2*>(dst[u] + i + half) = b;
                }
            }
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (!kind[u]) continue;
                const bool vec = dim_vec && (((reinterpret_cast<uintptr_t>(src[u]) |
                                               reinterpret_cast<uintptr_t>(dst[u])) & 15) == 0);
                if (kind[u] == 2) row_rotate(src[u], dst[u], c[u], s[u], head_dim, hl, vec);
                else row_copy(src[u], dst[u], head_dim, hl, vec);
            }
        }
    }
}

// Zeroes slots [slot0, slot0+n) of one layer of one stream: positions that were skipped over
// must read as zeros, as they do in the reference's zero-initialised ring
// (src/nn/fast_attention.rs:40-41).  mode 1 fills with N(0,1) values instead (bench caches).
__global__ void __launch_bounds__(256)
slots_fill_kernel(const int* __restrict__ pages, float* __restrict__ k_pool,
                  float* __restrict__ v_pool, long long pool_pages, int layer, int num_kv_heads,
                  int head_dim, int nv, long long slot0, long long n, int mode,
                  unsigned long long seed) {
    const int dp = nv * 4;
    const long long total = n * num_kv_heads * head_dim;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (long long)gridDim.x * blockDim.x) {
        const int d = int(e % head_dim);
        const long long rest = e / head_dim;
        const int h = int(rest % num_kv_heads);
        const long long i = rest / num_kv_heads;
        const int slot = int(slot0 + i);
        const size_t off = slot_offset(pages, pool_pages, layer, num_kv_heads, h, slot, dp) + d;
        if (mode == 0) {
            k_pool[off] = 0.f;
            v_pool[off] = 0.f;
        } else {
            const unsigned long long idx =
                ((unsigned long long)(slot) * num_kv_heads + h) * head_dim + d;
            k_pool[off] = normal_from(seed, 2ull * idx);
            v_pool[off] = normal_from(seed, 2ull * idx + 1ull);
        }
    }
}

// Gathers slots [slot0, slot0+n) of every KV head into dense [Hkv, n, D] buffers.
__global__ void __launch_bounds__(256)
slots_gather_kernel(const int* __restrict__ pages, const float* __restrict__ k_pool,
                    const float* __restrict__ v_pool, long long pool_pages, int layer,
                    int num_kv_heads, int head_dim, int nv, long long slot0, long long n,
                    float* __restrict__ k_out, float* __restrict__ v_out) {
    const int dp = nv * 4;
    const long long total = n * num_kv_heads * head_dim;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (long long)gridDim.x * blockDim.x) {
        const int d = int(e % head_dim);
        const long long rest = e / head_dim;
        const long long i = rest % n;
        const int h = int(rest / n);
        const size_t off = slot_offset(pages, pool_pages, layer, num_kv_heads, h, int(slot0 + i), dp) + d;
        if (k_out) k_out[e] = k_pool[off];
        if (v_out) v_out[e] = v_pool[off];
    }
}

// Diagnostic: one thread waits on an mbarrier that nothing will ever complete, with a short limit,
// and reports the expiry the way the attention kernels do.  Exercises the host's handling of a
// bounded wait that ran out without disturbing the GPU.
__global__ void wait_probe_kernel(int* __restrict__ status, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
        if (!mbar_wait_bounded(&bar, 0, limit_ns)) report_status(status, kDevWaitFull);
    }
}

__global__ void __launch_bounds__(256)
fill_normal_kernel(float* __restrict__ dst, long long n, unsigned long long seed) {
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n;
         e += (long long)gridDim.x * blockDim.x)
        dst[e] = normal_from(seed, (unsigned long long)e);
}

}  // namespace xn
