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

// One warp per (new token, row), rows = [q heads (only when rotating)] + [k heads] + [v heads].
//   * K rows: the append loop of src/nn/fast_attention.rs:104-116 (slot = position % capacity),
//     preceded, when the request asks for it, by the rotation of src/nn/fast_attention_simd.rs:
//     380-387 with table row index_pos + t (src/tensor.rs:302-309).  The rotation is written
//     with explicitly unfused multiplies and add/sub so that the stored bits equal the
//     reference's.
//   * V rows: plain copy.
//   * Q rows: rotated into a dense [Hq, S, D] scratch read by the attention kernels.
// When one call carries more new tokens than the ring holds, only the last writer of a slot
// stores (the reference's sequential loop leaves exactly that value).
__global__ void __launch_bounds__(256)
rope_append_kernel(const ReqDev* __restrict__ reqs, const int* __restrict__ page_ids,
                   float* __restrict__ k_pool, float* __restrict__ v_pool,
                   const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                   long long pool_pages, int num_heads, int num_kv_heads, int head_dim, int nv) {
    const ReqDev& r = reqs[blockIdx.y];
    const bool rope = r.flags & 1u;
    const int rows_per_tok = (rope ? num_heads : 0) + 2 * num_kv_heads;
    const long long n_rows = (long long)r.seq_len * rows_per_tok;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half = head_dim / 2;
    const int dp = nv * 4;
    const int* pages = page_ids + r.page_off;
    for (long long row = (long long)blockIdx.x * 8 + warp; row < n_rows;
         row += (long long)gridDim.x * 8) {
        const int t = int(row / rows_per_tok);
        int rr = int(row % rows_per_tok);
        const int pos = r.index_pos + t;
        const float* c = cos_t + size_t(pos) * half;
        const float* s = sin_t + size_t(pos) * half;
        if (rope && rr < num_heads) {
            // query row -> rotation scratch (ReqDev::q points at it)
            const float* src = r.q_in + size_t(rr) * r.qi_hs + size_t(t) * r.qi_ts;
            float* dst = const_cast<float*>(r.q) + size_t(rr) * r.q_hs + size_t(t) * r.q_ts;
            for (int i = lane; i < half; i += 32) {
                const float x1 = src[i], x2 = src[i + half], cv = c[i], sv = s[i];
                dst[i] = __fsub_rn(__fmul_rn(x1, cv), __fmul_rn(x2, sv));
                dst[i + half] = __fadd_rn(__fmul_rn(x1, sv), __fmul_rn(x2, cv));
            }
            if ((head_dim & 1) && lane == 0) dst[head_dim - 1] = src[head_dim - 1];
            continue;
        }
        if (rope) rr -= num_heads;
        if ((long long)t + r.cap < (long long)r.seq_len) continue;  // overwritten later in this call
        const int slot = pos % r.cap;
        if (rr < num_kv_heads) {
            const float* src = r.k + size_t(rr) * r.kv_hs + size_t(t) * r.kv_ts;
            float* dst = k_pool + slot_offset(pages, pool_pages, r.layer, num_kv_heads, rr, slot, dp);
            if (rope) {
                for (int i = lane; i < half; i += 32) {
                    const float x1 = src[i], x2 = src[i + half], cv = c[i], sv = s[i];
                    dst[i] = __fsub_rn(__fmul_rn(x1, cv), __fmul_rn(x2, sv));
                    dst[i + half] = __fadd_rn(__fmul_rn(x1, sv), __fmul_rn(x2, cv));
                }
                if ((head_dim & 1) && lane == 0) dst[head_dim - 1] = src[head_dim - 1];
            } else {
                for (int i = lane; i < head_dim; i += 32) dst[i] = src[i];
            }
        } else {
            rr -= num_kv_heads;
            const float* src = r.v + size_t(rr) * r.kv_hs + size_t(t) * r.kv_ts;
            float* dst = v_pool + slot_offset(pages, pool_pages, r.layer, num_kv_heads, rr, slot, dp);
            for (int i = lane; i < head_dim; i += 32) dst[i] = src[i];
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

__global__ void __launch_bounds__(256)
fill_normal_kernel(float* __restrict__ dst, long long n, unsigned long long seed) {
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n;
         e += (long long)gridDim.x * blockDim.x)
        dst[e] = normal_from(seed, (unsigned long long)e);
}

}  // namespace xn
