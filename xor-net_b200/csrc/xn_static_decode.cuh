// Split-KV decode attention whose scratch lives in a statically allocated device array: the
// kernels of the allocation-free entry point xn_decode_attention_static.
#pragma once
#include "xn_common.cuh"

namespace xn {

constexpr int kStaticMaxRecords = 1024;  // (query head, split) partial records per call
constexpr int kStaticMaxDim = 256;       // head_dim limit
constexpr int kStaticRecFloats = kStaticMaxDim + 4;  // [m, l, 0, 0, acc[head_dim]]
constexpr size_t kStaticScratchFloats = size_t(kStaticMaxRecords) * kStaticRecFloats;

// One block per (split, query head): 4 warps walk the split's tokens one token per warp at a
// time, each warp keeping an online-softmax state; the block's merged state becomes one record
// of the scratch.  K and V are dense [Hkv, capacity, D] (the reference's ring layout,
// src/nn/fast_attention.rs:107-108).
__global__ void __launch_bounds__(128)
static_split_kernel(const float* __restrict__ q, const float* __restrict__ k_cache,
                    const float* __restrict__ v_cache, float* __restrict__ scratch, int num_heads,
                    int num_kv_heads, int head_dim, long long kv_len, long long capacity,
                    int splits, float scale) {
    __shared__ float s_m[4], s_l[4];
    __shared__ float s_acc[4][kStaticMaxDim];
    const int split = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h_kv = h / (num_heads / num_kv_heads);
    const long long chunk = (kv_len + splits - 1) / splits;
    const long long t0 = (long long)split * chunk;
    const long long t1 = t0 + chunk < kv_len ? t0 + chunk : kv_len;
    const float* kb = k_cache + (size_t)h_kv * capacity * head_dim;
    const float* vb = v_cache + (size_t)h_kv * capacity * head_dim;
    const float* qr = q + (size_t)h * head_dim;
    constexpr int kPer = kStaticMaxDim / 32;
    float qv[kPer], acc[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const int d = lane + 32 * j;
        qv[j] = d < head_dim ? qr[d] : 0.f;
        acc[j] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (long long t = t0 + warp; t < t1; t += 4) {
        const float* kr = kb + (size_t)t * head_dim;
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            const int d = lane + 32 * j;
            if (d < head_dim) dot = fmaf(qv[j], kr[d], dot);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float s = dot * scale;
        const float m_new = fmaxf(m, s);
        const float alpha = expf(m - m_new), p = expf(s - m_new);
        l = l * alpha + p;
        const float* vr = vb + (size_t)t * head_dim;
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            const int d = lane + 32 * j;
            if (d < head_dim) acc[j] = fmaf(p, vr[d], acc[j] * alpha);
        }
        m = m_new;
    }
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const int d = lane + 32 * j;
        if (d < head_dim) s_acc[warp][d] = acc[j];
    }
    __syncthreads();
    float M = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
    float f[4], L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        f[w] = (s_m[w] == -INFINITY) ? 0.f : expf(s_m[w] - M);
        L += s_l[w] * f[w];
    }
    float* rec = scratch + (size_t)(h * splits + split) * kStaticRecFloats;
    if (threadIdx.x == 0) { rec[0] = M; rec[1] = L; rec[2] = 0.f; rec[3] = 0.f; }
    for (int d = threadIdx.x; d < head_dim; d += 128)
        rec[4 + d] = s_acc[0][d] * f[0] + s_acc[1][d] * f[1] + s_acc[2][d] * f[2] + s_acc[3][d] * f[3];
}

// One block per query head: log-sum-exp combination of its `splits` records.
__global__ void __launch_bounds__(256)
static_merge_kernel(const float* __restrict__ scratch, float* __restrict__ out, int head_dim,
                    int splits) {
    const int h = blockIdx.x;
    const float* base = scratch + (size_t)h * splits * kStaticRecFloats;
    float M = -INFINITY;
    for (int i = 0; i < splits; ++i) M = fmaxf(M, base[(size_t)i * kStaticRecFloats]);
    float L = 0.f;
    for (int i = 0; i < splits; ++i) {
        const float mi = base[(size_t)i * kStaticRecFloats];
        L += (mi == -INFINITY) ? 0.f : base[(size_t)i * kStaticRecFloats + 1] * expf(mi - M);
    }
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float sum = 0.f;
        for (int i = 0; i < splits; ++i) {
            const float mi = base[(size_t)i * kStaticRecFloats];
            const float w = (mi == -INFINITY) ? 0.f : expf(mi - M);
            sum = fmaf(w, base[(size_t)i * kStaticRecFloats + 4 + d], sum);
        }
        out[(size_t)h * head_dim + d] = sum / L;
    }
}

}  // namespace xn
