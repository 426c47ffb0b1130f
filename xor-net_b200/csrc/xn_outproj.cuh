// The attention output block on the device: heads->sequence layout (done by the attention kernels'
// output strides), the optional sub-norm (RMSNorm), the i8 activation quantiser and the ternary
// output projection (src/models/llama/attention.rs:103-108 of the reference).
//
// Everything after the RMS sum is integer work or single rounded multiplies, so given the same
// attention output the projected rows equal the reference's bit for bit:
//   * rms_norm (src/nn/fast_attention_simd.rs:453-521): squares rounded to f32 and added to ONE
//     accumulator in index order (all three ISA bodies do that), rms = sqrt(sum/n + eps),
//     (x * (1/rms)) * weight;
//   * quantize_f32_to_i8, AVX-512 body (src/bit1_58/quantization.rs:97-143): scale = 127/max|x|,
//     whole 16-element chunks round to nearest EVEN after clamping, the tail rounds half away from
//     zero; inverse scale max|x|/127 (both 1 for an all-zero row);
//   * TernaryLinear::forward (src/bit1_58/layers.rs:262-313): (i32 dot as f32 * inv_scale) * w_scale.
#pragma once
#include "xn_common.cuh"

namespace xn {

// One token row of the block: where the attention output row lives (in_dim floats) and where the
// projected row goes (out_dim floats).
struct OutRowDev {
    const float* src;
    float* dst;
};

// Global layout of the quantised activations: [K / 128][row][128 bytes], and inside a row the
// eight 16-byte chunks permuted by (row & 7).  A tile of rows (starting at a multiple of 8) of one
// 128-column block is then contiguous AND already in the 128-byte-swizzled K-major layout the
// tensor cores read from shared memory.  rows_pad = rows of the buffer (a multiple of 256).
__host__ __device__ __forceinline__ size_t act_offset(long long row, int k, long long rows_pad) {
    return (size_t(k >> 7) * size_t(rows_pad) + size_t(row)) * 128 +
           size_t((((k >> 4) & 7) ^ int(row & 7)) << 4) + size_t(k & 15);
}

// Global layout of the 2-bit weight codes: [row / 32][K / 128][32 rows][32 bytes]: everything one
// thread block of the tensor-core kernel needs (32 output rows, all of K) is one contiguous piece.
// nkb = K / 128.
__host__ __device__ __forceinline__ size_t code_offset(int row, int k, int nkb) {
    return ((size_t(row >> 5) * size_t(nkb) + size_t(k >> 7)) * 32 + size_t(row & 31)) * 32 +
           size_t((k & 127) >> 2);
}

constexpr int kOutRowsTile = 64;    // token rows per GEMM block
constexpr int kOutKChunk = 1280;    // activation bytes per row staged at a time (multiple of 128)
constexpr int kOutMaxRowsPerCta = 32;
constexpr int kOutActStride = kOutKChunk + 16;  // conflict-free 16-byte reads by 8 consecutive lanes
constexpr int kOutGemmSmem = kOutRowsTile * kOutActStride + kOutMaxRowsPerCta * kOutKChunk;

// ---- sub-norm + quantiser: one block per token row ---------------------------------------------
//
// The sum of squares is a 1-thread dependent chain on purpose (see the header: the reference's
// order is the only one that reproduces its bits); the other threads stage the row, then
// normalise, reduce max|x| (order-free) and quantise.  Dynamic shared memory: the row, its
// squares and the norm weights, 3 * round_up(in_dim, 4) floats.
__global__ void __launch_bounds__(256)
subnorm_quant_kernel(const OutRowDev* __restrict__ rows, const float* __restrict__ norm_w, float eps,
                     int in_dim, int8_t* __restrict__ q_out, int q_stride, long long q_row0,
                     long long q_rows_pad, float* __restrict__ inv_scale_out) {
    extern __shared__ float row_s[];
    __shared__ float red_s[8];
    __shared__ float bc_s;
    // the projection kernel behind this one may start now: its prologue (fetching and decoding its
    // weights) does not depend on anything written here, and it waits before it reads the rows
    pdl_launch_dependents();
    pdl_wait();   // this kernel itself may have been set up while the attention kernel still ran
    const int r = blockIdx.x;
    const float* src = rows[r].src;
    const int tid = threadIdx.x;
    const int pad = (in_dim + 3) & ~3;
    float* sq_s = row_s + pad;       // squares of the row
    float* nw_s = sq_s + pad;        // sub-norm weights, fetched while the row is
    const bool vec = (in_dim % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
    if (vec) {
        for (int i = tid * 4; i < in_dim; i += blockDim.x * 4) {
            const float4 x = *reinterpret_cast<const float4*>(src + i);
            *reinterpret_cast<float4*>(row_s + i) = x;
            // squares in parallel (each a single rounded multiply); the adds come later, in order
            *reinterpret_cast<float4*>(sq_s + i) = make_float4(__fmul_rn(x.x, x.x), __fmul_rn(x.y, x.y),
                                                                __fmul_rn(x.z, x.z), __fmul_rn(x.w, x.w));
            if (norm_w != nullptr)
                *reinterpret_cast<float4*>(nw_s + i) = *reinterpret_cast<const float4*>(norm_w + i);
        }
    } else {
        for (int i = tid; i < in_dim; i += blockDim.x) {
            const float x = src[i];
            row_s[i] = x;
            sq_s[i] = __fmul_rn(x, x);
            if (norm_w != nullptr) nw_s[i] = norm_w[i];
        }
    }
    __syncthreads();
    if (norm_w != nullptr) {
        if (tid < 32) {
            // the whole first warp runs the chain (same value in every lane: no divergence);
            // 16 elements per trip, the next 16 loaded before the adds of the current ones, which
            // keeps the chain at the 4-cycle latency of a dependent add
            float sum_sq = 0.f;
            const int n16 = in_dim >> 4;
            const float4* p = reinterpret_cast<const float4*>(sq_s);
            float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0, b2 = b0, b3 = b0;
            if (n16 > 0) { b0 = p[0]; b1 = p[1]; b2 = p[2]; b3 = p[3]; }
            for (int i = 0; i < n16; ++i) {
                const int nx = (i + 1 < n16 ? i + 1 : i) * 4;
                const float4 c0 = p[nx], c1 = p[nx + 1], c2 = p[nx + 2], c3 = p[nx + 3];
                sum_sq = __fadd_rn(sum_sq, b0.x); sum_sq = __fadd_rn(sum_sq, b0.y);
                sum_sq = __fadd_rn(sum_sq, b0.z); sum_sq = __fadd_rn(sum_sq, b0.w);
                sum_sq = __fadd_rn(sum_sq, b1.x); sum_sq = __fadd_rn(sum_sq, b1.y);
                sum_sq = __fadd_rn(sum_sq, b1.z); sum_sq = __fadd_rn(sum_sq, b1.w);
                sum_sq = __fadd_rn(sum_sq, b2.x); sum_sq = __fadd_rn(sum_sq, b2.y);
                sum_sq = __fadd_rn(sum_sq, b2.z); sum_sq = __fadd_rn(sum_sq, b2.w);
                sum_sq = __fadd_rn(sum_sq, b3.x); sum_sq = __fadd_rn(sum_sq, b3.y);
                sum_sq = __fadd_rn(sum_sq, b3.z); sum_sq = __fadd_rn(sum_sq, b3.w);
                b0 = c0; b1 = c1; b2 = c2; b3 = c3;
            }
            for (int i = n16 << 4; i < in_dim; ++i) sum_sq = __fadd_rn(sum_sq, sq_s[i]);
            const float rms = __fsqrt_rn(__fadd_rn(__fdiv_rn(sum_sq, float(in_dim)), eps));
            if (tid == 0) bc_s = __fdiv_rn(1.0f, rms);
        }
        __syncthreads();
    }
    // normalise (two rounded multiplies) and take max |x| in one pass; consecutive threads take
    // consecutive groups of four elements, which keeps shared memory and the global stores dense
    const float inv_rms = norm_w != nullptr ? bc_s : 1.0f;
    const int n4 = in_dim >> 2;
    float m = 0.f;
    for (int g = tid; g < n4; g += blockDim.x) {
        float4 v = *reinterpret_cast<const float4*>(row_s + 4 * g);
        if (norm_w != nullptr) {
            const float4 w = *reinterpret_cast<const float4*>(nw_s + 4 * g);
            v.x = __fmul_rn(__fmul_rn(v.x, inv_rms), w.x);
            v.y = __fmul_rn(__fmul_rn(v.y, inv_rms), w.y);
            v.z = __fmul_rn(__fmul_rn(v.z, inv_rms), w.z);
            v.w = __fmul_rn(__fmul_rn(v.w, inv_rms), w.w);
            *reinterpret_cast<float4*>(row_s + 4 * g) = v;
        }
        m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    for (int i = (n4 << 2) + tid; i < in_dim; i += blockDim.x) {
        float v = row_s[i];
        if (norm_w != nullptr) {
            v = __fmul_rn(__fmul_rn(v, inv_rms), nw_s[i]);
            row_s[i] = v;
        }
        m = fmaxf(m, fabsf(v));
    }
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & 31) == 0) red_s[tid >> 5] = m;
    __syncthreads();
    m = red_s[0];
    for (int w = 1; w < int(blockDim.x >> 5); ++w) m = fmaxf(m, red_s[w]);
    const float scale = m > 0.f ? __fdiv_rn(127.0f, m) : 1.0f;
    if (tid == 0) inv_scale_out[q_row0 + r] = m > 0.f ? __fdiv_rn(m, 127.0f) : 1.0f;
    // whole 16-element chunks round to nearest even after clamping, the tail half away from zero
    const int simd_end = (in_dim / 16) * 16;
    for (int g = tid; g < (q_stride >> 2); g += blockDim.x) {
        const int i0 = g << 2;
        uint32_t packed = 0u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = i0 + j;
            int v = 0;
            if (i < in_dim) {
                const float sc = __fmul_rn(row_s[i], scale);
                if (i < simd_end) v = __float2int_rn(fmaxf(-127.0f, fminf(127.0f, sc)));
                else v = int(fmaxf(-127.0f, fminf(127.0f, roundf(sc))));
            }
            packed |= uint32_t(v & 0xff) << (j * 8);
        }
        *reinterpret_cast<uint32_t*>(q_out + act_offset(q_row0 + r, i0, q_rows_pad)) = packed;
    }
}

// ---- ternary projection: i8 activations x 2-bit weights -> f32 rows ---------------------------
//
// Device weight format: 2 bits per weight, weight i of a row in bits 2(i%4).. of byte i/4 with the
// reference's pack4 codes (0 -> -1, 1 -> 0, 2 -> +1, 3 -> 0; bit1_58/quantization.rs:7-47); rows
// padded with code 1 (and code 3 re-coded as 1) to a multiple of 128 weights.  pack5 weights are re-coded on the host.
//
// Block = 64 token rows x `rows_per_cta` output rows.  The activations of the tile and the decoded
// weights are staged in shared memory one 1280-column chunk at a time; lane l of each warp owns
// tokens l and l+32, warp w the output rows w, w+8, ...; every 16 columns cost two 16-byte
// activation reads plus, per output row, one broadcast 16-byte weight read and eight dp4a.

__device__ __forceinline__ uint32_t decode4(uint32_t byte_codes) {
    // four 2-bit codes (one byte) -> four i8 in one word
    const uint32_t x = (byte_codes | (byte_codes << 6) | (byte_codes << 12) | (byte_codes << 18)) & 0x03030303u;
    const uint32_t nz = (x & 0x01010101u) ^ 0x01010101u;      // 1 where the code is even (weight != 0)
    const uint32_t pos = (x >> 1) & nz;                       // 1 where the weight is +1
    const uint32_t neg = nz ^ pos;                            // 1 where the weight is -1
    return pos | ((neg << 8) - neg);                          // -1 = 0xff per byte
}

__global__ void __launch_bounds__(256)
ternary_gemm_kernel(const int8_t* __restrict__ q, int q_stride, long long q_row0, long long q_rows_pad,
                    const float* __restrict__ inv_scale, const uint8_t* __restrict__ w2,
                    const float* __restrict__ w_scales, const OutRowDev* __restrict__ rows, int n_rows,
                    int out_dim, int rows_per_cta) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    int8_t* act_s = reinterpret_cast<int8_t*>(smem_raw);
    int8_t* w_s = act_s + kOutRowsTile * kOutActStride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int o0 = blockIdx.x * rows_per_cta;
    const int R = min(rows_per_cta, out_dim - o0);
    const int t0 = blockIdx.y * kOutRowsTile;
    int acc[2][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[a][j] = 0;

    for (int k0 = 0; k0 < q_stride; k0 += kOutKChunk) {
        const int kc = min(kOutKChunk, q_stride - k0);  // multiple of 16
        const int kv = kc / 16;
        for (int e = tid; e < kOutRowsTile * kv; e += blockDim.x) {
            const int t = e / kv, c = e % kv;
            int4 v = make_int4(0, 0, 0, 0);
            if (t0 + t < n_rows)
                v = *reinterpret_cast<const int4*>(q + act_offset(q_row0 + t0 + t, k0 + c * 16, q_rows_pad));
            *reinterpret_cast<int4*>(act_s + t * kOutActStride + c * 16) = v;
        }
        for (int e = tid; e < R * kv; e += blockDim.x) {
            const int rr = e / kv, c = e % kv;
            const uint32_t codes = *reinterpret_cast<const uint32_t*>(
                w2 + code_offset(o0 + rr, k0 + c * 16, q_stride >> 7));
            int4 v;
            v.x = int(decode4(codes & 0xffu));
            v.y = int(decode4((codes >> 8) & 0xffu));
            v.z = int(decode4((codes >> 16) & 0xffu));
            v.w = int(decode4(codes >> 24));
            *reinterpret_cast<int4*>(w_s + rr * kOutKChunk + c * 16) = v;
        }
        __syncthreads();
        const int8_t* a0p = act_s + lane * kOutActStride;
        const int8_t* a1p = act_s + (lane + 32) * kOutActStride;
        for (int c = 0; c < kv; ++c) {
            const int4 a0 = *reinterpret_cast<const int4*>(a0p + c * 16);
            const int4 a1 = *reinterpret_cast<const int4*>(a1p + c * 16);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int rr = warp + 8 * j;
                if (rr < R) {
                    const int4 w = *reinterpret_cast<const int4*>(w_s + rr * kOutKChunk + c * 16);
                    acc[0][j] = __dp4a(a0.x, w.x, acc[0][j]);
                    acc[0][j] = __dp4a(a0.y, w.y, acc[0][j]);
                    acc[0][j] = __dp4a(a0.z, w.z, acc[0][j]);
                    acc[0][j] = __dp4a(a0.w, w.w, acc[0][j]);
                    acc[1][j] = __dp4a(a1.x, w.x, acc[1][j]);
                    acc[1][j] = __dp4a(a1.y, w.y, acc[1][j]);
                    acc[1][j] = __dp4a(a1.z, w.z, acc[1][j]);
                    acc[1][j] = __dp4a(a1.w, w.w, acc[1][j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 2; ++a) {
        const int t = t0 + lane + 32 * a;
        if (t >= n_rows) continue;
        const float is = inv_scale[q_row0 + t];
        float* dst = rows[t].dst;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int rr = warp + 8 * j;
            if (rr < R) dst[o0 + rr] = __fmul_rn(__fmul_rn(float(acc[a][j]), is), w_scales[o0 + rr]);
        }
    }
}

}  // namespace xn
