/*
 * xn_oracle_outproj.c -- CPU restatement of what xor-net runs on the attention output:
 * heads->sequence layout, the optional sub-norm (RMSNorm) and the ternary output projection
 * (src/models/llama/attention.rs:103-108).
 *
 * TEST INFRASTRUCTURE ONLY, like xn_oracle.c: the checker of the CUDA library and the timed CPU
 * baseline.  Nothing in the shipped library calls it.
 *
 * Parity status: PINNED against the reference's own known-answer tests for these routines
 * (tests/bit1_58_tests.rs, tests/quantization_158bit_tests.rs, tests/tensor_rmsnorm_tests.rs,
 * tests/tensor_ops_tests.rs:70-110 and :318-341), whose vectors are formulas or literals
 * reproduced in this repository's oracle tests.  The reference is Rust and cannot be compiled
 * where this was written, so no output of the reference binary itself backs it.
 *
 * All integer work (packing, i8 quantisation, ternary dot products) is exact; the float steps
 * keep the reference's order of operations (build with -ffp-contract=off).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define XO_API __attribute__((visibility("default")))

/* 1 when the reference's has_avx512f() dispatch (src/bit1_58/quantization.rs:148-165) would pick
 * the AVX-512 quantiser under the ISA level selected in xn_oracle.c. */
int xo_quant_uses_avx512(void);

enum { XO_PACK4 = 4, XO_PACK5 = 5 };

/* ------------------------------------------------------------------------- */
/* rms_norm  (src/nn/fast_attention_simd.rs:411-521)                          */
/* ------------------------------------------------------------------------- */

/* The AVX-512 (:453-498), AVX2 (:411-450) and scalar (:502-521) bodies do the same arithmetic:
 * squares rounded to f32, added to one scalar accumulator in index order (the SIMD bodies store
 * the squared lanes and add them one by one), rms = sqrt(sum/n + eps), inv = 1/rms, then
 * (x * inv) * weight.  One body therefore restates all three. */
XO_API void xo_rms_norm(float* x, const float* weight, float eps, size_t n) {
    float sum_sq = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        const float sq = x[i] * x[i];
        sum_sq += sq;
    }
    const float rms = sqrtf(sum_sq / (float)n + eps);
    const float inv_rms = 1.0f / rms;
    for (size_t i = 0; i < n; ++i) {
        const float normalized = x[i] * inv_rms;
        x[i] = normalized * weight[i];
    }
}

/* FastTensor::rmsnorm, src/tensor.rs:242-265: every row of `hidden` elements independently. */
XO_API void xo_tensor_rmsnorm(const float* in, float* out, const float* weight, float eps,
                              size_t rows, size_t hidden) {
    for (size_t r = 0; r < rows; ++r) {
        memcpy(out + r * hidden, in + r * hidden, hidden * sizeof(float));
        xo_rms_norm(out + r * hidden, weight, eps, hidden);
    }
}

/* ------------------------------------------------------------------------- */
/* quantize_f32_to_i8  (src/bit1_58/quantization.rs:95-187)                    */
/* ------------------------------------------------------------------------- */

/* AVX-512 body (:97-143): absolute maximum; scale = 127/max, inv_scale = max/127 (both 1.0 for
 * an all-zero row); whole 16-element chunks are scaled, clamped to [-127,127] and converted with
 * _mm512_cvtps_epi32, i.e. round-to-nearest-EVEN (lrintf under the default rounding mode is the
 * same conversion); the <16 tail uses f32::round, i.e. half AWAY from zero, then clamps.
 * Scalar body (:167-187): f32::round then clamp for every element. */
XO_API float xo_quantize_f32_to_i8(const float* a, size_t n, int8_t* q) {
    float max_abs = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        const float v = fabsf(a[i]);
        if (v > max_abs) max_abs = v;
    }
    const float scale = max_abs > 0.0f ? 127.0f / max_abs : 1.0f;
    const float inv_scale = max_abs > 0.0f ? max_abs / 127.0f : 1.0f;
    const size_t simd_end = xo_quant_uses_avx512() ? (n / 16) * 16 : 0;
    for (size_t i = 0; i < simd_end; ++i) {
        float s = a[i] * scale;
        s = s < 127.0f ? s : 127.0f;   /* _mm512_min_ps(v_max, scaled) */
        s = s > -127.0f ? s : -127.0f; /* _mm512_max_ps(v_min, ...)    */
        q[i] = (int8_t)lrintf(s);
    }
    for (size_t i = simd_end; i < n; ++i) {
        float r = roundf(a[i] * scale);
        if (r > 127.0f) r = 127.0f;
        else if (r < -127.0f) r = -127.0f;
        q[i] = (int8_t)r;
    }
    return inv_scale;
}

/* ------------------------------------------------------------------------- */
/* ternary packing  (src/bit1_58/quantization.rs:7-93)                         */
/* ------------------------------------------------------------------------- */

/* code of one weight: 0 -> -1, 1 -> 0, 2 -> +1 (:12-20, :54-62) */
static unsigned ternary_code(float w, float w_scale) {
    const float scaled = w_scale > 0.0f ? w / w_scale : 0.0f;
    float qv = roundf(scaled);
    if (qv < -1.0f) qv = -1.0f;
    if (qv > 1.0f) qv = 1.0f;
    return qv < -0.5f ? 0u : (qv > 0.5f ? 2u : 1u);
}

XO_API size_t xo_packed_row_bytes(size_t n, int pack_type) {
    return pack_type == XO_PACK5 ? (n + 4) / 5 : (n + 3) / 4;
}

/* pack_1_58bit_4pack (:7-27): four 2-bit codes per byte, weight i in bits 2i..2i+1. */
XO_API void xo_pack4(const float* w, size_t n, float w_scale, uint8_t* out) {
    for (size_t b = 0; b < (n + 3) / 4; ++b) {
        unsigned byte = 0;
        for (size_t i = 0; i < 4 && b * 4 + i < n; ++i)
            byte |= ternary_code(w[b * 4 + i], w_scale) << (i * 2);
        out[b] = (uint8_t)byte;
    }
}

/* unpack_1_58bit_4pack (:29-47): 00 -> -1, 10 -> +1, anything else -> 0. */
XO_API void xo_unpack4(const uint8_t* packed, size_t n, float* out) {
    for (size_t i = 0; i < n; ++i) {
        const unsigned v = (packed[i / 4] >> ((i % 4) * 2)) & 3u;
        out[i] = v == 0u ? -1.0f : (v == 2u ? 1.0f : 0.0f);
    }
}

/* pack_1_58bit_5pack (:49-72): five base-3 digits per byte, weight i the digit of 3^i. */
XO_API void xo_pack5(const float* w, size_t n, float w_scale, uint8_t* out) {
    for (size_t b = 0; b < (n + 4) / 5; ++b) {
        unsigned byte = 0, mult = 1;
        for (size_t i = 0; i < 5 && b * 5 + i < n; ++i) {
            byte += ternary_code(w[b * 5 + i], w_scale) * mult;
            mult *= 3;
        }
        out[b] = (uint8_t)byte;
    }
}

/* unpack_1_58bit_5pack (:74-93) */
XO_API void xo_unpack5(const uint8_t* packed, size_t n, float* out) {
    for (size_t i = 0; i < n; ++i) {
        unsigned cur = packed[i / 5];
        for (size_t j = 0; j < i % 5; ++j) cur /= 3;
        const unsigned v = cur % 3;
        out[i] = v == 0u ? -1.0f : (v == 2u ? 1.0f : 0.0f);
    }
}

/* ------------------------------------------------------------------------- */
/* ternary dot products  (src/bit1_58/simd.rs)                                 */
/* ------------------------------------------------------------------------- */

/* ternary_dot_product_pack4, scalar definition (:372-381).  The AVX2 / AVX-512 / VNNI bodies
 * (:29-356) compute the same i32 sum; integer addition makes the order irrelevant. */
XO_API int32_t xo_ternary_dot_pack4(const int8_t* a, const uint8_t* w, size_t n) {
    int32_t total = 0;
    for (size_t i = 0; i < n; ++i) {
        const unsigned v = (w[i / 4] >> ((i % 4) * 2)) & 3u;
        const int32_t wv = v == 0u ? -1 : (v == 2u ? 1 : 0);
        total += (int32_t)a[i] * wv;
    }
    return total;
}

/* ternary_dot_product_pack5_scalar (:388-418) */
XO_API int32_t xo_ternary_dot_pack5(const int8_t* a, const uint8_t* w, size_t n) {
    int32_t total = 0;
    for (size_t b = 0; b * 5 < n; ++b) {
        unsigned cur = w[b];
        for (size_t j = 0; j < 5 && b * 5 + j < n; ++j) {
            const unsigned v = cur % 3;
            cur /= 3;
            const int32_t wv = v == 0u ? -1 : (v == 2u ? 1 : 0);
            total += (int32_t)a[b * 5 + j] * wv;
        }
    }
    return total;
}

/* ------------------------------------------------------------------------- */
/* TernaryLinear  (src/bit1_58/layers.rs)                                      */
/* ------------------------------------------------------------------------- */

/* TernaryLinear::new, dense representation (:91-149).  `provided_scale` NaN stands for None.
 * Weights that are already exactly ternary keep scale `provided_scale` (1.0 when None); others
 * use the provided global scale, or, without one, the per-row mean absolute value (summed in
 * index order). */
XO_API void xo_ternary_linear_pack(size_t in_dim, size_t out_dim, const float* weights,
                                   int pack_type, float provided_scale, uint8_t* packed,
                                   float* w_scales) {
    int already = 1;
    for (size_t i = 0; i < in_dim * out_dim; ++i)
        if (!(weights[i] == -1.0f || weights[i] == 0.0f || weights[i] == 1.0f)) { already = 0; break; }
    const int has_scale = !isnan(provided_scale);
    const size_t bpr = xo_packed_row_bytes(in_dim, pack_type);
    for (size_t o = 0; o < out_dim; ++o) {
        const float* row = weights + o * in_dim;
        float s;
        if (already) s = has_scale ? provided_scale : 1.0f;
        else if (has_scale) s = provided_scale;
        else {
            float sum_abs = 0.0f;
            for (size_t i = 0; i < in_dim; ++i) sum_abs += fabsf(row[i]);
            s = in_dim == 0 ? 1.0f : sum_abs / (float)in_dim;
        }
        w_scales[o] = s;
        if (pack_type == XO_PACK5) xo_pack5(row, in_dim, s, packed + o * bpr);
        else xo_pack4(row, in_dim, s, packed + o * bpr);
    }
}

/* TernaryLinear::forward (:262-313): each input row is quantised to i8 on its own, then
 * out[b][o] = (dot_i32 as f32 * inv_scale) * w_scales[o]. */
XO_API void xo_ternary_linear_forward(const float* x, size_t rows, size_t in_dim, size_t out_dim,
                                      int pack_type, const uint8_t* packed, const float* w_scales,
                                      float* out, int threads) {
    const size_t bpr = xo_packed_row_bytes(in_dim, pack_type);
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#else
    (void)threads;
#endif
    /* The weights are decoded to i8 once per call (the reference decodes them inside its SIMD dot
     * product); the i32 sums are the same. */
    int8_t* w8 = (int8_t*)malloc(out_dim * in_dim + 1);
#pragma omp parallel for schedule(static) num_threads(threads)
    for (long long o = 0; o < (long long)out_dim; ++o) {
        const uint8_t* pw = packed + (size_t)o * bpr;
        int8_t* dst = w8 + (size_t)o * in_dim;
        if (pack_type == XO_PACK5) {
            for (size_t b = 0; b * 5 < in_dim; ++b) {
                unsigned cur = pw[b];
                for (size_t j = 0; j < 5 && b * 5 + j < in_dim; ++j) {
                    const unsigned v = cur % 3;
                    cur /= 3;
                    dst[b * 5 + j] = v == 0u ? -1 : (v == 2u ? 1 : 0);
                }
            }
        } else {
            for (size_t i = 0; i < in_dim; ++i) {
                const unsigned v = (pw[i / 4] >> ((i % 4) * 2)) & 3u;
                dst[i] = v == 0u ? -1 : (v == 2u ? 1 : 0);
            }
        }
    }
#pragma omp parallel num_threads(threads)
    {
        int8_t* q = (int8_t*)malloc(in_dim ? in_dim : 1);
#pragma omp for schedule(static)
        for (long long b = 0; b < (long long)rows; ++b) {
            const float inv_scale = xo_quantize_f32_to_i8(x + (size_t)b * in_dim, in_dim, q);
            for (size_t o = 0; o < out_dim; ++o) {
                const int8_t* wr = w8 + o * in_dim;
                int32_t dot = 0;
                for (size_t i = 0; i < in_dim; ++i) dot += (int32_t)q[i] * (int32_t)wr[i];
                const float scaled = (float)dot * inv_scale;
                out[(size_t)b * out_dim + o] = scaled * w_scales[o];
            }
        }
        free(q);
    }
    free(w8);
}

/* The tail of CausalSelfAttention::forward, src/models/llama/attention.rs:103-108:
 * y [1,Hq,S,D] -> transpose_heads_to_seq -> optional sub-norm -> o_proj -> [S, out_dim]. */
XO_API void xo_attention_out_block(const float* y_heads, size_t num_heads, size_t seq_len,
                                   size_t head_dim, const float* norm_weight, float eps,
                                   size_t out_dim, int pack_type, const uint8_t* packed,
                                   const float* w_scales, float* out, int threads) {
    const size_t hidden = num_heads * head_dim;
    float* seq = (float*)malloc((seq_len * hidden + 1) * sizeof(float));
    for (size_t t = 0; t < seq_len; ++t)
        for (size_t h = 0; h < num_heads; ++h)
            memcpy(seq + t * hidden + h * head_dim, y_heads + (h * seq_len + t) * head_dim,
                   head_dim * sizeof(float));
    if (norm_weight)
        for (size_t t = 0; t < seq_len; ++t) xo_rms_norm(seq + t * hidden, norm_weight, eps, hidden);
    xo_ternary_linear_forward(seq, seq_len, hidden, out_dim, pack_type, packed, w_scales, out, threads);
    free(seq);
}

/* ------------------------------------------------------------------------- */
/* XorSparse rows  (src/bit1_58/sparse.rs)                                     */
/* ------------------------------------------------------------------------- */

/* ternarize_row (src/bit1_58/layers.rs:45-88) for one weight.  (A non-positive scale maps to 0
 * here as in the dense packers, quantization.rs:12.) */
static int ternary_value(float w, float w_scale, int already_ternary) {
    if (already_ternary) return (int)w;
    return (int)ternary_code(w, w_scale) - 1;
}

/* encode_sparse_row_into (sparse.rs:62-89): u32 num_blocks, then per 64-element block the u64
 * mask of non-zero positions and ceil(nnz/8) bytes of sign bits in scan order (bit set = -1).
 * Returns the bytes written (the caller provides 4 + ceil(in_dim/64)*16 bytes). */
XO_API size_t xo_sparse_encode_row(const int8_t* vals, size_t in_dim, uint8_t* out) {
    const uint32_t num_blocks = (uint32_t)((in_dim + 63) / 64);
    size_t p = 0;
    for (int i = 0; i < 4; ++i) out[p++] = (uint8_t)(num_blocks >> (8 * i));
    for (uint32_t b = 0; b < num_blocks; ++b) {
        const size_t start = (size_t)b * 64, end = start + 64 < in_dim ? start + 64 : in_dim;
        uint64_t mask = 0, signs = 0;
        unsigned si = 0;
        for (size_t i = start; i < end; ++i)
            if (vals[i] != 0) {
                mask |= (uint64_t)1 << (i - start);
                if (vals[i] < 0) signs |= (uint64_t)1 << si;
                ++si;
            }
        for (int i = 0; i < 8; ++i) out[p++] = (uint8_t)(mask >> (8 * i));
        for (unsigned i = 0; i < (si + 7) / 8; ++i) out[p++] = (uint8_t)(signs >> (8 * i));
    }
    return p;
}

/* SparseTernary::decode_row (sparse.rs:206-249).  Returns the bytes of the row. */
XO_API size_t xo_sparse_decode_row(const uint8_t* row, size_t in_dim, int8_t* out) {
    const uint32_t num_blocks = (uint32_t)row[0] | (uint32_t)row[1] << 8 | (uint32_t)row[2] << 16 |
                                (uint32_t)row[3] << 24;
    size_t p = 4;
    memset(out, 0, in_dim);
    for (uint32_t b = 0; b < num_blocks; ++b) {
        const size_t start = (size_t)b * 64, end = start + 64 < in_dim ? start + 64 : in_dim;
        uint64_t mask = 0, sb = 0;
        for (int i = 0; i < 8; ++i) mask |= (uint64_t)row[p + i] << (8 * i);
        p += 8;
        const unsigned nnz = (unsigned)__builtin_popcountll(mask);
        for (unsigned k = 0; k < (nnz + 7) / 8; ++k) sb |= (uint64_t)row[p + k] << (8 * k);
        p += (nnz + 7) / 8;
        unsigned si = 0;
        for (size_t i = start; i < end; ++i)
            if ((mask >> (i - start)) & 1) {
                out[i] = ((sb >> si) & 1) ? -1 : 1;
                ++si;
            }
    }
    return p;
}

/* ternary_dot_product_sparse_scalar over one row of the blob (src/bit1_58/simd.rs:425-461, with the
 * lane-order sign expansion of SparseTernary::from_blob, sparse.rs:160-177, folded in). */
XO_API int32_t xo_ternary_dot_sparse(const int8_t* a, const uint8_t* row, size_t in_dim) {
    const uint32_t num_blocks = (uint32_t)row[0] | (uint32_t)row[1] << 8 | (uint32_t)row[2] << 16 |
                                (uint32_t)row[3] << 24;
    size_t p = 4;
    int32_t total = 0;
    for (uint32_t b = 0; b < num_blocks; ++b) {
        uint64_t mask = 0, sb = 0;
        for (int i = 0; i < 8; ++i) mask |= (uint64_t)row[p + i] << (8 * i);
        p += 8;
        const unsigned nnz = (unsigned)__builtin_popcountll(mask);
        for (unsigned k = 0; k < (nnz + 7) / 8; ++k) sb |= (uint64_t)row[p + k] << (8 * k);
        p += (nnz + 7) / 8;
        unsigned si = 0;
        for (unsigned lane = 0; lane < 64 && (size_t)b * 64 + lane < in_dim; ++lane)
            if ((mask >> lane) & 1) {
                total += (int32_t)a[(size_t)b * 64 + lane] * (((sb >> si) & 1) ? -1 : 1);
                ++si;
            }
    }
    return total;
}

/* TernaryLinear::new_sparse (src/bit1_58/layers.rs:151-181): ternarise each row like the dense
 * constructor and encode it.  blob must hold out_dim * (4 + ceil(in_dim/64)*16) bytes; returns the
 * bytes used. */
XO_API size_t xo_ternary_linear_pack_sparse(size_t in_dim, size_t out_dim, const float* weights,
                                            float provided_scale, uint8_t* blob, float* w_scales) {
    int already = 1;
    for (size_t i = 0; i < in_dim * out_dim; ++i)
        if (!(weights[i] == -1.0f || weights[i] == 0.0f || weights[i] == 1.0f)) { already = 0; break; }
    const int has_scale = !isnan(provided_scale);
    int8_t* vals = (int8_t*)malloc(in_dim + 1);
    size_t p = 0;
    for (size_t o = 0; o < out_dim; ++o) {
        const float* row = weights + o * in_dim;
        float s;
        if (already) s = has_scale ? provided_scale : 1.0f;
        else if (has_scale) s = provided_scale;
        else {
            float sum_abs = 0.0f;
            for (size_t i = 0; i < in_dim; ++i) sum_abs += fabsf(row[i]);
            s = in_dim == 0 ? 1.0f : sum_abs / (float)in_dim;
        }
        w_scales[o] = s;
        for (size_t i = 0; i < in_dim; ++i) vals[i] = (int8_t)ternary_value(row[i], s, already);
        p += xo_sparse_encode_row(vals, in_dim, blob + p);
    }
    free(vals);
    return p;
}
