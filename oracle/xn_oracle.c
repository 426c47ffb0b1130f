/*
 * xn_oracle.c -- CPU restatement of xor-net's causal GQA attention path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is
 * compared against and the timed CPU baseline.  Nothing in the shipped library
 * calls it; only the test-suite, the smoke check and the benchmark's CPU
 * baseline leg may load it.
 *
 * Parity status: PINNED against the reference's own known-answer tests
 * (tests/attention_numerics_tests.rs, tests/fast_attention_tests.rs,
 * tests/tensor_ops_tests.rs:226-315, tests/tensor_rope_tests.rs,
 * tests/tensor_layout_tests.rs), all of which generate their vectors from
 * formulas that are reproduced in this repository's oracle tests.  The
 * reference is Rust and cannot be compiled where this was written, so no
 * output of the reference binary itself backs it.
 *
 * Every routine cites the reference lines it follows.  Build with
 *   gcc -O3 -ffp-contract=off -fopenmp -shared -fPIC
 * (-ffp-contract=off: rustc/LLVM never fuses a*b+c on its own, gcc does; the
 * fused multiply-adds below are the ones the reference writes explicitly).
 * The AVX2 / AVX-512 bodies carry per-function target attributes and are chosen
 * at run time the way the reference's is_x86_feature_detected! dispatch does.
 */
#include <immintrin.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define XO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* ISA selection: 0 = like the reference (best available), 1 scalar, 2 AVX2,  */
/* 3 AVX-512.  A forced level that the CPU lacks falls back to auto.          */
/* ------------------------------------------------------------------------- */
enum { XO_ISA_AUTO = 0, XO_ISA_SCALAR = 1, XO_ISA_AVX2 = 2, XO_ISA_AVX512 = 3 };
static int g_isa_force = XO_ISA_AUTO;

static int cpu_has_avx512(void) {
    return __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw");
}
static int cpu_has_avx512f(void) { return __builtin_cpu_supports("avx512f"); }
static int cpu_has_avx2_fma(void) {
    return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
}
static int cpu_has_avx2(void) { return __builtin_cpu_supports("avx2"); }

XO_API int xo_set_isa(int isa) {
    if (isa < 0 || isa > 3) return -1;
    if (isa == XO_ISA_AVX512 && !cpu_has_avx512()) return -2;
    if (isa == XO_ISA_AVX2 && !cpu_has_avx2_fma()) return -2;
    g_isa_force = isa;
    return 0;
}

/* ISA level the dot-product dispatch resolves to (fast_attention_simd.rs:645-651). */
XO_API int xo_active_isa(void) {
    if (g_isa_force != XO_ISA_AUTO) return g_isa_force;
    if (cpu_has_avx512()) return XO_ISA_AVX512;
    if (cpu_has_avx2_fma()) return XO_ISA_AVX2;
    return XO_ISA_SCALAR;
}

/* Whether the i8 activation quantiser takes its AVX-512 body: the reference tests avx512f alone
 * there (src/bit1_58/quantization.rs:148-165).  Used by xn_oracle_outproj.c. */
static int g_quant_body = -1; /* -1: follow the ISA level; 0 scalar body; 1 AVX-512 body */

/* Selects the quantiser body regardless of the CPU (both are restated in portable C), so that the
 * rounding of either build of the reference can be checked anywhere. */
XO_API int xo_set_quant_body(int body) {
    if (body < -1 || body > 1) return -1;
    g_quant_body = body;
    return 0;
}

int xo_quant_uses_avx512(void) {
    if (g_quant_body >= 0) return g_quant_body;
    if (g_isa_force == XO_ISA_SCALAR || g_isa_force == XO_ISA_AVX2) return 0;
    if (g_isa_force == XO_ISA_AVX512) return 1;
    return cpu_has_avx512f();
}

/* ------------------------------------------------------------------------- */
/* batched_dot_product  (src/nn/fast_attention_simd.rs:527-664)               */
/* ------------------------------------------------------------------------- */

/* fast_attention_simd.rs:594-630: one 16-lane accumulator, FMA per 16-chunk,
 * horizontal add, then an unfused scalar tail. */
__attribute__((target("avx512f,avx512bw")))
static void batched_dot_avx512(const float* q, const float* k_buf, size_t h_kv, size_t max_seq_len,
                               size_t head_dim, size_t t_start, size_t t_end, float* out) {
    size_t k_stride = max_seq_len * head_dim;
    size_t h_offset = h_kv * k_stride;
    for (size_t t_k = t_start; t_k < t_end; ++t_k) {
        const float* k_vec = k_buf + h_offset + (t_k % max_seq_len) * head_dim;
        __m512 acc = _mm512_setzero_ps();
        size_t i = 0;
        while (i + 16 <= head_dim) {
            __m512 vq = _mm512_loadu_ps(q + i);
            __m512 vk = _mm512_loadu_ps(k_vec + i);
            acc = _mm512_fmadd_ps(vq, vk, acc);
            i += 16;
        }
        float sum = _mm512_reduce_add_ps(acc);
        while (i < head_dim) {
            sum += q[i] * k_vec[i];
            i += 1;
        }
        out[t_k - t_start] = sum;
    }
}

/* fast_attention_simd.rs:529-590: four 8-lane accumulators over 32-chunks, pairwise
 * combine, 8-chunks into the combined register, lane sum left to right, scalar tail. */
__attribute__((target("avx2,fma")))
static void batched_dot_avx2(const float* q, const float* k_buf, size_t h_kv, size_t max_seq_len,
                             size_t head_dim, size_t t_start, size_t t_end, float* out) {
    size_t k_stride = max_seq_len * head_dim;
    size_t h_offset = h_kv * k_stride;
    for (size_t t_k = t_start; t_k < t_end; ++t_k) {
        const float* k_vec = k_buf + h_offset + (t_k % max_seq_len) * head_dim;
        __m256 s0 = _mm256_setzero_ps(), s1 = _mm256_setzero_ps();
        __m256 s2 = _mm256_setzero_ps(), s3 = _mm256_setzero_ps();
        size_t i = 0;
        while (i + 32 <= head_dim) {
            s0 = _mm256_fmadd_ps(_mm256_loadu_ps(q + i), _mm256_loadu_ps(k_vec + i), s0);
            s1 = _mm256_fmadd_ps(_mm256_loadu_ps(q + i + 8), _mm256_loadu_ps(k_vec + i + 8), s1);
            s2 = _mm256_fmadd_ps(_mm256_loadu_ps(q + i + 16), _mm256_loadu_ps(k_vec + i + 16), s2);
            s3 = _mm256_fmadd_ps(_mm256_loadu_ps(q + i + 24), _mm256_loadu_ps(k_vec + i + 24), s3);
            i += 32;
        }
        __m256 s8 = _mm256_add_ps(_mm256_add_ps(s0, s1), _mm256_add_ps(s2, s3));
        while (i + 8 <= head_dim) {
            s8 = _mm256_fmadd_ps(_mm256_loadu_ps(q + i), _mm256_loadu_ps(k_vec + i), s8);
            i += 8;
        }
        float tmp[8];
        _mm256_storeu_ps(tmp, s8);
        float total = tmp[0] + tmp[1] + tmp[2] + tmp[3] + tmp[4] + tmp[5] + tmp[6] + tmp[7];
        while (i < head_dim) {
            total += q[i] * k_vec[i];
            i += 1;
        }
        out[t_k - t_start] = total;
    }
}

/* fast_attention_simd.rs:653-663 */
static void batched_dot_scalar(const float* q, const float* k_buf, size_t h_kv, size_t max_seq_len,
                               size_t head_dim, size_t t_start, size_t t_end, float* out) {
    size_t k_stride = max_seq_len * head_dim;
    size_t h_offset = h_kv * k_stride;
    for (size_t t_k = t_start; t_k < t_end; ++t_k) {
        const float* k_vec = k_buf + h_offset + (t_k % max_seq_len) * head_dim;
        float sum = 0.0f;
        for (size_t i = 0; i < head_dim; ++i) sum += q[i] * k_vec[i];
        out[t_k - t_start] = sum;
    }
}

/* Dispatch of fast_attention_simd.rs:633-664: AVX-512 needs avx512f AND avx512bw,
 * AVX2 needs avx2 AND fma. */
XO_API void xo_batched_dot_product(const float* q, const float* k_buf, size_t h_kv,
                                   size_t max_seq_len, size_t head_dim, size_t t_start,
                                   size_t t_end, float* out) {
    int isa = g_isa_force;
    if (isa == XO_ISA_AVX512 || (isa == XO_ISA_AUTO && cpu_has_avx512())) {
        batched_dot_avx512(q, k_buf, h_kv, max_seq_len, head_dim, t_start, t_end, out);
        return;
    }
    if (isa == XO_ISA_AVX2 || (isa == XO_ISA_AUTO && cpu_has_avx2_fma())) {
        batched_dot_avx2(q, k_buf, h_kv, max_seq_len, head_dim, t_start, t_end, out);
        return;
    }
    batched_dot_scalar(q, k_buf, h_kv, max_seq_len, head_dim, t_start, t_end, out);
}

/* ------------------------------------------------------------------------- */
/* softmax_inplace  (src/nn/fast_attention_simd.rs:195-368)                    */
/*                                                                             */
/* All three ISA bodies of the reference compute the same values: the running  */
/* maximum is an exact operation, exp is the scalar libm call per element      */
/* (:261-268, :332-339), the sum is accumulated one element at a time in index */
/* order (:303-308), and every element is multiplied by the same 1/sum.  The   */
/* vector bodies below keep the reference's structure so that the timed        */
/* baseline does the same work.                                                */
/* ------------------------------------------------------------------------- */

/* fast_attention_simd.rs:272-329 */
__attribute__((target("avx512f")))
static void softmax_avx512(float* scores, size_t len) {
    float max_val = -INFINITY;
    size_t i = 0;
    while (i + 16 <= len) {
        __m512 v = _mm512_loadu_ps(scores + i);
        __m512 max_vec = _mm512_max_ps(_mm512_set1_ps(max_val), v);
        float tmp[16];
        _mm512_storeu_ps(tmp, max_vec);
        for (int j = 0; j < 16; ++j)
            if (tmp[j] > max_val) max_val = tmp[j];
        i += 16;
    }
    while (i < len) {
        if (scores[i] > max_val) max_val = scores[i];
        i += 1;
    }
    __m512 max_vec = _mm512_set1_ps(max_val);
    float sum_exp = 0.0f;
    i = 0;
    while (i + 16 <= len) {
        __m512 v = _mm512_sub_ps(_mm512_loadu_ps(scores + i), max_vec);
        float arr[16];
        _mm512_storeu_ps(arr, v);
        for (int j = 0; j < 16; ++j) arr[j] = expf(arr[j]);
        _mm512_storeu_ps(scores + i, _mm512_loadu_ps(arr));
        for (int j = 0; j < 16; ++j) sum_exp += arr[j];
        i += 16;
    }
    while (i < len) {
        scores[i] = expf(scores[i] - max_val);
        sum_exp += scores[i];
        i += 1;
    }
    __m512 inv_sum = _mm512_set1_ps(1.0f / sum_exp);
    i = 0;
    while (i + 16 <= len) {
        _mm512_storeu_ps(scores + i, _mm512_mul_ps(_mm512_loadu_ps(scores + i), inv_sum));
        i += 16;
    }
    while (i < len) {
        scores[i] *= 1.0f / sum_exp;
        i += 1;
    }
}

/* fast_attention_simd.rs:197-258 */
__attribute__((target("avx2")))
static void softmax_avx2(float* scores, size_t len) {
    float max_val = -INFINITY;
    size_t i = 0;
    while (i + 8 <= len) {
        __m256 v = _mm256_loadu_ps(scores + i);
        __m256 max_vec = _mm256_max_ps(_mm256_set1_ps(max_val), v);
        float tmp[8];
        _mm256_storeu_ps(tmp, max_vec);
        for (int j = 0; j < 8; ++j)
            if (tmp[j] > max_val) max_val = tmp[j];
        i += 8;
    }
    while (i < len) {
        if (scores[i] > max_val) max_val = scores[i];
        i += 1;
    }
    __m256 max_vec = _mm256_set1_ps(max_val);
    float sum_exp = 0.0f;
    i = 0;
    while (i + 8 <= len) {
        __m256 v = _mm256_sub_ps(_mm256_loadu_ps(scores + i), max_vec);
        float arr[8];
        _mm256_storeu_ps(arr, v);
        for (int j = 0; j < 8; ++j) arr[j] = expf(arr[j]);
        _mm256_storeu_ps(scores + i, _mm256_loadu_ps(arr));
        for (int j = 0; j < 8; ++j) sum_exp += arr[j];
        i += 8;
    }
    while (i < len) {
        scores[i] = expf(scores[i] - max_val);
        sum_exp += scores[i];
        i += 1;
    }
    __m256 inv_sum = _mm256_set1_ps(1.0f / sum_exp);
    i = 0;
    while (i + 8 <= len) {
        _mm256_storeu_ps(scores + i, _mm256_mul_ps(_mm256_loadu_ps(scores + i), inv_sum));
        i += 8;
    }
    while (i < len) {
        scores[i] *= 1.0f / sum_exp;
        i += 1;
    }
}

/* fast_attention_simd.rs:353-367 */
static void softmax_scalar(float* scores, size_t len) {
    float max_val = -INFINITY;
    for (size_t i = 0; i < len; ++i)
        if (scores[i] > max_val) max_val = scores[i];
    float sum_exp = 0.0f;
    for (size_t i = 0; i < len; ++i) {
        scores[i] = expf(scores[i] - max_val);
        sum_exp += scores[i];
    }
    float inv_sum = 1.0f / sum_exp;
    for (size_t i = 0; i < len; ++i) scores[i] *= inv_sum;
}

/* Dispatch of fast_attention_simd.rs:342-351: avx512f alone selects the 512 body. */
XO_API void xo_softmax_inplace(float* scores, size_t len) {
    int isa = g_isa_force;
    if (isa == XO_ISA_AVX512 || (isa == XO_ISA_AUTO && cpu_has_avx512f())) {
        softmax_avx512(scores, len);
        return;
    }
    if (isa == XO_ISA_AVX2 || (isa == XO_ISA_AUTO && cpu_has_avx2())) {
        softmax_avx2(scores, len);
        return;
    }
    softmax_scalar(scores, len);
}

/* ------------------------------------------------------------------------- */
/* weighted_sum  (src/nn/fast_attention_simd.rs:95-193)                        */
/* ------------------------------------------------------------------------- */

/* fast_attention_simd.rs:132-163: per 16-wide column block, FMA over t in order. */
__attribute__((target("avx512f")))
static void weighted_sum_avx512(float* out, const float* scores, const float* v_buf, size_t h_kv,
                                size_t max_seq_len, size_t head_dim, size_t total_kv_len) {
    size_t base = h_kv * (max_seq_len * head_dim);
    size_t i = 0;
    while (i + 16 <= head_dim) {
        __m512 sum = _mm512_setzero_ps();
        for (size_t t_k = 0; t_k < total_kv_len; ++t_k) {
            size_t v_offset = base + (t_k % max_seq_len) * head_dim + i;
            __m512 v_vec = _mm512_loadu_ps(v_buf + v_offset);
            __m512 w = _mm512_set1_ps(scores[t_k]);
            sum = _mm512_fmadd_ps(w, v_vec, sum);
        }
        _mm512_storeu_ps(out + i, sum);
        i += 16;
    }
    while (i < head_dim) {
        float s = 0.0f;
        for (size_t t_k = 0; t_k < total_kv_len; ++t_k) {
            size_t v_offset = base + (t_k % max_seq_len) * head_dim + i;
            s += scores[t_k] * v_buf[v_offset];
        }
        out[i] = s;
        i += 1;
    }
}

/* fast_attention_simd.rs:97-128.  The reference enables only "avx2" on this body
 * yet calls _mm256_fmadd_ps; the fma feature is needed for the same instruction. */
__attribute__((target("avx2,fma")))
static void weighted_sum_avx2(float* out, const float* scores, const float* v_buf, size_t h_kv,
                              size_t max_seq_len, size_t head_dim, size_t total_kv_len) {
    size_t base = h_kv * (max_seq_len * head_dim);
    size_t i = 0;
    while (i + 8 <= head_dim) {
        __m256 sum = _mm256_setzero_ps();
        for (size_t t_k = 0; t_k < total_kv_len; ++t_k) {
            size_t v_offset = base + (t_k % max_seq_len) * head_dim + i;
            __m256 v_vec = _mm256_loadu_ps(v_buf + v_offset);
            __m256 w = _mm256_set1_ps(scores[t_k]);
            sum = _mm256_fmadd_ps(w, v_vec, sum);
        }
        _mm256_storeu_ps(out + i, sum);
        i += 8;
    }
    while (i < head_dim) {
        float s = 0.0f;
        for (size_t t_k = 0; t_k < total_kv_len; ++t_k) {
            size_t v_offset = base + (t_k % max_seq_len) * head_dim + i;
            s += scores[t_k] * v_buf[v_offset];
        }
        out[i] = s;
        i += 1;
    }
}

/* fast_attention_simd.rs:185-192 */
static void weighted_sum_scalar(float* out, const float* scores, const float* v_buf, size_t h_kv,
                                size_t max_seq_len, size_t head_dim, size_t total_kv_len) {
    size_t base = h_kv * (max_seq_len * head_dim);
    for (size_t i = 0; i < head_dim; ++i) {
        float s = 0.0f;
        for (size_t t_k = 0; t_k < total_kv_len; ++t_k) {
            size_t v_offset = base + (t_k % max_seq_len) * head_dim + i;
            s += scores[t_k] * v_buf[v_offset];
        }
        out[i] = s;
    }
}

/* Dispatch of fast_attention_simd.rs:166-183. */
XO_API void xo_weighted_sum(float* out, const float* scores, const float* v_buf, size_t h_kv,
                            size_t max_seq_len, size_t head_dim, size_t total_kv_len) {
    int isa = g_isa_force;
    if (isa == XO_ISA_AVX512 || (isa == XO_ISA_AUTO && cpu_has_avx512f())) {
        weighted_sum_avx512(out, scores, v_buf, h_kv, max_seq_len, head_dim, total_kv_len);
        return;
    }
    if (isa == XO_ISA_AVX2 || (isa == XO_ISA_AUTO && cpu_has_avx2_fma())) {
        weighted_sum_avx2(out, scores, v_buf, h_kv, max_seq_len, head_dim, total_kv_len);
        return;
    }
    weighted_sum_scalar(out, scores, v_buf, h_kv, max_seq_len, head_dim, total_kv_len);
}

/* ------------------------------------------------------------------------- */
/* RoPE                                                                        */
/* ------------------------------------------------------------------------- */

/* One token vector: src/nn/fast_attention_simd.rs:380-387 (and the identical
 * scalar body :399-406).  Rotate-half pairs (x[i], x[i+D/2]); plain mul/mul/sub
 * and mul/mul/add, no fused multiply-add. */
XO_API void xo_rope_vec(float* x, const float* cos_row, const float* sin_row, size_t head_dim) {
    size_t half_dim = head_dim / 2;
    for (size_t i = 0; i < half_dim; ++i) {
        float c = cos_row[i];
        float s = sin_row[i];
        float x1 = x[i];
        float x2 = x[i + half_dim];
        x[i] = x1 * c - x2 * s;
        x[i + half_dim] = x1 * s + x2 * c;
    }
}

/* FastTensor::rope_inplace, src/tensor.rs:295-316: x is [1, num_heads, seq_len,
 * head_dim]; token t of every head uses table row index_pos + t. */
XO_API void xo_tensor_rope_inplace(float* x, size_t num_heads, size_t seq_len, size_t head_dim,
                                   const float* cos, const float* sin, size_t index_pos) {
    size_t half = head_dim / 2;
    for (size_t h = 0; h < num_heads; ++h) {
        float* head = x + h * seq_len * head_dim;
        for (size_t t = 0; t < seq_len; ++t) {
            size_t pos = index_pos + t;
            xo_rope_vec(head + t * head_dim, cos + pos * half, sin + pos * half, head_dim);
        }
    }
}

/* Cache::new table builder, src/models/llama/mod.rs:210-265.
 *   inv_freq[j] = 1 / theta^(2j / D)            (:210-216, f32 powf)
 *   optional Llama-3 frequency scaling           (:226-249); enabled when factor > 0
 *   angle = (pos as f32) * inv_freq[j]; cos/sin  (:252-262, f32 libm)
 * cos and sin are [max_pos, D/2]. */
XO_API void xo_rope_tables(float theta, size_t head_dim, size_t max_pos, float factor,
                           float low_freq_factor, float high_freq_factor, size_t original_max_pos,
                           float* cos_out, float* sin_out) {
    size_t half = head_dim / 2;
    size_t nfreq = (head_dim + 1) / 2; /* (0..head_dim).step_by(2) */
    float* inv_freq = (float*)malloc(sizeof(float) * (nfreq ? nfreq : 1));
    for (size_t j = 0; j < nfreq; ++j) {
        float i = (float)(2 * j);
        inv_freq[j] = 1.0f / powf(theta, i / (float)head_dim);
    }
    if (factor > 0.0f) {
        const float PI_F = 3.14159265358979323846f;
        float low_freq_wavelen = (float)original_max_pos / low_freq_factor;
        float high_freq_wavelen = (float)original_max_pos / high_freq_factor;
        for (size_t j = 0; j < nfreq; ++j) {
            float freq = inv_freq[j];
            float wavelen = 2.0f * PI_F / freq;
            if (wavelen < high_freq_wavelen) {
                /* unchanged */
            } else if (wavelen > low_freq_wavelen) {
                inv_freq[j] = freq / factor;
            } else {
                float smooth = ((float)original_max_pos / wavelen - low_freq_factor) /
                               (high_freq_factor - low_freq_factor);
                inv_freq[j] = (1.0f - smooth) * freq / factor + smooth * freq;
            }
        }
    }
    for (size_t pos = 0; pos < max_pos; ++pos) {
        for (size_t i = 0; i < half; ++i) {
            float a = (float)pos * inv_freq[i];
            cos_out[pos * half + i] = cosf(a);
            sin_out[pos * half + i] = sinf(a);
        }
    }
    free(inv_freq);
}

/* ------------------------------------------------------------------------- */
/* Layout steps either side of the call (src/tensor.rs:332-376)               */
/* ------------------------------------------------------------------------- */

/* [1, S, H*D] -> [1, H, S, D]   (tensor.rs:332-354) */
XO_API void xo_transpose_seq_to_heads(const float* in, float* out, size_t seq_len, size_t num_heads,
                                      size_t head_dim) {
    for (size_t h = 0; h < num_heads; ++h)
        for (size_t t = 0; t < seq_len; ++t)
            memcpy(out + h * seq_len * head_dim + t * head_dim,
                   in + t * num_heads * head_dim + h * head_dim, head_dim * sizeof(float));
}

/* [1, H, S, D] -> [1, S, H*D]   (tensor.rs:356-376) */
XO_API void xo_transpose_heads_to_seq(const float* in, float* out, size_t seq_len, size_t num_heads,
                                      size_t head_dim) {
    for (size_t t = 0; t < seq_len; ++t)
        for (size_t h = 0; h < num_heads; ++h)
            memcpy(out + t * num_heads * head_dim + h * head_dim,
                   in + h * seq_len * head_dim + t * head_dim, head_dim * sizeof(float));
}

/* ------------------------------------------------------------------------- */
/* CpuRingCache + fast_attention  (src/nn/fast_attention.rs)                   */
/* ------------------------------------------------------------------------- */

/* CpuRingCache, fast_attention.rs:18-60.  The u8 shadow (:62-71, :117-128) is
 * write-only in the reference -- nothing reads it back -- so it does not take
 * part in any result of the f32 cache; its quantiser is restated below
 * (xo_quantize_to_u8) for the opt-in u8 cache format of the CUDA library. */
typedef struct xo_ring_cache {
    size_t num_layers, num_kv_heads, max_seq_len, head_dim;
    float** k_buffers; /* [layer][h*cap*D + t*D + d], zero initialised (:40-41) */
    float** v_buffers;
} xo_ring_cache;

XO_API xo_ring_cache* xo_cache_new(size_t num_layers, size_t num_kv_heads, size_t max_seq_len,
                                   size_t head_dim) {
    xo_ring_cache* c = (xo_ring_cache*)calloc(1, sizeof(*c));
    if (!c) return NULL;
    c->num_layers = num_layers;
    c->num_kv_heads = num_kv_heads;
    c->max_seq_len = max_seq_len;
    c->head_dim = head_dim;
    c->k_buffers = (float**)calloc(num_layers ? num_layers : 1, sizeof(float*));
    c->v_buffers = (float**)calloc(num_layers ? num_layers : 1, sizeof(float*));
    size_t size = num_kv_heads * max_seq_len * head_dim;
    for (size_t l = 0; l < num_layers; ++l) {
        c->k_buffers[l] = (float*)calloc(size ? size : 1, sizeof(float));
        c->v_buffers[l] = (float*)calloc(size ? size : 1, sizeof(float));
    }
    return c;
}

XO_API void xo_cache_free(xo_ring_cache* c) {
    if (!c) return;
    for (size_t l = 0; l < c->num_layers; ++l) {
        free(c->k_buffers[l]);
        free(c->v_buffers[l]);
    }
    free(c->k_buffers);
    free(c->v_buffers);
    free(c);
}

/* Views of the reference's pub fields k_buffers[layer] / v_buffers[layer]. */
XO_API float* xo_cache_k(xo_ring_cache* c, size_t layer) { return c->k_buffers[layer]; }
XO_API float* xo_cache_v(xo_ring_cache* c, size_t layer) { return c->v_buffers[layer]; }

/* Append step only, fast_attention.rs:104-116 (positions fold modulo capacity). */
static void cache_append(xo_ring_cache* cache, size_t layer_idx, size_t index_pos, size_t seq_len,
                         const float* k_data, const float* v_data) {
    float* k_buf = cache->k_buffers[layer_idx];
    float* v_buf = cache->v_buffers[layer_idx];
    size_t max_seq_len = cache->max_seq_len, head_dim = cache->head_dim;
    for (size_t h_kv = 0; h_kv < cache->num_kv_heads; ++h_kv) {
        for (size_t t_new = 0; t_new < seq_len; ++t_new) {
            size_t t_abs = index_pos + t_new;
            size_t wrapped_t = t_abs % max_seq_len;
            size_t dest = h_kv * (max_seq_len * head_dim) + wrapped_t * head_dim;
            size_t src = h_kv * (seq_len * head_dim) + t_new * head_dim;
            memcpy(k_buf + dest, k_data + src, head_dim * sizeof(float));
            memcpy(v_buf + dest, v_data + src, head_dim * sizeof(float));
        }
    }
}

/* CpuRingCache::quantize_to_u8, fast_attention.rs:62-71, applied to `rows` rows of n floats (the
 * reference calls it once per (KV head, new token) slice, :120-121): max_abs folds f32::max over
 * |x| from 0.0 (NaNs are ignored), scale = max_abs / 127 or 1.0, inv_scale = 1 / scale, and each
 * byte is ((x * inv_scale) + 128).round().clamp(0, 255) as u8 -- round half away from zero, the
 * multiply and the add separate roundings, NaN -> 0.
 * PARITY UNPINNED: the reference holds no test or golden vector for the shadow. */
XO_API void xo_quantize_to_u8(const float* data, size_t rows, size_t n, uint8_t* out, float* scales) {
    for (size_t r = 0; r < rows; ++r) {
        const float* x = data + r * n;
        float max_abs = 0.0f;
        for (size_t i = 0; i < n; ++i) {
            float a = fabsf(x[i]);
            if (a > max_abs) max_abs = a; /* f32::max: a NaN operand loses */
        }
        float scale = max_abs > 0.0f ? max_abs / 127.0f : 1.0f;
        float inv_scale = 1.0f / scale;
        for (size_t i = 0; i < n; ++i) {
            float v = roundf((x[i] * inv_scale) + 128.0f);
            uint8_t b;
            if (v != v) b = 0;            /* NaN as u8 */
            else if (v < 0.0f) b = 0;
            else if (v > 255.0f) b = 255;
            else b = (uint8_t)v;
            out[r * n + i] = b;
        }
        scales[r] = scale;
    }
}

/* The values a reader of the u8 cache sees: (byte - 128) * scale.  (The reference never wrote its
 * "lazy dequantisation"; this is the inverse of the quantiser above.) */
XO_API void xo_dequantize_u8(const uint8_t* q, const float* scales, size_t rows, size_t n, float* out) {
    for (size_t r = 0; r < rows; ++r)
        for (size_t i = 0; i < n; ++i) out[r * n + i] = ((float)q[r * n + i] - 128.0f) * scales[r];
}

XO_API void xo_cache_append(xo_ring_cache* cache, size_t layer_idx, size_t index_pos,
                            size_t seq_len, const float* k_data, const float* v_data) {
    cache_append(cache, layer_idx, index_pos, seq_len, k_data, v_data);
}

/* Attention for one KV head: the closure body of fast_attention.rs:140-200.
 * scores is scratch of at least index_pos + seq_len floats. */
static void attend_kv_head(const xo_ring_cache* cache, size_t layer_idx, size_t index_pos,
                           size_t seq_len, size_t heads_per_kv, size_t head_dim, size_t h_kv,
                           const float* q_data, float* out_data, float* scores, float scale) {
    const float* k_buf = cache->k_buffers[layer_idx];
    const float* v_buf = cache->v_buffers[layer_idx];
    size_t max_seq_len = cache->max_seq_len;
    size_t q_head_start = h_kv * heads_per_kv;
    size_t q_head_end = q_head_start + heads_per_kv;
    for (size_t h = q_head_start; h < q_head_end; ++h) {
        for (size_t t_q = 0; t_q < seq_len; ++t_q) {
            const float* q_vec = q_data + h * (seq_len * head_dim) + t_q * head_dim;
            float* out_vec = out_data + h * (seq_len * head_dim) + t_q * head_dim;
            size_t limit = index_pos + t_q;
            size_t total_kv_len = limit + 1;
            size_t t_k = 0;
            while (t_k <= limit) { /* :166-182, batches of 16 keys */
                size_t batch_end = t_k + 16 < limit + 1 ? t_k + 16 : limit + 1;
                size_t batch_len = batch_end - t_k;
                float batch_scores[16] = {0};
                xo_batched_dot_product(q_vec, k_buf, h_kv, max_seq_len, head_dim, t_k, batch_end,
                                       batch_scores);
                for (size_t i = 0; i < batch_len; ++i) scores[t_k + i] = batch_scores[i] * scale;
                t_k = batch_end;
            }
            xo_softmax_inplace(scores, total_kv_len);                  /* :185-186 */
            memset(out_vec, 0, head_dim * sizeof(float));              /* :189 */
            xo_weighted_sum(out_vec, scores, v_buf, h_kv, max_seq_len, head_dim, total_kv_len);
        }
    }
}

/* fast_attention, fast_attention.rs:75-204.
 * q is [1, num_heads, seq_len, head_dim]; k, v are [1, num_kv_heads, seq_len,
 * head_dim]; out is [1, num_heads, seq_len, head_dim].  q_ndim / q_batch carry the
 * shape facts the reference checks (:86-92): returns 1 for a non-4-D Q, 2 for a
 * batch other than 1, 0 on success.  threads <= 0 uses the OpenMP default; the
 * parallel loop is over KV heads like the reference's rayon split (:138). */
XO_API int xo_fast_attention(const float* q, const float* k, const float* v, size_t layer_idx,
                             size_t index_pos, xo_ring_cache* cache, size_t num_heads,
                             size_t num_kv_heads, size_t head_dim, size_t seq_len, int q_ndim,
                             size_t q_batch, float* out, int threads) {
    if (q_ndim != 4) return 1;
    if (q_batch != 1) return 2;
    cache_append(cache, layer_idx, index_pos, seq_len, k, v);
    size_t heads_per_kv = num_heads / num_kv_heads;
    float scale = 1.0f / sqrtf((float)head_dim);
    size_t max_kv_len = index_pos + seq_len;
    memset(out, 0, num_heads * seq_len * head_dim * sizeof(float)); /* :134 */
#ifdef _OPENMP
    int nthreads = threads > 0 ? threads : omp_get_max_threads();
#pragma omp parallel for schedule(dynamic, 1) num_threads(nthreads)
#endif
    for (long h_kv = 0; h_kv < (long)num_kv_heads; ++h_kv) {
        float* scores = (float*)malloc(sizeof(float) * (max_kv_len ? max_kv_len : 1)); /* :151 */
        attend_kv_head(cache, layer_idx, index_pos, seq_len, heads_per_kv, head_dim, (size_t)h_kv,
                       q, out, scores, scale);
        free(scores);
    }
    (void)threads;
    return 0;
}

/* Many independent streams at once: stream i calls fast_attention on its own
 * cache, which is how the reference's server and batch_bench run concurrent
 * requests (server/main.rs:176-199, examples/batch_bench.rs:138-151: one thread
 * per stream).  Here the (stream, KV head) pairs are spread over OpenMP threads;
 * each pair computes exactly what xo_fast_attention computes for it.
 * Arrays are indexed by stream; all streams share layer_idx and the head shape. */
XO_API int xo_fast_attention_streams(size_t n_streams, const float* const* q, const float* const* k,
                                     const float* const* v, size_t layer_idx,
                                     const size_t* index_pos, const size_t* seq_len,
                                     xo_ring_cache* const* caches, size_t num_heads,
                                     size_t num_kv_heads, size_t head_dim, float* const* out,
                                     int threads) {
    size_t heads_per_kv = num_heads / num_kv_heads;
    float scale = 1.0f / sqrtf((float)head_dim);
    for (size_t s = 0; s < n_streams; ++s) {
        cache_append(caches[s], layer_idx, index_pos[s], seq_len[s], k[s], v[s]);
        memset(out[s], 0, num_heads * seq_len[s] * head_dim * sizeof(float));
    }
    long total = (long)(n_streams * num_kv_heads);
#ifdef _OPENMP
    int nthreads = threads > 0 ? threads : omp_get_max_threads();
#pragma omp parallel for schedule(dynamic, 1) num_threads(nthreads)
#endif
    for (long w = 0; w < total; ++w) {
        size_t s = (size_t)w / num_kv_heads, h_kv = (size_t)w % num_kv_heads;
        size_t max_kv_len = index_pos[s] + seq_len[s];
        float* scores = (float*)malloc(sizeof(float) * (max_kv_len ? max_kv_len : 1));
        attend_kv_head(caches[s], layer_idx, index_pos[s], seq_len[s], heads_per_kv, head_dim, h_kv,
                       q[s], out[s], scores, scale);
        free(scores);
    }
    (void)threads;
    return 0;
}

XO_API int xo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
