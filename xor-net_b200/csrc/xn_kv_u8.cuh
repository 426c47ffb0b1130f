// Opt-in compressed KV pages: the reference's u8 shadow cache made the cache itself, sm_100a.
//
// The reference quantises every appended K / V row to u8 with one f32 scale per (KV head, token)
// and keeps the result beside the f32 ring (src/nn/fast_attention.rs:5-16 the buffers, :62-71 the
// quantiser, :117-128 the append); its own attention never reads the shadow.  A context created
// with the u8 cache format stores ONLY that representation -- the same bytes and scales, bit for
// bit -- and attends over the dequantised values (byte - 128) * scale, a quarter of the f32
// cache's bytes per token.  Results differ from the f32 cache by the quantisation error, which is
// why the format is opt-in.
//
// Pool layout, one block per (layer, page, KV head), kPageTokens = 64 tokens each:
//     K bytes [64][dq] | V bytes [64][dq] | K scales [64] f32 | V scales [64] f32
// dq = head_dim rounded up to a power of two >= 16; padding bytes hold 128 (dequantised 0).
// Never-written slots hold byte 128 and scale 0.0 as in the reference (:45-48).
#pragma once
#include "xn_common.cuh"

namespace xn {
namespace kv8 {

__host__ __device__ __forceinline__ size_t block_bytes(int dq) {
    return size_t(kPageTokens) * (2 * size_t(dq) + 8);
}
inline int row_bytes_for(int head_dim) {
    int dq = 16;
    while (dq < head_dim) dq *= 2;
    return dq;
}

__device__ __forceinline__ uint8_t* block_ptr(uint8_t* pool, const int* pages, long long pool_pages,
                                              int layer, int num_kv_heads, int kv_head, int slot, int dq) {
    return pool + ((size_t(layer) * size_t(pool_pages) + size_t(pages[slot / kPageTokens])) * num_kv_heads +
                   kv_head) * block_bytes(dq);
}

// CpuRingCache::quantize_to_u8 (src/nn/fast_attention.rs:62-71) for one row held by a warp, element
// i = lane + 32 j in x[j]: scale = max|x| / 127 (1.0 for an all-zero row), byte =
// clamp(round_half_away(x * (1 / scale) + 128), 0, 255).  Unfused multiply and add, IEEE division:
// the stored bytes and the scale equal the reference's.  Bytes head_dim..dq-1 are written as 128.
__device__ __forceinline__ void quantize_row_store(const float (&x)[8], int head_dim, int dq,
                                                   uint8_t* __restrict__ dst_row,
                                                   float* __restrict__ dst_scale, int lane) {
    float mx = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j)
        if (lane + 32 * j < head_dim) mx = fmaxf(mx, fabsf(x[j]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float scale = mx > 0.f ? __fdiv_rn(mx, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = lane + 32 * j;
        if (i >= dq) break;
        uint8_t b = 128;
        if (i < head_dim) {
            float r = roundf(__fadd_rn(__fmul_rn(x[j], inv), 128.0f));
            r = fminf(fmaxf(r, 0.0f), 255.0f);   // a NaN becomes 0, as `NaN as u8` does
            b = uint8_t(r);
        }
        dst_row[i] = b;
    }
    if (lane == 0) *dst_scale = scale;
}

// The append of src/nn/fast_attention.rs:104-128 for the u8 format, one warp per (new token, row),
// rows = [q heads (when the request asks for the scratch copy)] + [k heads] + [v heads]:
//   * Q rows: copied, rotated when asked, into the dense f32 scratch ReqDev::q points at;
//   * K rows: rotated when asked (src/nn/fast_attention_simd.rs:380-387, table row index_pos + t,
//     unfused multiplies), then quantised and stored;  V rows: quantised and stored.
// A slot that a later token of the same call overwrites is skipped (the reference's sequential
// loop leaves the last writer's value).
__global__ void __launch_bounds__(256)
rope_append_u8_kernel(const ReqDev* __restrict__ reqs, const int* __restrict__ page_ids,
                      uint8_t* __restrict__ pool, const float* __restrict__ cos_t,
                      const float* __restrict__ sin_t, long long pool_pages, int num_heads,
                      int num_kv_heads, int head_dim, int dq) {
    const ReqDev& r = reqs[blockIdx.y];
    const bool rope = r.flags & 1u;
    const bool q_rows = r.flags & 3u;
    const int rows_per_tok = (q_rows ? num_heads : 0) + 2 * num_kv_heads;
    const long long n_rows = (long long)r.seq_len * rows_per_tok;
    const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
    const int half = head_dim / 2;
    const int* pages = page_ids + r.page_off;
    for (long long row = (long long)blockIdx.x * 8 + wp; row < n_rows; row += (long long)gridDim.x * 8) {
        const int t = int(row / rows_per_tok);
        int rr = int(row % rows_per_tok);
        const int pos = r.index_pos + t;
        const float* src;
        int kind;  // 0 query, 1 key, 2 value
        if (q_rows && rr < num_heads) {
            src = r.q_in + size_t(rr) * r.qi_hs + size_t(t) * r.qi_ts;
            kind = 0;
        } else {
            if (q_rows) rr -= num_heads;
            if ((long long)t + r.cap < (long long)r.seq_len) continue;  // overwritten later in this call
            if (rr < num_kv_heads) {
                src = r.k + size_t(rr) * r.kv_hs + size_t(t) * r.kv_ts;
                kind = 1;
            } else {
                rr -= num_kv_heads;
                src = r.v + size_t(rr) * r.kv_hs + size_t(t) * r.kv_ts;
                kind = 2;
            }
        }
        const bool rotate = rope && kind != 2;
        const float* c = cos_t + size_t(pos) * half;
        const float* s = sin_t + size_t(pos) * half;
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = lane + 32 * j;
            float val = 0.f;
            if (i < head_dim) {
                if (rotate && i < half) {
                    val = __fsub_rn(__fmul_rn(src[i], c[i]), __fmul_rn(src[i + half], s[i]));
                } else if (rotate && i < 2 * half) {
                    const int ii = i - half;
                    val = __fadd_rn(__fmul_rn(src[ii], s[ii]), __fmul_rn(src[i], c[ii]));
                } else {
                    val = src[i];
                }
            }
            x[j] = val;
        }
        if (kind == 0) {
            float* dst = const_cast<float*>(r.q) + size_t(rr) * r.q_hs + size_t(t) * r.q_ts;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (lane + 32 * j < head_dim) dst[lane + 32 * j] = x[j];
        } else {
            const int slot = pos % r.cap;
            uint8_t* blk = block_ptr(pool, pages, pool_pages, r.layer, num_kv_heads, rr, slot, dq);
            const int tk = slot % kPageTokens;
            uint8_t* row_dst = blk + (kind == 1 ? 0 : size_t(kPageTokens) * dq) + size_t(tk) * dq;
            float* sc_dst = reinterpret_cast<float*>(blk + 2 * size_t(kPageTokens) * dq) +
                            (kind == 1 ? 0 : kPageTokens) + tk;
            quantize_row_store(x, head_dim, dq, row_dst, sc_dst, lane);
        }
    }
}

// Slots [slot0, slot0+n) of one layer of one stream, one warp per (slot, KV head): mode 0 restores
// the never-written state (byte 128, scale 0.0: skipped positions must read as zeros, as in the
// reference's freshly built shadow, src/nn/fast_attention.rs:45-48); mode 1 quantises the N(0,1)
// rows the f32 fill kernel would have written (same generator, same indices).
__global__ void __launch_bounds__(256)
slots_fill_u8_kernel(const int* __restrict__ pages, uint8_t* __restrict__ pool, long long pool_pages,
                     int layer, int num_kv_heads, int head_dim, int dq, long long slot0, long long n,
                     int mode, unsigned long long seed) {
    const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
    const long long total = n * num_kv_heads;
    for (long long e = (long long)blockIdx.x * 8 + wp; e < total; e += (long long)gridDim.x * 8) {
        const int h = int(e % num_kv_heads);
        const int slot = int(slot0 + e / num_kv_heads);
        uint8_t* blk = block_ptr(pool, pages, pool_pages, layer, num_kv_heads, h, slot, dq);
        const int tk = slot % kPageTokens;
        uint8_t* k_row = blk + size_t(tk) * dq;
        uint8_t* v_row = blk + size_t(kPageTokens) * dq + size_t(tk) * dq;
        float* k_sc = reinterpret_cast<float*>(blk + 2 * size_t(kPageTokens) * dq) + tk;
        float* v_sc = k_sc + kPageTokens;
        if (mode == 0) {
            for (int i = lane; i < dq; i += 32) {
                k_row[i] = 128;
                v_row[i] = 128;
            }
            if (lane == 0) {
                *k_sc = 0.f;
                *v_sc = 0.f;
            }
        } else {
            float kx[8], vx[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int d = lane + 32 * j;
                const unsigned long long idx =
                    ((unsigned long long)(slot) * num_kv_heads + h) * head_dim + d;
                kx[j] = d < head_dim ? normal_from(seed, 2ull * idx) : 0.f;
                vx[j] = d < head_dim ? normal_from(seed, 2ull * idx + 1ull) : 0.f;
            }
            quantize_row_store(kx, head_dim, dq, k_row, k_sc, lane);
            quantize_row_store(vx, head_dim, dq, v_row, v_sc, lane);
        }
    }
}

// Every block of the pool into the never-written state.
__global__ void __launch_bounds__(256)
pool_init_u8_kernel(uint8_t* __restrict__ pool, long long n_blocks, int dq) {
    const size_t bb = block_bytes(dq);
    const size_t data = 2 * size_t(kPageTokens) * dq;   // bytes before the scales
    const size_t words = bb / 4;
    for (long long b = blockIdx.x; b < n_blocks; b += gridDim.x) {
        uint32_t* w = reinterpret_cast<uint32_t*>(pool + size_t(b) * bb);
        for (size_t i = threadIdx.x; i < words; i += blockDim.x) w[i] = (i * 4 < data) ? 0x80808080u : 0u;
    }
}

// Gathers slots [slot0, slot0+n) of every KV head: dequantised rows into dense f32 [Hkv, n, D]
// buffers and / or the stored representation itself (bytes [Hkv, n, D], scales [Hkv, n]).  Any
// output may be null.
__global__ void __launch_bounds__(256)
slots_gather_u8_kernel(const int* __restrict__ pages, const uint8_t* __restrict__ pool,
                       long long pool_pages, int layer, int num_kv_heads, int head_dim, int dq,
                       long long slot0, long long n, float* __restrict__ k_out,
                       float* __restrict__ v_out, uint8_t* __restrict__ k_raw,
                       uint8_t* __restrict__ v_raw, float* __restrict__ k_sc_out,
                       float* __restrict__ v_sc_out) {
    const long long total = n * num_kv_heads * head_dim;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (long long)gridDim.x * blockDim.x) {
        const int d = int(e % head_dim);
        const long long rest = e / head_dim;
        const long long i = rest % n;
        const int h = int(rest / n);
        const int slot = int(slot0 + i);
        const uint8_t* blk = block_ptr(const_cast<uint8_t*>(pool), pages, pool_pages, layer, num_kv_heads,
                                       h, slot, dq);
        const int tk = slot % kPageTokens;
        const uint8_t kb = blk[size_t(tk) * dq + d];
        const uint8_t vb = blk[size_t(kPageTokens) * dq + size_t(tk) * dq + d];
        const float* sc = reinterpret_cast<const float*>(blk + 2 * size_t(kPageTokens) * dq);
        const float ks = sc[tk], vs = sc[kPageTokens + tk];
        if (k_out) k_out[e] = (float(kb) - 128.0f) * ks;
        if (v_out) v_out[e] = (float(vb) - 128.0f) * vs;
        if (k_raw) k_raw[e] = kb;
        if (v_raw) v_raw[e] = vb;
        if (d == 0) {
            if (k_sc_out) k_sc_out[rest] = ks;
            if (v_sc_out) v_sc_out[rest] = vs;
        }
    }
}

// ---- split-KV attention over u8 pages --------------------------------------------------------

constexpr int kThreads = 256;
constexpr int kWarps = 8;
#ifndef XN_KV8_PREFETCH
#define XN_KV8_PREFETCH 2
#endif

__host__ __device__ constexpr size_t red_floats(int gt) { return size_t(4096) * gt; }
// partial record of one (item, head): [m (base-2 log domain), l, 0, 0, acc[dq]]
__host__ __device__ __forceinline__ size_t part_stride(int dq) { return size_t(dq) + 4; }

// 16 stored bytes -> 16 exact f32 values (byte - 128): the byte is dropped into the mantissa of
// 2^23 (one PRMT) and 2^23 + 128 is subtracted (exact).
__device__ __forceinline__ void dequant16(const uint4& w, float2 (&f)[8]) {
    const unsigned ws[4] = {w.x, w.y, w.z, w.w};
    const float2 c = make_float2(-8388736.0f, -8388736.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float a0 = __uint_as_float(__byte_perm(ws[i], 0x4B000000u, 0x7650));
        const float a1 = __uint_as_float(__byte_perm(ws[i], 0x4B000000u, 0x7651));
        const float a2 = __uint_as_float(__byte_perm(ws[i], 0x4B000000u, 0x7652));
        const float a3 = __uint_as_float(__byte_perm(ws[i], 0x4B000000u, 0x7653));
        f[2 * i] = __fadd2_rn(make_float2(a0, a1), c);
        f[2 * i + 1] = __fadd2_rn(make_float2(a2, a3), c);
    }
}

struct Fetch {
    uint4 k, v;
    float ks, vs;
};

// Same work decomposition and plan as the f32 kernel (units, items, chunks taken dynamically by
// one block per SM, partial records combined by the block that delivers a cut unit's last one),
// but no staging: a row is dq bytes, so the LPK = dq / 16 lanes that share a key fetch it with one
// 16-byte load each, straight into registers, XN_KV8_PREFETCH warp iterations ahead of its use.
// Every group of LPK lanes keeps its own online-softmax state for the keys it sees and its own
// partial accumulator for its 16 output dims; the states meet once per item, through shared
// memory.  Scores carry log2(e) (exp2f softmax).  No waits on other blocks or on copies: the
// kernel cannot hang.
template <int LPK, int GT>
__global__ void __launch_bounds__(kThreads, 1)
attn_splitkv_u8_kernel(const ReqDev* __restrict__ reqs, const UnitDev* __restrict__ units,
                       const ItemDev* __restrict__ items, const int* __restrict__ chunk_item_begin,
                       int n_chunks, const int* __restrict__ page_ids,
                       const uint8_t* __restrict__ pool, float* __restrict__ partials,
                       int* __restrict__ sync, long long pool_pages, int num_kv_heads, int head_dim,
                       float scale_log2) {
    constexpr int KPI = 32 / LPK;       // keys per warp iteration
    constexpr int DQ = LPK * 16;        // bytes per stored row
    constexpr int STEP = kWarps * KPI;  // keys per block iteration
    constexpr int PF = XN_KV8_PREFETCH;
    constexpr unsigned kFull = 0xffffffffu;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* red = reinterpret_cast<float*>(smem_raw);  // [kWarps * KPI groups][GT][DQ]
    __shared__ float sm_m[kWarps][4], sm_l[kWarps][4];
    __shared__ int sm_next, sm_last;

    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int sub = lane % LPK, grp = lane / LPK;
    const size_t blk_bytes = block_bytes(DQ);
    const size_t page_stride = size_t(num_kv_heads) * blk_bytes;
    const size_t pstride = part_stride(DQ);

    int chunk = blockIdx.x;
    while (chunk < n_chunks) {
        const int it_lo = chunk_item_begin[chunk], it_hi = chunk_item_begin[chunk + 1];
        for (int it = it_lo; it < it_hi; ++it) {
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

            float2 q2[GT][8];
#pragma unroll
            for (int hh = 0; hh < GT; ++hh)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int d = sub * 16 + 2 * e;
                    float a = 0.f, b = 0.f;
                    if (hh < u.nheads) {
                        if (d < head_dim) a = qrow[size_t(hh) * q_hs + d];
                        if (d + 1 < head_dim) b = qrow[size_t(hh) * q_hs + d + 1];
                    }
                    q2[hh][e] = make_float2(a, b);
                }
            float m[GT], l[GT];
            float2 acc[GT][8];
#pragma unroll
            for (int hh = 0; hh < GT; ++hh) {
                m[hh] = -INFINITY;
                l[hh] = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[hh][e] = make_float2(0.f, 0.f);
            }

            auto fetch = [&](Fetch& f, int kk) {
                const int key = kk + grp;
                if (key < tok_end) {
                    const uint8_t* b = base + size_t(pages[kk / kPageTokens]) * page_stride;
                    const int tk = key % kPageTokens;
                    f.k = __ldg(reinterpret_cast<const uint4*>(b + size_t(tk) * DQ + sub * 16));
                    f.v = __ldg(reinterpret_cast<const uint4*>(b + size_t(kPageTokens + tk) * DQ + sub * 16));
                    const float* sc = reinterpret_cast<const float*>(b + 2 * size_t(kPageTokens) * DQ);
                    f.ks = __ldg(sc + tk);
                    f.vs = __ldg(sc + kPageTokens + tk);
                } else {
                    f.k = f.v = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
                    f.ks = f.vs = 0.f;
                }
            };

            Fetch f[PF];
            int key0 = tok_begin + w * KPI;
#pragma unroll
            for (int p = 0; p < PF; ++p) fetch(f[p], key0 + p * STEP);
            for (; key0 < tok_end; key0 += PF * STEP) {
#pragma unroll
                for (int p = 0; p < PF; ++p) {
                    const int kk = key0 + p * STEP;
                    if (kk >= tok_end) break;  // the same for every lane of the warp
                    const Fetch cur = f[p];
                    fetch(f[p], kk + PF * STEP);
                    const bool valid = kk + grp < tok_end;

                    // ---- scores of this group's key for the unit's heads ----
                    float2 kf[8];
                    dequant16(cur.k, kf);
                    float dot[GT];
#pragma unroll
                    for (int hh = 0; hh < GT; ++hh) {
                        float2 a = make_float2(0.f, 0.f);
#pragma unroll
                        for (int e = 0; e < 8; ++e) a = __ffma2_rn(q2[hh][e], kf[e], a);
                        dot[hh] = a.x + a.y;
                    }
#pragma unroll
                    for (int o = 1; o < LPK; o <<= 1)
#pragma unroll
                        for (int hh = 0; hh < GT; ++hh) dot[hh] += __shfl_xor_sync(kFull, dot[hh], o);

                    // ---- online softmax, per group ----
                    const float ksc = cur.ks * scale_log2;
                    float s[GT];
                    bool moved = false;
#pragma unroll
                    for (int hh = 0; hh < GT; ++hh) {
                        s[hh] = valid ? dot[hh] * ksc : -INFINITY;
                        moved |= s[hh] > m[hh];
                    }
                    if (__any_sync(kFull, moved)) {
#pragma unroll
                        for (int hh = 0; hh < GT; ++hh) {
                            const float m_new = fmaxf(m[hh], s[hh]);
                            const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m[hh] - m_new);
                            m[hh] = m_new;
                            l[hh] *= alpha;
                            const float2 a2 = make_float2(alpha, alpha);
#pragma unroll
                            for (int e = 0; e < 8; ++e) acc[hh][e] = __fmul2_rn(acc[hh][e], a2);
                        }
                    }
                    float2 vf[8];
                    dequant16(cur.v, vf);
#pragma unroll
                    for (int hh = 0; hh < GT; ++hh) {
                        const float p = valid ? exp2f(s[hh] - m[hh]) : 0.f;
                        l[hh] += p;
                        const float pv = p * cur.vs;
                        const float2 p2 = make_float2(pv, pv);
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[hh][e] = __ffma2_rn(p2, vf[e], acc[hh][e]);
                    }
                }
            }

            // ---- the block's group states meet ----
#pragma unroll
            for (int hh = 0; hh < GT; ++hh) {
                float wm = m[hh];
#pragma unroll
                for (int o = LPK; o < 32; o <<= 1) wm = fmaxf(wm, __shfl_xor_sync(kFull, wm, o));
                if (lane == 0) sm_m[w][hh] = wm;
            }
            __syncthreads();
            float* mine = red + (size_t(w * KPI + grp) * GT) * DQ + sub * 16;
#pragma unroll
            for (int hh = 0; hh < GT; ++hh) {
                float M = -INFINITY;
#pragma unroll
                for (int ww = 0; ww < kWarps; ++ww) M = fmaxf(M, sm_m[ww][hh]);
                const float fct = (m[hh] == -INFINITY) ? 0.f : exp2f(m[hh] - M);
                float lv = (sub == 0) ? l[hh] * fct : 0.f;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) lv += __shfl_xor_sync(kFull, lv, o);
                if (lane == 0) sm_l[w][hh] = lv;
#pragma unroll
                for (int e = 0; e < 8; e += 2)
                    *reinterpret_cast<float4*>(mine + size_t(hh) * DQ + 2 * e) =
                        make_float4(acc[hh][e].x * fct, acc[hh][e].y * fct, acc[hh][e + 1].x * fct,
                                    acc[hh][e + 1].y * fct);
            }
            __syncthreads();
            for (int e = tid; e < GT * DQ; e += kThreads) {
                const int hh = e / DQ, d = e % DQ;
                if (hh >= u.nheads) continue;
                float sum = 0.f;
#pragma unroll 8
                for (int g = 0; g < kWarps * KPI; ++g) sum += red[(size_t(g) * GT + hh) * DQ + d];
                float M = -INFINITY, L = 0.f;
#pragma unroll
                for (int ww = 0; ww < kWarps; ++ww) {
                    M = fmaxf(M, sm_m[ww][hh]);
                    L += sm_l[ww][hh];
                }
                if (item.part < 0) {
                    if (d < head_dim) orow[size_t(hh) * o_hs + d] = sum / L;
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
                // the unit was cut: whoever delivers its last partial combines them all (one thread
                // fences and counts after the block barrier; the fence is cumulative)
                __syncthreads();
                if (tid == 0) {
                    __threadfence();
                    const int old = atomicAdd(&sync[kSyncMerge0 + u.merge_slot], 1);
                    const int last = old == u.part_count - 1;
                    if (last) {
                        sync[kSyncMerge0 + u.merge_slot] = 0;  // re-armed for the next launch
                        __threadfence();
                    }
                    sm_last = last;
                }
                __syncthreads();
                if (sm_last) {
                    for (int e = tid; e < GT * DQ; e += kThreads) {
                        const int hh = e / DQ, d = e % DQ;
                        if (hh >= u.nheads || d >= head_dim) continue;
                        float M = -INFINITY;
                        for (int i = 0; i < u.part_count; ++i)
                            M = fmaxf(M, __ldcg(partials + (size_t(u.part_begin + i) * GT + hh) * pstride));
                        float L = 0.f, sum = 0.f;
                        for (int i = 0; i < u.part_count; ++i) {
                            const float* rec = partials + (size_t(u.part_begin + i) * GT + hh) * pstride;
                            const float mi = __ldcg(rec);
                            const float wgt = (mi == -INFINITY) ? 0.f : exp2f(mi - M);
                            L += __ldcg(rec + 1) * wgt;
                            sum = fmaf(wgt, __ldcg(rec + 4 + d), sum);
                        }
                        orow[size_t(hh) * o_hs + d] = sum / L;
                    }
                }
            }
            __syncthreads();  // red, sm_m, sm_l and sm_last are rewritten by the next item
        }
        if (tid == 0) sm_next = atomicAdd(&sync[kSyncChunk], 1) + int(gridDim.x);
        __syncthreads();
        chunk = sm_next;
        __syncthreads();
    }
    if (tid == 0) {
        // the last block to finish re-arms the chunk counter for the next launch
        __threadfence();
        if (atomicAdd(&sync[kSyncDone], 1) == int(gridDim.x) - 1) {
            sync[kSyncChunk] = 0;
            sync[kSyncDone] = 0;
        }
    }
}

}  // namespace kv8
}  // namespace xn
