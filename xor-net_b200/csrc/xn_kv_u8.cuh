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
#include "xn_decode.cuh"

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

// Pages [0, n_pages) of one stream and layer, dequantised into an f32 staging area laid out as the
// tensor-core prefill kernel expects its pool: [staging page = position / 64][KV head][64][head_dim]
// (head_dim a multiple of 4).  One block per (page, KV head); whole pages are written, so the
// staging area only ever holds finite values.
__global__ void __launch_bounds__(256)
dequant_pages_u8_kernel(const uint8_t* __restrict__ pool, const int* __restrict__ pages, int n_pages,
                        int layer, long long pool_pages, int num_kv_heads, int head_dim, int dq,
                        float* __restrict__ k_stage, float* __restrict__ v_stage) {
    const int p = blockIdx.x / num_kv_heads, h = blockIdx.x % num_kv_heads;
    if (p >= n_pages) return;
    const uint8_t* blk = pool + ((size_t(layer) * size_t(pool_pages) + size_t(pages[p])) * num_kv_heads + h) *
                                    block_bytes(dq);
    const float* sc = reinterpret_cast<const float*>(blk + 2 * size_t(kPageTokens) * dq);
    const size_t out0 = (size_t(p) * num_kv_heads + h) * kPageTokens * head_dim;
    const int quads = head_dim / 4;
    for (int e = threadIdx.x; e < kPageTokens * quads; e += blockDim.x) {
        const int t = e / quads, d = (e % quads) * 4;
        const uchar4 kb = *reinterpret_cast<const uchar4*>(blk + size_t(t) * dq + d);
        const uchar4 vb = *reinterpret_cast<const uchar4*>(blk + size_t(kPageTokens + t) * dq + d);
        const float ks = sc[t], vs = sc[kPageTokens + t];
        *reinterpret_cast<float4*>(k_stage + out0 + size_t(t) * head_dim + d) =
            make_float4((float(kb.x) - 128.0f) * ks, (float(kb.y) - 128.0f) * ks, (float(kb.z) - 128.0f) * ks,
                        (float(kb.w) - 128.0f) * ks);
        *reinterpret_cast<float4*>(v_stage + out0 + size_t(t) * head_dim + d) =
            make_float4((float(vb.x) - 128.0f) * vs, (float(vb.y) - 128.0f) * vs, (float(vb.z) - 128.0f) * vs,
                        (float(vb.w) - 128.0f) * vs);
    }
}

// ---- split-KV attention over u8 pages --------------------------------------------------------

// One warp per thread block, many blocks per SM: every warp walks its own item, so the chain of
// dependent loads that opens an item (descriptors, query rows, page ids, first copies) overlaps
// with the other warps' arithmetic instead of idling a whole 8-warp block.
// (Measured on the config-3 batch: eight-warp blocks, one per SM, 127 us per launch; one-warp
// blocks, eight per SM, 104 us.)
constexpr int kWarps = 1;
constexpr int kThreads = 32 * kWarps;
// Bytes of a row one lane handles (EPL): 16 keeps the per-key bookkeeping lowest, 8 halves the
// registers a lane needs for its query slice and accumulators and so doubles the resident warps.
// (The register file is split over the SM's four schedulers, 16384 registers each: a one-warp
// block of up to 168 registers per thread fits three times per scheduler, up to 128 four times.)
#ifndef XN_KV8_BLOCKS_EPL16
#define XN_KV8_BLOCKS_EPL16 12
#endif
__host__ __device__ constexpr int blocks_per_sm(int epl) { return (epl == 8 ? 16 : XN_KV8_BLOCKS_EPL16) / kWarps; }
#ifndef XN_KV8_PREFETCH
#define XN_KV8_PREFETCH 8
#endif
#ifndef XN_KV8_KEYS_PER_TRIP
#define XN_KV8_KEYS_PER_TRIP 2
#endif
constexpr int kKeysPerTrip = XN_KV8_KEYS_PER_TRIP;   // keys a lane handles between two waits on its copies
constexpr int kPrefetch = XN_KV8_PREFETCH;   // warp iterations a thread's copies run ahead of their use

// reduction buffer of an item's end: [groups of the block][gt][dq] floats = 32 * epl * gt per warp
__host__ __device__ constexpr size_t red_floats(int gt, int epl) { return size_t(32) * epl * kWarps * gt; }
// ring of per-thread copy slots: [kPrefetch][kThreads] x (epl K bytes, epl V bytes, K scale, V scale)
__host__ __device__ constexpr size_t ring_bytes(int epl) { return size_t(kPrefetch) * kThreads * (2 * epl + 8); }
// the two are never live at the same time and share the block's dynamic shared memory
__host__ __device__ constexpr size_t smem_bytes(int gt, int epl) {
    return ring_bytes(epl) > red_floats(gt, epl) * 4 ? ring_bytes(epl) : red_floats(gt, epl) * 4;
}

// Per-thread asynchronous copies global -> shared (LDGSTS): no register holds the data in flight,
// completion is awaited per commit group by the issuing thread, which is also the only reader of
// what it copied -- no barrier between threads is involved.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async8(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// partial record of one (item, head): [m (base-2 log domain), l, 0, 0, acc[dq]]
__host__ __device__ __forceinline__ size_t part_stride(int dq) { return size_t(dq) + 4; }

// 4 * W stored bytes -> exact f32 values (byte - 128): the byte is dropped into the mantissa of
// 2^23 (one PRMT) and 2^23 + 128 is subtracted (exact).
template <int W>
__device__ __forceinline__ void dequant(const uint32_t (&ws)[W], float2 (&f)[2 * W]) {
    const float2 c = make_float2(-8388736.0f, -8388736.0f);
#pragma unroll
    for (int i = 0; i < W; ++i) {
        const float a0 = __uint_as_float(__byte_perm(ws[i], 0x4B000000u, 0x7650));
        const float a1 = __uint_as_float(__byte_perm(ws[i], 0x4B000000u, 0x7651));
        const float a2 = __uint_as_float(__byte_perm(ws[i], 0x4B000000u, 0x7652));
        const float a3 = __uint_as_float(__byte_perm(ws[i], 0x4B000000u, 0x7653));
        f[2 * i] = __fadd2_rn(make_float2(a0, a1), c);
        f[2 * i + 1] = __fadd2_rn(make_float2(a2, a3), c);
    }
}

// 2^x for the softmax weights in the key loop: one MUFU instruction (about 2 ulp), without exp2f's
// extra handling of results below 2^-126, which may flush to 0 here (85.6 against 88.1 us per
// launch on the config-3 batch).  Arguments are <= kLazy.
__device__ __forceinline__ float exp2_weight(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr float kLazy = 8.0f;   // log2 units the running softmax reference may lag the true maximum

// the lane (within a group of LPK lanes) whose owned_head<GT>() is hh
template <int GT>
__device__ __forceinline__ constexpr int src_sub(int hh) {
    return GT == 4 ? (hh == 1 ? 2 : (hh == 2 ? 1 : hh)) : (GT == 2 ? hh : 0);
}

// quantize_to_u8 (src/nn/fast_attention.rs:62-71) for a row spread over the LPK lanes of a group,
// EPL elements per lane: the same operations as quantize_row_store, so the same bytes and scale.
template <int LPK, int EPL>
__device__ __forceinline__ void quantize_group(const float (&x)[EPL], uint32_t (&w)[EPL / 4], float& scale) {
    float mx = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) mx = fmaxf(mx, fabsf(x[j]));
#pragma unroll
    for (int o = 1; o < LPK; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    scale = mx > 0.f ? __fdiv_rn(mx, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
#pragma unroll
    for (int i = 0; i < EPL / 4; ++i) w[i] = 0u;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        float r = roundf(__fadd_rn(__fmul_rn(x[j], inv), 128.0f));
        r = fminf(fmaxf(r, 0.0f), 255.0f);
        w[j / 4] |= uint32_t(r) << (8 * (j % 4));
    }
}

// Rotate-half RoPE (src/nn/fast_attention_simd.rs:380-387) of a row spread over the LPK >= 2 lanes of a
// group with head_dim == LPK * EPL: the partner of element (sub, j) sits on lane sub ^ (LPK / 2)
// at the same j.  cs / sn are the table rows of the position.  Unfused multiplies, as the reference.
template <int LPK, int EPL>
__device__ __forceinline__ void rope_group(float (&x)[EPL], const float* __restrict__ cs,
                                           const float* __restrict__ sn, int sub) {
    const bool lo = sub < LPK / 2;
    const int d0 = (sub % (LPK / 2)) * EPL;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, x[j], LPK / 2);
        const float c = cs[d0 + j], s = sn[d0 + j];
        x[j] = lo ? __fsub_rn(__fmul_rn(x[j], c), __fmul_rn(other, s))
                  : __fadd_rn(__fmul_rn(other, s), __fmul_rn(x[j], c));
    }
}

template <int W>
struct Fetch {
    uint32_t k[W], v[W];
    float ks, vs;
};

// Same work decomposition and plan as the f32 kernel (units, items, chunks taken dynamically by
// the resident blocks, partial records combined by the block that delivers a cut unit's last one),
// but no producer warp and no barriers on the data path: a row is dq bytes, so the LPK = dq / EPL
// lanes that share a key fetch it with one EPL-byte asynchronous copy each into a slot of shared
// memory that only the copying thread reads back, kPrefetch warp iterations ahead of its use
// (80 to 100 KB in flight per SM: enough to cover the HBM latency at full bandwidth).
// Every group of LPK lanes keeps its own online-softmax state for the keys it sees and its own
// partial accumulator for its EPL output dims; the states meet once per item, through shared
// memory.  Scores carry log2(e) (exp2f softmax).  No waits on other blocks or on copies: the
// kernel cannot hang.
template <int LPK, int GT, int EPL>
__global__ void __launch_bounds__(kThreads, blocks_per_sm(EPL))
attn_splitkv_u8_kernel(const ReqDev* __restrict__ reqs, const UnitDev* __restrict__ units,
                       const ItemDev* __restrict__ items, const int* __restrict__ chunk_item_begin,
                       int n_chunks, const int* __restrict__ page_ids,
                       const uint8_t* __restrict__ pool, float* __restrict__ partials,
                       int* __restrict__ sync, long long pool_pages, int num_kv_heads, int head_dim,
                       float scale_log2, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, int* __restrict__ status) {
    (void)status;                       // this kernel waits on nothing that could fail
    constexpr int KPI = 32 / LPK;       // keys per warp iteration
    constexpr int DQ = LPK * EPL;       // bytes per stored row
    constexpr int WE = EPL / 4;         // 32-bit words of a row per lane
    constexpr int HE = EPL / 2;         // float2 of a row per lane
    constexpr int STEP = kWarps * KPI;  // keys per block iteration
    constexpr int PF = kPrefetch;
    constexpr int U = kKeysPerTrip;
    static_assert(PF % U == 0, "the ring must hold a whole number of trips");
    constexpr unsigned kFull = 0xffffffffu;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint32_t* ring_k = reinterpret_cast<uint32_t*>(smem_raw);           // [PF][kThreads][WE]
    uint32_t* ring_v = ring_k + PF * kThreads * WE;                     // [PF][kThreads][WE]
    float2* ring_s = reinterpret_cast<float2*>(ring_v + PF * kThreads * WE);  // [PF][kThreads] (K scale, V scale)
    float* red = reinterpret_cast<float*>(smem_raw);  // [kWarps * KPI groups][GT][DQ], while the ring is idle
    __shared__ float sm_m[kWarps][4], sm_l[kWarps][4];
    __shared__ int sm_next, sm_last;

    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int sub = lane % LPK, grp = lane / LPK, gbase = lane - sub;
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

            float2 q2[GT][HE];
#pragma unroll
            for (int hh = 0; hh < GT; ++hh)
#pragma unroll
                for (int e = 0; e < HE; ++e) {
                    const int d = sub * EPL + 2 * e;
                    float a = 0.f, b = 0.f;
                    if (hh < u.nheads) {
                        if (d < head_dim) a = qrow[size_t(hh) * q_hs + d];
                        if (d + 1 < head_dim) b = qrow[size_t(hh) * q_hs + d + 1];
                    }
                    q2[hh][e] = make_float2(a, b);
                }
            // Fused append (ReqDev flag 8: one new token, not yet in the cache): the unit's last key is
            // taken from the request, rotated when asked, quantised here and stored by the unit
            // that owns the store; the query rows are rotated here as well.  Needs head_dim == DQ.
            const bool fused = r.flags & 8u;
            const bool fused_rope = fused && (r.flags & 1u);
            const bool fused_new = fused && tok_end == u.kv_len;
            const int loop_end = fused_new ? tok_end - 1 : tok_end;
            if constexpr (LPK >= 2) {
                if (fused_rope) {
                    const int half = head_dim / 2;
                    const float* cs = cos_t + size_t(r.index_pos) * half;
                    const float* sn = sin_t + size_t(r.index_pos) * half;
#pragma unroll
                    for (int hh = 0; hh < GT; ++hh) {
                        float x[EPL];
#pragma unroll
                        for (int e = 0; e < HE; ++e) {
                            x[2 * e] = q2[hh][e].x;
                            x[2 * e + 1] = q2[hh][e].y;
                        }
                        rope_group<LPK, EPL>(x, cs, sn, sub);
#pragma unroll
                        for (int e = 0; e < HE; ++e) q2[hh][e] = make_float2(x[2 * e], x[2 * e + 1]);
                    }
                }
            }
            float m[GT], l[GT];
            float2 acc[GT][HE];
#pragma unroll
            for (int hh = 0; hh < GT; ++hh) {
                m[hh] = -INFINITY;
                l[hh] = 0.f;
#pragma unroll
                for (int e = 0; e < HE; ++e) acc[hh][e] = make_float2(0.f, 0.f);
            }

            // one commit group per warp iteration, empty past the item's end, so that "all but the
            // newest PF - 1 groups" always names the iteration about to be used
            // (an item starts on a page boundary and a warp iteration never straddles one, so the
            // page's block address only changes when kk reaches a multiple of the page size)
            // (the id of the page after the current one is fetched a page ahead, so that its latency is
            // not paid when the boundary is reached)
            const uint8_t* page_blk = nullptr;
            int next_page = pages[tok_begin / kPageTokens];
            auto issue = [&](int stage, int kk) {
                const int key = kk + grp;
                if (kk < loop_end && (kk % kPageTokens) == w * KPI) {
                    page_blk = base + size_t(next_page) * page_stride;
                    if (kk - w * KPI + kPageTokens < loop_end) next_page = pages[kk / kPageTokens + 1];
                }
                if (key < loop_end) {
                    const uint8_t* b = page_blk;
                    const int tk = key % kPageTokens;
                    const int slot = stage * kThreads + tid;
                    if constexpr (EPL == 16) {
                        cp_async16(ring_k + slot * WE, b + size_t(tk) * DQ + sub * EPL);
                        cp_async16(ring_v + slot * WE, b + size_t(kPageTokens + tk) * DQ + sub * EPL);
                    } else {
                        cp_async8(ring_k + slot * WE, b + size_t(tk) * DQ + sub * EPL);
                        cp_async8(ring_v + slot * WE, b + size_t(kPageTokens + tk) * DQ + sub * EPL);
                    }
                    const float* sc = reinterpret_cast<const float*>(b + 2 * size_t(kPageTokens) * DQ);
                    cp_async4(&ring_s[slot].x, sc + tk);
                    cp_async4(&ring_s[slot].y, sc + kPageTokens + tk);
                }
                cp_async_commit();
            };

            const int key_first = tok_begin + w * KPI;
#pragma unroll
            for (int p = 0; p < PF; ++p) issue(p, key_first + p * STEP);
            // One trip: U keys per lane (their instruction chains are independent up to the softmax
            // bookkeeping, which they share).
            auto trip = [&](const Fetch<WE> (&cur)[U], const bool (&valid)[U]) {
                // ---- scores of this group's keys for the unit's heads ----
                float dot[U][GT];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    float2 kf[HE];
                    dequant<WE>(cur[u].k, kf);
#pragma unroll
                    for (int hh = 0; hh < GT; ++hh) {
                        float2 a = make_float2(0.f, 0.f);
#pragma unroll
                        for (int e = 0; e < HE; ++e) a = __ffma2_rn(q2[hh][e], kf[e], a);
                        dot[u][hh] = a.x + a.y;
                    }
                }
                // ---- online softmax.  The running reference m only has to stay within
                // 2^kLazy of the true maximum (weights up to 2^8 are harmless in f32), so it
                // moves -- and the accumulators are rescaled -- only on a jump of more than kLazy.
                float pv[U][GT];
                if constexpr (LPK >= GT) {
                    // every lane ends up with the score of ONE head (owned_head(sub)): GT - 1 +
                    // log2(LPK / GT) shuffles instead of GT * log2(LPK), one exp2f instead of GT
                    float s_own[U], smax = -INFINITY;
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const float d = group_reduce<GT, LPK>(dot[u], sub);
                        s_own[u] = valid[u] ? d * (cur[u].ks * scale_log2) : -INFINITY;
                        smax = fmaxf(smax, s_own[u]);
                    }
                    const bool moved = smax > m[0] + kLazy;
                    if (__any_sync(kFull, moved)) {
                        const float alpha = moved ? exp2_weight(m[0] - smax) : 1.f;
                        if (moved) m[0] = smax;
                        l[0] *= alpha;
#pragma unroll
                        for (int hh = 0; hh < GT; ++hh) {
                            const float a = __shfl_sync(kFull, alpha, gbase + src_sub<GT>(hh));
                            const float2 a2 = make_float2(a, a);
#pragma unroll
                            for (int e = 0; e < HE; ++e) acc[hh][e] = __fmul2_rn(acc[hh][e], a2);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const float pw = valid[u] ? exp2_weight(s_own[u] - m[0]) : 0.f;
                        l[0] += pw;
                        const float pvs = valid[u] ? pw * cur[u].vs : 0.f;   // (a stale scale may be anything)
#pragma unroll
                        for (int hh = 0; hh < GT; ++hh)
                            pv[u][hh] = __shfl_sync(kFull, pvs, gbase + src_sub<GT>(hh));
                    }
                } else {
                    float sc_all[U][GT], smax[GT];
#pragma unroll
                    for (int hh = 0; hh < GT; ++hh) smax[hh] = -INFINITY;
#pragma unroll
                    for (int u = 0; u < U; ++u) {
#pragma unroll
                        for (int o = 1; o < LPK; o <<= 1)
#pragma unroll
                            for (int hh = 0; hh < GT; ++hh)
                                dot[u][hh] += __shfl_xor_sync(kFull, dot[u][hh], o);
#pragma unroll
                        for (int hh = 0; hh < GT; ++hh) {
                            sc_all[u][hh] = valid[u] ? dot[u][hh] * (cur[u].ks * scale_log2) : -INFINITY;
                            smax[hh] = fmaxf(smax[hh], sc_all[u][hh]);
                        }
                    }
                    bool moved = false;
#pragma unroll
                    for (int hh = 0; hh < GT; ++hh) moved |= smax[hh] > m[hh] + kLazy;
                    if (__any_sync(kFull, moved)) {
#pragma unroll
                        for (int hh = 0; hh < GT; ++hh) {
                            const bool mv = smax[hh] > m[hh] + kLazy;
                            const float alpha = mv ? exp2_weight(m[hh] - smax[hh]) : 1.f;
                            if (mv) m[hh] = smax[hh];
                            l[hh] *= alpha;
                            const float2 a2 = make_float2(alpha, alpha);
#pragma unroll
                            for (int e = 0; e < HE; ++e) acc[hh][e] = __fmul2_rn(acc[hh][e], a2);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < U; ++u)
#pragma unroll
                        for (int hh = 0; hh < GT; ++hh) {
                            const float pw = valid[u] ? exp2_weight(sc_all[u][hh] - m[hh]) : 0.f;
                            l[hh] += pw;
                            pv[u][hh] = valid[u] ? pw * cur[u].vs : 0.f;
                        }
                }
                // ---- weighted V rows ----
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    float2 vf[HE];
                    dequant<WE>(cur[u].v, vf);
#pragma unroll
                    for (int hh = 0; hh < GT; ++hh) {
                        const float2 p2 = make_float2(pv[u][hh], pv[u][hh]);
#pragma unroll
                        for (int e = 0; e < HE; ++e) acc[hh][e] = __ffma2_rn(p2, vf[e], acc[hh][e]);
                    }
                }
            };

            for (int key0 = key_first; key0 < loop_end; key0 += PF * STEP) {
#pragma unroll
                for (int p = 0; p < PF; p += U) {
                    const int kk = key0 + p * STEP;
                    if (kk >= loop_end) break;  // the same for every lane of the warp
                    // U keys per lane and trip: their instruction chains are independent up to the
                    // softmax bookkeeping, which they share
                    cp_async_wait<PF - U>();
                    Fetch<WE> cur[U];
                    bool valid[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        // a lane past the item's end reads whatever its slot holds: its score is
                        // forced to -inf and its weight to 0 below; stored bytes are always finite
                        const int slot = (p + u) * kThreads + tid;
                        if constexpr (EPL == 16) {
                            const uint4 a = *reinterpret_cast<const uint4*>(ring_k + slot * WE);
                            const uint4 b = *reinterpret_cast<const uint4*>(ring_v + slot * WE);
                            cur[u].k[0] = a.x; cur[u].k[1] = a.y; cur[u].k[2] = a.z; cur[u].k[3] = a.w;
                            cur[u].v[0] = b.x; cur[u].v[1] = b.y; cur[u].v[2] = b.z; cur[u].v[3] = b.w;
                        } else {
                            const uint2 a = *reinterpret_cast<const uint2*>(ring_k + slot * WE);
                            const uint2 b = *reinterpret_cast<const uint2*>(ring_v + slot * WE);
                            cur[u].k[0] = a.x; cur[u].k[1] = a.y;
                            cur[u].v[0] = b.x; cur[u].v[1] = b.y;
                        }
                        const float2 sc = ring_s[slot];
                        cur[u].ks = sc.x;
                        cur[u].vs = sc.y;
                        valid[u] = kk + u * STEP + grp < loop_end;
                    }
#pragma unroll
                    for (int u = 0; u < U; ++u) issue(p + u, kk + (PF + u) * STEP);  // the slots' next use

                    trip(cur, valid);
                }
            }
            if (fused_new) {   // (the same for every lane of the block)
                // the request's new token, on the lanes of group 0
                Fetch<WE> cur[U];
                bool valid[U];
#pragma unroll
                for (int uu = 0; uu < U; ++uu) {
                    valid[uu] = false;
                    cur[uu].ks = cur[uu].vs = 0.f;
#pragma unroll
                    for (int i = 0; i < WE; ++i) cur[uu].k[i] = cur[uu].v[i] = 0x80808080u;
                }
                const float* kn = r.k + size_t(u.kv_head) * r.kv_hs;
                const float* vn = r.v + size_t(u.kv_head) * r.kv_hs;
                float kx[EPL], vx[EPL];
#pragma unroll
                for (int j = 0; j < EPL; ++j) {
                    const int d = sub * EPL + j;
                    kx[j] = (grp == 0 && d < head_dim) ? kn[d] : 0.f;
                    vx[j] = (grp == 0 && d < head_dim) ? vn[d] : 0.f;
                }
                if constexpr (LPK >= 2) {
                    if (fused_rope) {
                        const int half = head_dim / 2;
                        rope_group<LPK, EPL>(kx, cos_t + size_t(r.index_pos) * half,
                                             sin_t + size_t(r.index_pos) * half, sub);
                    }
                }
                quantize_group<LPK, EPL>(kx, cur[0].k, cur[0].ks);
                quantize_group<LPK, EPL>(vx, cur[0].v, cur[0].vs);
                valid[0] = grp == 0;
                if (u.store_new && grp == 0) {
                    const int slot_new = u.kv_len - 1;
                    uint8_t* blk = const_cast<uint8_t*>(base) + size_t(pages[slot_new / kPageTokens]) * page_stride;
                    const int tk = slot_new % kPageTokens;
                    uint32_t* kd = reinterpret_cast<uint32_t*>(blk + size_t(tk) * DQ + sub * EPL);
                    uint32_t* vd = reinterpret_cast<uint32_t*>(blk + size_t(kPageTokens + tk) * DQ + sub * EPL);
#pragma unroll
                    for (int i = 0; i < WE; ++i) {
                        kd[i] = cur[0].k[i];
                        vd[i] = cur[0].v[i];
                    }
                    if (sub == 0) {
                        float* sc = reinterpret_cast<float*>(blk + 2 * size_t(kPageTokens) * DQ);
                        sc[tk] = cur[0].ks;
                        sc[kPageTokens + tk] = cur[0].vs;
                    }
                }
                trip(cur, valid);
            }

            if constexpr (LPK >= GT) {
                // back to one (m, l) per head on every lane of the group, for the merge below
                const float m_own = m[0], l_own = l[0];
#pragma unroll
                for (int hh = 0; hh < GT; ++hh) {
                    m[hh] = __shfl_sync(kFull, m_own, gbase + src_sub<GT>(hh));
                    l[hh] = __shfl_sync(kFull, l_own, gbase + src_sub<GT>(hh));
                }
            }
            cp_async_wait<0>();   // nothing of this item is still on its way into the ring

            // ---- the block's group states meet ----
#pragma unroll
            for (int hh = 0; hh < GT; ++hh) {
                float wm = m[hh];
#pragma unroll
                for (int o = LPK; o < 32; o <<= 1) wm = fmaxf(wm, __shfl_xor_sync(kFull, wm, o));
                if (lane == 0) sm_m[w][hh] = wm;
            }
            __syncthreads();
            float* mine = red + (size_t(w * KPI + grp) * GT) * DQ + sub * EPL;
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
                for (int e = 0; e < HE; e += 2)
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
                if (sm_last && w == 0) {
                    // One warp combines the unit's partial records, all heads at once.  Lane i takes
                    // the (m, l) pairs of record i (32 records at a time, merged online), the
                    // weights travel by shuffle, and the accumulator loads of several records are
                    // all independent of one another, so they overlap instead of paying the L2
                    // latency one by one.
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
