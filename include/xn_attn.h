/*
 * xn_attn.h -- C ABI of the B200 (sm_100a) replacement for xor-net's causal
 * grouped-query attention path: `fast_attention` and the KV cache it owns.
 *
 * Every entry point is extern "C", takes plain pointers, integers and
 * plain-old-data structs, returns an xn_status, never throws and never calls
 * back.  A language binding (Rust FFI, ctypes, cgo ...) needs nothing else.
 *
 * Reference interface replaced (paths inside the xor-net source tree):
 *   src/nn/fast_attention.rs:75-85    pub fn fast_attention(q, k, v, layer_idx,
 *                                     index_pos, cache, num_heads, num_kv_heads, head_dim)
 *   src/nn/fast_attention.rs:18-60    pub struct CpuRingCache + CpuRingCache::new
 *   src/models/llama/mod.rs:210-265   RoPE table construction in Cache::new
 *   src/tensor.rs:295-316             FastTensor::rope_inplace (fused entry only)
 *
 * Tensor layout contract (same as the reference): row-major f32,
 *   q   [1, num_heads,    seq_len, head_dim]
 *   k,v [1, num_kv_heads, seq_len, head_dim]
 *   out [1, num_heads,    seq_len, head_dim]
 * Query head h reads KV head h / (num_heads / num_kv_heads).
 *
 * Cache contract: logical coordinate (layer, kv_head, t, d) with the reference's
 * ring rule slot = t % max_seq_len.  Storage is device memory in 64-token pages
 * taken from one pool per context; a stream (= one reference `Cache`) owns a
 * page table shared by all layers.  The reference's public `k_buffers` view is
 * served by xn_kv_read / xn_kv_read_range.
 */
#ifndef XN_ATTN_H
#define XN_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define XN_API __attribute__((visibility("default")))
#else
#define XN_API
#endif

typedef struct xn_ctx xn_ctx;       /* one per GPU: page pool, kernels' workspaces, CUDA stream */
typedef struct xn_stream xn_stream; /* one per sequence: replaces one CpuRingCache            */

typedef enum xn_status {
    XN_OK = 0,
    XN_ERR_ARG = 1,          /* null pointer, negative size, bad flag combination               */
    XN_ERR_SHAPE = 2,        /* head counts / head_dim outside what the kernels support          */
    XN_ERR_HANDLE = 3,       /* context or stream handle is not live                             */
    XN_ERR_OUT_OF_PAGES = 4, /* page pool exhausted                                              */
    XN_ERR_CAPACITY = 5,     /* position beyond the RoPE table, or request too large             */
    XN_ERR_CUDA = 6,         /* a CUDA runtime call failed; text in xn_last_error                */
    XN_ERR_DEVICE_WAIT = 7,  /* a kernel gave up on a bounded wait and reported it               */
    XN_ERR_NO_TABLES = 8,    /* fused-RoPE entry used on a context created without cos/sin       */
    XN_ERR_NOMEM = 9,        /* host allocation failed                                           */
    XN_ERR_NO_DEVICE = 10,   /* no usable CUDA device: there is no CPU fallback                  */
    XN_ERR_GUARD = 11        /* xn_debug_check_guards found bytes written outside a device buffer */
} xn_status;

/* Prefill kernel choice (xn_ctx_desc.prefill_mode). */
enum {
    XN_PREFILL_AUTO = 0, /* tensor-core TF32 kernel where the shape allows, exact f32 otherwise */
    XN_PREFILL_F32 = 1,  /* always the exact-f32 CUDA-core path                                 */
    XN_PREFILL_TF32 = 2  /* TF32 kernel whenever it supports the shape                          */
};

/* KV cache format (xn_ctx_desc.kv_format). */
enum {
    XN_KV_F32 = 0, /* f32 rows: what fast_attention reads (k_buffers / v_buffers,                 */
                   /* fast_attention.rs:20-21); results equal the reference's                      */
    XN_KV_U8 = 1   /* opt-in: ONLY the reference's u8 shadow is kept (one byte per element, one    */
                   /* f32 scale per KV head and token; U8CacheLayer fast_attention.rs:5-16, the    */
                   /* quantiser :62-71, the append :117-128) and attention runs over the           */
                   /* dequantised values (byte - 128) * scale.  A quarter of the cache bytes; the  */
                   /* stored bytes and scales equal the reference's shadow bit for bit, the        */
                   /* attention output differs from the f32 cache's by the quantisation error.     */
                   /* Prefills served by the tensor-core kernel first dequantise the stream's      */
                   /* pages of the layer into an f32 staging area (grown on demand).               */
};

typedef struct xn_ctx_desc {
    int32_t device;       /* CUDA ordinal                                                        */
    int32_t num_layers;   /* CpuRingCache::new(num_layers, ...)   fast_attention.rs:31-34        */
    int32_t num_heads;    /* query heads                                                         */
    int32_t num_kv_heads; /* must divide num_heads                                               */
    int32_t head_dim;     /* 1..256                                                              */
    int32_t page_tokens;  /* 0 or 64                                                             */
    int64_t pool_pages;   /* pages in the pool (each holds 64 tokens of every layer); if 0,      */
    int64_t pool_bytes;   /*   derived from pool_bytes; if that is 0 too, from XORNET_ATTN_POOL_MB */
                          /*   or, when unset, half of the device memory that is free             */
    uint64_t shuffle_seed;/* 0: pages handed out in ascending order; else a seeded permutation   */
    int32_t max_pos;      /* rows of the RoPE tables, 0 if none                                  */
    int32_t prefill_mode; /* XN_PREFILL_*                                                        */
    const float* rope_cos;/* host [max_pos, head_dim/2] (models/llama/mod.rs:252-265), or NULL   */
    const float* rope_sin;
    void* cuda_stream;    /* cudaStream_t to launch on; NULL: the context creates its own        */
    int32_t batch_window_us; /* how long a lone xn_attention caller waits for company            */
    int32_t kv_format;       /* XN_KV_*                                                           */
} xn_ctx_desc;

/* Request flags. */
enum {
    XN_REQ_DEVICE_PTRS = 1u << 0, /* q,k,v,out are device pointers; the call only enqueues work  */
    XN_REQ_ROPE = 1u << 1,        /* q,k are pre-RoPE; rotate with the context's tables          */
    XN_REQ_SEQ_MAJOR = 1u << 2,   /* q,k,v,out are [seq_len, heads*head_dim] (the layout before  */
                                  /* transpose_seq_to_heads, tensor.rs:332-354, and after        */
                                  /* transpose_heads_to_seq, tensor.rs:356-376)                  */
    XN_REQ_HOST_PINNED = 1u << 3, /* host pointers are page-locked, device-mapped memory         */
                                  /* (cudaHostAlloc / cudaHostRegister): the kernels read the    */
                                  /* inputs over PCIe themselves and the library's staging       */
                                  /* copies are skipped.  Outputs that lie back to back in host  */
                                  /* memory (>= 128 KB in all, e.g. one tensor for the batch)    */
                                  /* are produced on the device and leave in ONE transfer;       */
                                  /* scattered outputs are stored by the kernels directly, which */
                                  /* is about three times slower per byte.  The call still       */
                                  /* blocks until the output is complete.  All requests of a     */
                                  /* batch must agree on this flag.                              */
    XN_REQ_OUT_PROJ = 1u << 4,    /* `out` receives [seq_len, out_dim]: the attention output run */
                                  /* through the layer's output block (xn_out_proj_set) on the   */
                                  /* device, i.e. what models/llama/attention.rs:103-108 does    */
                                  /* after fast_attention returns                                */
    XN_REQ_QKV_PROJ = 1u << 5     /* `q` points at the hidden states x [seq_len, hidden] that    */
                                  /* CausalSelfAttention::forward receives; k and v are ignored. */
                                  /* The layer's q/k/v projections (xn_qkv_proj_set), the heads  */
                                  /* layout and the rotation run on the device                   */
                                  /* (models/llama/attention.rs:52-89); needs RoPE tables        */
};

typedef struct xn_req {
    xn_stream* stream;
    int32_t layer;     /* layer_idx  */
    int32_t seq_len;   /* new tokens in this call (1 = decode) */
    int64_t index_pos; /* position of the first new token      */
    const float* q;
    const float* k;
    const float* v;
    float* out;
    uint32_t flags;
    uint32_t reserved;
} xn_req;

typedef struct xn_stats {
    uint64_t calls;            /* requests served                                               */
    uint64_t batches;          /* batched submissions (one group of launches each)              */
    uint64_t kernel_launches;  /* kernels of this library launched                              */
    uint64_t decode_launches;  /* launches of the split-KV attention kernel                     */
    uint64_t prefill_launches; /* launches of the tiled prefill kernels                         */
    uint64_t h2d_bytes;
    uint64_t d2h_bytes;
    uint64_t pages_total;
    uint64_t pages_in_use;
    uint64_t streams_live;
    uint64_t device_wait_errors;
    uint64_t coalesced_max;    /* largest number of blocking callers merged into one batch      */
    uint64_t out_proj_rows;    /* token rows run through a projection block (q/k/v or output)   */
    uint64_t plan_reuses;      /* decode submissions that reused the previous one's plan        */
    uint64_t out_transfers;    /* submissions whose page-locked outputs left in one transfer    */
} xn_stats;

/* ---- context --------------------------------------------------------------------------------- */

/* Replaces the allocation half of CpuRingCache::new (fast_attention.rs:31-60) for all streams of
 * one GPU: reserves the page pool once instead of max_seq_len rows per request. */
XN_API int32_t xn_ctx_create(const xn_ctx_desc* desc, xn_ctx** out_ctx);
XN_API int32_t xn_ctx_destroy(xn_ctx* ctx);
/* Waits for everything enqueued on the context's CUDA stream; reports bounded-wait failures. */
XN_API int32_t xn_ctx_synchronize(xn_ctx* ctx);
/* The cudaStream_t the context launches on (for callers that time with CUDA events). */
XN_API void* xn_ctx_cuda_stream(xn_ctx* ctx);
XN_API int32_t xn_stats_get(xn_ctx* ctx, xn_stats* out);
/* Text of the most recent failure on this context (or of context creation when ctx is NULL). */
XN_API const char* xn_last_error(xn_ctx* ctx);

/* Device-side timing of the two attention kernels: when enabled, every launch of the split-KV
 * kernel and of the tensor-core prefill kernel is bracketed by CUDA events on the context's
 * stream.  xn_profile_read waits for the stream, adds up the elapsed times recorded since the
 * last read and returns them (milliseconds) with the number of launches they cover; any output
 * pointer may be NULL. */
XN_API int32_t xn_profile_enable(xn_ctx* ctx, int32_t on);
/* The same for every timed kind: ms and launches are arrays of XN_PROFILE_KINDS entries
 * (0 split-KV attention, 1 tensor-core prefill, 2 output block = sub-norm + projection pair,
 * 3 q/k/v block = quantiser + projection pair). */
#define XN_PROFILE_KINDS 4
XN_API int32_t xn_profile_read_all(xn_ctx* ctx, double* ms, uint64_t* launches);
XN_API int32_t xn_profile_read(xn_ctx* ctx, double* splitkv_ms, uint64_t* splitkv_launches,
                               double* prefill_ms, uint64_t* prefill_launches);

/* ---- device groups ---------------------------------------------------------------------------- */

/* The reference's server and batch_bench are ONE process whose slot threads share one model
 * (server/main.rs:635-645, examples/batch_bench.rs:138-151) and each own a `Cache`
 * (server/main.rs:92, batch_bench.rs:188).  A group puts every GPU of the box behind that one
 * process: one context per device, and each new stream (one per `Cache::new`, i.e. per
 * CpuRingCache::new, fast_attention.rs:31-34) is placed on one of them for its whole life.  The
 * blocking calls of streams on different devices then run in parallel: every context has its own
 * queue that merges its own concurrent callers. */
typedef struct xn_group xn_group;

enum {
    XN_PLACE_LEAST_LOADED = 0, /* the device holding the fewest cached (or announced) tokens; ties: */
                               /* the fewest live streams, then round-robin                          */
    XN_PLACE_ROUND_ROBIN = 1   /* device = stream number mod number of devices                      */
};

/* One context per listed CUDA ordinal, all created from `desc` (its `device` and `cuda_stream` are
 * ignored; pool_pages / pool_bytes apply per device).  n_devices = 0: the ordinals named by the
 * environment variable XORNET_ATTN_DEVICES ("0,1,5"), or every visible device when it is unset. */
XN_API int32_t xn_group_create(const xn_ctx_desc* desc, const int32_t* devices, int32_t n_devices,
                               xn_group** out_group);
/* Destroys the contexts of the group (and with them their streams). */
XN_API int32_t xn_group_destroy(xn_group* group);
XN_API int32_t xn_group_size(xn_group* group);          /* number of devices, or a negative xn_status */
XN_API xn_ctx* xn_group_ctx(xn_group* group, int32_t i); /* the i-th device's context, or NULL        */
/* xn_stream_create on the device the policy picks.  expected_tokens (0 = unknown) announces how many
 * tokens the stream is going to hold, so that streams created before they are filled still spread by
 * load.  *ctx_out receives the context that owns the stream: pass it with the stream to every call. */
XN_API int32_t xn_group_stream_create(xn_group* group, int64_t max_seq_len, int64_t expected_tokens,
                                      int32_t policy, xn_ctx** ctx_out, xn_stream** out_stream);
/* The placement rule on its own (no GPU needed): tokens[i] and live_streams[i] describe device i,
 * ticket is the number of streams placed so far.  Returns the chosen index or a negative xn_status. */
XN_API int32_t xn_place_stream(int32_t n_devices, const int64_t* tokens, const int64_t* live_streams,
                               uint64_t ticket, int32_t policy);

/* ---- streams (one per reference `Cache`, models/llama/mod.rs:202-279) ------------------------ */

/* max_seq_len is the reference's ring capacity (CpuRingCache.max_seq_len): positions fold modulo
 * it.  Pages are taken from the pool only as positions are written. */
XN_API int32_t xn_stream_create(xn_ctx* ctx, int64_t max_seq_len, xn_stream** out_stream);
/* Forget all cached tokens and return the pages (a fresh Cache::new in the reference). */
XN_API int32_t xn_stream_reset(xn_ctx* ctx, xn_stream* stream);
XN_API int32_t xn_stream_destroy(xn_ctx* ctx, xn_stream* stream);

/* ---- the hot path ---------------------------------------------------------------------------- */

/* Drop-in for fast_attention (fast_attention.rs:75-204): host pointers, q and k already rotated.
 * Appends k,v at positions index_pos.. then attends every new query row to positions
 * 0..=index_pos+t.  Blocks until `out` is written.  Calls made at the same time from different
 * threads (one per stream, as xor-net's server slots and batch_bench do) are merged into one
 * batched launch. */
XN_API int32_t xn_attention(xn_ctx* ctx, xn_stream* stream, int32_t layer, int64_t index_pos,
                            int32_t seq_len, const float* q, const float* k, const float* v,
                            float* out);

/* Same, with q and k before RoPE: fuses FastTensor::rope_inplace (tensor.rs:295-316, call site
 * models/llama/attention.rs:88-89) into the cache-append kernel. */
XN_API int32_t xn_attention_rope(xn_ctx* ctx, xn_stream* stream, int32_t layer, int64_t index_pos,
                                 int32_t seq_len, const float* q, const float* k, const float* v,
                                 float* out);

/* Explicit batch: n independent requests (distinct streams) in one submission.  With
 * XN_REQ_DEVICE_PTRS on every request the call returns after enqueueing; otherwise it blocks
 * until the host outputs are written.  Mixing host and device requests is an error. */
XN_API int32_t xn_attention_batch(xn_ctx* ctx, int32_t n, const xn_req* reqs);

/* No counterpart in the reference: decode attention for callers that must not allocate.
 *
 * Some users of this library run where cudaMalloc is off limits -- a serving loop that has handed
 * all device memory to its own arena, a latency-critical thread where an allocation's implicit
 * device synchronisation is unacceptable, a plugin host that forbids it.  This one entry point
 * computes single-token attention (one query row per head over kv_len cached positions, q.k *
 * 1/sqrt(head_dim), softmax, weighted V sum; query head h reads KV head h / (num_heads /
 * num_kv_heads)) without allocating anything: it calls no cudaMalloc, cudaFree or other
 * allocating routine, and creates no context.  The split-KV partial results go to a fixed scratch
 * array inside the library image (about 1.0 MiB of every GPU that loads the library, held until
 * the process exits).
 *
 * All pointers are device memory owned by the caller on the current device:
 *   q [num_heads, head_dim], out [num_heads, head_dim],
 *   k_cache, v_cache [num_kv_heads, capacity, head_dim] (the reference's ring layout,
 *   fast_attention.rs:107-108) with positions 0..kv_len-1 already written, the new token included.
 * Work is enqueued on cuda_stream (NULL = the default stream); the call does not wait for it.
 *
 * Limits, rejected with XN_ERR_CAPACITY and a message in xn_last_error(NULL): head_dim <= 256 and
 * num_heads <= 1024 (the scratch holds 1024 partial records of 260 floats).
 *
 * The first call on each device looks up the scratch array's device address; make that first
 * call before starting any stream capture.  Every call on a device shares the one scratch array:
 * two calls whose kernels overlap on the GPU (different streams, or different threads on
 * different streams) race on it -- keep calls on one stream or order them yourself.  Nothing in
 * the scratch has to start at zero; each call rewrites every record it later reads. */
XN_API int32_t xn_decode_attention_static(const float* q, const float* k_cache, const float* v_cache,
                                          float* out, int32_t num_heads, int32_t num_kv_heads,
                                          int32_t head_dim, int64_t kv_len, int64_t capacity,
                                          void* cuda_stream);

/* ---- RoPE tables ----------------------------------------------------------------------------- */

/* Builds cos/sin [max_pos, head_dim/2] exactly as Cache::new does (models/llama/mod.rs:210-265):
 * f32 powf / cosf / sinf on the host.  factor <= 0 disables the Llama-3 frequency scaling
 * (:226-249). */
XN_API int32_t xn_rope_tables(float theta, int32_t head_dim, int32_t max_pos, float factor,
                              float low_freq_factor, float high_freq_factor,
                              int32_t original_max_pos, float* cos_out, float* sin_out);

/* ---- cache inspection and synthetic fill (tests, benches) ------------------------------------ */

/* One cached row: the reference's k_buffers[layer][h*cap*D + (t%cap)*D ..] (fast_attention.rs:
 * 107-108).  Either output may be NULL.  Rows never written read as zeros. */
XN_API int32_t xn_kv_read(xn_ctx* ctx, xn_stream* stream, int32_t layer, int32_t kv_head, int64_t t,
                          float* k_row, float* v_row);
/* Slots [t0, t0+n) of every KV head: k_out, v_out are [num_kv_heads, n, head_dim]. */
XN_API int32_t xn_kv_read_range(xn_ctx* ctx, xn_stream* stream, int32_t layer, int64_t t0,
                                int64_t n, float* k_out, float* v_out);
/* XN_KV_U8 contexts only: the stored representation of slots [t0, t0+n) of every KV head, i.e.
 * the reference's u8_k / u8_v [num_kv_heads, n, head_dim] and k_scales / v_scales
 * [num_kv_heads, n] (fast_attention.rs:8-15).  Any output may be NULL.  Never-written slots read
 * as byte 128 with scale 0.0 (:45-48).  (xn_kv_read and xn_kv_read_range return the dequantised
 * rows in this format.) */
XN_API int32_t xn_kv_read_u8(xn_ctx* ctx, xn_stream* stream, int32_t layer, int64_t t0, int64_t n,
                             uint8_t* k_u8, uint8_t* v_u8, float* k_scales, float* v_scales);
/* Fills slots [t0, t0+n) of one layer with N(0,1) values from a counter-based generator on the
 * device (no host copy) so that benchmarks can build large caches. */
XN_API int32_t xn_kv_fill_normal(xn_ctx* ctx, xn_stream* stream, int32_t layer, int64_t t0,
                                 int64_t n, uint64_t seed);
/* N(0,1) fill of any device buffer with the same generator. */
XN_API int32_t xn_fill_normal(xn_ctx* ctx, float* device_ptr, int64_t n, uint64_t seed);
/* Number of cached positions of a stream in one layer (highest written position + 1). */
XN_API int64_t xn_stream_len(xn_ctx* ctx, xn_stream* stream, int32_t layer);
/* Copies the stream's page table (page ids in position order) into `out`; returns the count. */
XN_API int64_t xn_stream_pages(xn_ctx* ctx, xn_stream* stream, int32_t* out, int64_t max_out);

/* ---- attention output block: sub-norm + ternary o_proj ---------------------------------------- */

/* Packing of ternary weights, TernaryPackType (src/bit1_58/quantization.rs:1-5). */
enum {
    XN_PACK4 = 4, /* four 2-bit codes per byte  (pack_1_58bit_4pack, quantization.rs:7-27)        */
    XN_PACK5 = 5, /* five base-3 digits per byte (pack_1_58bit_5pack, quantization.rs:49-72)      */
    XN_SPARSE = 64 /* the XorSparse blob of TernaryRep::Sparse (src/bit1_58/sparse.rs:9-17): rows   */
                   /* back to back, each u32 num_blocks + per 64-element block {u64 mask of the    */
                   /* non-zero positions, ceil(popcount/8) bytes of sign bits}.  Lossless, so the  */
                   /* results equal the dense representation's                                    */
};

/* The tensors CausalSelfAttention holds for the tail of its forward pass
 * (src/models/llama/attention.rs:38-40, loaded at :147-163): the o_proj TernaryLinear in its
 * dense (src/bit1_58/layers.rs:34-41: packed rows + per-row scales) or sparse (XN_SPARSE: the blob of
 * SparseTernary) representation and the optional inner_attn_ln / attn_sub_norm FastRmsNorm
 * (src/nn/fast_rmsnorm.rs:5-17). */
typedef struct xn_out_proj_desc {
    int32_t layer;
    int32_t in_dim;           /* must equal num_heads * head_dim                                  */
    int32_t out_dim;
    int32_t pack_type;        /* XN_PACK4 or XN_PACK5                                             */
    const uint8_t* packed;    /* host: out_dim rows of ceil(in_dim/4) or ceil(in_dim/5) bytes, or */
                              /*       the XorSparse blob of out_dim rows                         */
    const float* w_scales;    /* host: [out_dim]                                                  */
    const float* norm_weight; /* host: [in_dim], or NULL when the model has no sub-norm           */
    float norm_eps;
    uint32_t reserved;
} xn_out_proj_desc;

/* The q_proj / k_proj / v_proj TernaryLinears of one layer (src/models/llama/attention.rs:34-36),
 * dense representation, all with in_dim = hidden size; out dims are num_heads * head_dim for q and
 * num_kv_heads * head_dim for k and v. */
typedef struct xn_qkv_proj_desc {
    int32_t layer;
    int32_t in_dim;
    int32_t pack_type;        /* XN_PACK4, XN_PACK5 or XN_SPARSE, the same for the three          */
    int32_t reserved;
    const uint8_t* q_packed;
    const float* q_scales;
    const uint8_t* k_packed;
    const float* k_scales;
    const uint8_t* v_packed;
    const float* v_scales;
} xn_qkv_proj_desc;

/* Uploads (or replaces) the q/k/v projections of one layer.  Requests of that layer may then
 * carry XN_REQ_QKV_PROJ: the rows of x are quantised to i8 once (quantize_f32_to_i8,
 * src/bit1_58/quantization.rs:95-187, AVX-512 body) and projected by all three
 * (TernaryLinear::forward / fused_forward_qkv, src/bit1_58/layers.rs:262-424); given the same x
 * the projected q, k, v equal the reference's bit for bit, and so do the cached K and V. */
XN_API int32_t xn_qkv_proj_set(xn_ctx* ctx, const xn_qkv_proj_desc* desc);

/* Uploads (or replaces) the output block of one layer.  Requests of that layer may then carry
 * XN_REQ_OUT_PROJ. */
XN_API int32_t xn_out_proj_set(xn_ctx* ctx, const xn_out_proj_desc* desc);

/* The output block on its own: y is [rows, in_dim] (the sequence-major attention output), out is
 * [rows, out_dim] = o_proj(sub_norm(y)): FastRmsNorm::forward (src/nn/fast_rmsnorm.rs:15-17,
 * src/tensor.rs:242-265) then TernaryLinear::forward (src/bit1_58/layers.rs:262-313).  flags: 0 for
 * host pointers (blocks), XN_REQ_DEVICE_PTRS for device pointers (enqueues).  Given the same y the
 * result equals the reference's AVX-512 build bit for bit (integer dot products; the float steps
 * keep its order of operations). */
XN_API int32_t xn_out_proj(xn_ctx* ctx, int32_t layer, int32_t rows, const float* y, float* out,
                           uint32_t flags);

/* TernaryLinear::new with the dense representation (src/bit1_58/layers.rs:91-149), on the host:
 * ternarises and packs `weights` [out_dim, in_dim].  provided_scale: NaN for None.  packed must
 * hold out_dim * ceil(in_dim / pack) bytes, w_scales out_dim floats.  No GPU needed. */
XN_API int32_t xn_ternary_pack(int32_t in_dim, int32_t out_dim, const float* weights,
                               int32_t pack_type, float provided_scale, uint8_t* packed,
                               float* w_scales);

/* TernaryLinear::new_sparse (src/bit1_58/layers.rs:151-181), on the host: ternarises `weights`
 * [out_dim, in_dim] like xn_ternary_pack and encodes the rows as an XorSparse blob.  blob_cap is the
 * capacity of `blob` (out_dim * (4 + ceil(in_dim/64) * 16) bytes always suffice); *blob_len
 * receives the bytes written.  Returns XN_ERR_CAPACITY when the blob does not fit.  No GPU needed. */
XN_API int32_t xn_ternary_pack_sparse(int32_t in_dim, int32_t out_dim, const float* weights,
                                      float provided_scale, uint8_t* blob, int64_t blob_cap,
                                      int64_t* blob_len, float* w_scales);

/* ---- host-side planning, exposed for tests (no GPU needed) ----------------------------------- */

/* Splits `n_units` attention units of kv_len[i] cached tokens into tiles of `tile_tokens` and
 * deals the tiles evenly to at most `max_ctas` thread blocks, the way the split-KV kernel is
 * launched.  Outputs (capacity `max_items` items): item_unit, item_tile_begin, item_tile_end,
 * item_part (-1 when the unit is covered by one block and written directly), and
 * cta_item_begin[ctas+1].  Returns the number of thread blocks, or a negative xn_status. */
XN_API int32_t xn_plan_split(int32_t n_units, const int32_t* kv_len, int32_t tile_tokens,
                             int32_t max_ctas, int32_t max_items, int32_t* item_unit,
                             int32_t* item_tile_begin, int32_t* item_tile_end, int32_t* item_part,
                             int32_t* cta_item_begin, int32_t* n_items_out, int32_t* n_parts_out);

/* Diagnostic for the error path of the kernels' bounded waits: launches a one-thread kernel
 * that waits, for at most timeout_ms (1..1000), on a barrier nothing will complete, then
 * synchronises.  Returns XN_ERR_DEVICE_WAIT (the expected outcome); the context stays usable. */
XN_API int32_t xn_debug_expire_wait(xn_ctx* ctx, int32_t timeout_ms);

/* Memory-safety check that needs no external tool: every device buffer of a context (page pools,
 * split-KV partials, rotation scratch, projection rows, staging, plan slots ...) is allocated between
 * two 256-byte guard areas filled with a known pattern.  This call waits for the context's stream,
 * reads the guard areas back and returns XN_ERR_GUARD (the text names the buffer and the side) when
 * any byte changed, XN_OK otherwise.  The test-suite calls it before it destroys a context. */
XN_API int32_t xn_debug_check_guards(xn_ctx* ctx);

/* Forgets the plan the context keeps on the device for reuse by the next decode submission of the
 * same geometry (xn_stats.plan_reuses).  In real decoding the first layer of every step plans afresh
 * because the position moved on; a benchmark that re-submits the SAME positions step after step
 * calls this once per step so that it measures that, and not thirty reuses out of thirty. */
XN_API int32_t xn_debug_drop_plan(xn_ctx* ctx);

/* Library build identification: "xn_attn <version> sm_100a". */
XN_API const char* xn_version(void);

#ifdef __cplusplus
}
#endif
#endif /* XN_ATTN_H */
