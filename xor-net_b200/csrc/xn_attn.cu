// C ABI, context, page allocator, batch planner and launch logic of the sm_100a attention
// library.  Declarations and the reference interfaces they replace: include/xn_attn.h.
#include "../../include/xn_attn.h"

#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <thread>
#include <mutex>
#include <string>
#include <unordered_set>
#include <vector>

#include "xn_append.cuh"
#include "xn_common.cuh"
#include "xn_decode.cuh"
#include "xn_kv_u8.cuh"
#include "xn_kv_u8_mma.cuh"
#include "xn_outproj.cuh"
#include "xn_outproj_tc.cuh"
#include "xn_plan.hpp"
#include "xn_prefill_f32.cuh"
#include "xn_prefill_tf32.cuh"
#include "xn_static_decode.cuh"
#include "xn_ternary.hpp"

using namespace xn;

namespace {

constexpr uint32_t kCtxMagic = 0x786e4354u;     // "xnCT"
constexpr uint32_t kStreamMagic = 0x786e5354u;  // "xnST"
constexpr int kPlanSlots = 4;
constexpr long long kMaxUnits = 1ll << 22;

std::mutex g_err_mu;
std::string g_create_error;

struct PlanSlot {
    unsigned char* host = nullptr;
    unsigned char* dev = nullptr;
    size_t cap = 0;
    cudaEvent_t ev = nullptr;     // recorded after the last launch that reads the slot
    cudaEvent_t up_ev = nullptr;  // recorded after the plan upload on the copy stream
    bool used = false;
};

// The plan of the last pure-decode submission, kept on the device.  The layers of one decode step
// submit the same streams at the same positions one after another; only the tensors' addresses
// and the layer differ, and those travel as a kernel parameter (ReqPatchTable).  A submission
// that matches therefore skips planning and the plan upload altogether.
struct PlanCache {
    struct Entry {
        xn_stream* stream;
        int64_t index_pos;
        uint32_t flags;
        int n_pages;
    };
    bool valid = false;
    bool host_mode = false, pinned = false;
    PlanSlot* slot = nullptr;
    std::vector<Entry> ent;
    size_t o_req = 0, o_unit = 0, o_item = 0, o_cta = 0, o_page = 0;
    int ctas = 0;
    uint64_t h2d_bytes = 0, d2h_bytes = 0;   // what the kernel moves over PCIe itself (page-locked callers)
    bool out_dma = false;                    // outputs staged on the device, one copy to the host behind the kernel
    size_t out_bytes = 0;                    // of all requests together
    ReqPatchTable table;
};

// Output block of one layer on the device (xn_out_proj_set).
struct OutProj {
    bool set = false;
    int in_dim = 0, out_dim = 0;
    int q_stride = 0;  // bytes per quantised activation row (in_dim rounded up to 128)
    int w_stride = 0;  // bytes per 2-bit weight row (q_stride / 4)
    uint8_t* w2 = nullptr;
    float* w_scales = nullptr;
    float* norm_w = nullptr;  // nullptr: no sub-norm
    float eps = 0.f;
};

// A run of consecutive token rows that go through the same layer's output block.
struct OutRun {
    int layer;
    int row_begin, row_count;  // rows of the submission's row table
    size_t q_row0;             // first row in the quantised-activation buffer (multiple of 256)
};

// One blocking caller of xn_attention waiting in the context's queue.  Every caller sleeps on its
// own condition variable: waking sixty-four slot threads one by one costs less than letting them
// all fight for one lock.
// Page-locked rows that collect the outputs of one merged group of blocking callers back to back,
// so that they leave the device in one transfer; every caller then copies its own row out.  Two of
// them alternate: a slab is handed to a new group only after the last caller of the group that
// used it before has taken its row.
struct OutSlab {
    unsigned char* host = nullptr;
    size_t cap = 0;
    std::atomic<int> readers{0};
};

struct Pending {
    OutSlab* slab = nullptr;     // set when `req.out` points into a slab: decrement `readers` when done
    xn_req req;
    int32_t status = XN_OK;
    bool done = false;      // served: status is final          (guarded by the context's q_mu)
    bool promoted = false;  // not served yet, but now the leader (guarded by the context's q_mu)
    std::condition_variable cv;
    float* user_out = nullptr;   // where the caller wants the output when the request was re-pointed
    size_t out_bytes = 0;        // at the stream's page-locked call buffer
};

}  // namespace

struct xn_stream {
    uint32_t magic = kStreamMagic;
    xn_ctx* ctx = nullptr;
    int64_t cap = 0;
    std::vector<int32_t> pages;   // page id of slots [64*i, 64*i+64)
    std::vector<int64_t> hw;      // per layer: highest written position + 1
    int64_t expected = 0;         // tokens the creator said the stream will hold (placement only)
    // Page-locked, device-mapped buffer for the tensors of one blocking single-token call
    // [q | k | v | out]: the caller copies its pageable tensors in and out itself, in parallel
    // with the other callers, and the kernels read and write the buffer over PCIe directly.
    unsigned char* call_buf = nullptr;
    size_t call_cap = 0;
};

// One context per GPU of a box behind one handle; streams are placed on the least-loaded one.
struct xn_group {
    uint32_t magic = 0x786e4752u;  // "xnGR"
    std::vector<xn_ctx*> ctxs;
    std::mutex mu;
    uint64_t ticket = 0;           // streams created so far
};

struct xn_ctx {
    uint32_t magic = kCtxMagic;
    int device = 0, num_layers = 0, num_heads = 0, num_kv_heads = 0, head_dim = 0;
    int group = 1, gt = 1, subs = 1;  // query heads per KV head; heads per unit; units per KV head
    int nv = 0;                       // float4 per cached row (row length padded to 4 floats)
    int nv_class = 0;                 // template NV of the kernel instantiation
    bool nv_exact = false;
    int tile_tokens = 64;
    float scale = 1.f;
    long long pool_pages = 0;
    int max_pos = 0;
    int prefill_mode = 0;
    int batch_window_us = 0;
    int auto_window_us = 0;     // >0: a leader waits this long for the previous group's callers to return
    int sm_count = 0;
    int decode_ctas = 0;     // thread blocks of the split-KV launch (one per SM)
    int decode_chunks = 0;   // chunks the tile list is cut into (several per block)
    bool fuse_append = true; // decode batches: the attention kernel appends the new token itself
    bool fuse_pinned = true; // ... also when q,k,v live in page-locked host memory
    bool plan_reuse = true;  // a decode submission of the previous one's geometry reuses its plan
    bool pf_rope_q = true;   // the tensor-core prefill kernel rotates the query rows itself
    bool pf_multi = true;    // several tensor-core prefills of one submission share one launch
    PlanCache pcache;
    size_t stage_direct_bytes = size_t(2) << 20;  // small staged calls: kernels use the pinned staging itself
    bool out_tc = true;      // output projection on the tensor cores (else the dp4a kernel)
    bool out_pdl = true;     // ... launched as a programmatic dependent of the quantiser kernel
    bool out_rows_kernel = true;  // ... and, for more than 128 rows, the many-row variant
    bool pf_pdl = true;      // tensor-core prefill launched as a programmatic dependent of the append
    bool f32_tiled = true;   // exact-f32 prefills of f32_tiled_min_rows rows or more: the tiled kernel
    int f32_tiled_min_rows = 32;   // (shorter ones are served row by row by the split-KV kernel)
    int* sync_d = nullptr;   // chunk counter, done counter, per-unit arrival counters
    size_t sync_cap = 0;     // ints
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    cudaStream_t copy_stream = nullptr;  // plan uploads run here, off the launch stream's critical path
    float* k_pool = nullptr;
    float* v_pool = nullptr;
    // u8 cache format: one pool of K bytes | V bytes | scales blocks instead of the two f32 pools
    bool kv_u8 = false;
    int dq = 0;                  // bytes per stored row
    int kv8_epl = 16;            // bytes of a row one lane of the attention kernel handles
    bool kv8_mma = true;         // q.k of the u8 attention kernel on the integer tensor-core path ...
    long long kv8_mma_min_rows = 1 << 19;  // ... for submissions that attend at least this many cached rows.
                                 // (Smaller ones are latency bound and the kernel that also appends wins:
                                 // measured on the config-3 shape, 1.75 against 1.80 ms per 30-layer step at
                                 // 32 streams = 315 k rows, 2.64 against 2.42 at 64 streams = 676 k rows.)
    uint8_t* pool8 = nullptr;
    // ... and the f32 staging area the tensor-core prefill kernel reads in that format: the pages of
    // one stream and layer, dequantised, addressed through an identity page table
    float* k_stage = nullptr;
    float* v_stage = nullptr;
    long long stage_pages = 0;
    int* stage_ident_d = nullptr;
    CUtensorMap k_stage_map, v_stage_map;
    float* cos_d = nullptr;
    float* sin_d = nullptr;
    std::vector<int32_t> free_pages;  // stack: back() is handed out next
    std::unordered_set<xn_stream*> streams;

    std::mutex mu;  // serialises submissions and every mutation below
    PlanSlot slots[kPlanSlots];
    int next_slot = 0;
    float* q_rot = nullptr;    size_t q_rot_cap = 0;      // floats
    // Outputs of page-locked callers whose `out` tensors lie back to back in host memory are
    // produced here and leave with ONE copy-engine transfer: stores of the SMs into host memory
    // cross PCIe at about a third of that rate.
    float* out_stage = nullptr; size_t out_stage_cap = 0; // floats
    bool pinned_out_dma = true;
    size_t out_dma_min_bytes = 128 << 10;   // below this the kernels' own stores are quicker than a transfer
    OutSlab slabs[2];
    int slab_next = 0;
    // Merged groups of blocking callers are enqueued under the context's lock and waited for
    // outside it (one event each), so that the next group's kernels queue up behind them.
    bool defer_groups = true;
    std::vector<cudaEvent_t> done_events;   // idle events
    float* partials = nullptr; size_t partials_cap = 0;   // floats
    // attention output block (sub-norm + ternary o_proj)
    std::vector<OutProj> out_proj;                         // per layer
    std::vector<OutProj> qkv_proj;                         // per layer: q, k, v rows stacked, no norm
    float* qkv_seq = nullptr; size_t qkv_seq_cap = 0;      // floats: projected [row][q | k | v]
    float* attn_seq = nullptr; size_t attn_seq_cap = 0;    // floats: sequence-major attention rows
    float* q8 = nullptr; size_t q8_cap = 0;                // floats: i8 activation rows + inverse scales
    unsigned char* io_host = nullptr; unsigned char* io_dev = nullptr; size_t io_cap = 0;
    // Error word of the kernels' bounded waits: page-locked host memory that the kernels write
    // directly (they only ever write it when a wait ran out), so reading it needs no copy.
    int* status_d = nullptr;  // device-side address of the same word
    int* status_h = nullptr;
    // every device buffer of the context sits between two 256-byte guard areas (see guarded_malloc)
    struct GuardRec {
        unsigned char* user;
        size_t bytes;       // rounded up to 256
        const char* name;
    };
    std::vector<GuardRec> guards;
    xn_stats stats{};
    std::mutex err_mu;       // guards last_error only: readers never wait for a submission
    std::string last_error;

    // tensor-core prefill (tcgen05 TF32): tensor maps over the K and V pools
    bool tf32_ok = false;
    int tf32_min_rows = 128;
    CUtensorMap k_map, v_map;

    // optional device timing of the split-KV kernel
    bool profile = false;
    std::vector<cudaEvent_t> prof_events;  // pairs (start, stop), reused
    std::vector<int> prof_kind;            // per pair: 0 split-KV, 1 prefill, 2 output block, 3 q/k/v block
    size_t prof_used = 0;

    // combining of concurrent blocking callers
    std::mutex q_mu;
    std::condition_variable q_cv;
    std::vector<Pending*> queue;
    bool leader_active = false;
    size_t last_group = 1;          // callers merged into the previous submission
    bool leader_in_window = false;  // the leader is waiting for company: arrivals tell it
    // Groups whose kernels are enqueued but not finished (guarded by q_mu).  A leader that is
    // promoted while one is in flight enqueues behind it only once its own group is as large as
    // the one its callers formed last time (groups alternate: the size two groups back);
    // otherwise it keeps collecting until the GPU is idle.  At most two groups are in flight.
    int in_flight = 0;
    size_t group_before_last = 1;
    std::condition_variable flight_cv;
};

namespace {

int32_t fail(xn_ctx* ctx, int32_t code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx) {
        std::lock_guard<std::mutex> g(ctx->err_mu);
        ctx->last_error = buf;
    } else {
        std::lock_guard<std::mutex> g(g_err_mu);
        g_create_error = buf;
    }
    return code;
}

#define XN_CUDA(ctx, expr)                                                                    \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess)                                                               \
            return fail(ctx, XN_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));   \
    } while (0)

bool ctx_ok(const xn_ctx* c) { return c && c->magic == kCtxMagic; }
bool stream_ok(const xn_ctx* c, const xn_stream* s) {
    return s && s->magic == kStreamMagic && s->ctx == c;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---- guarded device allocations -----------------------------------------------------------
// compute-sanitizer is not always available where this library runs, and the kernels do raw
// pointer arithmetic from host-built descriptors.  Every device buffer of a context is therefore
// allocated with 256 bytes of a known pattern before and behind it; xn_debug_check_guards reads
// the patterns back and names the buffer whose neighbourhood was written.
constexpr size_t kGuardBytes = 256;
constexpr int kGuardByte = 0xA5;

cudaError_t guarded_malloc(xn_ctx* c, void** out, size_t bytes, const char* name) {
    *out = nullptr;
    const size_t body = align_up(std::max<size_t>(bytes, 1), kGuardBytes);
    unsigned char* base = nullptr;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&base), body + 2 * kGuardBytes);
    if (e != cudaSuccess) return e;
    e = cudaMemset(base, kGuardByte, kGuardBytes);
    if (e == cudaSuccess) e = cudaMemset(base + kGuardBytes + body, kGuardByte, kGuardBytes);
    if (e != cudaSuccess) {
        cudaFree(base);
        return e;
    }
    c->guards.push_back({base + kGuardBytes, body, name});
    *out = base + kGuardBytes;
    return cudaSuccess;
}

cudaError_t guarded_free(xn_ctx* c, void* user) {
    if (!user) return cudaSuccess;
    for (size_t i = 0; i < c->guards.size(); ++i)
        if (c->guards[i].user == user) {
            c->guards.erase(c->guards.begin() + long(i));
            return cudaFree(static_cast<unsigned char*>(user) - kGuardBytes);
        }
    return cudaFree(user);   // not one of ours (never happens): free it as it is
}

// ---- kernel dispatch table ---------------------------------------------------------------

using SplitFn = void (*)(const ReqDev*, const UnitDev*, const ItemDev*, const int*, int, const int*,
                         const float*, const float*, float*, int*, long long, int, int, int, float,
                         const float*, const float*, int*, const ReqPatchTable);

struct SplitKernel {
    SplitFn fn;
    size_t smem;
    int threads;
    int tile_tokens;
};

template <int NV, int GT, bool EXACT>
SplitKernel make_split() {
    return {attn_splitkv_kernel<NV, GT, EXACT>, DecodeSmem<NV, GT>::kBytes, DecodeCfg<NV>::kThreads,
            DecodeCfg<NV>::kTPS};
}

template <int NV, bool EXACT>
SplitKernel pick_gt(int gt) {
    if (gt == 4) return make_split<NV, 4, EXACT>();
    if (gt == 2) return make_split<NV, 2, EXACT>();
    return make_split<NV, 1, EXACT>();
}

// Exact instantiations exist for the row lengths of head_dim 64, 100, 128 and 256.
SplitKernel pick_split(int nv_class, int gt, bool exact) {
    switch (nv_class) {
        case 8: return pick_gt<8, false>(gt);
        case 16: return exact ? pick_gt<16, true>(gt) : pick_gt<16, false>(gt);
        case 25: return pick_gt<25, true>(gt);
        case 32: return exact ? pick_gt<32, true>(gt) : pick_gt<32, false>(gt);
        default: return exact ? pick_gt<64, true>(gt) : pick_gt<64, false>(gt);
    }
}

using Split8Fn = void (*)(const ReqDev*, const UnitDev*, const ItemDev*, const int*, int, const int*,
                          const uint8_t*, float*, int*, long long, int, int, float, const float*,
                          const float*, int*);

template <int DQ, int EPL>
Split8Fn pick8_gt(int gt) {
    if (gt == 4) return kv8::attn_splitkv_u8_kernel<DQ / EPL, 4, EPL>;
    if (gt == 2) return kv8::attn_splitkv_u8_kernel<DQ / EPL, 2, EPL>;
    return kv8::attn_splitkv_u8_kernel<DQ / EPL, 1, EPL>;
}

template <int EPL>
Split8Fn pick8_dq(int dq, int gt) {
    switch (dq) {
        case 16: return pick8_gt<16, EPL>(gt);
        case 32: return pick8_gt<32, EPL>(gt);
        case 64: return pick8_gt<64, EPL>(gt);
        case 128: return pick8_gt<128, EPL>(gt);
        default: return pick8_gt<256, EPL>(gt);
    }
}

// epl: bytes of a row per lane.  Only 16 is built: with 8 a lane needs half the registers and
// twice the warps fit, but every key then costs 1.5x the instructions (the per-key bookkeeping is
// spread over half as many elements) and the config-3 batch ran at 134 us per launch against 104.
Split8Fn pick_split8(int dq, int gt, int epl) {
    (void)epl;
    return pick8_dq<16>(dq, gt);
}

// the variant with q.k on the integer tensor-core path: row widths 64 and 128 only
Split8Fn pick_split8_mma(int dq, int gt) {
    if (dq == 128)
        return gt == 4 ? kv8m::attn_splitkv_u8_mma_kernel<8, 4>
                       : (gt == 2 ? kv8m::attn_splitkv_u8_mma_kernel<8, 2> : kv8m::attn_splitkv_u8_mma_kernel<8, 1>);
    return gt == 4 ? kv8m::attn_splitkv_u8_mma_kernel<4, 4>
                   : (gt == 2 ? kv8m::attn_splitkv_u8_mma_kernel<4, 2> : kv8m::attn_splitkv_u8_mma_kernel<4, 1>);
}

int nv_class_for(int nv) {
    if (nv == 25) return 25;
    if (nv <= 8) return 8;
    if (nv <= 16) return 16;
    if (nv <= 32) return 32;
    return 64;
}

// ---- tiled exact-f32 prefill: instantiation by row length ------------------------------------

using PrefillF32Fn = void (*)(const ReqDev*, const F32Item*, const int*, const float*, const float*, long long,
                              int, int, int, int, float, int*);
struct PrefillF32Kernel {
    PrefillF32Fn fn;
    size_t smem;      // dynamic shared memory of a launch for this row length
    size_t smem_max;  // ... for the longest rows the instantiation serves: the per-function limit is
                      // shared by all contexts of the process, whatever their head_dim
};
PrefillF32Kernel pick_prefill_f32(int nv) {
    const int dp = nv * 4;
    if (dp <= 64) return {prefill_f32_kernel<64, 1>, pf32::smem_bytes(dp, 64), pf32::smem_bytes(64, 64)};
    if (dp <= 128) return {prefill_f32_kernel<64, 2>, pf32::smem_bytes(dp, 64), pf32::smem_bytes(128, 64)};
    return {prefill_f32_kernel<32, 4>, pf32::smem_bytes(dp, 32), pf32::smem_bytes(256, 32)};
}

// ---- TMA tensor maps (driver entry point resolved at run time; libcuda is not linked) -------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// f32 tensor of `rank` dims (dims[0] innermost, contiguous), byte strides for dims 1..rank-1,
// box of box[] elements, the given 128-byte swizzle flavour, zero fill outside the tensor.
bool make_map(CUtensorMap* map, CUtensorMapDataType type, const void* base, int rank,
              const cuuint64_t* dims, const cuuint64_t* strides_bytes, const cuuint32_t* box,
              CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return fn(map, type, cuuint32_t(rank), const_cast<void*>(base), dims, strides_bytes, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_map_f32(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims,
                  const cuuint64_t* strides_bytes, const cuuint32_t* box,
                  CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    return make_map(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rank, dims, strides_bytes, box, swizzle);
}

// ---- buffers -----------------------------------------------------------------------------

int32_t grow_device(xn_ctx* c, float** buf, size_t* cap, size_t need_floats) {
    if (need_floats <= *cap) return XN_OK;
    XN_CUDA(c, cudaStreamSynchronize(c->stream));  // nothing in flight may still use the old one
    if (*buf) XN_CUDA(c, guarded_free(c, *buf));
    *buf = nullptr;
    *cap = 0;
    size_t want = std::max(need_floats, size_t(1) << 18);
    want = align_up(want + want / 4, 1024);
    XN_CUDA(c, guarded_malloc(c, reinterpret_cast<void**>(buf), want * sizeof(float), "workspace"));
    *cap = want;
    return XN_OK;
}

int32_t grow_io(xn_ctx* c, size_t need_bytes) {
    if (need_bytes <= c->io_cap) return XN_OK;
    XN_CUDA(c, cudaStreamSynchronize(c->stream));
    if (c->io_host) XN_CUDA(c, cudaFreeHost(c->io_host));
    if (c->io_dev) XN_CUDA(c, guarded_free(c, c->io_dev));
    c->io_host = c->io_dev = nullptr;
    c->io_cap = 0;
    size_t want = align_up(std::max(need_bytes + need_bytes / 4, size_t(1) << 20), 4096);
    XN_CUDA(c, cudaMallocHost(reinterpret_cast<void**>(&c->io_host), want));
    XN_CUDA(c, guarded_malloc(c, reinterpret_cast<void**>(&c->io_dev), want, "staging"));
    c->io_cap = want;
    return XN_OK;
}

int32_t acquire_slot(xn_ctx* c, size_t need_bytes, PlanSlot** out) {
    // the slot whose plan is kept for reuse stays out of the rotation while that plan is valid
    if (c->pcache.valid && c->pcache.slot == &c->slots[c->next_slot]) c->next_slot = (c->next_slot + 1) % kPlanSlots;
    PlanSlot& s = c->slots[c->next_slot];
    c->next_slot = (c->next_slot + 1) % kPlanSlots;
    if (s.used) XN_CUDA(c, cudaEventSynchronize(s.ev));
    s.used = false;
    if (need_bytes > s.cap) {
        if (s.host) XN_CUDA(c, cudaFreeHost(s.host));
        if (s.dev) XN_CUDA(c, guarded_free(c, s.dev));
        s.host = s.dev = nullptr;
        s.cap = 0;
        size_t want = align_up(std::max(need_bytes * 2, size_t(1) << 16), 4096);
        XN_CUDA(c, cudaMallocHost(reinterpret_cast<void**>(&s.host), want));
        XN_CUDA(c, guarded_malloc(c, reinterpret_cast<void**>(&s.dev), want, "plan"));
        s.cap = want;
    }
    if (!s.ev) XN_CUDA(c, cudaEventCreateWithFlags(&s.ev, cudaEventDisableTiming));
    if (!s.up_ev) XN_CUDA(c, cudaEventCreateWithFlags(&s.up_ev, cudaEventDisableTiming));
    *out = &s;
    return XN_OK;
}

int32_t ensure_pages(xn_ctx* c, xn_stream* s, int64_t slots_needed) {
    const int64_t need = (slots_needed + kPageTokens - 1) / kPageTokens;
    while (int64_t(s->pages.size()) < need) {
        if (c->free_pages.empty())
            return fail(c, XN_ERR_OUT_OF_PAGES, "page pool exhausted (%lld pages, all in use)",
                        c->pool_pages);
        s->pages.push_back(c->free_pages.back());
        c->free_pages.pop_back();
    }
    return XN_OK;
}

void free_call_buffer(xn_stream* s) {
    if (s->call_buf) cudaFreeHost(s->call_buf);
    s->call_buf = nullptr;
    s->call_cap = 0;
}

void release_pages(xn_ctx* c, xn_stream* s) {
    c->pcache.valid = false;   // the kept plan may name this stream's pages
    for (auto it = s->pages.rbegin(); it != s->pages.rend(); ++it) c->free_pages.push_back(*it);
    s->pages.clear();
    std::fill(s->hw.begin(), s->hw.end(), 0);
}

int32_t check_device_status(xn_ctx* c) {
    if (*c->status_h != kDevOk) {
        int code = *c->status_h;
        *c->status_h = kDevOk;
        c->stats.device_wait_errors += 1;
        // a kernel that gave up may have left its arrival counters half-way
        cudaMemsetAsync(c->sync_d, 0, c->sync_cap * sizeof(int), c->stream);
        return fail(c, XN_ERR_DEVICE_WAIT, "a kernel gave up on a bounded wait (code %d)", code);
    }
    return XN_OK;
}

int32_t profile_begin(xn_ctx* c, int kind) {
    if (c->prof_used + 2 > c->prof_events.size()) {
        cudaEvent_t a, b;
        XN_CUDA(c, cudaEventCreate(&a));
        XN_CUDA(c, cudaEventCreate(&b));
        c->prof_events.push_back(a);
        c->prof_events.push_back(b);
        c->prof_kind.push_back(kind);
    }
    c->prof_kind[c->prof_used / 2] = kind;
    XN_CUDA(c, cudaEventRecord(c->prof_events[c->prof_used], c->stream));
    return XN_OK;
}

int32_t profile_end(xn_ctx* c) {
    XN_CUDA(c, cudaEventRecord(c->prof_events[c->prof_used + 1], c->stream));
    c->prof_used += 2;
    return XN_OK;
}

// ---- attention output block ----------------------------------------------------------------

// Floats of the quantised-activation buffer for `rows_pad` rows (a multiple of 256): the tiled i8
// rows, then one inverse scale per row.
size_t q8_floats(size_t q_stride, size_t rows_pad) { return rows_pad * q_stride / 4 + rows_pad + 4; }

// Sub-norm, quantiser and ternary projection of `n_rows` token rows; rows_d[i] names the source
// row (in_dim floats) and the destination row (out_dim floats) of row i.  The rows occupy rows
// [q_row0, q_row0 + n_rows) of the context's quantised-activation buffer, which holds q_rows_pad
// rows (both multiples of 256).
int32_t launch_out_block(xn_ctx* c, const OutProj& op, const OutRowDev* rows_d, int n_rows, size_t q_row0,
                         size_t q_rows_pad) {
    int8_t* q = reinterpret_cast<int8_t*>(c->q8);
    float* inv = c->q8 + q_rows_pad * size_t(op.q_stride) / 4;
    {
        // a programmatic dependent of whatever kernel precedes it in the stream (the attention
        // kernel when the block runs behind one): its launch overlaps that kernel's tail
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(unsigned(n_rows));
        cfg.blockDim = dim3(256);
        cfg.dynamicSmemBytes = align_up(size_t(op.in_dim), 4) * 12;
        cfg.stream = c->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = c->out_pdl ? 1 : 0;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        XN_CUDA(c, cudaLaunchKernelEx(&cfg, subnorm_quant_kernel, rows_d, (const float*)op.norm_w, op.eps,
                                      op.in_dim, q, op.q_stride, (long long)q_row0, (long long)q_rows_pad,
                                      inv));
    }
    if (c->out_tc && op.q_stride / tg::kBK <= tg::max_nkb()) {
        // tensor cores: 128 token rows x 32 output rows per block, the block's weights resident
        TernaryGemmArgs ga;
        ga.q = q; ga.w2 = op.w2; ga.q_rows_pad = (long long)q_rows_pad; ga.q_row0 = (long long)q_row0;
        ga.w_scales = op.w_scales; ga.inv_scale = inv; ga.rows = rows_d;
        ga.n_rows = n_rows; ga.out_dim = op.out_dim; ga.k_bytes = op.q_stride;
        ga.status = c->status_d;
        // up to 128 rows: one 128 x 32 tile per block; more rows: blocks that keep 64 output rows'
        // weights resident and walk over the token tiles
        const int nkb = op.q_stride / tg::kBK;
        const bool many = c->out_rows_kernel && n_rows > tg::kTM && nkb <= tgr::max_nkb();
        dim3 grid(unsigned((op.out_dim + tg::kTN - 1) / tg::kTN), unsigned((n_rows + tg::kTM - 1) / tg::kTM));
        if (many) {
            const int o_tiles = (op.out_dim + tgr::kTN - 1) / tgr::kTN;
            const int n_tiles = (n_rows + tgr::kTM - 1) / tgr::kTM;
            grid = dim3(unsigned(o_tiles), unsigned(std::max(1, std::min(n_tiles, c->sm_count / std::max(1, o_tiles)))));
        }
        // programmatic dependent launch: the blocks may start while the quantiser kernel still
        // runs (it releases them at its start) and decode their weights in the meantime
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(many ? tgr::kThreads : tg::kThreads);
        cfg.dynamicSmemBytes = size_t(many ? tgr::smem_bytes(nkb) : tg::smem_bytes(nkb));
        cfg.stream = c->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = c->out_pdl ? 1 : 0;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (many) XN_CUDA(c, cudaLaunchKernelEx(&cfg, ternary_gemm_rows_kernel, ga));
        else XN_CUDA(c, cudaLaunchKernelEx(&cfg, ternary_gemm_tc_kernel, ga));
    } else {
        const int R = std::max(1, std::min(kOutMaxRowsPerCta, (op.out_dim + c->sm_count - 1) / c->sm_count));
        dim3 grid(unsigned((op.out_dim + R - 1) / R), unsigned((n_rows + kOutRowsTile - 1) / kOutRowsTile));
        ternary_gemm_kernel<<<grid, 256, kOutGemmSmem, c->stream>>>(
            q, op.q_stride, (long long)q_row0, (long long)q_rows_pad, inv, op.w2, op.w_scales, rows_d,
            n_rows, op.out_dim, R);
    }
    c->stats.kernel_launches += 2;
    c->stats.out_proj_rows += uint64_t(n_rows);
    XN_CUDA(c, cudaGetLastError());
    return XN_OK;
}

// u8 cache format: room for `pages` dequantised pages of one layer, with tensor maps over it.
int32_t ensure_stage(xn_ctx* c, long long pages) {
    if (pages <= c->stage_pages) return XN_OK;
    XN_CUDA(c, cudaStreamSynchronize(c->stream));  // nothing in flight may still use the old area
    guarded_free(c, c->k_stage);
    guarded_free(c, c->v_stage);
    guarded_free(c, c->stage_ident_d);
    const long long np = std::max<long long>({pages, 2 * c->stage_pages, 32});
    c->k_stage = c->v_stage = nullptr;
    c->stage_ident_d = nullptr;
    c->stage_pages = 0;
    const size_t rows = size_t(np) * c->num_kv_heads * kPageTokens;
    const size_t bytes = rows * size_t(c->head_dim) * 4;
    XN_CUDA(c, guarded_malloc(c, reinterpret_cast<void**>(&c->k_stage), bytes, "k_stage"));
    XN_CUDA(c, guarded_malloc(c, reinterpret_cast<void**>(&c->v_stage), bytes, "v_stage"));
    XN_CUDA(c, cudaMemset(c->k_stage, 0, bytes));
    XN_CUDA(c, cudaMemset(c->v_stage, 0, bytes));
    std::vector<int32_t> ident(size_t(np), 0);
    for (long long i = 0; i < np; ++i) ident[size_t(i)] = int32_t(i);
    XN_CUDA(c, guarded_malloc(c, reinterpret_cast<void**>(&c->stage_ident_d), size_t(np) * 4, "stage page table"));
    XN_CUDA(c, cudaMemcpy(c->stage_ident_d, ident.data(), size_t(np) * 4, cudaMemcpyHostToDevice));
    const cuuint64_t dims[2] = {cuuint64_t(c->head_dim), cuuint64_t(rows)};
    const cuuint64_t str[1] = {cuuint64_t(c->head_dim) * 4};
    const cuuint32_t box[2] = {32, cuuint32_t(pf::kPage)};
    if (rows >= (1ull << 31) || !make_map_f32(&c->k_stage_map, c->k_stage, 2, dims, str, box) ||
        !make_map_f32(&c->v_stage_map, c->v_stage, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))
        return fail(c, XN_ERR_CUDA, "tensor maps over the prefill staging area could not be encoded");
    c->stage_pages = np;
    return XN_OK;
}

// ---- one batched submission ----------------------------------------------------------------

struct GapFill {
    int req;
    int64_t slot0, n;
};

// Validates one request against the context; returns XN_OK or the error (text in last_error).
int32_t validate_req(xn_ctx* c, const xn_req& r) {
    if (!stream_ok(c, r.stream)) return fail(c, XN_ERR_HANDLE, "stream handle is not live");
    if (r.layer < 0 || r.layer >= c->num_layers)
        return fail(c, XN_ERR_ARG, "layer %d outside 0..%d", r.layer, c->num_layers - 1);
    if (r.seq_len < 0 || r.index_pos < 0) return fail(c, XN_ERR_ARG, "negative seq_len or index_pos");
    const bool qkv = r.flags & XN_REQ_QKV_PROJ;   // k and v are produced by the library then
    if (r.seq_len > 0 && (!r.q || !r.out || (!qkv && (!r.k || !r.v))))
        return fail(c, XN_ERR_ARG, "null tensor pointer");
    if (r.index_pos + r.seq_len > (int64_t(1) << 30))
        return fail(c, XN_ERR_CAPACITY, "position %lld too large", (long long)(r.index_pos + r.seq_len));
    if (qkv && !c->qkv_proj[size_t(r.layer)].set)
        return fail(c, XN_ERR_ARG, "XN_REQ_QKV_PROJ: layer %d has no q/k/v projections (xn_qkv_proj_set)", r.layer);
    if ((r.flags & XN_REQ_ROPE) || qkv) {
        if (!c->cos_d) return fail(c, XN_ERR_NO_TABLES, "context was created without RoPE tables");
        if (r.index_pos + r.seq_len > c->max_pos)
            return fail(c, XN_ERR_CAPACITY, "position %lld beyond the RoPE table (%d rows)",
                        (long long)(r.index_pos + r.seq_len), c->max_pos);
    }
    if ((r.flags & XN_REQ_OUT_PROJ) && !c->out_proj[size_t(r.layer)].set)
        return fail(c, XN_ERR_ARG, "XN_REQ_OUT_PROJ: layer %d has no output block (xn_out_proj_set)", r.layer);
    return XN_OK;
}

// Whether a request goes to the tcgen05 prefill kernel: mode, shape, and 16-byte aligned rows
// where the kernel touches the caller's memory itself (`direct`: device or page-locked host
// pointers; pageable host tensors pass through the library's own aligned staging).  Anything
// else is served by the exact-f32 path.
bool use_tf32(const xn_ctx* c, const xn_req& r, bool direct) {
    if (!c->tf32_ok || c->prefill_mode == XN_PREFILL_F32) return false;
    if (r.index_pos + r.seq_len > r.stream->cap) return false;
    if (direct) {
        // with XN_REQ_OUT_PROJ the kernel writes into the library's own (aligned) row buffer
        uintptr_t bits = (r.flags & XN_REQ_OUT_PROJ) ? 0 : reinterpret_cast<uintptr_t>(r.out);
        const bool q_scratch = (r.flags & (XN_REQ_ROPE | XN_REQ_HOST_PINNED | XN_REQ_QKV_PROJ)) != 0;  // q read from the rotation scratch
        if (!q_scratch) bits |= reinterpret_cast<uintptr_t>(r.q);
        if (bits & 15) return false;
    }
    return r.seq_len >= (c->prefill_mode == XN_PREFILL_TF32 ? 2 : c->tf32_min_rows);
}

// The tensor-core prefill kernel rotates the query rows itself (head_dim 64 / 128, rows it can read
// as float4 from device memory): the append kernel then handles K and V only and no rotated copy
// of q is written and read back.
bool rope_in_prefill(const xn_ctx* c, const xn_req& r, bool direct, bool pinned) {
    if (!c->pf_rope_q || c->kv_u8 || pinned) return false;
    const bool qkv = r.flags & XN_REQ_QKV_PROJ;
    if (!((r.flags & XN_REQ_ROPE) || qkv)) return false;
    if (c->head_dim != 64 && c->head_dim != 128) return false;
    if (direct && !qkv && (reinterpret_cast<uintptr_t>(r.q) & 15)) return false;
    return use_tf32(c, r, direct);
}

// What a submission changes in its streams before its first launch (pages taken from the pool,
// the per-layer high-water marks).  Unless commit() is called, the destructor puts every stream
// back as it was, so a submission that fails on the way to its launches leaves no position
// claimed that was never written.
struct StreamRollback {
    struct Entry {
        xn_stream* s;
        size_t n_pages;
        int layer;
        int64_t hw;
    };
    xn_ctx* c;
    std::vector<Entry> entries;
    bool committed = false;
    explicit StreamRollback(xn_ctx* ctx) : c(ctx) {}
    void note(xn_stream* s, int layer) { entries.push_back({s, s->pages.size(), layer, s->hw[size_t(layer)]}); }
    void commit() { committed = true; }
    ~StreamRollback() {
        if (committed) return;
        for (auto it = entries.rbegin(); it != entries.rend(); ++it) {
            xn_stream* s = it->s;
            while (s->pages.size() > it->n_pages) {
                c->free_pages.push_back(s->pages.back());
                s->pages.pop_back();
            }
            s->hw[size_t(it->layer)] = it->hw;
        }
    }
};

// Whether a request that the tensor-core kernel does not take goes to the tiled exact-f32 kernel
// (f32 cache format, no ring fold, enough rows to fill a tile usefully).
bool use_f32_tiled(const xn_ctx* c, const xn_req& r) {
    return c->f32_tiled && !c->kv_u8 && r.seq_len >= c->f32_tiled_min_rows &&
           r.index_pos + r.seq_len <= r.stream->cap;
}

// reqs[i] are valid, on distinct streams, all host-mode or all device-mode.
// Arguments of the tensor-core prefill kernel for one request of a submission.
PrefillArgs make_prefill_args(const xn_ctx* c, const ReqDev& d, const int* pages_d) {
    PrefillArgs pa;
    pa.q = d.q;
    pa.q_hs = d.q_hs;
    pa.q_ts = d.q_ts;
    pa.cos_t = c->cos_d;
    pa.sin_t = c->sin_d;
    pa.rope_q = (d.flags & 16u) ? 1 : 0;
    pa.pages = c->kv_u8 ? c->stage_ident_d : pages_d + d.page_off;
    pa.out = d.out;
    pa.o_hs = d.o_hs;
    pa.o_ts = d.o_ts;
    pa.layer_page_base = c->kv_u8 ? 0 : (long long)d.layer * c->pool_pages;
    pa.pool_pages = c->kv_u8 ? c->stage_pages : c->pool_pages;
    pa.num_kv_heads = c->num_kv_heads;
    pa.group = c->group;
    pa.seq_len = d.seq_len;
    pa.index_pos = d.index_pos;
    pa.head_dim = c->head_dim;
    pa.scale_log2 = c->scale * 1.4426950408889634f;
    pa.status = c->status_d;
    return pa;
}

// A decode submission with the geometry of the plan kept on the device: the same streams, in the
// same order, at the same positions, one token each, all on one layer (any layer), nothing to
// zero-fill.  Launches the attention kernel over the kept plan with this call's addresses and layer
// as a kernel parameter.  Returns false when the submission does not match (nothing was touched).
bool submit_reusing_plan(xn_ctx* c, int n, const xn_req* reqs, bool host_mode, int32_t* rc_out,
                         cudaEvent_t defer) {
    PlanCache& pc = c->pcache;
    if (!pc.valid || !c->plan_reuse || n != int(pc.ent.size()) || host_mode != pc.host_mode) return false;
    const bool pinned = host_mode && (reqs[0].flags & XN_REQ_HOST_PINNED);
    if (pinned != pc.pinned) return false;
    const int layer = reqs[0].layer;
    for (int i = 0; i < n; ++i) {
        const xn_req& r = reqs[i];
        const PlanCache::Entry& e = pc.ent[size_t(i)];
        if (r.stream != e.stream || r.seq_len != 1 || r.index_pos != e.index_pos || r.flags != e.flags ||
            r.layer != layer || int(r.stream->pages.size()) != e.n_pages ||
            r.index_pos > r.stream->hw[size_t(layer)])
            return false;
        if ((reinterpret_cast<uintptr_t>(r.q) | reinterpret_cast<uintptr_t>(r.k) |
             reinterpret_cast<uintptr_t>(r.v)) & 15)
            return false;
    }
    // outputs staged on the device (one copy home) only while they are still one run of host memory
    const size_t row_bytes = size_t(c->num_heads) * c->head_dim * 4;
    bool out_dma = pc.out_dma;
    for (int i = 1; i < n && out_dma; ++i)
        if (reinterpret_cast<unsigned char*>(reqs[i].out) != reinterpret_cast<unsigned char*>(reqs[0].out) + size_t(i) * row_bytes)
            out_dma = false;
    if (out_dma != pc.out_dma) return false;
    auto run = [&]() -> int32_t {
        ReqPatchTable& t = pc.table;
        t.n = n;
        t.layer = layer;
        for (int i = 0; i < n; ++i)
            t.e[i] = {reqs[i].q, reqs[i].k, reqs[i].v,
                      out_dma ? c->out_stage + size_t(i) * (row_bytes / 4) : reqs[i].out};
        const unsigned char* dev = pc.slot->dev;
        int32_t rc;
        SplitKernel k = pick_split(c->nv_class, c->gt, c->nv_exact);
        if (c->profile && (rc = profile_begin(c, 0)) != XN_OK) return rc;
        k.fn<<<std::min(pc.ctas, c->decode_ctas), k.threads, k.smem, c->stream>>>(
            reinterpret_cast<const ReqDev*>(dev + pc.o_req), reinterpret_cast<const UnitDev*>(dev + pc.o_unit),
            reinterpret_cast<const ItemDev*>(dev + pc.o_item), reinterpret_cast<const int*>(dev + pc.o_cta),
            pc.ctas, reinterpret_cast<const int*>(dev + pc.o_page), c->k_pool, c->v_pool, c->partials,
            c->sync_d, c->pool_pages, c->num_kv_heads, c->head_dim, c->nv, c->scale, c->cos_d, c->sin_d,
            c->status_d, t);
        t.n = 0;
        XN_CUDA(c, cudaGetLastError());
        if (c->profile && (rc = profile_end(c)) != XN_OK) return rc;
        if (out_dma) {
            XN_CUDA(c, cudaMemcpyAsync(reqs[0].out, c->out_stage, size_t(n) * row_bytes, cudaMemcpyDeviceToHost, c->stream));
            c->stats.out_transfers += 1;
        }
        for (int i = 0; i < n; ++i) {
            int64_t& hw = reqs[i].stream->hw[size_t(layer)];
            hw = std::max(hw, reqs[i].index_pos + 1);
        }
        XN_CUDA(c, cudaEventRecord(pc.slot->ev, c->stream));
        pc.slot->used = true;
        c->stats.kernel_launches += 1;
        c->stats.decode_launches += 1;
        c->stats.batches += 1;
        c->stats.calls += uint64_t(n);
        c->stats.plan_reuses += 1;
        c->stats.h2d_bytes += pc.h2d_bytes;
        c->stats.d2h_bytes += pc.d2h_bytes;
        if (host_mode && defer) {   // the caller waits for this event outside the context's lock
            XN_CUDA(c, cudaEventRecord(defer, c->stream));
        } else if (host_mode) {
            XN_CUDA(c, cudaStreamSynchronize(c->stream));
            if ((rc = check_device_status(c)) != XN_OK) return rc;
        }
        return XN_OK;
    };
    *rc_out = run();
    return true;
}

// defer: (page-locked host pointers only) do not wait for the GPU: record this event behind the
// submission's last operation and return; the caller synchronises on it without holding the
// context's lock, so that the next group of blocking callers can be enqueued meanwhile, and then
// reads the device status itself.
int32_t submit_locked(xn_ctx* c, int n, const xn_req* reqs, bool host_mode, cudaEvent_t defer = nullptr) {
    const int Hq = c->num_heads, Hkv = c->num_kv_heads, D = c->head_dim, nv = c->nv;
    XN_CUDA(c, cudaSetDevice(c->device));
    {
        int32_t rc;
        if (n > 0 && submit_reusing_plan(c, n, reqs, host_mode, &rc, defer)) return rc;
    }

    // host memory that is page-locked and device-mapped is read and written by the kernels directly
    const bool pinned = host_mode && (reqs[0].flags & XN_REQ_HOST_PINNED);
    const bool direct = !host_mode || pinned;
    // -- the whole batch must fit the page pool before any stream is touched
    {
        long long new_pages = 0;
        for (int i = 0; i < n; ++i) {
            const xn_req& r = reqs[i];
            if (r.seq_len == 0) continue;
            const int64_t slots = std::min<int64_t>(r.index_pos + r.seq_len, r.stream->cap);
            const int64_t need = (slots + kPageTokens - 1) / kPageTokens;
            new_pages += std::max<int64_t>(0, need - int64_t(r.stream->pages.size()));
        }
        if (new_pages > (long long)c->free_pages.size())
            return fail(c, XN_ERR_OUT_OF_PAGES,
                        "page pool exhausted: the batch needs %lld more pages, %zu of %lld are free",
                        new_pages, c->free_pages.size(), c->pool_pages);
    }
    // -- pages, gaps, staging sizes
    StreamRollback undo(c);   // until the launches are certain, every early return restores the streams
    std::vector<GapFill> gaps;
    size_t io_in = 0, io_out = 0, qrot_floats = 0, n_page_ids = 0, out_rows = 0, qkv_rows = 0;
    const size_t qkv_width = size_t(Hq + 2 * Hkv) * D;   // floats of one projected row [q | k | v]
    long long n_units = 0, n_ring_rows = 0, stage_need = 0, key_rows = 0;
    int max_rows = 0;
    for (int i = 0; i < n; ++i) {
        const xn_req& r = reqs[i];
        if (r.seq_len == 0) continue;
        xn_stream* s = r.stream;
        const int64_t end = r.index_pos + r.seq_len;
        undo.note(s, r.layer);
        int32_t rc = ensure_pages(c, s, std::min<int64_t>(end, s->cap));
        if (rc != XN_OK) return rc;
        int64_t& hw = s->hw[r.layer];
        if (r.index_pos > hw && hw < s->cap)
            gaps.push_back({i, hw, std::min<int64_t>(r.index_pos, s->cap) - hw});
        hw = std::max(hw, end);
        n_page_ids += s->pages.size();
        const size_t qf = size_t(Hq) * r.seq_len * D, kvf = size_t(Hkv) * r.seq_len * D;
        const bool proj = r.flags & XN_REQ_OUT_PROJ;
        const size_t of = proj ? size_t(r.seq_len) * c->out_proj[size_t(r.layer)].out_dim : qf;  // floats returned
        if (proj) out_rows += size_t(r.seq_len);
        const bool qkv = r.flags & XN_REQ_QKV_PROJ;
        const size_t xf = qkv ? size_t(r.seq_len) * c->qkv_proj[size_t(r.layer)].in_dim : 0;  // floats of x
        if (qkv) qkv_rows += size_t(r.seq_len);
        if (host_mode && !pinned) {
            io_in += qkv ? align_up(xf * 4, 16) : align_up(qf * 4, 16) + 2 * align_up(kvf * 4, 16);
            io_out += align_up(of * 4, 16);
        }
        if (((r.flags & XN_REQ_ROPE) || pinned || qkv) && !rope_in_prefill(c, r, direct, pinned))
            qrot_floats += align_up(qf, 4);
        if (end > s->cap) n_ring_rows += r.seq_len;
        else if (use_tf32(c, r, direct)) {   // served by the tensor-core prefill kernel
            stage_need = std::max<long long>(stage_need, (end + kPageTokens - 1) / kPageTokens);
        }
        else if (!use_f32_tiled(c, r)) {
            n_units += (long long)r.seq_len * Hkv * c->subs;
            key_rows += (long long)Hkv * c->subs *
                        ((long long)r.seq_len * r.index_pos + (long long)r.seq_len * (r.seq_len + 1) / 2);
        }
        // rows the append kernel moves for this request (the query rows stay where they are when
        // the prefill kernel rotates them itself)
        max_rows = std::max<long long>(max_rows, (long long)r.seq_len *
                                                     ((rope_in_prefill(c, r, direct, pinned) ? 0 : Hq) + 2 * Hkv));
        if (pinned) {  // bytes the kernels move over PCIe themselves
            c->stats.h2d_bytes += (qkv ? xf : qf + 2 * kvf) * 4;
            c->stats.d2h_bytes += of * 4;
        }
    }
    // Pure decode batches (one new token per request) let the attention kernel append, and rotate,
    // the new token itself: no separate append launch.  Needs rows the bulk copies can take
    // (head_dim % 4 == 0, 16-byte aligned pointers) and, for RoPE, the pair layout of head_dim
    // 64 / 128.
    // (u8 cache format: rows without padding, i.e. head_dim a power of two >= 16; the rotation needs
    // at least two lanes per row; plain loads, so no alignment condition.)
    const bool mma_now = c->kv_u8 && c->kv8_mma && key_rows >= c->kv8_mma_min_rows;
    bool fused = c->fuse_append && n_ring_rows == 0 && !mma_now &&
                 (c->kv_u8 ? D == c->dq : (D % 4 == 0 && c->nv_class <= 32));
    for (int i = 0; i < n && fused; ++i) {
        const xn_req& r = reqs[i];
        if (r.seq_len != 1) { fused = false; break; }
        const bool qkv = r.flags & XN_REQ_QKV_PROJ;   // q, k, v then live in the library's aligned rows
        if (((r.flags & XN_REQ_ROPE) || qkv) &&
            !(c->kv_u8 ? c->dq >= 32 : (c->nv_exact && (c->nv == 16 || c->nv == 32))))
            fused = false;
        // (u8 kernel: a lane reads its slice of q, k and v with plain 4-byte loads, which is slow
        // over PCIe; page-locked host rows go through the append kernel's coalesced copy instead)
        if (pinned && (c->kv_u8 || !c->fuse_pinned)) fused = false;
        if ((!host_mode || pinned) && !qkv && !c->kv_u8)
            if ((reinterpret_cast<uintptr_t>(r.q) | reinterpret_cast<uintptr_t>(r.k) |
                 reinterpret_cast<uintptr_t>(r.v)) & 15)
                fused = false;
    }
    if (fused) {
        qrot_floats = 0;
        max_rows = 0;
    }
    if (n_units > kMaxUnits)
        return fail(c, XN_ERR_CAPACITY, "%lld attention rows in one submission exceed the limit %lld",
                    n_units, kMaxUnits);

    // Page-locked callers whose outputs are one contiguous run of host memory (a batch tensor, a
    // prompt's output): the kernels write into a device buffer and one transfer carries it home.
    bool out_dma = pinned && c->pinned_out_dma;
    size_t out_dma_bytes = 0;
    float* out_dma_host = nullptr;
    if (out_dma) {
        for (int i = 0; i < n; ++i) {
            const xn_req& r = reqs[i];
            if (r.seq_len == 0) continue;
            const size_t of = (r.flags & XN_REQ_OUT_PROJ)
                                  ? size_t(r.seq_len) * c->out_proj[size_t(r.layer)].out_dim
                                  : size_t(Hq) * r.seq_len * D;
            if (!out_dma_host) out_dma_host = r.out;
            if (reinterpret_cast<unsigned char*>(r.out) != reinterpret_cast<unsigned char*>(out_dma_host) + out_dma_bytes ||
                (of & 3)) { out_dma = false; break; }
            out_dma_bytes += of * 4;
        }
        if (!out_dma_host || out_dma_bytes < c->out_dma_min_bytes) out_dma = false;
    }

    // Small staged calls skip the two DMA copies: the library's page-locked staging buffer is
    // device-accessible, so the kernels read the inputs from it and write the outputs into it
    // over PCIe themselves; what remains is one plan upload, the launches and the wait.
    const bool stage_direct = host_mode && !pinned && io_in + io_out <= c->stage_direct_bytes;
    int32_t rc;
    if (c->kv_u8 && stage_need && (rc = ensure_stage(c, stage_need)) != XN_OK) return rc;
    if ((rc = grow_device(c, &c->q_rot, &c->q_rot_cap, qrot_floats)) != XN_OK) return rc;
    if (out_rows) {
        if ((rc = grow_device(c, &c->attn_seq, &c->attn_seq_cap, out_rows * size_t(Hq) * D)) != XN_OK) return rc;
    }
    if (qkv_rows && (rc = grow_device(c, &c->qkv_seq, &c->qkv_seq_cap, qkv_rows * qkv_width)) != XN_OK) return rc;
    if (out_dma && (rc = grow_device(c, &c->out_stage, &c->out_stage_cap, out_dma_bytes / 4)) != XN_OK) return rc;
    if (host_mode && (rc = grow_io(c, io_in + io_out)) != XN_OK) return rc;
    // (inputs are read in place either way; outputs above the transfer threshold are produced on the
    // device and copied into the staging buffer: stores of the SMs into host memory are the slow part)
    unsigned char* const in_base = stage_direct ? c->io_host : c->io_dev;
    const bool out_direct = stage_direct && io_out < c->out_dma_min_bytes;
    unsigned char* const out_base = out_direct ? c->io_host : c->io_dev;

    // -- request descriptors, page ids, units
    std::vector<ReqDev> rd(n);
    std::vector<int32_t> page_ids;
    page_ids.reserve(n_page_ids);
    std::vector<UnitDev> units;
    units.reserve(size_t(n_units));
    std::vector<int32_t> kv_lens;
    kv_lens.reserve(size_t(n_units));
    std::vector<int32_t> ring_rows;
    std::vector<int> tf32_reqs;
    std::vector<F32Item> f32_items;
    std::vector<OutRowDev> out_row_tab;
    out_row_tab.reserve(out_rows);
    std::vector<OutRun> out_runs;
    std::vector<OutRowDev> qkv_row_tab;
    qkv_row_tab.reserve(qkv_rows);
    std::vector<OutRun> qkv_runs;
    size_t in_off = 0, out_off = io_in, qrot_off = 0;
    for (int i = 0; i < n; ++i) {
        const xn_req& r = reqs[i];
        ReqDev& d = rd[i];
        memset(&d, 0, sizeof d);
        if (r.seq_len == 0) continue;
        xn_stream* s = r.stream;
        const int S = r.seq_len;
        const size_t qf = size_t(Hq) * S * D, kvf = size_t(Hkv) * S * D;
        const float *q_dev = r.q, *k_dev = r.k, *v_dev = r.v;
        float* o_dev = r.out;
        if (out_dma) o_dev = c->out_stage + (reinterpret_cast<unsigned char*>(r.out) -
                                             reinterpret_cast<unsigned char*>(out_dma_host)) / 4;
        const bool qkv = r.flags & XN_REQ_QKV_PROJ;
        if (host_mode && !pinned) {
            if (qkv) {
                const size_t xf = size_t(S) * c->qkv_proj[size_t(r.layer)].in_dim;
                memcpy(c->io_host + in_off, r.q, xf * 4);
                q_dev = reinterpret_cast<const float*>(in_base + in_off);   // x, for now
                in_off += align_up(xf * 4, 16);
            } else {
                memcpy(c->io_host + in_off, r.q, qf * 4);
                q_dev = reinterpret_cast<const float*>(in_base + in_off);
                in_off += align_up(qf * 4, 16);
                memcpy(c->io_host + in_off, r.k, kvf * 4);
                k_dev = reinterpret_cast<const float*>(in_base + in_off);
                in_off += align_up(kvf * 4, 16);
                memcpy(c->io_host + in_off, r.v, kvf * 4);
                v_dev = reinterpret_cast<const float*>(in_base + in_off);
                in_off += align_up(kvf * 4, 16);
            }
            o_dev = reinterpret_cast<float*>(out_base + out_off);
            out_off += align_up(((r.flags & XN_REQ_OUT_PROJ)
                                     ? size_t(S) * c->out_proj[size_t(r.layer)].out_dim : qf) * 4, 16);
        }
        const bool seq_major = (r.flags & XN_REQ_SEQ_MAJOR) || qkv;
        const bool rope = (r.flags & XN_REQ_ROPE) || qkv;
        long long q_hs = seq_major ? D : (long long)S * D, q_ts = seq_major ? (long long)Hq * D : D;
        long long kv_hs = seq_major ? D : (long long)S * D, kv_ts = seq_major ? (long long)Hkv * D : D;
        const long long o_hs = q_hs, o_ts = q_ts;
        if (qkv) {
            // x rows -> projected rows [q | k | v] in the library's buffer; the attention kernels read
            // q, k, v out of those rows through their strides
            const OutProj& op = c->qkv_proj[size_t(r.layer)];
            const size_t row0 = qkv_row_tab.size();
            float* rows = c->qkv_seq + row0 * qkv_width;
            for (int t = 0; t < S; ++t)
                qkv_row_tab.push_back({q_dev + size_t(t) * op.in_dim, rows + size_t(t) * qkv_width});
            if (!qkv_runs.empty() && qkv_runs.back().layer == r.layer) qkv_runs.back().row_count += S;
            else qkv_runs.push_back({r.layer, int(row0), S, 0});
            q_dev = rows;
            k_dev = rows + size_t(Hq) * D;
            v_dev = k_dev + size_t(Hkv) * D;
            q_ts = kv_ts = (long long)qkv_width;
        }
        d.q_in = q_dev; d.qi_hs = q_hs; d.qi_ts = q_ts;
        const bool to_tf32 = r.index_pos + S <= s->cap && use_tf32(c, r, direct);
        if (fused) {
            d.q = q_dev; d.q_hs = q_hs; d.q_ts = q_ts;
            d.flags = 8u | (rope ? 1u : 0u);
        } else if (rope_in_prefill(c, r, direct, pinned)) {
            d.q = q_dev; d.q_hs = q_hs; d.q_ts = q_ts;
            d.flags = 1u | 16u;   // rotate k here, q in the prefill kernel
        } else if (rope || pinned) {
            d.q = c->q_rot + qrot_off;
            d.q_hs = (long long)S * D; d.q_ts = D;
            qrot_off += align_up(qf, 4);
            d.flags = rope ? 1u : 2u;
        } else {
            d.q = q_dev; d.q_hs = q_hs; d.q_ts = q_ts;
        }
        d.k = k_dev; d.v = v_dev; d.kv_hs = kv_hs; d.kv_ts = kv_ts;
        d.out = o_dev; d.o_hs = o_hs; d.o_ts = o_ts;
        if (r.flags & XN_REQ_OUT_PROJ) {
            // the attention kernels write sequence-major rows into the block's input buffer
            const OutProj& op = c->out_proj[size_t(r.layer)];
            const size_t row0 = out_row_tab.size();
            float* rows = c->attn_seq + row0 * size_t(op.in_dim);
            d.out = rows; d.o_hs = D; d.o_ts = op.in_dim;
            for (int t = 0; t < S; ++t)
                out_row_tab.push_back({rows + size_t(t) * op.in_dim, o_dev + size_t(t) * op.out_dim});
            if (!out_runs.empty() && out_runs.back().layer == r.layer) out_runs.back().row_count += S;
            else out_runs.push_back({r.layer, int(row0), S, 0});
        }
        d.page_off = int(page_ids.size());
        d.n_pages = int(s->pages.size());
        page_ids.insert(page_ids.end(), s->pages.begin(), s->pages.end());
        d.layer = r.layer; d.seq_len = S; d.index_pos = int(r.index_pos);
        d.cap = int(std::min<int64_t>(s->cap, int64_t(1) << 30));
        if (r.index_pos + S > s->cap) {
            for (int t = 0; t < S; ++t) { ring_rows.push_back(i); ring_rows.push_back(t); }
        } else if (to_tf32) {
            tf32_reqs.push_back(i);
        } else if (use_f32_tiled(c, r)) {
            // heaviest query tiles first (blocks are handed to SMs in index order)
            for (int qt = (S + pf32::kTQ - 1) / pf32::kTQ - 1; qt >= 0; --qt)
                for (int h = 0; h < Hq; ++h) f32_items.push_back({i, h, qt, 0});
        } else {
            for (int h = 0; h < Hkv; ++h)
                for (int sb = 0; sb < c->subs; ++sb)
                    for (int t = 0; t < S; ++t) {
                        UnitDev u;
                        u.req = i; u.kv_head = h;
                        u.head0 = h * c->group + sb * c->gt;
                        u.nheads = std::min(c->gt, c->group - sb * c->gt);
                        u.t_q = t; u.kv_len = int(r.index_pos) + t + 1;
                        u.part_begin = -1; u.part_count = 1; u.merge_slot = -1;
                        u.store_new = sb == 0 ? 1 : 0;
                        units.push_back(u);
                        kv_lens.push_back(u.kv_len);
                    }
        }
    }

    SplitPlan sp = plan_split(kv_lens.data(), int(units.size()), c->tile_tokens, c->decode_chunks);
    int n_cut = 0;
    for (size_t u = 0; u < units.size(); ++u) {
        units[u].part_begin = sp.unit_part_begin[u];
        units[u].part_count = sp.unit_part_count[u];
        units[u].merge_slot = sp.unit_part_count[u] > 1 ? n_cut++ : -1;
    }
    if (size_t(n_cut) + 2 > c->sync_cap)
        return fail(c, XN_ERR_CAPACITY, "internal: %d cut units exceed the arrival counters", n_cut);
    if ((rc = grow_device(c, &c->partials, &c->partials_cap,
                          size_t(sp.n_parts) * c->gt *
                              (c->kv_u8 ? kv8::part_stride(c->dq) : part_stride_floats(nv)))) != XN_OK)
        return rc;

    // -- pack the plan: one pinned buffer, one copy
    size_t off = 0;
    auto place = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 16); return o; };
    const size_t o_req = place(sizeof(ReqDev) * n);
    const size_t o_unit = place(sizeof(UnitDev) * units.size());
    const size_t o_item = place(sizeof(ItemDev) * sp.items.size());
    const size_t o_cta = place(sizeof(int32_t) * sp.cta_item_begin.size());
    const size_t o_page = place(sizeof(int32_t) * page_ids.size());
    const size_t o_ring = place(sizeof(int32_t) * ring_rows.size());
    const size_t o_rows = place(sizeof(OutRowDev) * out_row_tab.size());
    const size_t o_qkv = place(sizeof(OutRowDev) * qkv_row_tab.size());
    const size_t o_f32 = place(sizeof(F32Item) * f32_items.size());
    // Several tensor-core prefills in one submission share one launch: a table of their arguments
    // and a list of (request, query tile, head) blocks, heaviest first over all of them.  (Not in
    // the u8 format, whose requests take turns in one staging area.)
    const bool multi_prefill = c->pf_multi && !c->kv_u8 && tf32_reqs.size() > 1;
    std::vector<PrefillBlock> pf_blocks;
    if (multi_prefill) {
        std::vector<std::pair<int, PrefillBlock>> weighted;
        for (size_t k = 0; k < tf32_reqs.size(); ++k) {
            const ReqDev& d = rd[size_t(tf32_reqs[k])];
            const int n_qt = (d.seq_len + pf::kBM - 1) / pf::kBM;
            for (int qt = 0; qt < n_qt; ++qt) {
                const int last_row = std::min((qt + 1) * pf::kBM, d.seq_len) - 1;
                const int tiles = ((d.index_pos + last_row) / kPageTokens + 2) / 2;
                for (int h = 0; h < Hq; ++h) weighted.push_back({tiles, {int(k), qt, h, 0}});
            }
        }
        std::stable_sort(weighted.begin(), weighted.end(),
                         [](const auto& x, const auto& y) { return x.first > y.first; });
        pf_blocks.reserve(weighted.size());
        for (const auto& w : weighted) pf_blocks.push_back(w.second);
    }
    const size_t o_pft = place(multi_prefill ? sizeof(PrefillArgs) * tf32_reqs.size() : 0);
    const size_t o_pfb = place(sizeof(PrefillBlock) * pf_blocks.size());
    PlanSlot* slot = nullptr;
    if ((rc = acquire_slot(c, off, &slot)) != XN_OK) return rc;
    memcpy(slot->host + o_req, rd.data(), sizeof(ReqDev) * n);
    if (!units.empty()) memcpy(slot->host + o_unit, units.data(), sizeof(UnitDev) * units.size());
    static_assert(sizeof(SplitItem) == sizeof(ItemDev), "plan item layouts must match");
    if (!sp.items.empty()) memcpy(slot->host + o_item, sp.items.data(), sizeof(ItemDev) * sp.items.size());
    memcpy(slot->host + o_cta, sp.cta_item_begin.data(), sizeof(int32_t) * sp.cta_item_begin.size());
    if (!page_ids.empty()) memcpy(slot->host + o_page, page_ids.data(), sizeof(int32_t) * page_ids.size());
    if (!ring_rows.empty()) memcpy(slot->host + o_ring, ring_rows.data(), sizeof(int32_t) * ring_rows.size());
    if (!out_row_tab.empty())
        memcpy(slot->host + o_rows, out_row_tab.data(), sizeof(OutRowDev) * out_row_tab.size());
    if (!qkv_row_tab.empty())
        memcpy(slot->host + o_qkv, qkv_row_tab.data(), sizeof(OutRowDev) * qkv_row_tab.size());
    if (!f32_items.empty()) memcpy(slot->host + o_f32, f32_items.data(), sizeof(F32Item) * f32_items.size());
    if (multi_prefill) {
        PrefillArgs* tab = reinterpret_cast<PrefillArgs*>(slot->host + o_pft);
        for (size_t k = 0; k < tf32_reqs.size(); ++k)
            tab[k] = make_prefill_args(c, rd[size_t(tf32_reqs[k])], reinterpret_cast<const int*>(slot->dev + o_page));
        memcpy(slot->host + o_pfb, pf_blocks.data(), sizeof(PrefillBlock) * pf_blocks.size());
    }
    // The plan does not depend on anything in flight: upload it on the copy stream so that it
    // overlaps the previous submission's kernels, and make the launch stream wait for it.
    // (A blocking host-pointer call has nothing in flight to overlap with: plain in-stream copy.)
    if (host_mode) {
        XN_CUDA(c, cudaMemcpyAsync(slot->dev, slot->host, off, cudaMemcpyHostToDevice, c->stream));
    } else {
        XN_CUDA(c, cudaMemcpyAsync(slot->dev, slot->host, off, cudaMemcpyHostToDevice, c->copy_stream));
        XN_CUDA(c, cudaEventRecord(slot->up_ev, c->copy_stream));
        XN_CUDA(c, cudaStreamWaitEvent(c->stream, slot->up_ev, 0));
    }
    c->stats.h2d_bytes += off;
    const ReqDev* reqs_d = reinterpret_cast<const ReqDev*>(slot->dev + o_req);
    const UnitDev* units_d = reinterpret_cast<const UnitDev*>(slot->dev + o_unit);
    const ItemDev* items_d = reinterpret_cast<const ItemDev*>(slot->dev + o_item);
    const int* cta_d = reinterpret_cast<const int*>(slot->dev + o_cta);
    const int* pages_d = reinterpret_cast<const int*>(slot->dev + o_page);
    const int* ring_d = reinterpret_cast<const int*>(slot->dev + o_ring);

    if (host_mode && !pinned && io_in) {
        if (!stage_direct)
            XN_CUDA(c, cudaMemcpyAsync(c->io_dev, c->io_host, io_in, cudaMemcpyHostToDevice, c->stream));
        c->stats.h2d_bytes += io_in;
    }

    // -- the two projection blocks share one quantised-activation buffer (they run one after the
    //    other); every run of rows starts on a 256-row boundary of it
    size_t qkv_rows_pad = 0, q_rows_pad = 0;
    for (OutRun& run : qkv_runs) {
        run.q_row0 = qkv_rows_pad;
        qkv_rows_pad += align_up(size_t(run.row_count), 256);
    }
    for (OutRun& run : out_runs) {
        run.q_row0 = q_rows_pad;
        q_rows_pad += align_up(size_t(run.row_count), 256);
    }
    {
        size_t need = 0;
        for (const OutRun& run : qkv_runs)
            need = std::max(need, q8_floats(size_t(c->qkv_proj[size_t(run.layer)].q_stride), qkv_rows_pad));
        for (const OutRun& run : out_runs)
            need = std::max(need, q8_floats(size_t(c->out_proj[size_t(run.layer)].q_stride), q_rows_pad));
        if (need && (rc = grow_device(c, &c->q8, &c->q8_cap, need)) != XN_OK) return rc;
    }

    // -- launches: every sizing step above has succeeded, the cache positions are going to be written
    undo.commit();
    for (const OutRun& run : qkv_runs) {   // x -> [q | k | v] rows, before anything reads them
        const OutRowDev* rows_d = reinterpret_cast<const OutRowDev*>(slot->dev + o_qkv) + run.row_begin;
        if (c->profile && (rc = profile_begin(c, 3)) != XN_OK) return rc;
        if ((rc = launch_out_block(c, c->qkv_proj[size_t(run.layer)], rows_d, run.row_count, run.q_row0,
                                   qkv_rows_pad)) != XN_OK)
            return rc;
        if (c->profile && (rc = profile_end(c)) != XN_OK) return rc;
    }
    for (const GapFill& g : gaps) {
        const long long total = g.n * Hkv * D;
        const int blocks = int(std::min<long long>((total + 255) / 256, 4096));
        if (c->kv_u8)
            kv8::slots_fill_u8_kernel<<<int(std::min<long long>((g.n * Hkv + 7) / 8, 4096)), 256, 0, c->stream>>>(
                pages_d + rd[g.req].page_off, c->pool8, c->pool_pages, rd[g.req].layer, Hkv, D, c->dq,
                g.slot0, g.n, 0, 0ull);
        else
        slots_fill_kernel<<<blocks, 256, 0, c->stream>>>(
            pages_d + rd[g.req].page_off, c->k_pool, c->v_pool, c->pool_pages, rd[g.req].layer, Hkv,
            D, nv, g.slot0, g.n, 0, 0ull);
        c->stats.kernel_launches += 1;
    }
    if (max_rows > 0) {
        dim3 grid(unsigned(std::min<long long>((max_rows + 63) / 64, 4096)), unsigned(n));
        if (c->kv_u8) {
            dim3 grid8(unsigned(std::min<long long>((max_rows + 7) / 8, 4096)), unsigned(n));
            kv8::rope_append_u8_kernel<<<grid8, 256, 0, c->stream>>>(reqs_d, pages_d, c->pool8, c->cos_d,
                                                                    c->sin_d, c->pool_pages, Hq, Hkv, D,
                                                                    c->dq);
        } else
        {
            auto append = (D % 8 != 0 && D % 4 == 0 && D <= 128) ? rope_append_kernel<true> : rope_append_kernel<false>;
            append<<<grid, 256, 0, c->stream>>>(reqs_d, pages_d, c->k_pool, c->v_pool, c->cos_d, c->sin_d,
                                                c->pool_pages, Hq, Hkv, D, nv);
        }
        c->stats.kernel_launches += 1;
    }
    if (sp.ctas > 0 && c->kv_u8) {
        if (c->profile && (rc = profile_begin(c, 0)) != XN_OK) return rc;
        const Split8Fn fn8 = mma_now ? pick_split8_mma(c->dq, c->gt) : pick_split8(c->dq, c->gt, c->kv8_epl);
        const size_t smem8 = mma_now ? kv8m::smem_bytes(c->gt, c->dq) : kv8::smem_bytes(c->gt, c->kv8_epl);
        fn8<<<std::min(sp.ctas, c->decode_ctas), kv8::kThreads, smem8, c->stream>>>(
            reqs_d, units_d, items_d, cta_d, sp.ctas, pages_d, c->pool8, c->partials, c->sync_d,
            c->pool_pages, Hkv, D, c->scale * 1.4426950408889634f, c->cos_d, c->sin_d, c->status_d);
        if (c->profile && (rc = profile_end(c)) != XN_OK) return rc;
        c->stats.kernel_launches += 1;
        c->stats.decode_launches += 1;
    } else if (sp.ctas > 0) {
        SplitKernel k = pick_split(c->nv_class, c->gt, c->nv_exact);
        if (c->profile && (rc = profile_begin(c, 0)) != XN_OK) return rc;
        // sp.ctas chunks, taken dynamically by at most one block per SM
        c->pcache.table.n = 0;
        k.fn<<<std::min(sp.ctas, c->decode_ctas), k.threads, k.smem, c->stream>>>(
            reqs_d, units_d, items_d, cta_d, sp.ctas, pages_d, c->k_pool, c->v_pool, c->partials,
            c->sync_d, c->pool_pages, Hkv, D, nv, c->scale, c->cos_d, c->sin_d, c->status_d,
            c->pcache.table);
        if (c->profile && (rc = profile_end(c)) != XN_OK) return rc;
        c->stats.kernel_launches += 1;
        c->stats.decode_launches += 1;
        // Keep the plan when the whole submission was this one launch: one new token per request,
        // appended by the kernel, tensors addressed directly (device or page-locked host memory).
        PlanCache& pc = c->pcache;
        pc.valid = false;
        if (c->plan_reuse && fused && direct && n <= kPatchReqs && gaps.empty() && out_runs.empty() &&
            qkv_runs.empty() && tf32_reqs.empty() && f32_items.empty() && ring_rows.empty()) {
            pc.ent.resize(size_t(n));
            bool all = true;
            for (int i = 0; i < n && all; ++i) {
                if (reqs[i].seq_len != 1) { all = false; break; }
                pc.ent[size_t(i)] = {reqs[i].stream, reqs[i].index_pos, reqs[i].flags,
                                     int(reqs[i].stream->pages.size())};
            }
            if (all) {
                pc.valid = true;
                pc.host_mode = host_mode; pc.pinned = pinned; pc.slot = slot;
                pc.o_req = o_req; pc.o_unit = o_unit; pc.o_item = o_item; pc.o_cta = o_cta; pc.o_page = o_page;
                pc.ctas = sp.ctas;
                pc.out_dma = out_dma;
                pc.out_bytes = out_dma_bytes;
                pc.h2d_bytes = pinned ? uint64_t(n) * size_t(Hq + 2 * Hkv) * D * 4 : 0;
                pc.d2h_bytes = pinned ? uint64_t(n) * size_t(Hq) * D * 4 : 0;
            }
        }
    }
    if (!f32_items.empty()) {
        const PrefillF32Kernel pk = pick_prefill_f32(nv);
        if (c->profile && (rc = profile_begin(c, 1)) != XN_OK) return rc;
        pk.fn<<<unsigned(f32_items.size()), pf32::kThreads, pk.smem, c->stream>>>(
            reqs_d, reinterpret_cast<const F32Item*>(slot->dev + o_f32), pages_d, c->k_pool, c->v_pool,
            c->pool_pages, Hkv, c->group, D, nv, c->scale, c->status_d);
        if (c->profile && (rc = profile_end(c)) != XN_OK) return rc;
        c->stats.kernel_launches += 1;
        c->stats.prefill_launches += 1;
    }
    auto prefill_args = [&](int i) { return make_prefill_args(c, rd[size_t(i)], pages_d); };
    // A programmatic dependent of the kernel before it (the append): its blocks set up while that
    // kernel drains; their reads of what it wrote wait inside the kernel.  Not behind another
    // prefill launch: two of them must not share the SMs' tensor memory.
    auto launch_prefill = [&](unsigned blocks, bool pdl, bool multi, const PrefillArgs& pa,
                              const PrefillArgs* table_d, const PrefillBlock* blocks_d) -> cudaError_t {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(blocks);
        cfg.blockDim = dim3(pf::kThreads);
        cfg.dynamicSmemBytes = pf::kSmemBytes;
        cfg.stream = c->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = (c->pf_pdl && pdl && !c->profile) ? 1 : 0;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const CUtensorMap& km = c->kv_u8 ? c->k_stage_map : c->k_map;
        const CUtensorMap& vm = c->kv_u8 ? c->v_stage_map : c->v_map;
        return multi ? cudaLaunchKernelEx(&cfg, prefill_tf32_kernel<true>, km, vm, pa, table_d, blocks_d)
                     : cudaLaunchKernelEx(&cfg, prefill_tf32_kernel<false>, km, vm, pa, table_d, blocks_d);
    };
    if (multi_prefill) {
        // several prompts in one submission: one launch, blocks of all requests heaviest first
        if (c->profile && (rc = profile_begin(c, 1)) != XN_OK) return rc;
        XN_CUDA(c, launch_prefill(unsigned(pf_blocks.size()), true, true, prefill_args(tf32_reqs.front()),
                                  reinterpret_cast<const PrefillArgs*>(slot->dev + o_pft),
                                  reinterpret_cast<const PrefillBlock*>(slot->dev + o_pfb)));
        if (c->profile && (rc = profile_end(c)) != XN_OK) return rc;
        c->stats.kernel_launches += 1;
        c->stats.prefill_launches += 1;
    } else
    for (int i : tf32_reqs) {
        const ReqDev& d = rd[size_t(i)];
        const PrefillArgs pa = prefill_args(i);
        if (c->profile && (rc = profile_begin(c, 1)) != XN_OK) return rc;
        if (c->kv_u8) {
            // the stream's pages of this layer (the new rows included: the append ran above),
            // dequantised into the staging area the kernel's tensor maps cover
            const int n_pages = (d.index_pos + d.seq_len + kPageTokens - 1) / kPageTokens;
            kv8::dequant_pages_u8_kernel<<<n_pages * Hkv, 256, 0, c->stream>>>(
                c->pool8, pages_d + d.page_off, n_pages, d.layer, c->pool_pages, Hkv, D, c->dq, c->k_stage,
                c->v_stage);
            c->stats.kernel_launches += 1;
        }
        XN_CUDA(c, launch_prefill(unsigned((d.seq_len + pf::kBM - 1) / pf::kBM) * unsigned(Hq),
                                  i == tf32_reqs.front(), false, pa, nullptr, nullptr));
        if (c->profile && (rc = profile_end(c)) != XN_OK) return rc;
        c->stats.kernel_launches += 1;
        c->stats.prefill_launches += 1;
    }
    if (!ring_rows.empty()) {
        const int rows = int(ring_rows.size() / 2);
        attn_ring_kernel<<<rows * Hq, 256, 0, c->stream>>>(reqs_d, ring_d, rows, pages_d, c->k_pool,
                                                           c->v_pool, c->pool_pages, Hq, Hkv, D, nv,
                                                           c->scale, c->pool8, c->dq);
        c->stats.kernel_launches += 1;
    }
    XN_CUDA(c, cudaGetLastError());
    for (const OutRun& run : out_runs) {
        const OutRowDev* rows_d = reinterpret_cast<const OutRowDev*>(slot->dev + o_rows) + run.row_begin;
        if (c->profile && (rc = profile_begin(c, 2)) != XN_OK) return rc;
        if ((rc = launch_out_block(c, c->out_proj[size_t(run.layer)], rows_d, run.row_count, run.q_row0,
                                   q_rows_pad)) != XN_OK)
            return rc;
        if (c->profile && (rc = profile_end(c)) != XN_OK) return rc;
    }

    if (out_dma) {
        XN_CUDA(c, cudaMemcpyAsync(out_dma_host, c->out_stage, out_dma_bytes, cudaMemcpyDeviceToHost, c->stream));
        c->stats.out_transfers += 1;
    }
    if (host_mode) {
        if (io_out) {
            if (!out_direct)
                XN_CUDA(c, cudaMemcpyAsync(c->io_host + io_in, c->io_dev + io_in, io_out,
                                           cudaMemcpyDeviceToHost, c->stream));
            c->stats.d2h_bytes += io_out;
        }
    }
    XN_CUDA(c, cudaEventRecord(slot->ev, c->stream));
    slot->used = true;
    c->stats.batches += 1;
    c->stats.calls += uint64_t(n);

    if (host_mode && pinned && defer) {
        XN_CUDA(c, cudaEventRecord(defer, c->stream));
        return XN_OK;
    }
    if (host_mode) {
        XN_CUDA(c, cudaStreamSynchronize(c->stream));
        if ((rc = check_device_status(c)) != XN_OK) return rc;
        if (pinned) return XN_OK;  // the kernels wrote the outputs in place
        size_t o = io_in;
        for (int i = 0; i < n; ++i) {
            if (reqs[i].seq_len == 0) continue;
            const size_t of = (reqs[i].flags & XN_REQ_OUT_PROJ)
                                  ? size_t(reqs[i].seq_len) * c->out_proj[size_t(reqs[i].layer)].out_dim
                                  : size_t(Hq) * reqs[i].seq_len * D;
            memcpy(reqs[i].out, c->io_host + o, of * 4);
            o += align_up(of * 4, 16);
        }
    }
    return XN_OK;
}

// Runs a group of blocking host-pointer requests.  Requests that fail validation, or that name a
// stream already in the group, get their own status and are left out.  The others go out as one
// submission per kind of memory they point at (the streams' page-locked call buffers, or pageable
// memory that the library stages).
// What the leader of a group still has to wait for after run_group returned: the page-locked part
// of the group is only enqueued; `ev` fires behind its last operation.
struct GroupWait {
    cudaEvent_t ev = nullptr;
    std::vector<Pending*> members;
};

void run_group(xn_ctx* c, std::vector<Pending*>& group, GroupWait* wait) {
    std::lock_guard<std::mutex> g(c->mu);
    std::vector<xn_req> ok[2];   // [0] pageable, [1] page-locked
    std::vector<Pending*> ok_p[2];
    std::unordered_set<xn_stream*> seen;
    for (Pending* p : group) {
        int32_t rc = validate_req(c, p->req);
        if (rc == XN_OK && !seen.insert(p->req.stream).second)
            rc = fail(c, XN_ERR_ARG, "two concurrent calls on one stream");
        p->status = rc;
        if (rc == XN_OK) {
            const int kind = (p->req.flags & XN_REQ_HOST_PINNED) ? 1 : 0;
            ok[kind].push_back(p->req);
            ok_p[kind].push_back(p);
        }
    }
    c->stats.coalesced_max = std::max<uint64_t>(c->stats.coalesced_max, ok[0].size() + ok[1].size());
    // Callers that went through their streams' call buffers: re-point their outputs at one slab,
    // back to back, when the group is large enough for one transfer to beat the kernels' own
    // stores into host memory.
    {
        const size_t row = size_t(c->num_heads) * c->head_dim * 4;
        bool all_staged = c->pinned_out_dma && !ok[1].empty() && ok[1].size() * row >= c->out_dma_min_bytes;
        for (Pending* p : ok_p[1]) all_staged = all_staged && p->user_out != nullptr && p->out_bytes == row;
        if (all_staged) {
            // a slab whose previous group has not finished reading is passed over (never waited
            // for: this runs under the context's lock, which that group's leader needs to finish);
            // with both busy the group's outputs go to the call buffers as before
            if (c->slabs[c->slab_next].readers.load(std::memory_order_acquire) > 0) c->slab_next ^= 1;
            OutSlab& sl = c->slabs[c->slab_next];
            bool usable = sl.readers.load(std::memory_order_acquire) == 0;
            const size_t need = ok[1].size() * row;
            if (usable && sl.cap < need) {
                if (sl.host) cudaFreeHost(sl.host);
                sl.host = nullptr;
                sl.cap = 0;
                void* p = nullptr;
                const size_t want = std::max(need * 2, size_t(1) << 20);
                if (cudaSetDevice(c->device) == cudaSuccess &&
                    cudaHostAlloc(&p, want, cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
                    sl.host = static_cast<unsigned char*>(p);
                    sl.cap = want;
                } else {
                    cudaGetLastError();
                    usable = false;
                }
            }
            if (usable) {
                c->slab_next ^= 1;
                sl.readers.store(int(ok[1].size()), std::memory_order_release);
                for (size_t i = 0; i < ok[1].size(); ++i) {
                    float* dst = reinterpret_cast<float*>(sl.host + i * row);
                    ok[1][i].out = dst;
                    ok_p[1][i]->req.out = dst;
                    ok_p[1][i]->slab = &sl;
                }
            }
        }
    }
    for (int kind = 1; kind >= 0; --kind) {
        if (ok[kind].empty()) continue;
        // the page-locked part (callers that came through their call buffers) is enqueued and
        // waited for outside this lock; the pageable part shares one staging area and stays inside
        cudaEvent_t ev = nullptr;
        if (kind == 1 && wait && c->defer_groups) {
            if (!c->done_events.empty()) {
                ev = c->done_events.back();
                c->done_events.pop_back();
            } else if (cudaSetDevice(c->device) != cudaSuccess ||
                       cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) {
                cudaGetLastError();
                ev = nullptr;
            }
        }
        int32_t rc = submit_locked(c, int(ok[kind].size()), ok[kind].data(), true, ev);
        for (Pending* p : ok_p[kind]) p->status = rc;
        if (ev && rc == XN_OK) {
            wait->ev = ev;
            wait->members = ok_p[kind];
        } else if (ev) {
            c->done_events.push_back(ev);
        }
        // The callers are independent, as in the reference: when the merged submission was
        // refused before anything ran (it left the streams untouched), one request that does not
        // fit must not fail the others.  Run them one by one; each gets its own status.
        if (ok[kind].size() > 1 && (rc == XN_ERR_OUT_OF_PAGES || rc == XN_ERR_CAPACITY || rc == XN_ERR_NOMEM))
            for (size_t i = 0; i < ok[kind].size(); ++i)
                ok_p[kind][i]->status = submit_locked(c, 1, &ok[kind][i], true);
    }
}

// A single-token call brings its tensors to the stream's page-locked call buffer itself (every
// caller in parallel, outside all locks) and is queued pointing there; the kernels then need no
// staging copy.  Larger calls stay as they are and go through the library's staging.
void stage_in_call_buffer(xn_ctx* c, Pending& me) {
    xn_req& r = me.req;
    xn_stream* s = r.stream;
    // (u8 cache format: its attention kernel reads the new rows with plain 4-byte loads, which is
    // slow over PCIe; those calls keep the staged path and its fused append)
    if (c->kv_u8 || r.seq_len != 1 || !stream_ok(c, s) || !r.q || !r.k || !r.v || !r.out ||
        (r.flags & ~uint32_t(XN_REQ_ROPE)))
        return;
    const size_t qb = align_up(size_t(c->num_heads) * c->head_dim * 4, 16);
    const size_t kb = align_up(size_t(c->num_kv_heads) * c->head_dim * 4, 16);
    if (s->call_cap < 2 * qb + 2 * kb) {
        if (s->call_buf) return;   // sized at first use; a stream's shape does not change
        void* p = nullptr;
        if (cudaSetDevice(c->device) != cudaSuccess ||
            cudaHostAlloc(&p, 2 * qb + 2 * kb, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
            cudaGetLastError();
            return;                // no page-locked memory to be had: the staged path serves the call
        }
        s->call_buf = static_cast<unsigned char*>(p);
        s->call_cap = 2 * qb + 2 * kb;
    }
    unsigned char* b = s->call_buf;
    memcpy(b, r.q, size_t(c->num_heads) * c->head_dim * 4);
    memcpy(b + qb, r.k, size_t(c->num_kv_heads) * c->head_dim * 4);
    memcpy(b + qb + kb, r.v, size_t(c->num_kv_heads) * c->head_dim * 4);
    me.user_out = r.out;
    me.out_bytes = size_t(c->num_heads) * c->head_dim * 4;
    r.q = reinterpret_cast<const float*>(b);
    r.k = reinterpret_cast<const float*>(b + qb);
    r.v = reinterpret_cast<const float*>(b + qb + kb);
    r.out = reinterpret_cast<float*>(b + qb + 2 * kb);
    r.flags |= XN_REQ_HOST_PINNED;
}

// The queue of blocking callers.  Whoever finds no leader becomes one: it takes everything queued
// (its own request included), runs it as one group, wakes the callers it served, and hands the
// lead to the first caller that arrived meanwhile.  When the previous group held several callers
// a new leader first waits briefly for as many to show up again: slot threads that were woken
// together come back together, one layer later.
int32_t attention_blocking(xn_ctx* c, const xn_req& req) {
    Pending me;
    me.req = req;
    stage_in_call_buffer(c, me);
    std::unique_lock<std::mutex> lk(c->q_mu);
    c->queue.push_back(&me);
    if (c->leader_active) {
        if (c->leader_in_window) c->q_cv.notify_one();
        c->flight_cv.notify_one();   // a leader may be waiting for its group to fill up
        me.cv.wait(lk, [&] { return me.done || me.promoted; });
    } else {
        c->leader_active = true;
        me.promoted = true;
    }
    if (!me.done) {
        // ---- leader
        const size_t target = c->batch_window_us > 0 ? std::max<size_t>(1, c->streams.size()) : c->last_group;
        const int window_us = c->batch_window_us > 0 ? c->batch_window_us : (c->last_group > 1 ? c->auto_window_us : 0);
        if (window_us > 0 && c->queue.size() < target) {
            c->leader_in_window = true;
            c->q_cv.wait_for(lk, std::chrono::microseconds(window_us), [&] { return c->queue.size() >= target; });
            c->leader_in_window = false;
        }
        if (c->in_flight > 0)
            c->flight_cv.wait(lk, [&] {
                return c->in_flight == 0 ||
                       (c->in_flight < 2 && c->queue.size() >= std::max<size_t>(2, c->group_before_last));
            });
        std::vector<Pending*> group;
        group.swap(c->queue);
        c->in_flight += 1;
        lk.unlock();
        GroupWait wait;
        run_group(c, group, &wait);
        lk.lock();
        c->group_before_last = c->last_group;
        c->last_group = group.size();
        // The lead passes on BEFORE this group's kernels have finished: whoever arrived meanwhile
        // (or arrives next) enqueues the next group right behind them.
        if (c->queue.empty()) {
            c->leader_active = false;
        } else {
            c->queue.front()->promoted = true;
            c->queue.front()->cv.notify_one();
        }
        if (wait.ev) {
            lk.unlock();
            const cudaError_t e = cudaEventSynchronize(wait.ev);
            {
                std::lock_guard<std::mutex> g(c->mu);
                int32_t rc = e == cudaSuccess ? check_device_status(c)
                                              : fail(c, XN_ERR_CUDA, "cudaEventSynchronize: %s", cudaGetErrorString(e));
                if (rc != XN_OK)
                    for (Pending* p : wait.members) p->status = rc;
                c->done_events.push_back(wait.ev);
            }
            lk.lock();
        }
        c->in_flight -= 1;
        c->flight_cv.notify_all();
        for (Pending* p : group) {
            p->done = true;
            if (p != &me) p->cv.notify_one();
        }
    }
    lk.unlock();
    if (me.user_out && me.status == XN_OK) memcpy(me.user_out, me.req.out, me.out_bytes);
    if (me.slab) me.slab->readers.fetch_sub(1, std::memory_order_release);
    return me.status;
}

}  // namespace

// ============================================================================================
// C ABI
// ============================================================================================

extern "C" {

const char* xn_version(void) { return "xn_attn 0.1 sm_100a"; }

const char* xn_last_error(xn_ctx* ctx) {
    // The text is copied into a buffer of the calling thread: other threads may fail, and rewrite
    // the context's message, while the caller still reads this one.
    static thread_local std::string copy;
    if (ctx_ok(ctx)) {
        std::lock_guard<std::mutex> g(ctx->err_mu);
        copy = ctx->last_error;
    } else {
        std::lock_guard<std::mutex> g(g_err_mu);
        copy = g_create_error;
    }
    return copy.c_str();
}

int32_t xn_ctx_create(const xn_ctx_desc* d, xn_ctx** out_ctx) {
    if (!d || !out_ctx) return fail(nullptr, XN_ERR_ARG, "null descriptor or output");
    *out_ctx = nullptr;
    if (d->num_layers <= 0 || d->num_heads <= 0 || d->num_kv_heads <= 0)
        return fail(nullptr, XN_ERR_SHAPE, "layer and head counts must be positive");
    if (d->num_heads % d->num_kv_heads != 0)
        return fail(nullptr, XN_ERR_SHAPE, "num_heads %d is not a multiple of num_kv_heads %d",
                    d->num_heads, d->num_kv_heads);
    if (d->head_dim < 1 || d->head_dim > 256)
        return fail(nullptr, XN_ERR_SHAPE, "head_dim %d outside 1..256", d->head_dim);
    if (d->page_tokens != 0 && d->page_tokens != kPageTokens)
        return fail(nullptr, XN_ERR_ARG, "page_tokens must be 0 or %d", kPageTokens);
    if (d->kv_format != XN_KV_F32 && d->kv_format != XN_KV_U8)
        return fail(nullptr, XN_ERR_ARG, "kv_format %d is neither XN_KV_F32 nor XN_KV_U8", d->kv_format);
    if ((d->rope_cos == nullptr) != (d->rope_sin == nullptr) || (d->rope_cos && d->max_pos <= 0))
        return fail(nullptr, XN_ERR_ARG, "rope tables need cos, sin and max_pos together");

    int n_dev = 0;
    cudaError_t e = cudaGetDeviceCount(&n_dev);
    if (e != cudaSuccess || n_dev <= 0)
        return fail(nullptr, XN_ERR_NO_DEVICE,
                    "no CUDA device (%s); this library has no CPU fallback",
                    e != cudaSuccess ? cudaGetErrorString(e) : "count is 0");
    if (d->device < 0 || d->device >= n_dev)
        return fail(nullptr, XN_ERR_ARG, "device ordinal %d outside 0..%d", d->device, n_dev - 1);
    cudaDeviceProp prop;
    XN_CUDA(nullptr, cudaSetDevice(d->device));
    XN_CUDA(nullptr, cudaGetDeviceProperties(&prop, d->device));
    if (prop.major != 10)
        return fail(nullptr, XN_ERR_NO_DEVICE, "device %d is sm_%d%d; this build targets sm_100a only",
                    d->device, prop.major, prop.minor);

    xn_ctx* c = new (std::nothrow) xn_ctx();
    if (!c) return fail(nullptr, XN_ERR_NOMEM, "out of host memory");
    c->device = d->device;
    c->num_layers = d->num_layers;
    c->num_heads = d->num_heads;
    c->num_kv_heads = d->num_kv_heads;
    c->head_dim = d->head_dim;
    c->group = d->num_heads / d->num_kv_heads;
    c->gt = (c->group >= 3) ? 4 : c->group;  // 1, 2 or 4 query heads share each K/V tile
    c->subs = (c->group + c->gt - 1) / c->gt;
    c->nv = (d->head_dim + 3) / 4;
    c->nv_class = nv_class_for(c->nv);
    c->nv_exact = c->nv_class == c->nv;
    c->tile_tokens = pick_split(c->nv_class, c->gt, c->nv_exact).tile_tokens;
    c->kv_u8 = d->kv_format == XN_KV_U8;
    if (c->kv_u8) {
        c->dq = kv8::row_bytes_for(d->head_dim);
        c->tile_tokens = kPageTokens;  // the u8 kernel's plan tile is one page
        if (const char* env = getenv("XORNET_ATTN_KV8_MMA")) c->kv8_mma = atoi(env) != 0;
        if (const char* env = getenv("XORNET_ATTN_KV8_MMA_MIN_ROWS")) c->kv8_mma_min_rows = atoll(env);
        c->kv8_mma = c->kv8_mma && d->head_dim == c->dq && (c->dq == 64 || c->dq == 128);
    }
    c->scale = 1.0f / sqrtf(float(d->head_dim));  // fast_attention.rs:135
    c->max_pos = d->max_pos;
    c->prefill_mode = d->prefill_mode;
    c->batch_window_us = d->batch_window_us;
    if (c->batch_window_us == 0)
        if (const char* env = getenv("XORNET_ATTN_BATCH_WINDOW_US")) c->batch_window_us = std::max(0, atoi(env));
    if (const char* env = getenv("XORNET_ATTN_AUTO_WINDOW_US")) c->auto_window_us = std::max(0, atoi(env));
    c->sm_count = prop.multiProcessorCount;
    c->out_proj.resize(size_t(d->num_layers));
    c->qkv_proj.resize(size_t(d->num_layers));
    c->decode_ctas = c->kv_u8 ? c->sm_count * (c->kv8_mma ? kv8m::kBlocksPerSm : kv8::blocks_per_sm(c->kv8_epl))
                              : c->sm_count;
    if (const char* env = getenv("XORNET_ATTN_DECODE_CTAS")) {
        int v = atoi(env);
        if (v > 0) c->decode_ctas = v;
    }
    int chunks_per_cta = 1;  // more chunks = dynamic balancing, at the cost of more cut units
    if (const char* env = getenv("XORNET_ATTN_DECODE_CHUNKS_PER_CTA")) {
        int v = atoi(env);
        if (v > 0) chunks_per_cta = v;
    }
    c->decode_chunks = c->decode_ctas * chunks_per_cta;
    if (const char* env = getenv("XORNET_ATTN_FUSE_APPEND")) c->fuse_append = atoi(env) != 0;
    if (const char* env = getenv("XORNET_ATTN_FUSE_PINNED")) c->fuse_pinned = atoi(env) != 0;
    if (const char* env = getenv("XORNET_ATTN_PLAN_REUSE")) c->plan_reuse = atoi(env) != 0;
    if (const char* env = getenv("XORNET_ATTN_PINNED_OUT_DMA")) c->pinned_out_dma = atoi(env) != 0;
    if (const char* env = getenv("XORNET_ATTN_DEFER_GROUPS")) c->defer_groups = atoi(env) != 0;
    if (const char* env = getenv("XORNET_ATTN_OUT_DMA_MIN_BYTES")) c->out_dma_min_bytes = size_t(std::max(0ll, atoll(env)));
    if (const char* env = getenv("XORNET_ATTN_PREFILL_ROPE_Q")) c->pf_rope_q = atoi(env) != 0;
    if (const char* env = getenv("XORNET_ATTN_PREFILL_MULTI")) c->pf_multi = atoi(env) != 0;
    if (const char* env = getenv("XORNET_ATTN_STAGE_DIRECT_BYTES")) c->stage_direct_bytes = size_t(atoll(env));
    if (const char* env = getenv("XORNET_ATTN_OUTPROJ_TC")) c->out_tc = atoi(env) != 0;
    if (const char* env = getenv("XORNET_ATTN_OUTPROJ_PDL")) c->out_pdl = atoi(env) != 0;
    if (const char* env = getenv("XORNET_ATTN_OUTPROJ_ROWS")) c->out_rows_kernel = atoi(env) != 0;
    if (const char* env = getenv("XORNET_ATTN_PREFILL_PDL")) c->pf_pdl = atoi(env) != 0;
    if (const char* env = getenv("XORNET_ATTN_F32_TILED")) c->f32_tiled = atoi(env) != 0;
    if (const char* env = getenv("XORNET_ATTN_F32_TILED_MIN_ROWS")) c->f32_tiled_min_rows = std::max(1, atoi(env));


    const size_t page_bytes =
        c->kv_u8 ? size_t(d->num_layers) * d->num_kv_heads * kv8::block_bytes(c->dq)
                 : size_t(d->num_layers) * d->num_kv_heads * kPageTokens * c->nv * 16 * 2;  // K and V
    long long pool_bytes = d->pool_bytes;
    if (d->pool_pages <= 0 && pool_bytes <= 0) {
        // neither given: a bounded byte budget -- XORNET_ATTN_POOL_MB, else half of what the device has free
        if (const char* env = getenv("XORNET_ATTN_POOL_MB")) pool_bytes = atoll(env) << 20;
        if (pool_bytes <= 0) {
            size_t free_b = 0, total_b = 0;
            if (cudaMemGetInfo(&free_b, &total_b) == cudaSuccess) pool_bytes = (long long)(free_b / 2);
        }
    }
    long long pages = d->pool_pages > 0 ? d->pool_pages : (pool_bytes > 0 ? pool_bytes / (long long)page_bytes : 0);
    if (pages <= 0 || pages > (1ll << 30)) {
        delete c;
        return fail(nullptr, XN_ERR_ARG, "pool_pages (or pool_bytes) must give at least one page");
    }
    c->pool_pages = pages;

    auto bail = [&](int32_t code) {
        std::string msg;
        { std::lock_guard<std::mutex> g(g_err_mu); msg = g_create_error; }
        xn_ctx_destroy(c);
        { std::lock_guard<std::mutex> g(g_err_mu); g_create_error = msg; }
        return code;
    };
#define XN_CREATE_CUDA(expr)                                                                   \
    do {                                                                                       \
        cudaError_t e__ = (expr);                                                              \
        if (e__ != cudaSuccess) {                                                              \
            fail(nullptr, XN_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));       \
            return bail(XN_ERR_CUDA);                                                          \
        }                                                                                      \
    } while (0)

    if (d->cuda_stream) {
        c->stream = static_cast<cudaStream_t>(d->cuda_stream);
    } else {
        XN_CREATE_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
        c->own_stream = true;
    }
    XN_CREATE_CUDA(cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking));
    if (c->kv_u8) {
        const long long n_blocks = pages * d->num_layers * d->num_kv_heads;
        XN_CREATE_CUDA(guarded_malloc(c, reinterpret_cast<void**>(&c->pool8), size_t(n_blocks) * kv8::block_bytes(c->dq), "pool8"));
        // every slot starts as the reference's shadow does: byte 128, scale 0.0
        kv8::pool_init_u8_kernel<<<unsigned(std::min<long long>(n_blocks, 4096)), 256, 0, c->stream>>>(
            c->pool8, n_blocks, c->dq);
        XN_CREATE_CUDA(cudaGetLastError());
    } else {
        const size_t pool_floats = size_t(pages) * d->num_layers * d->num_kv_heads * kPageTokens * c->nv * 4;
        XN_CREATE_CUDA(guarded_malloc(c, reinterpret_cast<void**>(&c->k_pool), pool_floats * 4, "k_pool"));
        XN_CREATE_CUDA(guarded_malloc(c, reinterpret_cast<void**>(&c->v_pool), pool_floats * 4, "v_pool"));
        // Row padding (head_dim rounded up to 4 floats) must hold zeros for the lifetime of the pool.
        XN_CREATE_CUDA(cudaMemsetAsync(c->k_pool, 0, pool_floats * 4, c->stream));
        XN_CREATE_CUDA(cudaMemsetAsync(c->v_pool, 0, pool_floats * 4, c->stream));
    }
    if (d->rope_cos) {
        const size_t tb = size_t(d->max_pos) * (d->head_dim / 2) * 4;
        XN_CREATE_CUDA(guarded_malloc(c, reinterpret_cast<void**>(&c->cos_d), std::max<size_t>(tb, 16), "cos table"));
        XN_CREATE_CUDA(guarded_malloc(c, reinterpret_cast<void**>(&c->sin_d), std::max<size_t>(tb, 16), "sin table"));
        XN_CREATE_CUDA(cudaMemcpyAsync(c->cos_d, d->rope_cos, tb, cudaMemcpyHostToDevice, c->stream));
        XN_CREATE_CUDA(cudaMemcpyAsync(c->sin_d, d->rope_sin, tb, cudaMemcpyHostToDevice, c->stream));
    }
    c->sync_cap = size_t(c->decode_chunks) + 8;  // a unit is cut at most once per chunk boundary
    XN_CREATE_CUDA(guarded_malloc(c, reinterpret_cast<void**>(&c->sync_d), c->sync_cap * sizeof(int), "arrival counters"));
    XN_CREATE_CUDA(cudaMemsetAsync(c->sync_d, 0, c->sync_cap * sizeof(int), c->stream));
    XN_CREATE_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&c->status_h), sizeof(int), cudaHostAllocMapped));
    *c->status_h = kDevOk;
    XN_CREATE_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&c->status_d), c->status_h, 0));

    if (c->kv_u8) {
        XN_CREATE_CUDA(cudaFuncSetAttribute(reinterpret_cast<const void*>(pick_split8(c->dq, c->gt, c->kv8_epl)),
                                            cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            int(kv8::smem_bytes(c->gt, c->kv8_epl))));
    } else {
        SplitKernel k = pick_split(c->nv_class, c->gt, c->nv_exact);
        XN_CREATE_CUDA(cudaFuncSetAttribute(reinterpret_cast<const void*>(k.fn),
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, int(k.smem)));
        const PrefillF32Kernel pk = pick_prefill_f32(c->nv);
        XN_CREATE_CUDA(cudaFuncSetAttribute(reinterpret_cast<const void*>(pk.fn),
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, int(pk.smem_max)));
    }

    // tensor-core prefill: possible when rows are exactly head_dim floats and TMA can address them
    {
        const unsigned long long rows = (unsigned long long)pages * d->num_layers * d->num_kv_heads * kPageTokens;
        if (c->kv_u8) {
            // the kernel reads a dequantised staging area, mapped when the first prefill needs it
            c->tf32_ok = d->head_dim % 4 == 0 && d->head_dim >= 16 && d->head_dim <= 128 && encode_tiled_fn() != nullptr;
            if (c->tf32_ok)
                XN_CREATE_CUDA(cudaFuncSetAttribute(reinterpret_cast<const void*>(prefill_tf32_kernel<false>),
                                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    pf::kSmemBytes));
        } else if (d->head_dim % 4 == 0 && d->head_dim >= 16 && d->head_dim <= 128 && rows < (1ull << 31)) {
            const cuuint64_t dims[2] = {cuuint64_t(d->head_dim), cuuint64_t(rows)};
            const cuuint64_t str[1] = {cuuint64_t(d->head_dim) * 4};
            const cuuint32_t box[2] = {32, cuuint32_t(pf::kPage)};
            c->tf32_ok = make_map_f32(&c->k_map, c->k_pool, 2, dims, str, box) &&
                         // V is consumed MN-major: 32-byte-chunk swizzle
                         make_map_f32(&c->v_map, c->v_pool, 2, dims, str, box,
                                      CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
            if (c->tf32_ok) {
                XN_CREATE_CUDA(cudaFuncSetAttribute(reinterpret_cast<const void*>(prefill_tf32_kernel<false>),
                                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    pf::kSmemBytes));
                XN_CREATE_CUDA(cudaFuncSetAttribute(reinterpret_cast<const void*>(prefill_tf32_kernel<true>),
                                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    pf::kSmemBytes));
            }
        }
        if (const char* env = getenv("XORNET_ATTN_TF32_MIN_ROWS")) {
            int v = atoi(env);
            if (v > 0) c->tf32_min_rows = v;
        }
        if (d->prefill_mode == XN_PREFILL_TF32 && !c->tf32_ok) {
            fail(nullptr, XN_ERR_SHAPE, "head_dim %d cannot use the TF32 prefill kernel", d->head_dim);
            return bail(XN_ERR_SHAPE);
        }
    }

    c->free_pages.resize(size_t(pages));
    for (long long i = 0; i < pages; ++i) c->free_pages[size_t(i)] = int32_t(pages - 1 - i);
    if (d->shuffle_seed) {  // Fisher-Yates with the counter-based generator
        uint64_t ctr = 0;
        for (size_t i = c->free_pages.size(); i > 1; --i) {
            size_t j = size_t(mix64(d->shuffle_seed * 0x9E3779B97F4A7C15ull + ctr++) % i);
            std::swap(c->free_pages[i - 1], c->free_pages[j]);
        }
    }
    c->stats.pages_total = uint64_t(pages);
    XN_CREATE_CUDA(cudaStreamSynchronize(c->stream));
#undef XN_CREATE_CUDA
    *out_ctx = c;
    return XN_OK;
}

int32_t xn_ctx_destroy(xn_ctx* c) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    for (xn_stream* s : c->streams) {
        free_call_buffer(s);
        s->magic = 0;
        delete s;
    }
    c->streams.clear();
    for (PlanSlot& s : c->slots) {
        if (s.host) cudaFreeHost(s.host);
        guarded_free(c, s.dev);
        if (s.ev) cudaEventDestroy(s.ev);
        if (s.up_ev) cudaEventDestroy(s.up_ev);
    }
    for (cudaEvent_t e : c->prof_events) cudaEventDestroy(e);
    for (std::vector<OutProj>* v : {&c->out_proj, &c->qkv_proj})
        for (OutProj& op : *v) {
            guarded_free(c, op.w2);
            guarded_free(c, op.w_scales);
            guarded_free(c, op.norm_w);
        }
    guarded_free(c, c->qkv_seq);
    guarded_free(c, c->attn_seq);
    guarded_free(c, c->q8);
    guarded_free(c, c->q_rot);
    if (c->out_stage) guarded_free(c, c->out_stage);
    for (cudaEvent_t ev : c->done_events) cudaEventDestroy(ev);
    for (OutSlab& sl : c->slabs)
        if (sl.host) cudaFreeHost(sl.host);
    guarded_free(c, c->partials);
    if (c->io_host) cudaFreeHost(c->io_host);
    guarded_free(c, c->io_dev);
    guarded_free(c, c->sync_d);
    if (c->status_h) cudaFreeHost(c->status_h);
    guarded_free(c, c->cos_d);
    guarded_free(c, c->sin_d);
    guarded_free(c, c->k_pool);
    guarded_free(c, c->v_pool);
    guarded_free(c, c->pool8);
    guarded_free(c, c->k_stage);
    guarded_free(c, c->v_stage);
    guarded_free(c, c->stage_ident_d);
    if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
    if (c->own_stream && c->stream) cudaStreamDestroy(c->stream);
    c->magic = 0;
    delete c;
    return XN_OK;
}

int32_t xn_ctx_synchronize(xn_ctx* c) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    XN_CUDA(c, cudaSetDevice(c->device));
    XN_CUDA(c, cudaStreamSynchronize(c->stream));
    return check_device_status(c);
}

void* xn_ctx_cuda_stream(xn_ctx* c) { return ctx_ok(c) ? static_cast<void*>(c->stream) : nullptr; }

int32_t xn_stats_get(xn_ctx* c, xn_stats* out) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    if (!out) return XN_ERR_ARG;
    std::lock_guard<std::mutex> g(c->mu);
    c->stats.pages_in_use = c->stats.pages_total - c->free_pages.size();
    c->stats.streams_live = c->streams.size();
    *out = c->stats;
    return XN_OK;
}

int32_t xn_profile_enable(xn_ctx* c, int32_t on) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    c->profile = on != 0;
    return XN_OK;
}

int32_t xn_profile_read_all(xn_ctx* c, double* ms, uint64_t* launches) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    XN_CUDA(c, cudaSetDevice(c->device));
    XN_CUDA(c, cudaStreamSynchronize(c->stream));
    double total[XN_PROFILE_KINDS] = {};
    uint64_t count[XN_PROFILE_KINDS] = {};
    for (size_t i = 0; i + 1 < c->prof_used; i += 2) {
        float t = 0.f;
        XN_CUDA(c, cudaEventElapsedTime(&t, c->prof_events[i], c->prof_events[i + 1]));
        const int kind = std::min(std::max(c->prof_kind[i / 2], 0), XN_PROFILE_KINDS - 1);
        total[kind] += t;
        count[kind] += 1;
    }
    for (int k = 0; k < XN_PROFILE_KINDS; ++k) {
        if (ms) ms[k] = total[k];
        if (launches) launches[k] = count[k];
    }
    c->prof_used = 0;
    return XN_OK;
}

int32_t xn_profile_read(xn_ctx* c, double* splitkv_ms, uint64_t* splitkv_launches,
                        double* prefill_ms, uint64_t* prefill_launches) {
    double ms[XN_PROFILE_KINDS];
    uint64_t n[XN_PROFILE_KINDS];
    const int32_t rc = xn_profile_read_all(c, ms, n);
    if (rc != XN_OK) return rc;
    if (splitkv_ms) *splitkv_ms = ms[0];
    if (splitkv_launches) *splitkv_launches = n[0];
    if (prefill_ms) *prefill_ms = ms[1];
    if (prefill_launches) *prefill_launches = n[1];
    return XN_OK;
}

int32_t xn_stream_create(xn_ctx* c, int64_t max_seq_len, xn_stream** out) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    if (!out) return XN_ERR_ARG;
    *out = nullptr;
    std::lock_guard<std::mutex> g(c->mu);
    if (max_seq_len <= 0) return fail(c, XN_ERR_ARG, "max_seq_len must be positive");
    xn_stream* s = new (std::nothrow) xn_stream();
    if (!s) return fail(c, XN_ERR_NOMEM, "out of host memory");
    s->ctx = c;
    s->cap = max_seq_len;
    s->hw.assign(size_t(c->num_layers), 0);
    {
        std::lock_guard<std::mutex> q(c->q_mu);
        c->streams.insert(s);
    }
    *out = s;
    return XN_OK;
}

int32_t xn_stream_reset(xn_ctx* c, xn_stream* s) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    if (!stream_ok(c, s)) return fail(c, XN_ERR_HANDLE, "stream handle is not live");
    // Pages may still be read by launches already enqueued: finish them before reuse.
    XN_CUDA(c, cudaSetDevice(c->device));
    XN_CUDA(c, cudaStreamSynchronize(c->stream));
    release_pages(c, s);
    return XN_OK;
}

int32_t xn_stream_destroy(xn_ctx* c, xn_stream* s) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    if (!stream_ok(c, s)) return fail(c, XN_ERR_HANDLE, "stream handle is not live");
    XN_CUDA(c, cudaSetDevice(c->device));
    XN_CUDA(c, cudaStreamSynchronize(c->stream));
    release_pages(c, s);
    {
        std::lock_guard<std::mutex> q(c->q_mu);
        c->streams.erase(s);
    }
    free_call_buffer(s);
    s->magic = 0;
    delete s;
    return XN_OK;
}

int32_t xn_attention(xn_ctx* c, xn_stream* s, int32_t layer, int64_t index_pos, int32_t seq_len,
                     const float* q, const float* k, const float* v, float* out) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    xn_req r{s, layer, seq_len, index_pos, q, k, v, out, 0u, 0u};
    return attention_blocking(c, r);
}

int32_t xn_attention_rope(xn_ctx* c, xn_stream* s, int32_t layer, int64_t index_pos,
                          int32_t seq_len, const float* q, const float* k, const float* v,
                          float* out) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    xn_req r{s, layer, seq_len, index_pos, q, k, v, out, XN_REQ_ROPE, 0u};
    return attention_blocking(c, r);
}

int32_t xn_attention_batch(xn_ctx* c, int32_t n, const xn_req* reqs) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    if (n < 0 || (n > 0 && !reqs)) return fail(c, XN_ERR_ARG, "bad request array");
    if (n == 0) return XN_OK;
    const bool dev = reqs[0].flags & XN_REQ_DEVICE_PTRS;
    std::unordered_set<xn_stream*> seen;
    for (int i = 0; i < n; ++i) {
        int32_t rc = validate_req(c, reqs[i]);
        if (rc != XN_OK) return rc;
        if (bool(reqs[i].flags & XN_REQ_DEVICE_PTRS) != dev)
            return fail(c, XN_ERR_ARG, "host and device requests mixed in one batch");
        if ((reqs[i].flags & XN_REQ_HOST_PINNED) != (reqs[0].flags & XN_REQ_HOST_PINNED) ||
            (dev && (reqs[i].flags & XN_REQ_HOST_PINNED)))
            return fail(c, XN_ERR_ARG, "XN_REQ_HOST_PINNED must be set on all host requests of a batch or on none");
        if (!seen.insert(reqs[i].stream).second)
            return fail(c, XN_ERR_ARG, "request %d repeats a stream of this batch", i);
    }
    return submit_locked(c, n, reqs, !dev);
}

// ---- device groups: one context per GPU, streams placed on the least-loaded one ----------------

int32_t xn_place_stream(int32_t n_devices, const int64_t* tokens, const int64_t* live_streams,
                        uint64_t ticket, int32_t policy) {
    if (n_devices <= 0) return -XN_ERR_ARG;
    const int start = int(ticket % uint64_t(n_devices));
    if (policy == XN_PLACE_ROUND_ROBIN || !tokens) return start;
    if (policy != XN_PLACE_LEAST_LOADED) return -XN_ERR_ARG;
    int best = start;
    for (int k = 1; k < n_devices; ++k) {   // ties go to the round-robin candidate, then onwards from it
        const int i = (start + k) % n_devices;
        const int64_t li = live_streams ? live_streams[i] : 0, lb = live_streams ? live_streams[best] : 0;
        if (tokens[i] < tokens[best] || (tokens[i] == tokens[best] && li < lb)) best = i;
    }
    return best;
}

static bool group_ok(const xn_group* g) { return g && g->magic == 0x786e4752u; }

int32_t xn_group_create(const xn_ctx_desc* desc, const int32_t* devices, int32_t n_devices, xn_group** out) {
    if (!desc || !out || n_devices < 0 || (n_devices > 0 && !devices))
        return fail(nullptr, XN_ERR_ARG, "null descriptor, output or device list");
    *out = nullptr;
    std::vector<int32_t> devs(devices, devices + n_devices);
    if (devs.empty()) {
        if (const char* env = getenv("XORNET_ATTN_DEVICES")) {   // "0,2,3"
            for (const char* p = env; *p;) {
                char* end = nullptr;
                const long v = strtol(p, &end, 10);
                if (end == p) break;
                devs.push_back(int32_t(v));
                p = *end ? end + 1 : end;
            }
        }
        if (devs.empty()) {
            int n = 0;
            if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0)
                return fail(nullptr, XN_ERR_NO_DEVICE, "no CUDA device; this library has no CPU fallback");
            for (int i = 0; i < n; ++i) devs.push_back(i);
        }
    }
    xn_group* g = new (std::nothrow) xn_group();
    if (!g) return fail(nullptr, XN_ERR_NOMEM, "out of host memory");
    for (int32_t dev : devs) {
        xn_ctx_desc d = *desc;
        d.device = dev;
        d.cuda_stream = nullptr;   // a caller's stream belongs to one device: each context makes its own
        xn_ctx* c = nullptr;
        const int32_t rc = xn_ctx_create(&d, &c);
        if (rc != XN_OK) {
            for (xn_ctx* made : g->ctxs) xn_ctx_destroy(made);
            g->magic = 0;
            delete g;
            return rc;   // the text of xn_ctx_create stays in xn_last_error(NULL)
        }
        g->ctxs.push_back(c);
    }
    *out = g;
    return XN_OK;
}

int32_t xn_group_destroy(xn_group* g) {
    if (!group_ok(g)) return XN_ERR_HANDLE;
    for (xn_ctx* c : g->ctxs) xn_ctx_destroy(c);
    g->magic = 0;
    delete g;
    return XN_OK;
}

int32_t xn_group_size(xn_group* g) { return group_ok(g) ? int32_t(g->ctxs.size()) : -XN_ERR_HANDLE; }

xn_ctx* xn_group_ctx(xn_group* g, int32_t i) {
    return group_ok(g) && i >= 0 && size_t(i) < g->ctxs.size() ? g->ctxs[size_t(i)] : nullptr;
}

int32_t xn_group_stream_create(xn_group* g, int64_t max_seq_len, int64_t expected_tokens, int32_t policy,
                               xn_ctx** ctx_out, xn_stream** stream_out) {
    if (!group_ok(g)) return XN_ERR_HANDLE;
    if (!ctx_out || !stream_out || expected_tokens < 0) return fail(nullptr, XN_ERR_ARG, "bad argument");
    *ctx_out = nullptr;
    *stream_out = nullptr;
    std::lock_guard<std::mutex> lk(g->mu);   // placements are decided one at a time
    const int n = int(g->ctxs.size());
    std::vector<int64_t> tokens(size_t(n), 0), live(size_t(n), 0);
    for (int i = 0; i < n; ++i) {
        xn_ctx* c = g->ctxs[size_t(i)];
        std::lock_guard<std::mutex> cl(c->mu);
        for (const xn_stream* s : c->streams) {   // what the stream holds, or what it was announced to hold
            int64_t len = 0;
            for (int64_t h : s->hw) len = std::max(len, std::min(h, s->cap));
            tokens[size_t(i)] += std::max(len, s->expected);
        }
        live[size_t(i)] = int64_t(c->streams.size());
    }
    const int where = xn_place_stream(n, tokens.data(), live.data(), g->ticket, policy);
    if (where < 0) return fail(nullptr, XN_ERR_ARG, "unknown placement policy %d", policy);
    xn_ctx* c = g->ctxs[size_t(where)];
    const int32_t rc = xn_stream_create(c, max_seq_len, stream_out);
    if (rc != XN_OK) return rc;
    {
        std::lock_guard<std::mutex> cl(c->mu);
        (*stream_out)->expected = std::min(expected_tokens, max_seq_len);
    }
    g->ticket += 1;
    *ctx_out = c;
    return XN_OK;
}

int32_t xn_rope_tables(float theta, int32_t head_dim, int32_t max_pos, float factor,
                       float low_freq_factor, float high_freq_factor, int32_t original_max_pos,
                       float* cos_out, float* sin_out) {
    if (head_dim <= 0 || max_pos < 0 || !cos_out || !sin_out) return XN_ERR_ARG;
    const int half = head_dim / 2;
    const int nfreq = (head_dim + 1) / 2;
    std::vector<float> inv;
    inv.resize(size_t(nfreq));
    for (int j = 0; j < nfreq; ++j)  // models/llama/mod.rs:210-216
        inv[size_t(j)] = 1.0f / powf(theta, float(2 * j) / float(head_dim));
    if (factor > 0.0f) {  // models/llama/mod.rs:226-249
        const float pi = 3.14159265358979323846f;
        const float low_wl = float(original_max_pos) / low_freq_factor;
        const float high_wl = float(original_max_pos) / high_freq_factor;
        for (float& fr : inv) {
            const float wl = 2.0f * pi / fr;
            if (wl < high_wl) continue;
            if (wl > low_wl) {
                fr = fr / factor;
            } else {
                const float smooth = (float(original_max_pos) / wl - low_freq_factor) /
                                     (high_freq_factor - low_freq_factor);
                fr = (1.0f - smooth) * fr / factor + smooth * fr;
            }
        }
    }
    for (int pos = 0; pos < max_pos; ++pos)  // models/llama/mod.rs:252-262
        for (int i = 0; i < half; ++i) {
            const float a = float(pos) * inv[size_t(i)];
            cos_out[size_t(pos) * half + i] = cosf(a);
            sin_out[size_t(pos) * half + i] = sinf(a);
        }
    return XN_OK;
}

// ---- cache inspection / synthetic fill ------------------------------------------------------

static int32_t upload_pages(xn_ctx* c, xn_stream* s, const int** pages_d, PlanSlot** slot_out) {
    PlanSlot* slot = nullptr;
    int32_t rc = acquire_slot(c, std::max<size_t>(16, s->pages.size() * 4), &slot);
    if (rc != XN_OK) return rc;
    memcpy(slot->host, s->pages.data(), s->pages.size() * 4);
    XN_CUDA(c, cudaMemcpyAsync(slot->dev, slot->host, std::max<size_t>(16, s->pages.size() * 4),
                               cudaMemcpyHostToDevice, c->stream));
    *pages_d = reinterpret_cast<const int*>(slot->dev);
    *slot_out = slot;
    return XN_OK;
}

// u8 cache format: dequantised rows and / or the stored bytes and scales of slots [t0, t0+n).
// Called with the context lock held and the arguments checked.
static int32_t kv_read_u8_locked(xn_ctx* c, xn_stream* s, int32_t layer, int64_t t0, int64_t n,
                                 float* k_out, float* v_out, uint8_t* k_u8, uint8_t* v_u8,
                                 float* k_sc, float* v_sc) {
    const size_t D = size_t(c->head_dim), H = size_t(c->num_kv_heads);
    const size_t elems = size_t(n) * H * D, rows = size_t(n) * H;
    if (k_out) memset(k_out, 0, elems * 4);
    if (v_out) memset(v_out, 0, elems * 4);
    if (k_u8) memset(k_u8, 128, elems);
    if (v_u8) memset(v_u8, 128, elems);
    if (k_sc) memset(k_sc, 0, rows * 4);
    if (v_sc) memset(v_sc, 0, rows * 4);
    const int64_t have = std::min<int64_t>(
        {int64_t(s->pages.size()) * kPageTokens, t0 + n, std::min<int64_t>(s->hw[size_t(layer)], s->cap)});
    if (have <= t0) return XN_OK;
    const int64_t m = have - t0;
    const size_t melems = size_t(m) * H * D, mrows = size_t(m) * H;
    const size_t o_v = melems * 4, o_ks = 2 * melems * 4, o_vs = o_ks + mrows * 4, o_kr = o_vs + mrows * 4,
                 o_vr = o_kr + melems, total_bytes = o_vr + melems;
    int32_t rc = grow_io(c, total_bytes);
    if (rc != XN_OK) return rc;
    const int* pages_d = nullptr;
    PlanSlot* slot = nullptr;
    if ((rc = upload_pages(c, s, &pages_d, &slot)) != XN_OK) return rc;
    unsigned char* b = c->io_dev;
    const int blocks = int(std::min<size_t>((melems + 255) / 256, 8192));
    kv8::slots_gather_u8_kernel<<<blocks, 256, 0, c->stream>>>(
        pages_d, c->pool8, c->pool_pages, layer, c->num_kv_heads, c->head_dim, c->dq, t0, m,
        reinterpret_cast<float*>(b), reinterpret_cast<float*>(b + o_v), b + o_kr, b + o_vr,
        reinterpret_cast<float*>(b + o_ks), reinterpret_cast<float*>(b + o_vs));
    c->stats.kernel_launches += 1;
    XN_CUDA(c, cudaGetLastError());
    XN_CUDA(c, cudaMemcpyAsync(c->io_host, c->io_dev, total_bytes, cudaMemcpyDeviceToHost, c->stream));
    XN_CUDA(c, cudaEventRecord(slot->ev, c->stream));
    slot->used = true;
    XN_CUDA(c, cudaStreamSynchronize(c->stream));
    const unsigned char* hb = c->io_host;
    for (size_t h = 0; h < H; ++h) {  // [Hkv, m, ...] -> [Hkv, n, ...]
        if (k_out) memcpy(k_out + h * n * D, hb + h * m * D * 4, size_t(m) * D * 4);
        if (v_out) memcpy(v_out + h * n * D, hb + o_v + h * m * D * 4, size_t(m) * D * 4);
        if (k_u8) memcpy(k_u8 + h * n * D, hb + o_kr + h * m * D, size_t(m) * D);
        if (v_u8) memcpy(v_u8 + h * n * D, hb + o_vr + h * m * D, size_t(m) * D);
        if (k_sc) memcpy(k_sc + h * n, hb + o_ks + h * m * 4, size_t(m) * 4);
        if (v_sc) memcpy(v_sc + h * n, hb + o_vs + h * m * 4, size_t(m) * 4);
    }
    return XN_OK;
}

int32_t xn_kv_read_u8(xn_ctx* c, xn_stream* s, int32_t layer, int64_t t0, int64_t n, uint8_t* k_u8,
                      uint8_t* v_u8, float* k_scales, float* v_scales) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    if (!stream_ok(c, s)) return fail(c, XN_ERR_HANDLE, "stream handle is not live");
    if (!c->kv_u8) return fail(c, XN_ERR_ARG, "xn_kv_read_u8: the context keeps the f32 cache format");
    if (layer < 0 || layer >= c->num_layers || t0 < 0 || n < 0 || t0 + n > s->cap)
        return fail(c, XN_ERR_ARG, "slot range outside the stream's capacity");
    if (n == 0) return XN_OK;
    XN_CUDA(c, cudaSetDevice(c->device));
    return kv_read_u8_locked(c, s, layer, t0, n, nullptr, nullptr, k_u8, v_u8, k_scales, v_scales);
}

int32_t xn_kv_read_range(xn_ctx* c, xn_stream* s, int32_t layer, int64_t t0, int64_t n,
                         float* k_out, float* v_out) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    if (!stream_ok(c, s)) return fail(c, XN_ERR_HANDLE, "stream handle is not live");
    if (layer < 0 || layer >= c->num_layers || t0 < 0 || n < 0 || t0 + n > s->cap)
        return fail(c, XN_ERR_ARG, "slot range outside the stream's capacity");
    if (n == 0) return XN_OK;
    XN_CUDA(c, cudaSetDevice(c->device));
    if (c->kv_u8) return kv_read_u8_locked(c, s, layer, t0, n, k_out, v_out, nullptr, nullptr, nullptr, nullptr);
    const size_t elems = size_t(n) * c->num_kv_heads * c->head_dim;
    if (k_out) memset(k_out, 0, elems * 4);
    if (v_out) memset(v_out, 0, elems * 4);
    // slots without a page were never written: zeros
    // slots at or beyond the highest written position of this layer were never written either
    const int64_t have = std::min<int64_t>(
        {int64_t(s->pages.size()) * kPageTokens, t0 + n, std::min<int64_t>(s->hw[size_t(layer)], s->cap)});
    if (have <= t0) return XN_OK;
    const int64_t m = have - t0;
    const size_t melems = size_t(m) * c->num_kv_heads * c->head_dim;
    int32_t rc = grow_io(c, 2 * melems * 4);
    if (rc != XN_OK) return rc;
    const int* pages_d = nullptr;
    PlanSlot* slot = nullptr;
    if ((rc = upload_pages(c, s, &pages_d, &slot)) != XN_OK) return rc;
    float* kd = reinterpret_cast<float*>(c->io_dev);
    float* vd = kd + melems;
    const int blocks = int(std::min<size_t>((melems + 255) / 256, 8192));
    slots_gather_kernel<<<blocks, 256, 0, c->stream>>>(pages_d, c->k_pool, c->v_pool, c->pool_pages,
                                                       layer, c->num_kv_heads, c->head_dim, c->nv,
                                                       t0, m, kd, vd);
    c->stats.kernel_launches += 1;
    XN_CUDA(c, cudaGetLastError());
    XN_CUDA(c, cudaMemcpyAsync(c->io_host, c->io_dev, 2 * melems * 4, cudaMemcpyDeviceToHost, c->stream));
    XN_CUDA(c, cudaEventRecord(slot->ev, c->stream));
    slot->used = true;
    XN_CUDA(c, cudaStreamSynchronize(c->stream));
    const float* kh = reinterpret_cast<const float*>(c->io_host);
    const float* vh = kh + melems;
    const size_t D = size_t(c->head_dim);
    for (int h = 0; h < c->num_kv_heads; ++h) {  // [Hkv, m, D] -> [Hkv, n, D]
        if (k_out) memcpy(k_out + size_t(h) * n * D, kh + size_t(h) * m * D, size_t(m) * D * 4);
        if (v_out) memcpy(v_out + size_t(h) * n * D, vh + size_t(h) * m * D, size_t(m) * D * 4);
    }
    return XN_OK;
}

int32_t xn_kv_read(xn_ctx* c, xn_stream* s, int32_t layer, int32_t kv_head, int64_t t, float* k_row,
                   float* v_row) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    if (!stream_ok(c, s)) return XN_ERR_HANDLE;
    if (kv_head < 0 || kv_head >= c->num_kv_heads || t < 0) return XN_ERR_ARG;
    const size_t D = size_t(c->head_dim);
    std::vector<float> kb(size_t(c->num_kv_heads) * D), vb(size_t(c->num_kv_heads) * D);
    int32_t rc = xn_kv_read_range(c, s, layer, t % s->cap, 1, kb.data(), vb.data());
    if (rc != XN_OK) return rc;
    if (k_row) memcpy(k_row, kb.data() + size_t(kv_head) * D, D * 4);
    if (v_row) memcpy(v_row, vb.data() + size_t(kv_head) * D, D * 4);
    return XN_OK;
}

int32_t xn_kv_fill_normal(xn_ctx* c, xn_stream* s, int32_t layer, int64_t t0, int64_t n,
                          uint64_t seed) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    if (!stream_ok(c, s)) return fail(c, XN_ERR_HANDLE, "stream handle is not live");
    if (layer < -1 || layer >= c->num_layers || t0 < 0 || n < 0 || t0 + n > s->cap)
        return fail(c, XN_ERR_ARG, "slot range outside the stream's capacity");
    if (n == 0) return XN_OK;
    XN_CUDA(c, cudaSetDevice(c->device));
    int32_t rc = ensure_pages(c, s, t0 + n);
    if (rc != XN_OK) return rc;
    const int* pages_d = nullptr;
    PlanSlot* slot = nullptr;
    if ((rc = upload_pages(c, s, &pages_d, &slot)) != XN_OK) return rc;
    const long long total = n * c->num_kv_heads * c->head_dim;
    const int blocks = int(std::min<long long>((total + 255) / 256, 8192));
    const int l0 = layer < 0 ? 0 : layer, l1 = layer < 0 ? c->num_layers : layer + 1;
    for (int l = l0; l < l1; ++l) {
        if (c->kv_u8)
            kv8::slots_fill_u8_kernel<<<int(std::min<long long>((n * c->num_kv_heads + 7) / 8, 8192)), 256, 0,
                                        c->stream>>>(pages_d, c->pool8, c->pool_pages, l, c->num_kv_heads,
                                                     c->head_dim, c->dq, t0, n, 1,
                                                     seed + 0x632BE59BD9B4E019ull * uint64_t(l));
        else
        slots_fill_kernel<<<blocks, 256, 0, c->stream>>>(pages_d, c->k_pool, c->v_pool, c->pool_pages,
                                                         l, c->num_kv_heads, c->head_dim, c->nv, t0,
                                                         n, 1, seed + 0x632BE59BD9B4E019ull * uint64_t(l));
        c->stats.kernel_launches += 1;
        s->hw[size_t(l)] = std::max<int64_t>(s->hw[size_t(l)], t0 + n);
    }
    XN_CUDA(c, cudaGetLastError());
    XN_CUDA(c, cudaEventRecord(slot->ev, c->stream));
    slot->used = true;
    return XN_OK;
}

int32_t xn_fill_normal(xn_ctx* c, float* device_ptr, int64_t n, uint64_t seed) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    if (!device_ptr || n < 0) return fail(c, XN_ERR_ARG, "bad buffer");
    if (n == 0) return XN_OK;
    XN_CUDA(c, cudaSetDevice(c->device));
    const int blocks = int(std::min<long long>((n + 255) / 256, 8192));
    fill_normal_kernel<<<blocks, 256, 0, c->stream>>>(device_ptr, n, seed);
    c->stats.kernel_launches += 1;
    XN_CUDA(c, cudaGetLastError());
    return XN_OK;
}

int64_t xn_stream_len(xn_ctx* c, xn_stream* s, int32_t layer) {
    if (!ctx_ok(c) || !stream_ok(c, s) || layer < 0 || layer >= c->num_layers) return -1;
    std::lock_guard<std::mutex> g(c->mu);
    return s->hw[size_t(layer)];
}

int64_t xn_stream_pages(xn_ctx* c, xn_stream* s, int32_t* out, int64_t max_out) {
    if (!ctx_ok(c) || !stream_ok(c, s)) return -1;
    std::lock_guard<std::mutex> g(c->mu);
    const int64_t n = int64_t(s->pages.size());
    for (int64_t i = 0; i < n && i < max_out && out; ++i) out[i] = s->pages[size_t(i)];
    return n;
}

// ---- attention output block ------------------------------------------------------------------

int32_t xn_ternary_pack(int32_t in_dim, int32_t out_dim, const float* weights, int32_t pack_type,
                        float provided_scale, uint8_t* packed, float* w_scales) {
    if (in_dim < 0 || out_dim < 0 || !weights || !packed || !w_scales) return XN_ERR_ARG;
    if (pack_type != XN_PACK4 && pack_type != XN_PACK5) return XN_ERR_ARG;
    ternary_linear_pack(size_t(in_dim), size_t(out_dim), weights, pack_type, !std::isnan(provided_scale),
                        provided_scale, packed, w_scales);
    return XN_OK;
}

namespace {
struct LinearPart {
    const uint8_t* packed;
    const float* scales;
    int rows;
};

// Builds the device form of a ternary linear layer whose rows are the concatenation of `parts`
// (all with the same in_dim and packing) and stores it in *slot, replacing what was there.
int32_t install_linear(xn_ctx* c, OutProj* slot, int in_dim, int pack_type, const LinearPart* parts,
                       int n_parts, const float* norm_weight, float norm_eps) {
    if (pack_type != XN_PACK4 && pack_type != XN_PACK5 && pack_type != XN_SPARSE)
        return fail(c, XN_ERR_ARG, "pack_type must be XN_PACK4, XN_PACK5 or XN_SPARSE");
    if (in_dim <= 0 || size_t(in_dim) * 12 > 200 * 1024)
        return fail(c, XN_ERR_CAPACITY, "in_dim %d outside what one block's shared memory holds", in_dim);
    long long out_dim = 0;
    for (int i = 0; i < n_parts; ++i) {
        if (!parts[i].packed || !parts[i].scales || parts[i].rows <= 0)
            return fail(c, XN_ERR_ARG, "null weight pointer or empty projection");
        out_dim += parts[i].rows;
    }
    if (out_dim > (1 << 20)) return fail(c, XN_ERR_SHAPE, "out_dim %lld outside 1..2^20", out_dim);
    XN_CUDA(c, cudaSetDevice(c->device));
    XN_CUDA(c, cudaStreamSynchronize(c->stream));  // launches in flight may still read the old weights

    OutProj op;
    op.in_dim = in_dim;
    op.out_dim = int(out_dim);
    op.q_stride = int(align_up(size_t(in_dim), 128));
    op.w_stride = op.q_stride / 4;
    op.eps = norm_eps;
    const size_t bpr = pack_type == XN_SPARSE ? 0 : packed_row_bytes(size_t(in_dim), pack_type);
    // device layout: [row / 32][K / 128][32 rows][32 bytes] (code_offset); rows past out_dim and
    // columns past in_dim hold code 1 = weight 0
    const int nkb = op.q_stride / 128;
    std::vector<uint8_t> w2(size_t((out_dim + 31) / 32) * nkb * 1024, uint8_t(0x55));
    std::vector<float> scales(size_t(out_dim), 0.f);
    std::vector<uint8_t> row_codes(size_t(op.w_stride));
    int o = 0;
    for (int i = 0; i < n_parts; ++i) {
        const uint8_t* sparse_row = parts[i].packed;   // XN_SPARSE: rows are found by walking the blob
        for (int rr = 0; rr < parts[i].rows; ++rr, ++o) {
            if (pack_type == XN_SPARSE) {
                const size_t used = recode_sparse_row_2bit(sparse_row, size_t(in_dim), row_codes.data(),
                                                           row_codes.size());
                if (used == 0)
                    return fail(c, XN_ERR_SHAPE, "sparse row %d does not describe %d columns", o, in_dim);
                sparse_row += used;
            } else {
                recode_row_2bit(parts[i].packed + size_t(rr) * bpr, size_t(in_dim), pack_type, row_codes.data(),
                                row_codes.size());
            }
            for (int kb = 0; kb < nkb; ++kb)
                memcpy(w2.data() + code_offset(o, kb * 128, nkb), row_codes.data() + size_t(kb) * 32, 32);
            scales[size_t(o)] = parts[i].scales[rr];
        }
    }
    auto upload = [&](void** dst, const void* src, size_t bytes) -> cudaError_t {
        cudaError_t e = guarded_malloc(c, dst, bytes, "projection weights");
        if (e != cudaSuccess) return e;
        return cudaMemcpy(*dst, src, bytes, cudaMemcpyHostToDevice);
    };
    cudaError_t e = upload(reinterpret_cast<void**>(&op.w2), w2.data(), w2.size());
    if (e == cudaSuccess) e = upload(reinterpret_cast<void**>(&op.w_scales), scales.data(), scales.size() * 4);
    if (e == cudaSuccess && norm_weight)
        e = upload(reinterpret_cast<void**>(&op.norm_w), norm_weight, size_t(in_dim) * 4);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(reinterpret_cast<const void*>(ternary_gemm_kernel),
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, kOutGemmSmem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(reinterpret_cast<const void*>(ternary_gemm_tc_kernel),
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, tg::smem_bytes(tg::max_nkb()));
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(reinterpret_cast<const void*>(ternary_gemm_rows_kernel),
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, tgr::smem_bytes(tgr::max_nkb()));
    if (e == cudaSuccess && align_up(size_t(in_dim), 4) * 12 > 40 * 1024)  // static shared memory counts too
        e = cudaFuncSetAttribute(reinterpret_cast<const void*>(subnorm_quant_kernel),
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(align_up(size_t(in_dim), 4) * 12));
    if (e != cudaSuccess) {
        guarded_free(c, op.w2);
        guarded_free(c, op.w_scales);
        guarded_free(c, op.norm_w);
        return fail(c, XN_ERR_CUDA, "uploading the weights failed: %s", cudaGetErrorString(e));
    }
    guarded_free(c, slot->w2);
    guarded_free(c, slot->w_scales);
    guarded_free(c, slot->norm_w);
    op.set = true;
    *slot = op;
    return XN_OK;
}
}  // namespace

int32_t xn_ternary_pack_sparse(int32_t in_dim, int32_t out_dim, const float* weights, float provided_scale,
                               uint8_t* blob, int64_t blob_cap, int64_t* blob_len, float* w_scales) {
    if (in_dim < 0 || out_dim < 0 || !weights || !blob || !blob_len || !w_scales || blob_cap < 0) return XN_ERR_ARG;
    const bool has_scale = !std::isnan(provided_scale);
    bool already = true;
    for (size_t i = 0; i < size_t(in_dim) * size_t(out_dim) && already; ++i)
        already = weights[i] == -1.0f || weights[i] == 0.0f || weights[i] == 1.0f;
    std::vector<uint8_t> buf;
    std::vector<int8_t> vals(size_t(in_dim) + 1);
    for (int o = 0; o < out_dim; ++o) {   // ternarize_row, src/bit1_58/layers.rs:45-88
        const float* row = weights + size_t(o) * in_dim;
        float s;
        if (already) s = has_scale ? provided_scale : 1.0f;
        else if (has_scale) s = provided_scale;
        else {
            float sum_abs = 0.0f;
            for (int i = 0; i < in_dim; ++i) sum_abs += std::fabs(row[i]);
            s = in_dim == 0 ? 1.0f : sum_abs / float(in_dim);
        }
        w_scales[o] = s;
        for (int i = 0; i < in_dim; ++i) vals[size_t(i)] = int8_t(ternary_value(row[i], s, already));
        sparse_encode_row(vals.data(), size_t(in_dim), buf);
    }
    *blob_len = int64_t(buf.size());
    if (int64_t(buf.size()) > blob_cap) return XN_ERR_CAPACITY;
    if (!buf.empty()) memcpy(blob, buf.data(), buf.size());
    return XN_OK;
}

int32_t xn_out_proj_set(xn_ctx* c, const xn_out_proj_desc* d) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    if (!d || !d->packed || !d->w_scales) return fail(c, XN_ERR_ARG, "null descriptor or weight pointer");
    if (d->layer < 0 || d->layer >= c->num_layers)
        return fail(c, XN_ERR_ARG, "layer %d outside 0..%d", d->layer, c->num_layers - 1);
    if (d->in_dim != c->num_heads * c->head_dim)
        return fail(c, XN_ERR_SHAPE, "Input dimension mismatch: expected %d, got %d",
                    c->num_heads * c->head_dim, d->in_dim);
    if (d->out_dim <= 0) return fail(c, XN_ERR_SHAPE, "out_dim %d must be positive", d->out_dim);
    const LinearPart part{d->packed, d->w_scales, d->out_dim};
    return install_linear(c, &c->out_proj[size_t(d->layer)], d->in_dim, d->pack_type, &part, 1,
                          d->norm_weight, d->norm_eps);
}

int32_t xn_qkv_proj_set(xn_ctx* c, const xn_qkv_proj_desc* d) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    if (!d) return fail(c, XN_ERR_ARG, "null descriptor");
    if (d->layer < 0 || d->layer >= c->num_layers)
        return fail(c, XN_ERR_ARG, "layer %d outside 0..%d", d->layer, c->num_layers - 1);
    const LinearPart parts[3] = {{d->q_packed, d->q_scales, c->num_heads * c->head_dim},
                                 {d->k_packed, d->k_scales, c->num_kv_heads * c->head_dim},
                                 {d->v_packed, d->v_scales, c->num_kv_heads * c->head_dim}};
    return install_linear(c, &c->qkv_proj[size_t(d->layer)], d->in_dim, d->pack_type, parts, 3, nullptr, 0.f);
}

int32_t xn_out_proj(xn_ctx* c, int32_t layer, int32_t rows, const float* y, float* out, uint32_t flags) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    if (layer < 0 || layer >= c->num_layers || !c->out_proj[size_t(layer)].set)
        return fail(c, XN_ERR_ARG, "layer %d has no output block (xn_out_proj_set)", layer);
    if (rows < 0 || (rows > 0 && (!y || !out))) return fail(c, XN_ERR_ARG, "bad rows or null tensor pointer");
    if (flags & ~uint32_t(XN_REQ_DEVICE_PTRS)) return fail(c, XN_ERR_ARG, "only XN_REQ_DEVICE_PTRS is accepted here");
    if (rows == 0) return XN_OK;
    XN_CUDA(c, cudaSetDevice(c->device));
    const OutProj& op = c->out_proj[size_t(layer)];
    const bool dev = flags & XN_REQ_DEVICE_PTRS;
    const size_t in_b = size_t(rows) * op.in_dim * 4, out_b = size_t(rows) * op.out_dim * 4;
    int32_t rc;
    const size_t q_rows_pad = align_up(size_t(rows), 256);
    if ((rc = grow_device(c, &c->q8, &c->q8_cap, q8_floats(size_t(op.q_stride), q_rows_pad))) != XN_OK) return rc;
    const float* src = y;
    float* dst = out;
    if (!dev) {
        if ((rc = grow_io(c, align_up(in_b, 16) + out_b)) != XN_OK) return rc;
        memcpy(c->io_host, y, in_b);
        XN_CUDA(c, cudaMemcpyAsync(c->io_dev, c->io_host, in_b, cudaMemcpyHostToDevice, c->stream));
        c->stats.h2d_bytes += in_b;
        src = reinterpret_cast<const float*>(c->io_dev);
        dst = reinterpret_cast<float*>(c->io_dev + align_up(in_b, 16));
    }
    PlanSlot* slot = nullptr;
    if ((rc = acquire_slot(c, sizeof(OutRowDev) * size_t(rows), &slot)) != XN_OK) return rc;
    OutRowDev* tab = reinterpret_cast<OutRowDev*>(slot->host);
    for (int t = 0; t < rows; ++t) tab[t] = {src + size_t(t) * op.in_dim, dst + size_t(t) * op.out_dim};
    XN_CUDA(c, cudaMemcpyAsync(slot->dev, slot->host, sizeof(OutRowDev) * size_t(rows),
                               cudaMemcpyHostToDevice, c->stream));
    rc = launch_out_block(c, op, reinterpret_cast<const OutRowDev*>(slot->dev), rows, 0, q_rows_pad);
    XN_CUDA(c, cudaEventRecord(slot->ev, c->stream));
    slot->used = true;
    if (rc != XN_OK) return rc;
    if (!dev) {
        XN_CUDA(c, cudaMemcpyAsync(c->io_host + align_up(in_b, 16), dst, out_b, cudaMemcpyDeviceToHost, c->stream));
        XN_CUDA(c, cudaStreamSynchronize(c->stream));
        c->stats.d2h_bytes += out_b;
        memcpy(out, c->io_host + align_up(in_b, 16), out_b);
    }
    return XN_OK;
}

int32_t xn_debug_expire_wait(xn_ctx* c, int32_t timeout_ms) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    if (timeout_ms < 1 || timeout_ms > 1000) return fail(c, XN_ERR_ARG, "timeout_ms outside 1..1000");
    XN_CUDA(c, cudaSetDevice(c->device));
    wait_probe_kernel<<<1, 32, 0, c->stream>>>(c->status_d, (unsigned long long)timeout_ms * 1000000ull);
    c->stats.kernel_launches += 1;
    XN_CUDA(c, cudaGetLastError());
    XN_CUDA(c, cudaStreamSynchronize(c->stream));
    return check_device_status(c);
}

int32_t xn_debug_drop_plan(xn_ctx* c) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    c->pcache.valid = false;
    return XN_OK;
}

int32_t xn_debug_check_guards(xn_ctx* c) {
    if (!ctx_ok(c)) return XN_ERR_HANDLE;
    std::lock_guard<std::mutex> g(c->mu);
    XN_CUDA(c, cudaSetDevice(c->device));
    XN_CUDA(c, cudaStreamSynchronize(c->stream));
    unsigned char host[2 * kGuardBytes];
    for (const xn_ctx::GuardRec& r : c->guards) {
        XN_CUDA(c, cudaMemcpy(host, r.user - kGuardBytes, kGuardBytes, cudaMemcpyDeviceToHost));
        XN_CUDA(c, cudaMemcpy(host + kGuardBytes, r.user + r.bytes, kGuardBytes, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < 2 * kGuardBytes; ++i)
            if (host[i] != kGuardByte)
                return fail(c, XN_ERR_GUARD, "a kernel wrote %s the device buffer '%s' (%zu bytes): guard byte %zu is 0x%02x",
                            i < kGuardBytes ? "in front of" : "behind", r.name, r.bytes, i % kGuardBytes, host[i]);
    }
    return XN_OK;
}

int32_t xn_plan_split(int32_t n_units, const int32_t* kv_len, int32_t tile_tokens, int32_t max_ctas,
                      int32_t max_items, int32_t* item_unit, int32_t* item_tile_begin,
                      int32_t* item_tile_end, int32_t* item_part, int32_t* cta_item_begin,
                      int32_t* n_items_out, int32_t* n_parts_out) {
    if (n_units < 0 || (n_units > 0 && !kv_len) || tile_tokens <= 0 || max_ctas <= 0) return -XN_ERR_ARG;
    SplitPlan p = plan_split(kv_len, n_units, tile_tokens, max_ctas);
    if (int32_t(p.items.size()) > max_items) return -XN_ERR_CAPACITY;
    for (size_t i = 0; i < p.items.size(); ++i) {
        if (item_unit) item_unit[i] = p.items[i].unit;
        if (item_tile_begin) item_tile_begin[i] = p.items[i].tile_begin;
        if (item_tile_end) item_tile_end[i] = p.items[i].tile_end;
        if (item_part) item_part[i] = p.items[i].part;
    }
    if (cta_item_begin)
        for (size_t i = 0; i < p.cta_item_begin.size(); ++i) cta_item_begin[i] = p.cta_item_begin[i];
    if (n_items_out) *n_items_out = int32_t(p.items.size());
    if (n_parts_out) *n_parts_out = p.n_parts;
    return p.ctas;
}

}  // extern "C"

// ============================================================================================
// Allocation-free decode entry point
// ============================================================================================

// Scratch of xn_decode_attention_static: partial (max, sum, accumulator) records of the split-KV
// pass.  It is part of the library image, so every GPU that loads the library holds these
// kStaticScratchFloats * 4 bytes (about 1.0 MiB) until the process exits.  In host code this name
// is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_static_scratch[xn::kStaticScratchFloats];

namespace {
constexpr int kStaticMaxDevices = 64;
std::mutex g_static_mu;
float* g_static_scratch_addr[kStaticMaxDevices] = {nullptr};  // per device, resolved once
}  // namespace

extern "C" int32_t xn_decode_attention_static(const float* q, const float* k_cache,
                                              const float* v_cache, float* out, int32_t num_heads,
                                              int32_t num_kv_heads, int32_t head_dim,
                                              int64_t kv_len, int64_t capacity, void* cuda_stream) {
    if (!q || !k_cache || !v_cache || !out) return fail(nullptr, XN_ERR_ARG, "null tensor pointer");
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail(nullptr, XN_ERR_SHAPE, "num_heads %d must be a positive multiple of num_kv_heads %d",
                    num_heads, num_kv_heads);
    if (head_dim < 1 || head_dim > kStaticMaxDim)
        return fail(nullptr, XN_ERR_CAPACITY,
                    "head_dim %d is beyond the static scratch limit of %d", head_dim, kStaticMaxDim);
    if (num_heads > kStaticMaxRecords)
        return fail(nullptr, XN_ERR_CAPACITY,
                    "num_heads %d is beyond the static scratch limit of %d partial records",
                    num_heads, kStaticMaxRecords);
    if (kv_len < 1 || capacity < kv_len || kv_len > (int64_t(1) << 40))
        return fail(nullptr, XN_ERR_ARG, "need 1 <= kv_len <= capacity");

    int dev = -1;
    XN_CUDA(nullptr, cudaGetDevice(&dev));
    if (dev < 0 || dev >= kStaticMaxDevices)
        return fail(nullptr, XN_ERR_ARG, "device ordinal %d outside 0..%d", dev, kStaticMaxDevices - 1);
    float* scratch = nullptr;
    {
        // First call on this device: resolve the device address of the static array, with this
        // device current.  Later calls reuse it.
        std::lock_guard<std::mutex> g(g_static_mu);
        if (!g_static_scratch_addr[dev]) {
            void* p = nullptr;
            XN_CUDA(nullptr, cudaGetSymbolAddress(&p, g_static_scratch));
            g_static_scratch_addr[dev] = static_cast<float*>(p);
        }
        scratch = g_static_scratch_addr[dev];
    }

    // as many splits as the record budget allows, at least 256 tokens each, at most ~4 waves
    int64_t splits = std::min<int64_t>(kStaticMaxRecords / num_heads, (kv_len + 255) / 256);
    splits = std::max<int64_t>(1, std::min<int64_t>(splits, std::max<int64_t>(1, 592 / num_heads)));
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const float scale = 1.0f / sqrtf(float(head_dim));
    static_split_kernel<<<dim3(unsigned(splits), unsigned(num_heads)), 128, 0, st>>>(
        q, k_cache, v_cache, scratch, num_heads, num_kv_heads, head_dim, kv_len, capacity,
        int(splits), scale);
    static_merge_kernel<<<unsigned(num_heads), 256, 0, st>>>(scratch, out, head_dim, int(splits));
    XN_CUDA(nullptr, cudaGetLastError());
    return XN_OK;
}
