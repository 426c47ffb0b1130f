// Ternary output projection on the 5th-generation tensor cores: i8 activations x 2-bit ternary
// weights -> i32 accumulators in tensor memory (tcgen05.mma.kind::i8), sm_100a only.
//
//   out[t][o] = (i32 dot(q[t], W[o]) as f32 * inv_scale[t]) * w_scale[o]
// is TernaryLinear::forward of the reference (src/bit1_58/layers.rs:262-313).  The dot products
// are integers, so the tensor-core result equals the CUDA-core kernel's and the reference's.
//
// One thread block = 128 token rows (the MMA's M: activations are operand A) x 32 output rows
// (N: weights are operand B), all of K.  80 blocks for the 2B model's 2560 outputs, whatever the
// number of tokens up to 128.  What shapes the kernel is latency, not throughput: one barrier
// hand-off costs ~100-200 cycles and a 128-column step only holds ~200 cycles of tensor work, so
//   * the block's whole weight slab [32 rows x K] is decoded ONCE into shared memory (80 KB for
//     K = 2560), in pieces of 512 columns, instead of being re-staged every step; the codes of
//     all pieces are fetched into registers up front;
//   * the activations stream through two 512-column stages that are contiguous in global memory
//     AND already laid out the way the tensor core reads them (act_offset), so a stage is four
//     plain bulk copies; tiled tensor-map loads of the same tiles were several times slower (one
//     request per row);
//   * one stage = one piece = 16 MMAs: five hand-offs for K = 2560; ring positions and phases
//     are counted, never divided out; the control warps run their loops converged with one lane
//     issuing, operand descriptors are built before the loop;
//   * the kernel is launched as a programmatic dependent of the quantiser kernel: its blocks start
//     while that kernel runs, fetch and decode their weights, and only then wait for the rows.
// Roles (320 threads):
//   warp 0      copy producer: activation stages (bulk async copies, no tensor map, no multicast);
//   warp 1      MMA issuer (one lane): sixteen tcgen05.mma (K = 32 each) per stage, both operands
//               from shared memory; tcgen05.commit frees the stage and finally signals the
//               epilogue; owns the tensor-memory allocation (32 columns);
//   warps 2..9  weight decoders: 64 weights (16 bytes of codes) per thread and piece, five
//               integer instructions per four weights, stored in the K-major 128-byte-swizzled
//               operand layout.  Afterwards the same warps are the epilogue: tcgen05.ld, a pass
//               through shared memory, then whole 128-byte row segments out with the two rounded
//               multiplies applied.
// Every wait is bounded; on expiry the kernel records a status code, drains and returns.
#pragma once
#include "xn_outproj.cuh"
#include "xn_prefill_tf32.cuh"

namespace xn {

namespace tg {
constexpr int kTM = 128;                 // token rows per block (MMA M)
constexpr int kTN = 32;                  // output rows per block (MMA N)
constexpr int kBK = 128;                 // K bytes (= i8 elements) per K-block
constexpr int kPieceKb = 4;              // K-blocks per piece = per activation stage
constexpr int kActBlock = kTM * kBK;     // 16 KB: one K-block of one token tile
constexpr int kActStage = kPieceKb * kActBlock;   // 64 KB
constexpr int kActStages = 2;
constexpr int kWBlock = kTN * kBK;       // 4 KB of decoded weights per K-block
constexpr int kCBlock = kTN * kBK / 4;   // 1 KB of codes per K-block
constexpr int kMaxPieces = 6;            // K <= 3072: 128 KB of stages + 96 KB of weights
constexpr int kThreads = 320;
constexpr int kDecoderWarps = 8;
constexpr int kOutStride = kTN + 1;      // floats per staged output row (conflict-free both ways)

__host__ __device__ constexpr int smem_bytes(int nkb) {
    return kActStages * kActStage + nkb * kWBlock + 1024 /* alignment slack */ + 512 /* barriers */;
}
__host__ __device__ constexpr int max_nkb() { return kMaxPieces * kPieceKb; }
static_assert(kTM * kOutStride * 4 <= kActStage, "the output tile is staged in a retired activation stage");

// Instruction descriptor, kind::i8: [4,6) D format 2 = s32, [7,10) A format 1 = s8, [10,13) B
// format 1 = s8, bits 15/16 A/B major 0 = K-major, [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_i8(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Four canonical 2-bit codes (0 -> -1, 1 -> 0, 2 -> +1; code 3 never occurs in the device
// format) in one byte -> four i8 in one word: spread the fields to the byte lanes, then
// code - 1 per byte without inter-byte borrows.
__device__ __forceinline__ uint32_t decode4_canon(uint32_t b) {
    const uint32_t t = b * 0x1001u;                       // b | b << 12 (disjoint fields)
    const uint32_t x = (t | (t << 6)) & 0x03030303u;      // code i in byte i
    return (x + 0x7F7F7F7Fu) ^ 0x80808080u;
}

// One lane polls (bounded) for the phase; every lane of the (converged) warp gets the outcome.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, int lane) {
    int ok = 1;
    if (lane == 0) ok = mbar_spin_bounded(bar, parity) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// True in exactly one lane of the (converged) warp.  Unlike `lane == 0`, the election tells the
// compiler that a single thread runs the guarded code.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void fence_generic_to_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, "
        "%12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
}  // namespace tg

struct TernaryGemmArgs {
    const int8_t* q;         // activations, tiled: act_offset()
    const uint8_t* w2;       // weight codes, tiled: code_offset()
    long long q_rows_pad;    // rows of the activation buffer (multiple of 256)
    long long q_row0;        // first activation row of this launch (multiple of 256)
    const float* w_scales;   // [out_dim]
    const float* inv_scale;  // [q_rows_pad], indexed like the activation rows
    const OutRowDev* rows;   // destination rows of this launch
    int n_rows;              // token rows of this launch
    int out_dim;
    int k_bytes;             // i8 elements per activation row, multiple of 128
    int* status;
};

__global__ void __launch_bounds__(tg::kThreads, 1)
ternary_gemm_tc_kernel(const TernaryGemmArgs a) {
    using namespace tg;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    const int nkb = a.k_bytes / kBK;
    const int n_pieces = (nkb + kPieceKb - 1) / kPieceKb;
    unsigned char* act_s = smem;                                  // [kActStages][kPieceKb][128 rows x 128 B]
    unsigned char* w_s = act_s + kActStages * kActStage;          // [nkb][32 rows x 128 B], decoded
    uint64_t* bars = reinterpret_cast<uint64_t*>(w_s + nkb * kWBlock);
    // one barrier per piece, used once: the activation copies' bytes AND the eight decoder warps'
    // arrivals complete it, so the MMA issuer pays one barrier wait per piece
    uint64_t* piece_full = bars;                     // [kMaxPieces]
    uint64_t* act_empty = piece_full + kMaxPieces;   // [kActStages] the MMAs that read the stage are done
    uint64_t* acc_full = act_empty + kActStages;     // all MMAs done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);
    static_assert((kActStages + kMaxPieces + 1) * 8 + 16 <= 512, "barrier area");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int o0 = blockIdx.x * kTN;
    const int t0 = blockIdx.y * kTM;

    // decoders: this thread's codes of every piece, requested before anything else happens
    // item = (K-block, row, half): 16 bytes of codes -> 64 i8; 64 items per K-block, so one pass of
    // the 256 decoder threads covers one piece of 4 K-blocks
    const int dtid = tid - 64;                   // 0..255 for decoder threads
    const int kb_in = (dtid >> 6) & 3;           // K-block inside the piece
    const int r = (dtid >> 1) & 31, h = dtid & 1;
    uint4 codes[kMaxPieces];
    if (warp >= 2) {
        const bool valid = o0 + r < a.out_dim;   // rows past the matrix decode to weight 0
        const uint8_t* src = a.w2 + (size_t(blockIdx.x) * nkb + kb_in) * kCBlock + r * 32 + h * 16;
#pragma unroll
        for (int p = 0; p < kMaxPieces; ++p) {
            codes[p] = make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u);
            if (valid && p * kPieceKb + kb_in < nkb)
                codes[p] = __ldg(reinterpret_cast<const uint4*>(src + size_t(p) * kPieceKb * kCBlock));
        }
    }

    if (tid == 0) {
        for (int s = 0; s < kActStages; ++s) mbar_init(&act_empty[s], 1);
        for (int p = 0; p < n_pieces; ++p) mbar_init(&piece_full[p], 1 + kDecoderWarps);
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(uint32_t(kTN))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pf::fence_before_sync();
    __syncthreads();
    pf::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ======================= copy producer: activation stages =======================
        pdl_wait();   // the activation rows are written by the kernel launched before this one
        const int8_t* src = a.q + size_t(a.q_row0 + t0) * kBK;
        const size_t kb_step = size_t(a.q_rows_pad) * kBK;   // one K-block further in global memory
        int st = 0;
        uint32_t wrap_par = 1;   // parity of the `empty` phase that frees the stage being refilled
        for (int p = 0; p < n_pieces; ++p) {
            if (p >= kActStages) {
                wrap_par ^= (st == 0) ? 1u : 0u;
                if (!warp_wait(&act_empty[st], wrap_par, lane)) {
                    if (lane == 0) {
                        report_status(a.status, kDevWaitEmpty);
                        *abort_flag = 1;
                    }
                    break;
                }
            }
            if (lane == 0) {
                const int kbs = min(kPieceKb, nkb - p * kPieceKb);
                mbar_arrive_expect_tx(&piece_full[p], uint32_t(kbs * kActBlock));
                for (int j = 0; j < kbs; ++j)
                    bulk_g2s(act_s + st * kActStage + j * kActBlock, src + size_t(j) * kb_step,
                             uint32_t(kActBlock), &piece_full[p]);
            }
            src += size_t(kPieceKb) * kb_step;
            st ^= 1;
            __syncwarp();
        }
    } else if (warp == 1) {
        // =============================== MMA issuer ===============================
        // Its first wait needs the activation copies, which cannot start before the preceding
        // kernels have finished: wait for them here, so that the 2 s limit of the bounded waits
        // below is measured from that moment and never counts a long predecessor's run time.
        pdl_wait();
        const uint32_t idesc = make_idesc_i8(kTM, kTN);
        // descriptor address fields advance by bytes >> 4
        const uint64_t adesc0 = pf::smem_desc(smem_u32(act_s), 0, 1024, pf::kLayoutSw128);
        uint64_t bdesc = pf::smem_desc(smem_u32(w_s), 0, 1024, pf::kLayoutSw128);
        bool ok = true;
        int st = 0;
        for (int p = 0; p < n_pieces; ++p) {
            ok = warp_wait(&piece_full[p], 0, lane);
            if (!ok || *abort_flag) { ok = false; break; }
            if (tg::elect_one()) {
                pf::fence_after_sync();
                const int kbs = min(kPieceKb, nkb - p * kPieceKb);
                const uint64_t adesc = adesc0 + uint64_t(st * (kActStage >> 4));
                // 32 bytes of K per instruction: +2 in the descriptor's address field
                if (kbs == kPieceKb) {
#pragma unroll
                    for (int j = 0; j < kPieceKb; ++j)
#pragma unroll
                        for (int k4 = 0; k4 < kBK / 32; ++k4)
                            mma_ss_i8(tmem_base, adesc + uint64_t(j * (kActBlock >> 4) + k4 * 2),
                                      bdesc + uint64_t(j * (kWBlock >> 4) + k4 * 2), idesc,
                                      uint32_t((p | j | k4) != 0));
                } else {
                    for (int j = 0; j < kbs; ++j)
#pragma unroll
                        for (int k4 = 0; k4 < kBK / 32; ++k4)
                            mma_ss_i8(tmem_base, adesc + uint64_t(j * (kActBlock >> 4) + k4 * 2),
                                      bdesc + uint64_t(j * (kWBlock >> 4) + k4 * 2), idesc,
                                      uint32_t((p | j | k4) != 0));
                }
                bdesc += uint64_t(kPieceKb * (kWBlock >> 4));
                pf::mma_commit(&act_empty[st]);
            }
            st ^= 1;
            __syncwarp();
        }
        if (tg::elect_one()) {
            if (ok) {
                pf::mma_commit(acc_full);
            } else {
                report_status(a.status, kDevWaitFull);
                *abort_flag = 1;
            }
        }
    } else {
        // =============================== weight decoders ===============================
        const int w_off = (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
        for (int p = 0; p < kMaxPieces; ++p) {
            if (p < n_pieces) {
                const int kb = p * kPieceKb + kb_in;
                if (kb < nkb) {
                    const uint32_t w[4] = {codes[p].x, codes[p].y, codes[p].z, codes[p].w};
                    unsigned char* dst = w_s + kb * kWBlock + w_off;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint4 v;
                        v.x = decode4_canon(w[j] & 0xffu);
                        v.y = decode4_canon((w[j] >> 8) & 0xffu);
                        v.z = decode4_canon((w[j] >> 16) & 0xffu);
                        v.w = decode4_canon(w[j] >> 24);
                        *reinterpret_cast<uint4*>(dst + (((h * 4 + j) ^ (r & 7)) << 4)) = v;
                    }
                }
                fence_generic_to_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&piece_full[p]);
            }
        }

        // =============================== epilogue ===============================
        // tensor memory -> registers (thread = token row; the two warps of a lane quarter split
        // the 32 output columns) -> shared memory -> whole 128-byte row segments out
        // (what the store pass needs from global memory is fetched before waiting for the MMAs)
        pdl_wait();   // the inverse scales come from the kernel launched before this one
        const int o = o0 + lane;
        const bool o_valid = o < a.out_dim;
        const float ws = o_valid ? a.w_scales[o] : 0.f;
        const int tw = (warp - 2) * 16;    // this warp's 16 token rows of the tile in the store pass
        const int t_mine = t0 + tw + (lane & 15);
        float* dst_mine = t_mine < a.n_rows ? a.rows[t_mine].dst : nullptr;
        const float is_mine = t_mine < a.n_rows ? a.inv_scale[a.q_row0 + t_mine] : 0.f;
        const bool acc_ok = warp_wait(acc_full, 0, lane) && !*abort_flag;
        pf::fence_after_sync();
        float* out_s = reinterpret_cast<float*>(act_s);   // every stage has been consumed by now
        if (acc_ok) {
            const int quarter = warp & 3;
            const int half = (warp - 2) >> 2;
            uint32_t acc[16];
            tmem_ld16(tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(half * 16), acc);
            pf::tmem_wait_ld();
            float* row = out_s + (quarter * 32 + lane) * kOutStride + half * 16;
#pragma unroll
            for (int i = 0; i < 16; ++i) row[i] = float(int(acc[i]));
        }
        named_bar_sync(1, kDecoderWarps * 32);
        if (acc_ok) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float* dst = reinterpret_cast<float*>(
                    __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(dst_mine), i));
                const float is = __shfl_sync(0xffffffffu, is_mine, i);
                const float v = out_s[(tw + i) * kOutStride + lane];
                if (dst != nullptr && o_valid) dst[o] = __fmul_rn(__fmul_rn(v, is), ws);
            }
        } else if (lane == 0 && !*abort_flag) {
            report_status(a.status, kDevWaitMma);
        }
    }

    pf::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        pf::fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(uint32_t(kTN))
                     : "memory");
    }
}

// ================================================================================================
// Many-row variant (prefill-size inputs): the same arithmetic, shaped for throughput.
//
// One thread block keeps the weights of 64 output rows resident (decoded once, 160 KB for
// K = 2560) and walks over token tiles of 128 rows: blockIdx.y, blockIdx.y + gridDim.y, ...  The
// activation ring, the MMA issuer and the epilogue never drain between tiles: two accumulators of
// 64 columns alternate in tensor memory, so tile i is stored while tile i + 1 is multiplied.
// Per 256-column stage: 8 MMAs with N = 64.  Roles as in ternary_gemm_tc_kernel (320 threads).
// ================================================================================================
namespace tgr {
constexpr int kTM = 128;
constexpr int kTN = 64;
constexpr int kBK = 128;
constexpr int kPieceKb = 2;
constexpr int kActBlock = kTM * kBK;               // 16 KB
constexpr int kActStage = kPieceKb * kActBlock;    // 32 KB
constexpr int kActStages = 2;
constexpr int kWBlock = kTN * kBK;                 // 8 KB of decoded weights per K-block
constexpr int kMaxPieces = 10;                     // K <= 2560
constexpr int kThreads = 320;
constexpr int kDecoderWarps = 8;
__host__ __device__ constexpr int smem_bytes(int nkb) {
    return kActStages * kActStage + nkb * kWBlock + 1024 /* alignment slack */ + 512 /* barriers */;
}
__host__ __device__ constexpr int max_nkb() { return kMaxPieces * kPieceKb; }
}  // namespace tgr

__global__ void __launch_bounds__(tgr::kThreads, 1)
ternary_gemm_rows_kernel(const TernaryGemmArgs a) {
    using namespace tgr;
    using tg::warp_wait;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    const int nkb = a.k_bytes / kBK;
    const int n_pieces = (nkb + kPieceKb - 1) / kPieceKb;
    const int n_tiles = (a.n_rows + kTM - 1) / kTM;
    unsigned char* act_s = smem;                                  // [2][2][128 rows x 128 B]
    unsigned char* w_s = act_s + kActStages * kActStage;          // [nkb][64 rows x 128 B], decoded
    uint64_t* bars = reinterpret_cast<uint64_t*>(w_s + nkb * kWBlock);
    uint64_t* w_full = bars;                         // [kMaxPieces] piece decoded (once)
    uint64_t* act_full = w_full + kMaxPieces;        // [2] stage landed
    uint64_t* act_empty = act_full + kActStages;     // [2] stage consumed
    uint64_t* acc_full = act_empty + kActStages;     // [2] accumulator complete
    uint64_t* acc_empty = acc_full + 2;              // [2] accumulator read out by the 8 epilogue warps
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);
    static_assert((kMaxPieces + 2 * kActStages + 4) * 8 + 16 <= 512, "barrier area");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int o0 = blockIdx.x * kTN;

    // decoders: item = (K-block, row 0..63, half); 128 items per K-block, so one pass of the 256
    // decoder threads covers one piece of 2 K-blocks.  All codes are requested up front.
    const int dtid = tid - 64;
    const int kb_in = (dtid >> 7) & 1;
    const int r = (dtid >> 1) & 63, h = dtid & 1;
    uint4 codes[kMaxPieces];
    if (warp >= 2) {
        const bool valid = o0 + r < a.out_dim;
        // the code layout groups 32 rows: this block's 64 rows are two consecutive groups
        const uint8_t* src = a.w2 + ((size_t(2 * blockIdx.x + (r >> 5)) * nkb + kb_in) * 32 + (r & 31)) * 32 + h * 16;
#pragma unroll
        for (int p = 0; p < kMaxPieces; ++p) {
            codes[p] = make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u);
            if (valid && p * kPieceKb + kb_in < nkb)
                codes[p] = __ldg(reinterpret_cast<const uint4*>(src + size_t(p) * kPieceKb * 1024));
        }
    }

    if (tid == 0) {
        for (int p = 0; p < n_pieces; ++p) mbar_init(&w_full[p], kDecoderWarps);
        for (int s = 0; s < kActStages; ++s) {
            mbar_init(&act_full[s], 1);
            mbar_init(&act_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], kDecoderWarps);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(uint32_t(2 * kTN))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pf::fence_before_sync();
    __syncthreads();
    pf::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ======================= copy producer: activation stages of every tile =======================
        pdl_wait();
        const size_t kb_step = size_t(a.q_rows_pad) * kBK;
        int st = 0;
        uint32_t wrap_par = 1;
        int issued = 0;
        bool ok = true;
        for (int tile = blockIdx.y; tile < n_tiles && ok; tile += gridDim.y) {
            const int8_t* src = a.q + size_t(a.q_row0 + size_t(tile) * kTM) * kBK;
            for (int p = 0; p < n_pieces; ++p, ++issued) {
                if (issued >= kActStages) {
                    wrap_par ^= (st == 0) ? 1u : 0u;
                    if (!warp_wait(&act_empty[st], wrap_par, lane)) {
                        if (lane == 0) {
                            report_status(a.status, kDevWaitEmpty);
                            *abort_flag = 1;
                        }
                        ok = false;
                        break;
                    }
                }
                if (lane == 0) {
                    const int kbs = min(kPieceKb, nkb - p * kPieceKb);
                    mbar_arrive_expect_tx(&act_full[st], uint32_t(kbs * kActBlock));
                    for (int j = 0; j < kbs; ++j)
                        bulk_g2s(act_s + st * kActStage + j * kActBlock, src + size_t(j) * kb_step,
                                 uint32_t(kActBlock), &act_full[st]);
                }
                src += size_t(kPieceKb) * kb_step;
                st ^= 1;
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // =============================== MMA issuer ===============================
        pdl_wait();   // as in ternary_gemm_tc_kernel: the bounded waits start counting here
        const uint32_t idesc = tg::make_idesc_i8(kTM, kTN);
        const uint64_t adesc0 = pf::smem_desc(smem_u32(act_s), 0, 1024, pf::kLayoutSw128);
        const uint64_t bdesc0 = pf::smem_desc(smem_u32(w_s), 0, 1024, pf::kLayoutSw128);
        bool ok = true;
        int st = 0;
        uint32_t par = 0;
        int tile_idx = 0;
        for (int tile = blockIdx.y; tile < n_tiles && ok; tile += gridDim.y, ++tile_idx) {
            const int b = tile_idx & 1;
            if (tile_idx >= 2)   // the epilogue must have read this accumulator's previous tile
                ok = warp_wait(&acc_empty[b], uint32_t(((tile_idx >> 1) - 1) & 1), lane);
            uint64_t bdesc = bdesc0;
            for (int p = 0; p < n_pieces && ok; ++p) {
                if (tile_idx == 0) ok = warp_wait(&w_full[p], 0, lane);
                ok = ok && warp_wait(&act_full[st], par, lane);
                if (!ok || *abort_flag) { ok = false; break; }
                if (tg::elect_one()) {
                    pf::fence_after_sync();
                    const int kbs = min(kPieceKb, nkb - p * kPieceKb);
                    const uint64_t adesc = adesc0 + uint64_t(st * (kActStage >> 4));
                    for (int j = 0; j < kbs; ++j)
#pragma unroll
                        for (int k4 = 0; k4 < kBK / 32; ++k4)
                            tg::mma_ss_i8(tmem_base + uint32_t(b * kTN),
                                          adesc + uint64_t(j * (kActBlock >> 4) + k4 * 2),
                                          bdesc + uint64_t(j * (kWBlock >> 4) + k4 * 2), idesc,
                                          uint32_t((p | j | k4) != 0));
                    pf::mma_commit(&act_empty[st]);
                }
                bdesc += uint64_t(kPieceKb * (kWBlock >> 4));
                par ^= uint32_t(st);
                st ^= 1;
                __syncwarp();
            }
            if (ok && tg::elect_one()) pf::mma_commit(&acc_full[b]);
            __syncwarp();
        }
        if (!ok && lane == 0) {
            report_status(a.status, kDevWaitFull);
            *abort_flag = 1;
        }
    } else {
        // =============================== weight decoders ===============================
        const int w_off = (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
        for (int p = 0; p < kMaxPieces; ++p) {
            if (p < n_pieces) {
                const int kb = p * kPieceKb + kb_in;
                if (kb < nkb) {
                    const uint32_t w[4] = {codes[p].x, codes[p].y, codes[p].z, codes[p].w};
                    unsigned char* dst = w_s + kb * kWBlock + w_off;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint4 v;
                        v.x = tg::decode4_canon(w[j] & 0xffu);
                        v.y = tg::decode4_canon((w[j] >> 8) & 0xffu);
                        v.z = tg::decode4_canon((w[j] >> 16) & 0xffu);
                        v.w = tg::decode4_canon(w[j] >> 24);
                        *reinterpret_cast<uint4*>(dst + (((h * 4 + j) ^ (r & 7)) << 4)) = v;
                    }
                }
                tg::fence_generic_to_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&w_full[p]);
            }
        }

        // =============================== epilogue, tile after tile ===============================
        // thread = token row; the two warps of a lane quarter take 32 of the 64 output columns each:
        // 128 contiguous bytes per thread
        pdl_wait();
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int oc = o0 + half * 32;
        int tile_idx = 0;
        for (int tile = blockIdx.y; tile < n_tiles; tile += gridDim.y, ++tile_idx) {
            const int b = tile_idx & 1;
            const int t = tile * kTM + quarter * 32 + lane;
            const bool t_valid = t < a.n_rows;
            float* dst = t_valid ? a.rows[t].dst + oc : nullptr;
            const float is = t_valid ? a.inv_scale[a.q_row0 + t] : 0.f;
            if (!warp_wait(&acc_full[b], uint32_t((tile_idx >> 1) & 1), lane) || *abort_flag) {
                if (lane == 0 && !*abort_flag) report_status(a.status, kDevWaitMma);
                break;
            }
            pf::fence_after_sync();
            uint32_t acc[32];
            pf::tmem_ld32(tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(b * kTN + half * 32), acc);
            pf::tmem_wait_ld();
            pf::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[b]);   // the MMA issuer may overwrite this accumulator
            if (t_valid) {
                if (oc + 32 <= a.out_dim && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const float4 ws = *reinterpret_cast<const float4*>(a.w_scales + oc + i);
                        float4 v;
                        v.x = __fmul_rn(__fmul_rn(float(int(acc[i + 0])), is), ws.x);
                        v.y = __fmul_rn(__fmul_rn(float(int(acc[i + 1])), is), ws.y);
                        v.z = __fmul_rn(__fmul_rn(float(int(acc[i + 2])), is), ws.z);
                        v.w = __fmul_rn(__fmul_rn(float(int(acc[i + 3])), is), ws.w);
                        *reinterpret_cast<float4*>(dst + i) = v;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (oc + i < a.out_dim)
                            dst[i] = __fmul_rn(__fmul_rn(float(int(acc[i])), is), a.w_scales[oc + i]);
                }
            }
        }
    }

    pf::fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        pf::fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(uint32_t(2 * kTN))
                     : "memory");
    }
}

}  // namespace xn
