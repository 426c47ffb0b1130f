// Host-side handling of the reference's ternary weight formats (src/bit1_58/quantization.rs,
// src/bit1_58/layers.rs:91-149): ternarising + packing f32 weights the way TernaryLinear::new does,
// and re-coding packed rows into the 2-bit device format of the projection kernel.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <vector>

namespace xn {

inline size_t packed_row_bytes(size_t n, int pack) { return pack == 5 ? (n + 4) / 5 : (n + 3) / 4; }

// 0 -> -1, 1 -> 0, 2 -> +1 after scaling, rounding (half away from zero) and clamping
// (quantization.rs:11-20 and :53-62).
inline unsigned ternary_code(float w, float w_scale) {
    const float scaled = w_scale > 0.0f ? w / w_scale : 0.0f;
    float q = std::round(scaled);
    q = q < -1.0f ? -1.0f : (q > 1.0f ? 1.0f : q);
    return q < -0.5f ? 0u : (q > 0.5f ? 2u : 1u);
}

inline void pack_row(const float* w, size_t n, float w_scale, int pack, uint8_t* out) {
    const size_t per = pack == 5 ? 5 : 4;
    for (size_t b = 0; b * per < n; ++b) {
        unsigned byte = 0, mult = 1;
        for (size_t i = 0; i < per && b * per + i < n; ++i) {
            const unsigned code = ternary_code(w[b * per + i], w_scale);
            if (pack == 5) { byte += code * mult; mult *= 3; }
            else byte |= code << (2 * i);
        }
        out[b] = uint8_t(byte);
    }
}

// TernaryLinear::new, dense representation (layers.rs:91-149).  has_scale == false stands for
// provided_scale == None.
inline void ternary_linear_pack(size_t in_dim, size_t out_dim, const float* weights, int pack,
                                bool has_scale, float provided_scale, uint8_t* packed,
                                float* w_scales) {
    bool already = true;
    for (size_t i = 0; i < in_dim * out_dim && already; ++i)
        already = weights[i] == -1.0f || weights[i] == 0.0f || weights[i] == 1.0f;
    const size_t bpr = packed_row_bytes(in_dim, pack);
    for (size_t o = 0; o < out_dim; ++o) {
        const float* row = weights + o * in_dim;
        float s;
        if (already) s = has_scale ? provided_scale : 1.0f;
        else if (has_scale) s = provided_scale;
        else {  // per-row mean absolute value, summed in index order (:128-133)
            float sum_abs = 0.0f;
            for (size_t i = 0; i < in_dim; ++i) sum_abs += std::fabs(row[i]);
            s = in_dim == 0 ? 1.0f : sum_abs / float(in_dim);
        }
        w_scales[o] = s;
        pack_row(row, in_dim, s, pack, packed + o * bpr);
    }
}

// One packed row -> the device format: 2-bit pack4 codes, `stride` bytes per row, positions
// past in_dim hold code 1 (weight 0).  Code 3 of a pack4 row decodes to 0 in the reference
// (quantization.rs:36-40) and becomes code 1 here; base-3 digits of a pack5 row map one to one.
inline void recode_row_2bit(const uint8_t* src, size_t in_dim, int pack, uint8_t* dst, size_t stride) {
    for (size_t b = 0; b < stride; ++b) dst[b] = 0x55u;
    for (size_t i = 0; i < in_dim; ++i) {
        unsigned code;
        if (pack == 5) {
            unsigned cur = src[i / 5];
            for (size_t j = 0; j < i % 5; ++j) cur /= 3;
            code = cur % 3;
        } else {
            code = (src[i / 4] >> ((i % 4) * 2)) & 3u;
            if (code == 3u) code = 1u;  // both decode to weight 0; the kernels rely on codes 0..2
        }
        uint8_t& byte = dst[i / 4];
        byte = uint8_t((byte & ~(3u << ((i % 4) * 2))) | (code << ((i % 4) * 2)));
    }
}

// ---- XorSparse rows (src/bit1_58/sparse.rs) ------------------------------------------------------
// per row: u32 num_blocks, then per 64-element block a u64 mask of the non-zero positions and
// ceil(popcount / 8) bytes of sign bits in scan order (bit set = weight -1); little-endian.

// ternarize_row (src/bit1_58/layers.rs:45-88): the weight of one position as -1 / 0 / +1
inline int ternary_value(float w, float w_scale, bool already_ternary) {
    if (already_ternary) return int(w);
    return int(ternary_code(w, w_scale)) - 1;
}

// encode_sparse_row_into (sparse.rs:62-89); returns the bytes appended
inline size_t sparse_encode_row(const int8_t* vals, size_t in_dim, std::vector<uint8_t>& buf) {
    const size_t before = buf.size();
    const uint32_t num_blocks = uint32_t((in_dim + 63) / 64);
    for (int i = 0; i < 4; ++i) buf.push_back(uint8_t(num_blocks >> (8 * i)));
    for (uint32_t b = 0; b < num_blocks; ++b) {
        uint64_t mask = 0, signs = 0;
        unsigned si = 0;
        for (size_t i = size_t(b) * 64; i < std::min(in_dim, size_t(b) * 64 + 64); ++i)
            if (vals[i] != 0) {
                mask |= uint64_t(1) << (i - size_t(b) * 64);
                if (vals[i] < 0) signs |= uint64_t(1) << si;
                ++si;
            }
        for (int i = 0; i < 8; ++i) buf.push_back(uint8_t(mask >> (8 * i)));
        for (unsigned i = 0; i < (si + 7) / 8; ++i) buf.push_back(uint8_t(signs >> (8 * i)));
    }
    return buf.size() - before;
}

// One sparse row -> the device's 2-bit codes (decode_row, sparse.rs:206-249).  Returns the bytes
// of the row in the blob, or 0 when the row does not describe in_dim columns.
inline size_t recode_sparse_row_2bit(const uint8_t* src, size_t in_dim, uint8_t* dst, size_t stride) {
    for (size_t b = 0; b < stride; ++b) dst[b] = 0x55u;
    const uint32_t num_blocks = uint32_t(src[0]) | uint32_t(src[1]) << 8 | uint32_t(src[2]) << 16 |
                                uint32_t(src[3]) << 24;
    if (size_t(num_blocks) != (in_dim + 63) / 64) return 0;
    size_t p = 4;
    for (uint32_t b = 0; b < num_blocks; ++b) {
        uint64_t mask = 0;
        for (int i = 0; i < 8; ++i) mask |= uint64_t(src[p + i]) << (8 * i);
        p += 8;
        unsigned nnz = 0;
        for (uint64_t m = mask; m; m &= m - 1) ++nnz;
        uint64_t sb = 0;
        for (unsigned k = 0; k < (nnz + 7) / 8; ++k) sb |= uint64_t(src[p + k]) << (8 * k);
        p += (nnz + 7) / 8;
        unsigned si = 0;
        for (size_t i = size_t(b) * 64; i < std::min(in_dim, size_t(b) * 64 + 64); ++i)
            if ((mask >> (i - size_t(b) * 64)) & 1) {
                const unsigned code = ((sb >> si) & 1) ? 0u : 2u;   // -1 : +1
                uint8_t& byte = dst[i / 4];
                byte = uint8_t((byte & ~(3u << ((i % 4) * 2))) | (code << ((i % 4) * 2)));
                ++si;
            }
    }
    return p;
}

}  // namespace xn
