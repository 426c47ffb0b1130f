// C++ host side above the C ABI: the reference's operator interface for this path with the same
// names, argument order and error behaviour, so that code written against xor-net's
// `xor_net::nn::{fast_attention, CpuRingCache}` reads the same here.
//
//   FastTensor        src/tensor.rs:6-40           { data: Vec<f32>, shape: Vec<usize> }
//   DeviceKvCache     src/nn/fast_attention.rs:18-60   stands where CpuRingCache stood
//   fast_attention    src/nn/fast_attention.rs:75-204  same signature; errors become exceptions
//                     carrying the reference's messages (:86-92)
//
// Header-only; link against libxn_attn.so.  All compute happens in the CUDA library.
#pragma once
#include <cstdlib>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

#include <cstdint>

#include "xn_attn.h"

namespace xor_net {

struct FastTensor {
    std::vector<float> data;
    std::vector<size_t> shape;
    FastTensor() = default;
    FastTensor(std::vector<float> d, std::vector<size_t> s) : data(std::move(d)), shape(std::move(s)) {}
    static FastTensor zeros(std::vector<size_t> s) {
        size_t n = 1;
        for (size_t x : s) n *= x;
        return FastTensor(std::vector<float>(n, 0.0f), std::move(s));
    }
    const std::vector<size_t>& dims() const { return shape; }
};

// Every GPU of the box behind one process, per model shape: one context (page pool, launch state,
// queue of concurrent callers) per device, shared by every cache of that shape -- the counterpart
// of the `Arc<Llama>` the reference's slot threads share (server/main.rs:613-645).  Devices:
// XORNET_ATTN_DEVICES ("0,1,5"; default every visible device).  Pool per device:
// XORNET_ATTN_POOL_PAGES pages, else XORNET_ATTN_POOL_MB megabytes, else half of the free memory.
class AttnGroup {
public:
    AttnGroup(int num_layers, int num_heads, int num_kv_heads, int head_dim) {
        xn_ctx_desc d{};
        d.num_layers = num_layers;
        d.num_heads = num_heads;
        d.num_kv_heads = num_kv_heads;
        d.head_dim = head_dim;
        d.page_tokens = 64;
        if (const char* env = std::getenv("XORNET_ATTN_POOL_PAGES")) d.pool_pages = std::atoll(env);
        if (const char* env = std::getenv("XORNET_ATTN_BATCH_WINDOW_US")) d.batch_window_us = std::atoi(env);
        if (xn_group_create(&d, nullptr, 0, &group_) != XN_OK)
            throw std::runtime_error(std::string("xn_group_create: ") + xn_last_error(nullptr));
    }
    ~AttnGroup() { xn_group_destroy(group_); }
    AttnGroup(const AttnGroup&) = delete;
    AttnGroup& operator=(const AttnGroup&) = delete;
    xn_group* get() const { return group_; }
    int size() const { return xn_group_size(group_); }
    xn_ctx* ctx(int i) const { return xn_group_ctx(group_, i); }

    static std::shared_ptr<AttnGroup> shared(int num_layers, int num_heads, int num_kv_heads, int head_dim) {
        static std::mutex mu;
        static std::map<std::tuple<int, int, int, int>, std::weak_ptr<AttnGroup>> all;
        std::lock_guard<std::mutex> g(mu);
        auto key = std::make_tuple(num_layers, num_heads, num_kv_heads, head_dim);
        if (auto sp = all[key].lock()) return sp;
        auto sp = std::make_shared<AttnGroup>(num_layers, num_heads, num_kv_heads, head_dim);
        all[key] = sp;
        return sp;
    }

private:
    xn_group* group_ = nullptr;
};

class DeviceKvCache {
public:
    size_t max_seq_len, num_kv_heads, head_dim, num_layers;

    // CpuRingCache::new(num_layers, num_kv_heads, max_seq_len, head_dim, use_u8).  The u8 shadow of
    // the reference is write-only (nothing reads it), so `use_u8` has no effect on any result.
    // The cache lands on the GPU that holds the fewest cached tokens (XORNET_ATTN_PLACEMENT=rr:
    // cache number mod number of GPUs) and stays there.  `expected_tokens` (0 = unknown) lets a
    // caller that creates its caches before filling them spread them by the load they will carry.
    // Unlike the reference's Cache it is not copyable: it names pages of a device pool.
    DeviceKvCache(size_t num_layers_, size_t num_kv_heads_, size_t max_seq_len_, size_t head_dim_,
                  bool /*use_u8*/ = false, size_t expected_tokens = 0)
        : max_seq_len(max_seq_len_), num_kv_heads(num_kv_heads_), head_dim(head_dim_),
          num_layers(num_layers_), expected_(expected_tokens) {}
    ~DeviceKvCache() {
        if (stream_) xn_stream_destroy(ctx_, stream_);
    }
    DeviceKvCache(const DeviceKvCache&) = delete;
    DeviceKvCache& operator=(const DeviceKvCache&) = delete;

    // The reference's pub field `k_buffers[layer]`: index h*cap*D + t*D + d.
    std::vector<float> k_buffer(size_t layer) const { return buffer(layer, true); }
    std::vector<float> v_buffer(size_t layer) const { return buffer(layer, false); }

    // binds to the shared group on first use (the query head count arrives with the first call)
    std::pair<xn_ctx*, xn_stream*> bind(size_t num_heads) {
        if (!stream_) {
            group_ = AttnGroup::shared(int(num_layers), int(num_heads), int(num_kv_heads), int(head_dim));
            int policy = XN_PLACE_LEAST_LOADED;
            if (const char* env = std::getenv("XORNET_ATTN_PLACEMENT"))
                if (std::string(env) == "rr" || std::string(env) == "round_robin") policy = XN_PLACE_ROUND_ROBIN;
            if (xn_group_stream_create(group_->get(), (int64_t)max_seq_len, (int64_t)expected_, policy, &ctx_,
                                       &stream_) != XN_OK)
                throw std::runtime_error(std::string("xn_group_stream_create: ") + xn_last_error(nullptr));
        }
        return {ctx_, stream_};
    }

private:
    std::vector<float> buffer(size_t layer, bool keys) const {
        std::vector<float> out(num_kv_heads * max_seq_len * head_dim, 0.0f);
        if (stream_) {
            int rc = xn_kv_read_range(ctx_, stream_, int(layer), 0, (int64_t)max_seq_len,
                                      keys ? out.data() : nullptr, keys ? nullptr : out.data());
            if (rc != XN_OK) throw std::runtime_error(std::string("xn_kv_read_range: ") + xn_last_error(ctx_));
        }
        return out;
    }
    size_t expected_;
    std::shared_ptr<AttnGroup> group_;
    xn_ctx* ctx_ = nullptr;
    xn_stream* stream_ = nullptr;
};

// fast_attention (src/nn/fast_attention.rs:75-85).  Throws std::runtime_error with the reference's
// text for its two checked errors; any library status becomes an exception too.
inline FastTensor fast_attention(const FastTensor& q, const FastTensor& k, const FastTensor& v,
                                 size_t layer_idx, size_t index_pos, DeviceKvCache& cache,
                                 size_t num_heads, size_t num_kv_heads, size_t head_dim) {
    if (q.shape.size() != 4) throw std::runtime_error("fast_attention: Q shape must be 4D");
    const size_t b_sz = q.shape[0], seq_len = q.shape[2];
    if (b_sz != 1)
        throw std::runtime_error("fast_attention currently only supports batch size 1, got " +
                                 std::to_string(b_sz));
    (void)num_kv_heads;
    auto [ctx, stream] = cache.bind(num_heads);
    FastTensor out = FastTensor::zeros({b_sz, num_heads, seq_len, head_dim});
    int rc = xn_attention(ctx, stream, int(layer_idx), (int64_t)index_pos, int(seq_len), q.data.data(),
                          k.data.data(), v.data.data(), out.data.data());
    if (rc != XN_OK)
        throw std::runtime_error("xn_attention failed (" + std::to_string(rc) + "): " + xn_last_error(ctx));
    return out;
}

// ---- attention output block (src/models/llama/attention.rs:103-108) ---------------------------

enum class TernaryPackType { Pack4 = XN_PACK4, Pack5 = XN_PACK5 };

// TernaryLinear with the dense packed representation (src/bit1_58/layers.rs:34-149): `create`
// ternarises and packs exactly like TernaryLinear::new; the forward pass runs on the device.
struct TernaryLinear {
    size_t in_dim = 0, out_dim = 0;
    TernaryPackType pack_type = TernaryPackType::Pack4;
    std::vector<uint8_t> packed;
    std::vector<float> w_scales;

    // provided_scale: NaN stands for None
    static TernaryLinear create(size_t in_dim, size_t out_dim, const std::vector<float>& weights_f32,
                                TernaryPackType pack_type, float provided_scale) {
        if (weights_f32.size() != in_dim * out_dim)
            throw std::runtime_error("Weight length must match in_dim * out_dim");
        TernaryLinear l;
        l.in_dim = in_dim;
        l.out_dim = out_dim;
        l.pack_type = pack_type;
        const size_t per = pack_type == TernaryPackType::Pack5 ? 5 : 4;
        l.packed.assign(out_dim * ((in_dim + per - 1) / per), 0);
        l.w_scales.assign(out_dim, 0.0f);
        if (xn_ternary_pack(int(in_dim), int(out_dim), weights_f32.data(), int(pack_type), provided_scale,
                            l.packed.data(), l.w_scales.data()) != XN_OK)
            throw std::runtime_error("xn_ternary_pack failed");
        return l;
    }
};

struct FastRmsNorm {  // src/nn/fast_rmsnorm.rs:5-17
    float eps = 1e-5f;
    std::vector<float> weight;
};

// Uploads a layer's o_proj (and optional sub-norm) to one device's context (every context of a
// group that serves the layer needs it).
inline void set_out_proj(xn_ctx* ctx, size_t layer, const TernaryLinear& o_proj,
                         const FastRmsNorm* sub_norm) {
    xn_out_proj_desc d{};
    d.layer = int(layer);
    d.in_dim = int(o_proj.in_dim);
    d.out_dim = int(o_proj.out_dim);
    d.pack_type = int(o_proj.pack_type);
    d.packed = o_proj.packed.data();
    d.w_scales = o_proj.w_scales.data();
    d.norm_weight = sub_norm ? sub_norm->weight.data() : nullptr;
    d.norm_eps = sub_norm ? sub_norm->eps : 0.0f;
    if (xn_out_proj_set(ctx, &d) != XN_OK)
        throw std::runtime_error(std::string("xn_out_proj_set: ") + xn_last_error(ctx));
}

// y [.., in_dim] -> o_proj(sub_norm(y)) [.., out_dim]: FastRmsNorm::forward + TernaryLinear::forward.
inline FastTensor out_proj_forward(xn_ctx* ctx, size_t layer, const FastTensor& y, size_t out_dim) {
    if (y.shape.empty()) throw std::runtime_error("Input must have at least 1 dimension");
    const size_t in_dim = y.shape.back();
    const size_t rows = in_dim ? y.data.size() / in_dim : 0;
    std::vector<size_t> shape = y.shape;
    shape.back() = out_dim;
    FastTensor out = FastTensor::zeros(shape);
    if (xn_out_proj(ctx, int(layer), int(rows), y.data.data(), out.data.data(), 0) != XN_OK)
        throw std::runtime_error(std::string("xn_out_proj: ") + xn_last_error(ctx));
    return out;
}

}  // namespace xor_net
