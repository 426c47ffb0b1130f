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

// One page pool and launch state per (device, model shape), shared by every cache of that shape:
// the counterpart of the `Arc<Llama>` the reference's slots share (server/main.rs:613-645).
class AttnContext {
public:
    AttnContext(int device, int num_layers, int num_heads, int num_kv_heads, int head_dim,
                long long pool_pages) {
        xn_ctx_desc d{};
        d.device = device;
        d.num_layers = num_layers;
        d.num_heads = num_heads;
        d.num_kv_heads = num_kv_heads;
        d.head_dim = head_dim;
        d.page_tokens = 64;
        d.pool_pages = pool_pages;
        if (xn_ctx_create(&d, &ctx_) != XN_OK)
            throw std::runtime_error(std::string("xn_ctx_create: ") + xn_last_error(nullptr));
    }
    ~AttnContext() { xn_ctx_destroy(ctx_); }
    AttnContext(const AttnContext&) = delete;
    AttnContext& operator=(const AttnContext&) = delete;
    xn_ctx* get() const { return ctx_; }

    // Pool size: XORNET_ATTN_POOL_PAGES pages if set, else enough for `max_seq_len` x 64 streams.
    static std::shared_ptr<AttnContext> shared(int device, int num_layers, int num_heads,
                                               int num_kv_heads, int head_dim, size_t max_seq_len) {
        static std::mutex mu;
        static std::map<std::tuple<int, int, int, int, int>, std::weak_ptr<AttnContext>> all;
        std::lock_guard<std::mutex> g(mu);
        auto key = std::make_tuple(device, num_layers, num_heads, num_kv_heads, head_dim);
        if (auto sp = all[key].lock()) return sp;
        long long pages = 0;
        if (const char* env = std::getenv("XORNET_ATTN_POOL_PAGES")) pages = std::atoll(env);
        if (pages <= 0) pages = (long long)((max_seq_len + 63) / 64) * 64;
        auto sp = std::make_shared<AttnContext>(device, num_layers, num_heads, num_kv_heads, head_dim, pages);
        all[key] = sp;
        return sp;
    }

private:
    xn_ctx* ctx_ = nullptr;
};

class DeviceKvCache {
public:
    size_t max_seq_len, num_kv_heads, head_dim, num_layers;

    // CpuRingCache::new(num_layers, num_kv_heads, max_seq_len, head_dim, use_u8).  The u8 shadow of
    // the reference is write-only (nothing reads it), so `use_u8` has no effect on any result.
    DeviceKvCache(size_t num_layers_, size_t num_kv_heads_, size_t max_seq_len_, size_t head_dim_,
                  bool /*use_u8*/ = false, int device = 0)
        : max_seq_len(max_seq_len_), num_kv_heads(num_kv_heads_), head_dim(head_dim_),
          num_layers(num_layers_), device_(device) {}
    ~DeviceKvCache() {
        if (stream_) xn_stream_destroy(ctx_->get(), stream_);
    }
    DeviceKvCache(const DeviceKvCache&) = delete;
    DeviceKvCache& operator=(const DeviceKvCache&) = delete;

    // The reference's pub field `k_buffers[layer]`: index h*cap*D + t*D + d.
    std::vector<float> k_buffer(size_t layer) const { return buffer(layer, true); }
    std::vector<float> v_buffer(size_t layer) const { return buffer(layer, false); }

    // binds to the shared context on first use (the query head count arrives with the first call)
    std::pair<xn_ctx*, xn_stream*> bind(size_t num_heads) {
        if (!stream_) {
            ctx_ = AttnContext::shared(device_, int(num_layers), int(num_heads), int(num_kv_heads),
                                       int(head_dim), max_seq_len);
            if (xn_stream_create(ctx_->get(), (int64_t)max_seq_len, &stream_) != XN_OK)
                throw std::runtime_error(std::string("xn_stream_create: ") + xn_last_error(ctx_->get()));
        }
        return {ctx_->get(), stream_};
    }

private:
    std::vector<float> buffer(size_t layer, bool keys) const {
        std::vector<float> out(num_kv_heads * max_seq_len * head_dim, 0.0f);
        if (stream_) {
            int rc = xn_kv_read_range(ctx_->get(), stream_, int(layer), 0, (int64_t)max_seq_len,
                                      keys ? out.data() : nullptr, keys ? nullptr : out.data());
            if (rc != XN_OK) throw std::runtime_error(std::string("xn_kv_read_range: ") + xn_last_error(ctx_->get()));
        }
        return out;
    }
    int device_;
    std::shared_ptr<AttnContext> ctx_;
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

// Uploads a layer's o_proj (and optional sub-norm) to the context.
inline void set_out_proj(AttnContext& ctx, size_t layer, const TernaryLinear& o_proj,
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
    if (xn_out_proj_set(ctx.get(), &d) != XN_OK)
        throw std::runtime_error(std::string("xn_out_proj_set: ") + xn_last_error(ctx.get()));
}

// y [.., in_dim] -> o_proj(sub_norm(y)) [.., out_dim]: FastRmsNorm::forward + TernaryLinear::forward.
inline FastTensor out_proj_forward(AttnContext& ctx, size_t layer, const FastTensor& y, size_t out_dim) {
    if (y.shape.empty()) throw std::runtime_error("Input must have at least 1 dimension");
    const size_t in_dim = y.shape.back();
    const size_t rows = in_dim ? y.data.size() / in_dim : 0;
    std::vector<size_t> shape = y.shape;
    shape.back() = out_dim;
    FastTensor out = FastTensor::zeros(shape);
    if (xn_out_proj(ctx.get(), int(layer), int(rows), y.data.data(), out.data.data(), 0) != XN_OK)
        throw std::runtime_error(std::string("xn_out_proj: ") + xn_last_error(ctx.get()));
    return out;
}

}  // namespace xor_net
