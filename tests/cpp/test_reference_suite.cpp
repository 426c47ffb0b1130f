// The reference's own tests of this path (tests/attention_numerics_tests.rs and the ring-wrap
// test of tests/fast_attention_tests.rs), written against the C++ host mirror.  Exit code 0 = all
// passed.  Needs a B200; built and run by tests/test_gpu_cpp_host.py.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>

#include "xor_net_attn.hpp"

using xor_net::DeviceKvCache;
using xor_net::FastTensor;
using xor_net::fast_attention;

static int failures = 0;
#define CHECK(cond, msg)                                          \
    do {                                                          \
        if (!(cond)) {                                            \
            std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, msg); \
            ++failures;                                           \
        }                                                         \
    } while (0)

static const float EPS = 1e-4f;

static void attention_single_token_is_identity() {  // attention_numerics_tests.rs:10-30
    const size_t num_heads = 2, num_kv_heads = 2, head_dim = 4;
    DeviceKvCache cache(1, num_kv_heads, 32, head_dim, false);
    FastTensor q(std::vector<float>(num_heads * head_dim, 1.0f), {1, num_heads, 1, head_dim});
    FastTensor k(std::vector<float>(num_kv_heads * head_dim, 1.0f), {1, num_kv_heads, 1, head_dim});
    std::vector<float> v_data(num_kv_heads * head_dim);
    for (size_t i = 0; i < v_data.size(); ++i) v_data[i] = float(i);
    FastTensor v(v_data, {1, num_kv_heads, 1, head_dim});
    FastTensor out = fast_attention(q, k, v, 0, 0, cache, num_heads, num_kv_heads, head_dim);
    CHECK((out.shape == std::vector<size_t>{1, num_heads, 1, head_dim}), "shape");
    for (size_t i = 0; i < v_data.size(); ++i) CHECK(std::fabs(out.data[i] - v_data[i]) < EPS, "identity");
}

static void attention_causal_mask_second_token_no_future() {  // :33-70
    DeviceKvCache cache(1, 1, 32, 2, false);
    fast_attention(FastTensor({1, 0}, {1, 1, 1, 2}), FastTensor({1, 0}, {1, 1, 1, 2}),
                   FastTensor({10, 0}, {1, 1, 1, 2}), 0, 0, cache, 1, 1, 2);
    FastTensor out = fast_attention(FastTensor({1, 1}, {1, 1, 1, 2}), FastTensor({0, 1}, {1, 1, 1, 2}),
                                    FastTensor({0, 20}, {1, 1, 1, 2}), 0, 1, cache, 1, 1, 2);
    CHECK(std::fabs(out.data[0] - 5.0f) < EPS && std::fabs(out.data[1] - 10.0f) < EPS, "[5,10]");
}

static void attention_output_finite() {  // :73-99
    const size_t H = 4, Hkv = 2, D = 8, S = 6;
    DeviceKvCache cache(1, Hkv, 64, D, false);
    std::vector<float> qd(H * S * D), kd(Hkv * S * D), vd(Hkv * S * D);
    for (size_t i = 0; i < qd.size(); ++i) qd[i] = std::sin(float(i) * 0.1f);
    for (size_t i = 0; i < kd.size(); ++i) kd[i] = std::cos(float(i) * 0.07f);
    for (size_t i = 0; i < vd.size(); ++i) vd[i] = float(i) * 0.03f - 1.0f;
    FastTensor out = fast_attention(FastTensor(qd, {1, H, S, D}), FastTensor(kd, {1, Hkv, S, D}),
                                    FastTensor(vd, {1, Hkv, S, D}), 0, 0, cache, H, Hkv, D);
    for (float x : out.data) CHECK(std::isfinite(x), "finite");
}

static void cache_write_correctness() {  // :102-116
    DeviceKvCache cache(1, 1, 8, 2, false);
    fast_attention(FastTensor({1, 1}, {1, 1, 1, 2}), FastTensor({5, 6}, {1, 1, 1, 2}),
                   FastTensor({0, 0}, {1, 1, 1, 2}), 0, 0, cache, 1, 1, 2);
    auto kb = cache.k_buffer(0);
    CHECK(kb[0] == 5.0f && kb[1] == 6.0f, "k_buffers[0][0..1]");
}

static void ring_wrapping_correctness() {  // fast_attention_tests.rs:191-241
    const size_t H = 2, Hkv = 1, cap = 4, D = 4;
    DeviceKvCache cache(1, Hkv, cap, D, false);
    FastTensor ones_q(std::vector<float>(H * D, 1.0f), {1, H, 1, D});
    FastTensor ones_kv(std::vector<float>(Hkv * D, 1.0f), {1, Hkv, 1, D});
    for (size_t pos = 0; pos < 4; ++pos) fast_attention(ones_q, ones_kv, ones_kv, 0, pos, cache, H, Hkv, D);
    for (float x : cache.k_buffer(0)) CHECK(x == 1.0f, "all ones");
    FastTensor zq = FastTensor::zeros({1, H, 1, D}), zkv = FastTensor::zeros({1, Hkv, 1, D});
    fast_attention(zq, zkv, zkv, 0, 4, cache, H, Hkv, D);
    auto kb = cache.k_buffer(0);
    for (size_t d = 0; d < D; ++d) {
        CHECK(kb[0 * D + d] == 0.0f, "slot 0 overwritten");
        CHECK(kb[1 * D + d] == 1.0f, "slot 1 intact");
    }
}

static void shape_errors() {  // fast_attention.rs:86-92
    DeviceKvCache cache(1, 1, 8, 2, false);
    FastTensor z({0, 0}, {1, 1, 1, 2});
    bool threw = false;
    try {
        fast_attention(FastTensor({0, 0}, {1, 1, 2}), z, z, 0, 0, cache, 1, 1, 2);
    } catch (const std::runtime_error& e) {
        threw = std::string(e.what()) == "fast_attention: Q shape must be 4D";
    }
    CHECK(threw, "4D message");
    threw = false;
    try {
        fast_attention(FastTensor({0, 0, 0, 0}, {2, 1, 1, 2}), z, z, 0, 0, cache, 1, 1, 2);
    } catch (const std::runtime_error& e) {
        threw = std::string(e.what()) == "fast_attention currently only supports batch size 1, got 2";
    }
    CHECK(threw, "batch message");
}

// tests/bit1_58_tests.rs:68-92 (test_ternary_linear_layer): pack4 and pack5 give the same output,
// and the literals of that test, which belong to the global weight scale 5/8 it was written with.
static void ternary_linear_layer() {
    using namespace xor_net;
    AttnGroup grp(1, 1, 1, 4);
    xn_ctx* ctx = grp.ctx(0);
    const std::vector<float> w = {1, 0, -1, 1, 0, -1, 1, 0};
    const FastTensor x({0.5f, 1.0f, -0.5f, 2.0f}, {1, 4});
    set_out_proj(ctx, 0, TernaryLinear::create(4, 2, w, TernaryPackType::Pack4, 0.625f), nullptr);
    const FastTensor o4 = out_proj_forward(ctx, 0, x, 2);
    set_out_proj(ctx, 0, TernaryLinear::create(4, 2, w, TernaryPackType::Pack5, 0.625f), nullptr);
    const FastTensor o5 = out_proj_forward(ctx, 0, x, 2);
    CHECK(o4.data == o5.data, "pack4 == pack5");
    CHECK(std::fabs(o4.data[0] - 1.879921f) < 1e-4f, "o_proj[0]");
    CHECK(std::fabs(o4.data[1] + 0.944882f) < 1e-4f, "o_proj[1]");
    // tests/tensor_rmsnorm_tests.rs:20-31 through the block: identity weights, unit norm weight
    AttnGroup grp2(1, 1, 1, 2);
    xn_ctx* ctx2 = grp2.ctx(0);
    FastRmsNorm norm;
    norm.eps = 1e-6f;
    norm.weight = {1.0f, 1.0f};
    set_out_proj(ctx2, 0, TernaryLinear::create(2, 2, {1, 0, 0, 1}, TernaryPackType::Pack4, NAN), &norm);
    const FastTensor n = out_proj_forward(ctx2, 0, FastTensor({3.0f, 4.0f}, {1, 2}), 2);
    // normalised row (3,4)/sqrt(12.5) quantised to i8 with scale 127/max and dequantised again
    const float rms = std::sqrt(12.5f), mx = 4.0f / rms;
    CHECK(std::fabs(n.data[1] - mx) < 1e-5f, "sub-norm max element");
    CHECK(std::fabs(n.data[0] - std::round(3.0f / rms * (127.0f / mx)) * (mx / 127.0f)) < 1e-5f, "sub-norm other element");
}

int main() {
    setenv("XORNET_ATTN_POOL_MB", "64", 0);   // small pools: these tests hold a handful of tokens

    try {
        ternary_linear_layer();
        attention_single_token_is_identity();
        attention_causal_mask_second_token_no_future();
        attention_output_finite();
        cache_write_correctness();
        ring_wrapping_correctness();
        shape_errors();
    } catch (const std::exception& e) {
        std::printf("EXCEPTION %s\n", e.what());
        return 2;
    }
    std::printf("%s (%d failures)\n", failures ? "FAILED" : "all reference tests passed", failures);
    return failures ? 1 : 0;
}
