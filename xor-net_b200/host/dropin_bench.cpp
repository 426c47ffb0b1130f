// The drop-in call measured the way xor-net's own front-ends make it: one OS thread per stream
// (a server slot, server/main.rs:176-199; a batch_bench worker, examples/batch_bench.rs:138-151),
// each with its own cache (server/main.rs:92, batch_bench.rs:188) and ordinary pageable
// FastTensors, blocking in fast_attention once per layer (batch_bench.rs:194-199 through
// Llama::forward).  Nothing here batches: the library's per-device queue merges whoever calls at
// the same time.
//
//   dropin_bench <streams> <layers> <heads> <kv_heads> <head_dim> <len_lo> <len_hi> <steps> <warmup> <seed>
//
// Prints one JSON object.  Streams are created with their expected length, so that with several
// GPUs visible they spread by load; XORNET_ATTN_DEVICES / XORNET_ATTN_PLACEMENT /
// XORNET_ATTN_BATCH_WINDOW_US / XORNET_ATTN_POOL_MB apply as usual.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <random>
#include <thread>
#include <vector>

#include "xor_net_attn.hpp"

using xor_net::DeviceKvCache;
using xor_net::FastTensor;
using xor_net::fast_attention;

int main(int argc, char** argv) {
    if (argc < 11) {
        std::fprintf(stderr, "usage: %s streams layers heads kv_heads head_dim len_lo len_hi steps warmup seed\n", argv[0]);
        return 2;
    }
    const int n = std::atoi(argv[1]), layers = std::atoi(argv[2]), Hq = std::atoi(argv[3]), Hkv = std::atoi(argv[4]),
              D = std::atoi(argv[5]), lo = std::atoi(argv[6]), hi = std::atoi(argv[7]), steps = std::atoi(argv[8]),
              warmup = std::atoi(argv[9]);
    const unsigned long long seed = std::strtoull(argv[10], nullptr, 10);
    try {
        std::mt19937_64 rng(seed);
        std::uniform_int_distribution<int> len_dist(lo, hi);
        std::normal_distribution<float> normal(0.f, 1.f);
        std::vector<int> lens(static_cast<size_t>(n));
        for (int& L : lens) L = len_dist(rng);
        const size_t cap = size_t(hi) + size_t(steps + warmup) + 1;
        std::vector<std::unique_ptr<DeviceKvCache>> caches;
        long long total_tokens = 0;
        for (int i = 0; i < n; ++i) {
            caches.emplace_back(new DeviceKvCache(size_t(layers), size_t(Hkv), cap, size_t(D), false, size_t(lens[size_t(i)])));
            auto [ctx, st] = caches.back()->bind(size_t(Hq));   // placement happens here, in creation order
            if (lens[size_t(i)] > 1 &&
                xn_kv_fill_normal(ctx, st, -1, 0, lens[size_t(i)] - 1, seed + 1000003ull * (unsigned long long)i) != XN_OK)
                throw std::runtime_error(std::string("xn_kv_fill_normal: ") + xn_last_error(ctx));
            total_tokens += lens[size_t(i)];
        }
        auto group = xor_net::AttnGroup::shared(layers, Hq, Hkv, D);
        for (int g = 0; g < group->size(); ++g) xn_ctx_synchronize(group->ctx(g));

        // per-thread inputs: one token per step, the same tensors for every layer (their values do
        // not change the work)
        std::vector<FastTensor> qs, ks, vs;
        for (int i = 0; i < n; ++i) {
            std::vector<float> q(size_t(Hq) * D), k(size_t(Hkv) * D), v(size_t(Hkv) * D);
            for (float& x : q) x = normal(rng);
            for (float& x : k) x = normal(rng);
            for (float& x : v) x = normal(rng);
            qs.emplace_back(q, std::vector<size_t>{1, size_t(Hq), 1, size_t(D)});
            ks.emplace_back(k, std::vector<size_t>{1, size_t(Hkv), 1, size_t(D)});
            vs.emplace_back(v, std::vector<size_t>{1, size_t(Hkv), 1, size_t(D)});
        }

        std::atomic<int> at_start{0}, failures{0};
        std::atomic<bool> go{false};
        std::vector<double> done_at(static_cast<size_t>(n), 0.0);
        std::chrono::steady_clock::time_point t_go;
        std::vector<std::thread> threads;
        double checksum = 0.0;
        std::vector<double> sums(static_cast<size_t>(n), 0.0);
        for (int i = 0; i < n; ++i) {
            threads.emplace_back([&, i] {
                try {
                    size_t pos = size_t(lens[size_t(i)]) - 1;
                    for (int s = 0; s < warmup; ++s, ++pos)
                        for (int l = 0; l < layers; ++l)
                            fast_attention(qs[size_t(i)], ks[size_t(i)], vs[size_t(i)], size_t(l), pos, *caches[size_t(i)],
                                           size_t(Hq), size_t(Hkv), size_t(D));
                    at_start.fetch_add(1);
                    while (!go.load(std::memory_order_acquire)) std::this_thread::yield();
                    for (int s = 0; s < steps; ++s, ++pos)
                        for (int l = 0; l < layers; ++l) {
                            FastTensor out = fast_attention(qs[size_t(i)], ks[size_t(i)], vs[size_t(i)], size_t(l), pos,
                                                            *caches[size_t(i)], size_t(Hq), size_t(Hkv), size_t(D));
                            sums[size_t(i)] += out.data[0];
                        }
                    done_at[size_t(i)] =
                        std::chrono::duration<double>(std::chrono::steady_clock::now() - t_go).count();
                } catch (const std::exception& e) {
                    std::fprintf(stderr, "stream %d: %s\n", i, e.what());
                    failures.fetch_add(1);
                    at_start.fetch_add(1);
                }
            });
        }
        while (at_start.load() < n) std::this_thread::yield();
        xn_stats before{};
        std::vector<xn_stats> b0(static_cast<size_t>(group->size()));
        for (int g = 0; g < group->size(); ++g) xn_stats_get(group->ctx(g), &b0[size_t(g)]);
        t_go = std::chrono::steady_clock::now();
        go.store(true, std::memory_order_release);
        for (auto& t : threads) t.join();
        double wall = 0.0;
        for (double d : done_at) wall = std::max(wall, d);
        for (double x : sums) checksum += x;
        unsigned long long batches = 0, calls = 0, coalesced = 0;
        for (int g = 0; g < group->size(); ++g) {
            xn_stats a{};
            xn_stats_get(group->ctx(g), &a);
            batches += a.batches - b0[size_t(g)].batches;
            calls += a.calls - b0[size_t(g)].calls;
            coalesced = std::max<unsigned long long>(coalesced, a.coalesced_max);
        }
        (void)before;
        const char* win = std::getenv("XORNET_ATTN_BATCH_WINDOW_US");
        std::printf(
            "{\"streams\": %d, \"layers\": %d, \"steps\": %d, \"devices\": %d, \"kv_tokens\": %lld, "
            "\"wall_s\": %.6f, \"ms_per_step\": %.4f, \"tokens_per_s\": %.1f, \"calls\": %llu, "
            "\"batches\": %llu, \"batches_per_step\": %.2f, \"calls_per_batch\": %.2f, \"coalesced_max\": %llu, "
            "\"batch_window_us\": %d, \"failures\": %d, \"checksum\": %.6g}\n",
            n, layers, steps, group->size(), total_tokens, wall, wall / steps * 1e3, double(n) * steps / wall, calls,
            batches, double(batches) / steps, batches ? double(calls) / double(batches) : 0.0, coalesced,
            win ? std::atoi(win) : 0, failures.load(), checksum);
        caches.clear();
        return failures.load() ? 1 : 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "dropin_bench: %s\n", e.what());
        return 2;
    }
}
