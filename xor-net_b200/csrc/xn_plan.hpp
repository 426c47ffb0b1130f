// Host-side planning for the split-KV attention launch.  Pure C++ (no CUDA): unit-tested on
// machines without a GPU through xn_plan_split.
#pragma once
#include <cstdint>
#include <vector>

namespace xn {

struct SplitItem {
    int32_t unit, tile_begin, tile_end, part;
};

struct SplitPlan {
    std::vector<SplitItem> items;
    std::vector<int32_t> cta_item_begin;  // ctas + 1 entries
    std::vector<int32_t> unit_part_begin; // per unit: first partial slot or -1
    std::vector<int32_t> unit_part_count; // per unit: number of items covering it
    int32_t ctas = 0;
    int32_t n_parts = 0;
    int64_t total_tiles = 0;
};

// Deals the flattened tile sequence of all units evenly to at most max_ctas thread blocks.
// Block b receives tiles [b*T/ctas, (b+1)*T/ctas) of the sequence; every maximal run of tiles
// of one unit inside a block's range becomes an item.  A unit covered by a single item is
// written directly by that block (part = -1); otherwise each of its items gets a partial slot,
// numbered consecutively per unit.
inline SplitPlan plan_split(const int32_t* kv_len, int32_t n_units, int32_t tile_tokens,
                            int32_t max_ctas) {
    SplitPlan p;
    p.unit_part_begin.assign(n_units, -1);
    p.unit_part_count.assign(n_units, 0);
    std::vector<int64_t> first_tile(n_units + 1, 0);
    for (int32_t u = 0; u < n_units; ++u) {
        int64_t tiles = kv_len[u] > 0 ? (int64_t(kv_len[u]) + tile_tokens - 1) / tile_tokens : 0;
        first_tile[u + 1] = first_tile[u] + tiles;
    }
    const int64_t T = first_tile[n_units];
    p.total_tiles = T;
    if (T == 0 || max_ctas <= 0) {
        p.cta_item_begin.assign(1, 0);
        return p;
    }
    const int32_t ctas = int32_t(T < max_ctas ? T : max_ctas);
    p.ctas = ctas;
    p.cta_item_begin.reserve(ctas + 1);
    int32_t u = 0;
    for (int32_t b = 0; b < ctas; ++b) {
        const int64_t lo = T * b / ctas, hi = T * (b + 1) / ctas;
        p.cta_item_begin.push_back(int32_t(p.items.size()));
        int64_t cur = lo;
        while (cur < hi) {
            while (first_tile[u + 1] <= cur) ++u;
            const int64_t end = first_tile[u + 1] < hi ? first_tile[u + 1] : hi;
            p.items.push_back({u, int32_t(cur - first_tile[u]), int32_t(end - first_tile[u]), -1});
            p.unit_part_count[u] += 1;
            cur = end;
        }
    }
    p.cta_item_begin.push_back(int32_t(p.items.size()));
    int32_t next_part = 0;
    for (int32_t i = 0; i < n_units; ++i) {
        if (p.unit_part_count[i] > 1) {
            p.unit_part_begin[i] = next_part;
            next_part += p.unit_part_count[i];
        }
    }
    p.n_parts = next_part;
    std::vector<int32_t> seen(n_units, 0);
    for (auto& it : p.items) {
        if (p.unit_part_count[it.unit] > 1) it.part = p.unit_part_begin[it.unit] + seen[it.unit]++;
    }
    return p;
}

}  // namespace xn
