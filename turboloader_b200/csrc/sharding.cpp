// Host-only shard index math behind the C ABI (no CUDA).  Mirrors the rules of
// TurboLoader's src/distributed/sharding_strategies.hpp:150-316 (contiguous block with the
// remainder spread over the low ranks; stride-by-world; splitmix64 hash modulo world),
// DistributedSampler::get_indices (src/distributed/distributed_dataloader.hpp:111-149:
// Fisher-Yates with mt19937(seed+epoch), wrap-around padding, rank-strided pick) and
// DirectBatchCore::build_order (src/pipeline/direct_batch_loader.hpp:116-135:
// std::shuffle with mt19937_64(seed+epoch), then floor(total/world) block per rank).
// The shuffles call the same standard-library engines and algorithms as those sources,
// so the orders agree element for element when both are built with the same libstdc++.
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <random>
#include <vector>

#include "../../include/turboloader_b200.h"

namespace {

constexpr uint64_t kHashSeed = 0x517cc1b727220a95ULL;

uint64_t mix(uint64_t x) {
    x ^= x >> 30;
    x *= 0xbf58476d1ce4e5b9ULL;
    x ^= x >> 27;
    x *= 0x94d049bb133111ebULL;
    x ^= x >> 31;
    return x;
}

template <class It>
int64_t emit(It b, It e, int64_t* out, int64_t cap) {
    int64_t n = 0;
    for (; b != e; ++b, ++n)
        if (out && n < cap) out[n] = static_cast<int64_t>(*b);
    return n;
}

}  // namespace

extern "C" {

int64_t tlb_shard_indices(int32_t kind, int64_t total, int64_t world, int64_t rank, int64_t* out, int64_t cap) {
    if (world <= 0 || rank < 0 || rank >= world || total < 0 || kind < 0 || kind > 2) return -1;
    int64_t n = 0;
    auto put = [&](int64_t v) {
        if (out && n < cap) out[n] = v;
        ++n;
    };
    if (kind == 0) {
        const int64_t base = total / world, rem = total % world;
        const int64_t start = rank < rem ? rank * (base + 1) : rank * base + rem;
        const int64_t len = base + (rank < rem ? 1 : 0);
        for (int64_t i = 0; i < len; ++i) put(start + i);
    } else if (kind == 1) {
        for (int64_t i = rank; i < total; i += world) put(i);
    } else {
        for (int64_t i = 0; i < total; ++i)
            if (static_cast<int64_t>(mix(kHashSeed ^ static_cast<uint64_t>(i)) % static_cast<uint64_t>(world)) == rank) put(i);
    }
    return n;
}

int64_t tlb_sampler_indices(int64_t total, int32_t world, int32_t rank, int32_t shuffle, uint64_t seed, uint64_t epoch,
                            int32_t drop_last, int64_t* out, int64_t cap) {
    if (world < 1 || rank < 0 || rank >= world || total < 0) return -1;
    const size_t T = static_cast<size_t>(total), Wn = static_cast<size_t>(world);
    const size_t per = drop_last ? T / Wn : (T + Wn - 1) / Wn;
    const size_t padded = per * Wn;
    std::vector<size_t> idx(T);
    std::iota(idx.begin(), idx.end(), size_t{0});
    if (shuffle && T > 1) {
        std::mt19937 rng(static_cast<uint32_t>(seed + epoch));
        for (size_t i = T - 1; i > 0; --i) {
            std::uniform_int_distribution<size_t> pick(0, i);
            std::swap(idx[i], idx[pick(rng)]);
        }
    }
    if (!drop_last && T > 0)
        for (size_t i = 0; idx.size() < padded; ++i) idx.push_back(idx[i % T]);
    std::vector<size_t> shard;
    for (size_t i = static_cast<size_t>(rank); i < padded; i += Wn)
        if (i < idx.size()) shard.push_back(idx[i]);
    return emit(shard.begin(), shard.end(), out, cap);
}

int64_t tlb_direct_order(int64_t total, int32_t shuffle, int32_t seed, int32_t epoch, int32_t distributed, int32_t rank,
                         int32_t world, int64_t* out, int64_t cap) {
    if (total < 0 || (distributed && world > 1 && (rank < 0 || rank >= world))) return -1;
    std::vector<size_t> order(static_cast<size_t>(total));
    std::iota(order.begin(), order.end(), size_t{0});
    if (shuffle) {
        std::mt19937_64 rng(static_cast<uint64_t>(seed) + static_cast<uint64_t>(epoch));
        std::shuffle(order.begin(), order.end(), rng);
    }
    auto b = order.begin(), e = order.end();
    if (distributed && world > 1) {
        const size_t per = order.size() / static_cast<size_t>(world);
        b = order.begin() + static_cast<size_t>(rank) * per;
        e = b + per;
    }
    return emit(b, e, out, cap);
}

}  // extern "C"
