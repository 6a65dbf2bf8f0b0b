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
#include <cmath>
#include <cstdint>
#include <numeric>
#include <random>
#include <thread>
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


// RandomResizedCrop + horizontal-flip sampler of the direct-batch loader
// (DirectBatchCore::pick_crop, src/pipeline/direct_batch_loader.hpp:141-178): per sample a
// mt19937_64 seeded with (seed << 32) ^ (epoch << 20) ^ index; up to 10 attempts of
// area * U(0.08, 1) with a log-uniform aspect ratio in [3/4, 4/3], integer rect accepted when
// it fits; otherwise the central crop at the clamped aspect ratio; the flip flag is the last
// draw.  All arithmetic is in float, draws come from uniform_real_distribution<float>(0, 1),
// in the same order, so with the same libstdc++ the rects agree with that loader's.
int64_t tlb_pick_crops(int32_t seed, int32_t epoch, const int64_t* indices, const int32_t* sizes_wh, int64_t n,
                       float hflip_prob, int32_t* boxes_out, uint8_t* flips_out) {
    if (n < 0 || !sizes_wh || !boxes_out) return -1;
    const float lo = std::log(3.0f / 4.0f), hi = std::log(4.0f / 3.0f);
    // Every sample has its own generator, so the samples of a whole epoch are drawn on all host cores:
    // seeding a 64-bit Mersenne twister and regenerating its state costs ~1 us per sample, which for an
    // epoch of a million images would otherwise hold the loader back for a second.
    auto draw = [&](int64_t i0, int64_t i1) -> int64_t {
    for (int64_t i = i0; i < i1; ++i) {
        const int w = sizes_wh[2 * i], h = sizes_wh[2 * i + 1];
        if (w <= 0 || h <= 0) return -(i + 2);
        const uint64_t idx = static_cast<uint64_t>(indices ? indices[i] : i);
        std::mt19937_64 rng((static_cast<uint64_t>(seed) << 32) ^ (static_cast<uint64_t>(epoch) << 20) ^ idx);
        std::uniform_real_distribution<float> uni(0.0f, 1.0f);
        const float area = static_cast<float>(w) * h;
        int bx = 0, by = 0, bw = w, bh = h;
        bool found = false;
        for (int attempt = 0; attempt < 10 && !found; ++attempt) {
            const float target = area * (0.08f + uni(rng) * (1.0f - 0.08f));
            const float ratio = std::exp(lo + uni(rng) * (hi - lo));
            const int cw = static_cast<int>(std::lround(std::sqrt(target * ratio)));
            const int ch = static_cast<int>(std::lround(std::sqrt(target / ratio)));
            if (cw > 0 && ch > 0 && cw <= w && ch <= h) {
                bw = cw;
                bh = ch;
                bx = std::min(static_cast<int>(uni(rng) * (w - cw + 1)), w - cw);
                by = std::min(static_cast<int>(uni(rng) * (h - ch + 1)), h - ch);
                found = true;
            }
        }
        if (!found) {
            const float in_ratio = static_cast<float>(w) / h;
            if (in_ratio < 3.0f / 4.0f) {
                bw = w;
                bh = std::min(h, static_cast<int>(std::lround(w / (3.0f / 4.0f))));
            } else if (in_ratio > 4.0f / 3.0f) {
                bh = h;
                bw = std::min(w, static_cast<int>(std::lround(h * (4.0f / 3.0f))));
            }
            bx = (w - bw) / 2;
            by = (h - bh) / 2;
        }
        const bool flip = uni(rng) < hflip_prob;
        boxes_out[4 * i] = bx;
        boxes_out[4 * i + 1] = by;
        boxes_out[4 * i + 2] = bw;
        boxes_out[4 * i + 3] = bh;
        if (flips_out) flips_out[i] = flip ? 1 : 0;
    }
    return 0;
    };
    constexpr int64_t kPerThread = 4096;
    unsigned threads = std::thread::hardware_concurrency();
    threads = static_cast<unsigned>(std::min<int64_t>(std::min<unsigned>(threads ? threads : 1u, 32u), (n + kPerThread - 1) / kPerThread));
    if (threads <= 1) {
        const int64_t rc = draw(0, n);
        return rc < 0 ? rc : n;
    }
    std::vector<int64_t> rcs(threads, 0);
    std::vector<std::thread> pool;
    const int64_t chunk = (n + threads - 1) / threads;
    for (unsigned t = 1; t < threads; ++t)
        pool.emplace_back([&, t] { rcs[t] = draw(std::min<int64_t>(n, t * chunk), std::min<int64_t>(n, (t + 1) * chunk)); });
    rcs[0] = draw(0, std::min<int64_t>(n, chunk));
    for (auto& th : pool) th.join();
    for (int64_t rc : rcs)
        if (rc < 0) return rc;  // chunks are in index order: the first failing chunk holds the first bad sample
    return n;
}

}  // extern "C"
