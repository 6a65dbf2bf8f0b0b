// TEST INFRASTRUCTURE ONLY -- exposes the UNMODIFIED reference sharding headers
// (src/distributed/sharding_strategies.hpp, src/distributed/distributed_dataloader.hpp),
// compiled in place from the reference tree, through a C interface so the tests can
// compare the package's own index math with them and so tests/golden/ can be generated.
// (DirectBatchCore::build_order is exposed by ref_dbc_harness.cpp, which runs that class itself.)
#include <cstdint>
#include <vector>

#include "src/distributed/distributed_dataloader.hpp"
#include "src/distributed/sharding_strategies.hpp"

#define API extern "C" __attribute__((visibility("default")))

// kind: 0 contiguous, 1 interleaved, 2 hash.  Returns the shard size, or -1 on a
// constructor exception; writes at most cap indices.
API int64_t tlref_shard_indices(int kind, int64_t total, int64_t world, int64_t rank, int64_t* out,
                                int64_t cap) {
    try {
        auto s = turboloader::ShardingStrategy::create((turboloader::ShardingType)kind, (size_t)total,
                                                       (size_t)world, (size_t)rank);
        auto v = s->get_indices();
        for (size_t i = 0; i < v.size() && (int64_t)i < cap; ++i) out[i] = (int64_t)v[i];
        return (int64_t)v.size();
    } catch (...) {
        return -1;
    }
}

API int64_t tlref_sampler_indices(int64_t total, int world, int rank, int shuffle, uint64_t seed,
                                  uint64_t epoch, int drop_last, int64_t* out, int64_t cap) {
    try {
        turboloader::distributed::DistributedConfig cfg;
        cfg.world_size = world;
        cfg.rank = rank;
        cfg.drop_last = drop_last != 0;
        cfg.seed = (size_t)seed;
        cfg.shuffle = shuffle != 0;
        turboloader::distributed::DistributedSampler s((size_t)total, cfg);
        auto v = s.get_indices((size_t)epoch);
        for (size_t i = 0; i < v.size() && (int64_t)i < cap; ++i) out[i] = (int64_t)v[i];
        return (int64_t)v.size();
    } catch (...) {
        return -1;
    }
}
