// TEST INFRASTRUCTURE ONLY -- runs the reference's UNMODIFIED DirectBatchCore
// (src/pipeline/direct_batch_loader.hpp, compiled where it lies in the reference tree through
// the link directory oracle/Makefile builds) behind a C interface: epoch order, batch cursor,
// the RandomResizedCrop + flip sampler and the per-sample transform, fed from an in-memory TAR of
// pre-decoded "RAW8" samples (see standin/jpeg_decoder.hpp for the one stand-in).
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <numeric>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

// The sampler and the order are private members; the class itself is not edited.
#define private public
#include "src/pipeline/direct_batch_loader.hpp"
#undef private

#define API extern "C" __attribute__((visibility("default")))

using turboloader::DirectBatchCore;

API void* tlref_dbc_create(const uint8_t* tar, int64_t tar_bytes, int batch, int h, int w, int chw, int normalize_01,
                           const float* mean, const float* std_, int shuffle, int seed, int distributed, int rank,
                           int world, int drop_last, int antialias, int train_aug, float hflip_prob) {
    try {
        auto data = std::make_shared<std::vector<uint8_t>>(tar, tar + tar_bytes);
        std::vector<float> m, s;
        if (mean && std_) {
            m.assign(mean, mean + 3);
            s.assign(std_, std_ + 3);
        }
        return new DirectBatchCore("", data, static_cast<size_t>(batch), h, w, chw != 0, normalize_01 != 0, m, s,
                                   shuffle != 0, seed, distributed != 0, rank, world, drop_last != 0, antialias != 0,
                                   train_aug != 0, hflip_prob);
    } catch (...) {
        return nullptr;
    }
}

API void tlref_dbc_destroy(void* c) { delete static_cast<DirectBatchCore*>(c); }

API int64_t tlref_dbc_num_samples(void* c) { return static_cast<int64_t>(static_cast<DirectBatchCore*>(c)->num_samples()); }

API void tlref_dbc_begin_epoch(void* c, int epoch, int64_t start_batch) {
    static_cast<DirectBatchCore*>(c)->begin_epoch(epoch, static_cast<size_t>(start_batch));
}

// acquire_batch + fill_batch: writes the batch's sample indices and its float32 output; returns the
// batch size (0 at the end of the epoch).
API int tlref_dbc_next(void* c, int64_t* indices_out, float* out) {
    auto* core = static_cast<DirectBatchCore*>(c);
    std::vector<size_t> idx;
    const size_t bs = core->acquire_batch(idx);
    if (bs == 0) return 0;
    for (size_t i = 0; i < bs; ++i) indices_out[i] = static_cast<int64_t>(idx[i]);
    core->fill_batch(idx, out);
    return static_cast<int>(bs);
}

// The epoch's order as built by build_order (after begin_epoch).
API int64_t tlref_dbc_order(void* c, int64_t* out, int64_t cap) {
    auto* core = static_cast<DirectBatchCore*>(c);
    const auto& o = core->order_;
    for (size_t i = 0; i < o.size() && static_cast<int64_t>(i) < cap; ++i) out[i] = static_cast<int64_t>(o[i]);
    return static_cast<int64_t>(o.size());
}

// pick_crop for n samples: sizes_wh = n x (w, h), indices = n sample indices; out = n x (x, y, w, h, flip).
API void tlref_dbc_pick_crops(void* c, const int32_t* sizes_wh, const int64_t* indices, int64_t n, int32_t* out) {
    auto* core = static_cast<DirectBatchCore*>(c);
    for (int64_t i = 0; i < n; ++i) {
        const auto r = core->pick_crop(sizes_wh[2 * i], sizes_wh[2 * i + 1], static_cast<size_t>(indices[i]));
        out[5 * i] = r.x;
        out[5 * i + 1] = r.y;
        out[5 * i + 2] = r.w;
        out[5 * i + 3] = r.h;
        out[5 * i + 4] = r.flip ? 1 : 0;
    }
}

API int64_t tlref_dbc_decode_failures(void* c) {
    return static_cast<int64_t>(static_cast<DirectBatchCore*>(c)->decode_failures());
}
