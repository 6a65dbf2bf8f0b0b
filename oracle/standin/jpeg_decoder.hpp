// TEST INFRASTRUCTURE ONLY -- stand-in for the one dependency that keeps the reference's
// DirectBatchCore (src/pipeline/direct_batch_loader.hpp) from compiling on a machine without
// libjpeg: its JPEG wrapper (src/decode/jpeg_decoder.hpp).  oracle/Makefile (target `refdbc`)
// builds a directory of symbolic links in which direct_batch_loader.hpp and every other header
// it includes are the reference's own files, and only "../decode/jpeg_decoder.hpp" resolves to
// this file.  The class below has the one member DirectBatchCore calls.  Instead of JPEG it reads
// a trivial container for PRE-DECODED pixels, which is exactly the input of the path under test:
//     bytes 0-3  "RAW8"
//     bytes 4-7  width  (little-endian int32)
//     bytes 8-11 height (little-endian int32)
//     then       width*height*3 bytes, HWC, RGB
// so the reference's own batch loop (build_order, acquire_batch, fill_batch, pick_crop,
// process_one) runs unmodified on the same pixels the GPU path gets.
#pragma once

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <vector>

#include "../core/compat.hpp"

namespace turboloader {

class JPEGDecoder {
public:
    void decode_scaled(turboloader::span<const uint8_t> data, std::vector<uint8_t>& output, int /*target_width*/,
                       int /*target_height*/, int& actual_width, int& actual_height, int& channels) {
        if (data.size() < 12 || std::memcmp(data.data(), "RAW8", 4) != 0) throw std::runtime_error("not a RAW8 sample");
        int32_t w, h;
        std::memcpy(&w, data.data() + 4, 4);
        std::memcpy(&h, data.data() + 8, 4);
        const size_t bytes = static_cast<size_t>(w) * h * 3;
        if (w <= 0 || h <= 0 || data.size() < 12 + bytes) throw std::runtime_error("truncated RAW8 sample");
        output.assign(data.data() + 12, data.data() + 12 + bytes);
        actual_width = w;
        actual_height = h;
        channels = 3;
    }
};

}  // namespace turboloader
