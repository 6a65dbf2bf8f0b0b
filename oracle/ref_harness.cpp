// TEST INFRASTRUCTURE ONLY -- thin driver around the UNMODIFIED TurboLoader
// headers, compiled in place from the reference tree (never copied here) into
// oracle/_ref/ by oracle/Makefile.  It replays the transform half of
// DirectBatchCore::process_one (src/pipeline/direct_batch_loader.hpp:219-243)
// for explicit crop rects and flip flags, calling the reference's own
// resize_bilinear_simd and deinterleave_hwc_to_chw_f32
// (src/transforms/simd_utils.hpp) on the reference's own thread pool
// (src/core/parallel_for.hpp).  DirectBatchCore itself cannot be built here
// because it needs libjpeg/lz4/curl headers; the decode half it would add is
// outside the path anyway (inputs are pre-decoded pixels).
//
// Used (a) to pin the C restatement in fused_ref.c, (b) to generate
// tests/golden/, (c) as the timed CPU baseline ("kind": "reference").
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "src/core/parallel_for.hpp"
#include "src/transforms/simd_utils.hpp"

namespace tsimd = turboloader::transforms::simd;

extern "C" {

__attribute__((visibility("default"))) int tlref_threads() {
    return (int)turboloader::ThreadPool::global().concurrency();
}

// Which resize branch this build of the reference header selected.
__attribute__((visibility("default"))) const char* tlref_simd_branch() {
#if defined(TURBOLOADER_SIMD_AVX512)
    return "avx512-macro (scalar resize branch, avx2-width normalize)";
#elif defined(TURBOLOADER_SIMD_AVX2)
    return "avx2";
#elif defined(TURBOLOADER_SIMD_NEON)
    return "neon";
#else
    return "scalar";
#endif
}

__attribute__((visibility("default"))) void tlref_resize_bilinear(const uint8_t* src, uint8_t* dst,
                                                                  int sw, int sh, int dw, int dh) {
    tsimd::resize_bilinear_simd(src, dst, sw, sh, dw, dh, 3);
}

// Same argument meaning as tlo_fused_batch in fused_ref.c.  `threads` <= 1
// runs the samples on the calling thread; otherwise the reference pool
// (hardware_concurrency threads) is used, as fill_batch does
// (direct_batch_loader.hpp:106-113).
static int fused_batch_impl(
    const uint8_t* src, const int64_t* offsets, const int32_t* sizes, int64_t n_src,
    const int64_t* sel, const int32_t* boxes, const uint8_t* flips, int n, int dh, int dw,
    const float* mean, const float* std_, int normalize_01, float* out, int threads, bool antialias) {
    const float inv_std[3] = {1.0f / std_[0], 1.0f / std_[1], 1.0f / std_[2]};
    for (int i = 0; i < n; ++i) {
        int64_t s = sel ? sel[i] : i;
        if (s < 0 || s >= n_src) return -(i + 1);
        int iw = sizes[2 * s], ih = sizes[2 * s + 1];
        int cx = 0, cy = 0, cw = iw, ch = ih;
        if (boxes) { cx = boxes[4 * i]; cy = boxes[4 * i + 1]; cw = boxes[4 * i + 2]; ch = boxes[4 * i + 3]; }
        if (cw <= 0 || ch <= 0 || cx < 0 || cy < 0 || cx + cw > iw || cy + ch > ih) return -(i + 1);
    }
    const size_t npix = (size_t)dh * dw;
    auto one = [&](size_t i) {
        thread_local std::vector<uint8_t> cropped, resized;
        const int64_t s = sel ? sel[i] : (int64_t)i;
        const int iw = sizes[2 * s];
        const uint8_t* img = src + offsets[s];
        int cx = 0, cy = 0, cw = iw, ch = sizes[2 * s + 1];
        if (boxes) { cx = boxes[4 * i]; cy = boxes[4 * i + 1]; cw = boxes[4 * i + 2]; ch = boxes[4 * i + 3]; }
        cropped.resize((size_t)cw * ch * 3);
        for (int y = 0; y < ch; ++y)
            std::memcpy(cropped.data() + (size_t)y * cw * 3,
                        img + (((size_t)cy + y) * iw + cx) * 3, (size_t)cw * 3);
        resized.resize(npix * 3);
        if (cw == dw && ch == dh)
            std::memcpy(resized.data(), cropped.data(), resized.size());
        else if (antialias)  // direct_batch_loader.hpp:229-231
            tsimd::resize_triangle_antialias(cropped.data(), resized.data(), cw, ch, dw, dh, 3);
        else
            tsimd::resize_bilinear_simd(cropped.data(), resized.data(), cw, ch, dw, dh, 3);
        if (flips && flips[i]) {
            for (int y = 0; y < dh; ++y) {
                uint8_t* row = resized.data() + (size_t)y * dw * 3;
                for (int a = 0, b = dw - 1; a < b; ++a, --b)
                    for (int k = 0; k < 3; ++k) std::swap(row[a * 3 + k], row[b * 3 + k]);
            }
        }
        float* o = out + i * 3 * npix;
        tsimd::deinterleave_hwc_to_chw_f32(resized.data(), o, o + npix, o + 2 * npix, npix,
                                           normalize_01 != 0, mean, inv_std);
    };
    if (threads <= 1) {
        for (int i = 0; i < n; ++i) one((size_t)i);
    } else {
        turboloader::parallel_for((size_t)n, one);
    }
    return 0;
}

__attribute__((visibility("default"))) int tlref_fused_batch(
    const uint8_t* src, const int64_t* offsets, const int32_t* sizes, int64_t n_src,
    const int64_t* sel, const int32_t* boxes, const uint8_t* flips, int n, int dh, int dw,
    const float* mean, const float* std_, int normalize_01, float* out, int threads) {
    return fused_batch_impl(src, offsets, sizes, n_src, sel, boxes, flips, n, dh, dw, mean, std_, normalize_01, out,
                            threads, false);
}

// The same pipeline with DirectBatchCore's `antialias` option on.
__attribute__((visibility("default"))) int tlref_fused_batch_aa(
    const uint8_t* src, const int64_t* offsets, const int32_t* sizes, int64_t n_src,
    const int64_t* sel, const int32_t* boxes, const uint8_t* flips, int n, int dh, int dw,
    const float* mean, const float* std_, int normalize_01, float* out, int threads, int antialias) {
    return fused_batch_impl(src, offsets, sizes, n_src, sel, boxes, flips, n, dh, dw, mean, std_, normalize_01, out,
                            threads, antialias != 0);
}

}  // extern "C"
