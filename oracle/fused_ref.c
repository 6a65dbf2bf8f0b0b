/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of TurboLoader's fused image
 * transform, used as the parity oracle for the sm_100a kernels.  Nothing in
 * the shipped package may call into this file; only tests/, the smoke check
 * and the benchmark's cpu_baseline / reference arm may.
 *
 * Parity status: PINNED.  tests/test_oracle.py checks this restatement
 * bit-for-bit against (a) the golden vectors in tests/golden/ that were
 * generated from the reference's own headers, and (b) when the compiled
 * reference harness (oracle/_ref) is present, against the reference itself
 * on the size cases the reference's tests/test_simd_bilinear.cpp:111-251 use.
 *
 * Build: gcc -O2 -ffp-contract=off -fPIC -shared  (contraction must stay
 * off: the reference semantic is "every multiply and add rounds to fp32";
 * an FMA changes ~1e-4 of the uint8 results by one code value).
 *
 * Reference statements followed (paths are within the TurboLoader tree):
 *   src/transforms/simd_utils.hpp:97-103     resize_scale / resize_src_coord
 *   src/transforms/simd_utils.hpp:1897-1931  scalar bilinear u8 -> u8 (truncating)
 *   src/transforms/simd_utils.hpp:2201-2222  scalar u8 HWC -> f32 CHW normalize
 *   src/pipeline/direct_batch_loader.hpp:180-187  hflip of the RESIZED u8 image
 *   src/pipeline/direct_batch_loader.hpp:219-257  crop copy -> resize -> flip -> normalize
 *   src/pipeline/direct_batch_loader.hpp:55-59    inv_std = 1.0f / std
 *   src/python/turboloader_bindings.cpp:1198-1258 normalize_u8_gather (index gather)
 *   src/transforms/simd_utils.hpp:1939-2014  resize_triangle_antialias (opt-in quality resize)
 *   src/metal/metal_transforms.mm:111-115    colour jitter of the train_transform shader
 *       (PARITY UNPINNED for this one step: its only reference implementation is a Metal
 *       shader, which cannot be executed here; the restatement applies the shader's five
 *       lines to the CPU path's 8-bit code, each operation rounded separately)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(_WIN32)
#define TLO_API
#else
#define TLO_API __attribute__((visibility("default")))
#endif

/* simd_utils.hpp:97-99 */
static float tlo_scale(int src_dim, int dst_dim) {
    return (float)src_dim / (float)(dst_dim > 0 ? dst_dim : 1);
}

/* simd_utils.hpp:100-103 */
static float tlo_src_coord(int dst_idx, float scale) {
    float s = ((float)dst_idx + 0.5f) * scale - 0.5f;
    return s < 0.0f ? 0.0f : s;
}

/*
 * Bilinear u8 HWC -> u8 HWC, half-pixel centres, result TRUNCATED to uint8
 * after a [0,255] clamp (simd_utils.hpp:1897-1931).  `src` is a tightly
 * packed sw x sh x 3 image (the crop has already been copied out, so the
 * coordinate clamp is to the crop, not to the full image).
 */
TLO_API void tlo_resize_bilinear_u8(const uint8_t* src, uint8_t* dst, int sw, int sh,
                                    int dw, int dh) {
    const float xr = tlo_scale(sw, dw);
    const float yr = tlo_scale(sh, dh);
    for (int y = 0; y < dh; ++y) {
        float sy = tlo_src_coord(y, yr);
        int y0 = (int)sy;
        int y1 = y0 + 1 < sh - 1 ? y0 + 1 : sh - 1;
        float dy = sy - (float)y0;
        for (int x = 0; x < dw; ++x) {
            float sx = tlo_src_coord(x, xr);
            int x0 = (int)sx;
            int x1 = x0 + 1 < sw - 1 ? x0 + 1 : sw - 1;
            float dx = sx - (float)x0;
            for (int c = 0; c < 3; ++c) {
                float p00 = src[((size_t)y0 * sw + x0) * 3 + c];
                float p10 = src[((size_t)y0 * sw + x1) * 3 + c];
                float p01 = src[((size_t)y1 * sw + x0) * 3 + c];
                float p11 = src[((size_t)y1 * sw + x1) * 3 + c];
                float top = p00 * (1.0f - dx) + p10 * dx;
                float bot = p01 * (1.0f - dx) + p11 * dx;
                float val = top * (1.0f - dy) + bot * dy;
                float cl = val > 255.0f ? 255.0f : val;
                cl = cl < 0.0f ? 0.0f : cl;
                dst[((size_t)y * dw + x) * 3 + c] = (uint8_t)cl;
            }
        }
    }
}

/* u8 HWC -> f32 planes, (u8*s - mean)*inv_std (simd_utils.hpp:2201-2222). */
TLO_API void tlo_normalize_hwc_to_chw(const uint8_t* src, float* dst, size_t npix,
                                      int normalize_01, const float* mean,
                                      const float* inv_std) {
    const float s = normalize_01 ? (1.0f / 255.0f) : 1.0f;
    for (size_t i = 0; i < npix; ++i) {
        for (int c = 0; c < 3; ++c) {
            float v = (float)src[i * 3 + c] * s;
            if (mean && inv_std) v = (v - mean[c]) * inv_std[c];
            dst[(size_t)c * npix + i] = v;
        }
    }
}

/* fp32 -> bf16 bits, round to nearest even (the definition of the bf16 output). */
TLO_API uint16_t tlo_f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u); /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/*
 * One sample of DirectBatchCore::process_one's transform half
 * (direct_batch_loader.hpp:219-243) with an explicit rect and flip flag:
 * copy the crop rows out, resize (identity copy when the crop already has the
 * target size), flip the RESIZED u8 image, then normalize into three planes.
 * `scratch` must hold cw*ch*3 + dw*dh*3 bytes.
 */
/*
 * One axis of the antialiased triangle filter (simd_utils.hpp:1945-1975): for every output
 * index the first source tap, the tap count and the normalized weights.  `weights` has
 * dst_dim * max_taps entries.  Returns max_taps.
 */
static int tlo_aa_taps(int src_dim, int dst_dim, int* left, int* count, float* weights) {
    const float scale = tlo_scale(src_dim, dst_dim);
    const float support = scale > 1.0f ? scale : 1.0f;
    const int max_taps = (int)ceilf(support * 2.0f) + 2;
    if (!weights) return max_taps;
    for (int i = 0; i < dst_dim; ++i) {
        float* w = weights + (size_t)i * max_taps;
        const float center = ((float)i + 0.5f) * scale;
        int lo = (int)floorf(center - support);
        int hi = (int)ceilf(center + support);
        if (lo < 0) lo = 0;
        if (hi > src_dim) hi = src_dim;
        float wsum = 0.0f;
        int n = 0;
        for (int j = lo; j < hi && n < max_taps; ++j, ++n) {
            const float t = ((float)j + 0.5f - center) / support;
            float v = 1.0f - fabsf(t);
            if (v < 0.0f) v = 0.0f;
            w[n] = v;
            wsum += v;
        }
        if (wsum > 0.0f)
            for (int k = 0; k < n; ++k) w[k] /= wsum;
        left[i] = lo;
        count[i] = n;
    }
    return max_taps;
}

/*
 * Antialiased (triangle filter) resize u8 HWC -> u8 HWC (simd_utils.hpp:1939-2014): horizontal
 * pass into a float image, vertical pass, result rounded half up after a [0,255] clamp.  Every
 * accumulation is a sequential fp32 sum of separately rounded products, first tap first.
 */
TLO_API void tlo_resize_antialias_u8(const uint8_t* src, uint8_t* dst, int sw, int sh, int dw, int dh) {
    const int xt = tlo_aa_taps(sw, dw, NULL, NULL, NULL), yt = tlo_aa_taps(sh, dh, NULL, NULL, NULL);
    int* xl = (int*)malloc(sizeof(int) * 2 * ((size_t)dw + dh));
    int *xc = xl + dw, *yl = xc + dw, *yc = yl + dh;
    float* xw = (float*)calloc((size_t)dw * xt + (size_t)dh * yt, sizeof(float));
    float* yw = xw + (size_t)dw * xt;
    float* tmp = (float*)malloc(sizeof(float) * (size_t)sh * dw * 3);
    tlo_aa_taps(sw, dw, xl, xc, xw);
    tlo_aa_taps(sh, dh, yl, yc, yw);
    for (int y = 0; y < sh; ++y) {
        const uint8_t* srow = src + (size_t)y * sw * 3;
        float* trow = tmp + (size_t)y * dw * 3;
        for (int x = 0; x < dw; ++x) {
            const float* w = xw + (size_t)x * xt;
            for (int c = 0; c < 3; ++c) {
                float acc = 0.0f;
                for (int k = 0; k < xc[x]; ++k) acc += w[k] * (float)srow[(xl[x] + k) * 3 + c];
                trow[x * 3 + c] = acc;
            }
        }
    }
    for (int y = 0; y < dh; ++y) {
        const float* w = yw + (size_t)y * yt;
        for (int x = 0; x < dw; ++x)
            for (int c = 0; c < 3; ++c) {
                float acc = 0.0f;
                for (int k = 0; k < yc[y]; ++k) acc += w[k] * tmp[((size_t)(yl[y] + k) * dw + x) * 3 + c];
                float v = acc + 0.5f;
                v = v > 255.0f ? 255.0f : v;
                v = v < 0.0f ? 0.0f : v;
                dst[((size_t)y * dw + x) * 3 + c] = (uint8_t)v;
            }
    }
    free(tmp);
    free(xw);
    free(xl);
}

static int g_antialias = 0; /* set per call by tlo_fused_batch_aa; the oracle is single-threaded */
static const float* g_jitter = NULL; /* (brightness, contrast, saturation) of the current sample, or NULL */

/*
 * u8 HWC -> colour jitter -> f32 planes.  The jitter is the train_transform shader's
 * (src/metal/metal_transforms.mm:111-115), applied to rgb = u8 * (1/255):
 *   rgb *= brightness;  rgb = (rgb - 0.5)*contrast + 0.5;
 *   lum = dot(rgb, (0.299, 0.587, 0.114));  rgb = mix(lum, rgb, saturation);  clamp to [0,1]
 * with dot() summed left to right and mix(x, y, a) = x + (y - x)*a; every multiply, add and
 * subtract rounds to fp32 on its own (the file is compiled without contraction).
 */
static void tlo_jitter_normalize_hwc_to_chw(const uint8_t* src, float* dst, size_t npix, const float* jit,
                                            const float* mean, const float* inv_std) {
    const float s = 1.0f / 255.0f;
    for (size_t i = 0; i < npix; ++i) {
        float rgb[3];
        for (int c = 0; c < 3; ++c) {
            float v = (float)src[i * 3 + c] * s;
            v = v * jit[0];
            v = (v - 0.5f) * jit[1] + 0.5f;
            rgb[c] = v;
        }
        const float lum = (rgb[0] * 0.299f + rgb[1] * 0.587f) + rgb[2] * 0.114f;
        for (int c = 0; c < 3; ++c) {
            float v = lum + (rgb[c] - lum) * jit[2];
            v = v < 0.0f ? 0.0f : v;
            v = v > 1.0f ? 1.0f : v;
            dst[(size_t)c * npix + i] = (v - mean[c]) * inv_std[c];
        }
    }
}

static void tlo_one_sample(const uint8_t* img, int iw, int ih, int cx, int cy, int cw, int ch,
                           int flip, int dw, int dh, int normalize_01, const float* mean,
                           const float* inv_std, float* out_chw, uint8_t* scratch) {
    (void)ih;
    uint8_t* cropped = scratch;
    uint8_t* resized = scratch + (size_t)cw * ch * 3;
    for (int y = 0; y < ch; ++y)
        memcpy(cropped + (size_t)y * cw * 3, img + (((size_t)cy + y) * iw + cx) * 3,
               (size_t)cw * 3);
    if (cw == dw && ch == dh)
        memcpy(resized, cropped, (size_t)dw * dh * 3);
    else if (g_antialias)
        tlo_resize_antialias_u8(cropped, resized, cw, ch, dw, dh);
    else
        tlo_resize_bilinear_u8(cropped, resized, cw, ch, dw, dh);
    if (flip) {
        for (int y = 0; y < dh; ++y) {
            uint8_t* row = resized + (size_t)y * dw * 3;
            for (int a = 0, b = dw - 1; a < b; ++a, --b)
                for (int k = 0; k < 3; ++k) {
                    uint8_t t = row[a * 3 + k];
                    row[a * 3 + k] = row[b * 3 + k];
                    row[b * 3 + k] = t;
                }
        }
    }
    if (g_jitter)
        tlo_jitter_normalize_hwc_to_chw(resized, out_chw, (size_t)dw * dh, g_jitter, mean, inv_std);
    else
        tlo_normalize_hwc_to_chw(resized, out_chw, (size_t)dw * dh, normalize_01, mean, inv_std);
}

/*
 * Batch form used by the parity tests.
 *   src          packed u8 HWC images
 *   offsets[i]   byte offset of dataset image i inside src
 *   sizes[2i..]  (w, h) of dataset image i
 *   sel          n gather indices into the dataset, or NULL for 0..n-1
 *   boxes        n * (x, y, w, h) int32, or NULL for the full image
 *   flips        n flags, or NULL
 *   std_         per-channel std; 1.0f/std is formed in fp32 as the reference does
 *   out          n*3*dh*dw floats, NCHW
 * Returns 0, or -(i+1) when sample i has an invalid index or box.
 */
TLO_API int tlo_fused_batch(const uint8_t* src, const int64_t* offsets, const int32_t* sizes,
                            int64_t n_src, const int64_t* sel, const int32_t* boxes,
                            const uint8_t* flips, int n, int dh, int dw, const float* mean,
                            const float* std_, int normalize_01, float* out) {
    float inv_std[3];
    for (int c = 0; c < 3; ++c) inv_std[c] = 1.0f / std_[c];
    size_t cap = 0;
    uint8_t* scratch = NULL;
    for (int i = 0; i < n; ++i) {
        int64_t s = sel ? sel[i] : i;
        if (s < 0 || s >= n_src) { free(scratch); return -(i + 1); }
        int iw = sizes[2 * s], ih = sizes[2 * s + 1];
        int cx = 0, cy = 0, cw = iw, ch = ih;
        if (boxes) { cx = boxes[4 * i]; cy = boxes[4 * i + 1]; cw = boxes[4 * i + 2]; ch = boxes[4 * i + 3]; }
        if (cw <= 0 || ch <= 0 || cx < 0 || cy < 0 || cx + cw > iw || cy + ch > ih) {
            free(scratch);
            return -(i + 1);
        }
        size_t need = (size_t)cw * ch * 3 + (size_t)dw * dh * 3;
        if (need > cap) { free(scratch); scratch = (uint8_t*)malloc(need); cap = need; }
        tlo_one_sample(src + offsets[s], iw, ih, cx, cy, cw, ch, flips ? flips[i] : 0, dw, dh,
                       normalize_01, mean, inv_std, out + (size_t)i * 3 * dh * dw, scratch);
    }
    free(scratch);
    return 0;
}

/* Same, with the resize of direct_batch_loader.hpp:229-231 selected by `antialias`. */
TLO_API int tlo_fused_batch_aa(const uint8_t* src, const int64_t* offsets, const int32_t* sizes,
                               int64_t n_src, const int64_t* sel, const int32_t* boxes,
                               const uint8_t* flips, int n, int dh, int dw, const float* mean,
                               const float* std_, int normalize_01, float* out, int antialias) {
    g_antialias = antialias != 0;
    const int rc = tlo_fused_batch(src, offsets, sizes, n_src, sel, boxes, flips, n, dh, dw, mean, std_,
                                   normalize_01, out);
    g_antialias = 0;
    return rc;
}

/* Same as tlo_fused_batch with per-sample colour jitter: jitter = n x (brightness, contrast,
 * saturation).  mean/std are in [0,1] units (normalize_01 is implied). */
TLO_API int tlo_fused_batch_jitter(const uint8_t* src, const int64_t* offsets, const int32_t* sizes,
                                   int64_t n_src, const int64_t* sel, const int32_t* boxes,
                                   const uint8_t* flips, int n, int dh, int dw, const float* mean,
                                   const float* std_, const float* jitter, float* out) {
    for (int i = 0; i < n; ++i) {
        g_jitter = jitter + 3 * (size_t)i;
        const int64_t one_sel = sel ? sel[i] : i;
        const int rc = tlo_fused_batch(src, offsets, sizes, n_src, &one_sel, boxes ? boxes + 4 * (size_t)i : NULL,
                                       flips ? flips + i : NULL, 1, dh, dw, mean, std_, 1,
                                       out + (size_t)i * 3 * dh * dw);
        g_jitter = NULL;
        if (rc) return -(i + 1);
    }
    return 0;
}

/* ... and with the antialiased resize in front of the jitter (the reference has both options on
 * its training path: direct_batch_loader.hpp:229-231 picks the filter, the shader jitters the
 * resized 8-bit image). */
TLO_API int tlo_fused_batch_aa_jitter(const uint8_t* src, const int64_t* offsets, const int32_t* sizes,
                                      int64_t n_src, const int64_t* sel, const int32_t* boxes,
                                      const uint8_t* flips, int n, int dh, int dw, const float* mean,
                                      const float* std_, const float* jitter, float* out) {
    g_antialias = 1;
    const int rc = tlo_fused_batch_jitter(src, offsets, sizes, n_src, sel, boxes, flips, n, dh, dw, mean, std_,
                                          jitter, out);
    g_antialias = 0;
    return rc;
}

/* NCHW f32 -> NHWC f32 (same values, permuted). */
TLO_API void tlo_nchw_to_nhwc(const float* in, float* out, int n, int h, int w) {
    size_t hw = (size_t)h * w;
    for (int i = 0; i < n; ++i)
        for (size_t p = 0; p < hw; ++p)
            for (int c = 0; c < 3; ++c)
                out[((size_t)i * hw + p) * 3 + c] = in[((size_t)i * 3 + c) * hw + p];
}

TLO_API void tlo_f32_to_bf16_array(const float* in, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = tlo_f32_to_bf16(in[i]);
}
