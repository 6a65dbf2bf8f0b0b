/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of TurboLoader's fused YUV 4:2:0 video
 * transform (YUV -> RGB, optional crop window + horizontal flip, bilinear resize,
 * normalize, planar float output), used as the parity oracle for the sm_100a video
 * kernel.  Nothing in the shipped package may call into this file.
 *
 * The reference has no CPU implementation of this path: the statement followed is its CUDA
 * kernel source, read as plain C arithmetic with every multiply, add and divide rounded to
 * fp32 separately (build with -ffp-contract=off):
 *   src/cuda/cuda_transforms.cu:143-197  yuv420_resize_normalize_kernel (whole-frame resize)
 *   src/cuda/cuda_transforms.cu:207-268  yuv420_clip_crop_normalize_kernel (crop window + flip)
 *   src/cuda/cuda_transforms.cu:392-393, 453-455  inv_std = 1.0f / std on the host
 *
 * Parity status: PINNED ON THE GPU BOX.  tests/test_gpu_video.py runs the reference's own
 * kernels (compiled in place without FMA contraction, oracle/_ref/libtl_ref_cuda_nofma.so)
 * on the same inputs and requires bit-identical output from this restatement; the golden
 * vectors in tests/golden/video_*.npz were written by that reference build on a B200 and are
 * checked on CPU.  With the reference's default flags (contraction on) its kernels agree with
 * this file to rounding (~1e-6), which the same test also checks.
 */
#include <math.h>
#include <stdint.h>

#define TLO_API __attribute__((visibility("default")))

static float lerp2(const uint8_t* row, int i0, int i1, float w) {
    /* p0 * (1 - w) + p1 * w, bytes converted to float first */
    return (float)row[i0] * (1.0f - w) + (float)row[i1] * w;
}

/*
 * One frame -> out[3][dst_h][dst_w] (fp32).
 *   c_px_stride 1: I420 (separate cb / cr planes); 2: NV12 (cr = cb + 1 in one interleaved plane).
 *   use_crop 0: whole-frame sampling of the batch kernel (crop/flip ignored);
 *            1: crop window (x, y, w, h in source pixels, floats) + flip of the clip kernel.
 */
TLO_API void tlo_yuv420_frame(const uint8_t* yp, const uint8_t* cbp, const uint8_t* crp, int y_stride,
                              int c_stride, int c_px_stride, int src_w, int src_h, int dst_w, int dst_h,
                              int use_crop, const float* crop, int flip, int bt709, const float* mean,
                              const float* std_, float* out) {
    const float isd[3] = {1.0f / std_[0], 1.0f / std_[1], 1.0f / std_[2]};
    const int cw = (src_w + 1) / 2, ch = (src_h + 1) / 2;
    const float kY = 255.0f / 219.0f;
    for (int y = 0; y < dst_h; ++y) {
        float sy;
        if (use_crop) {
            sy = crop[1] + ((float)y + 0.5f) / (float)dst_h * crop[3] - 0.5f;
            sy = fminf(fmaxf(sy, 0.0f), (float)(src_h - 1));
        } else {
            sy = fmaxf(0.0f, ((float)y + 0.5f) * (float)src_h / (float)dst_h - 0.5f);
        }
        const int y0 = (int)sy;
        const int y1 = y0 + 1 < src_h - 1 ? y0 + 1 : src_h - 1;
        const float dy = sy - (float)y0;
        const float cyf = fminf(fmaxf(sy * 0.5f - 0.25f, 0.0f), (float)(ch - 1));
        const int cy0 = (int)cyf;
        const int cy1 = cy0 + 1 < ch - 1 ? cy0 + 1 : ch - 1;
        const float cdy = cyf - (float)cy0;
        for (int x = 0; x < dst_w; ++x) {
            float sx;
            if (use_crop) {
                const int ox = flip ? (dst_w - 1 - x) : x;
                sx = crop[0] + ((float)ox + 0.5f) / (float)dst_w * crop[2] - 0.5f;
                sx = fminf(fmaxf(sx, 0.0f), (float)(src_w - 1));
            } else {
                sx = fmaxf(0.0f, ((float)x + 0.5f) * (float)src_w / (float)dst_w - 0.5f);
            }
            const int x0 = (int)sx;
            const int x1 = x0 + 1 < src_w - 1 ? x0 + 1 : src_w - 1;
            const float dx = sx - (float)x0;
            const float ytop = lerp2(yp + (long)y0 * y_stride, x0, x1, dx);
            const float ybot = lerp2(yp + (long)y1 * y_stride, x0, x1, dx);
            const float yv0 = ytop * (1.0f - dy) + ybot * dy;

            const float cxf = fminf(fmaxf(sx * 0.5f, 0.0f), (float)(cw - 1));
            const int cx0 = (int)cxf;
            const int cx1 = cx0 + 1 < cw - 1 ? cx0 + 1 : cw - 1;
            const float cdx = cxf - (float)cx0;
            const int i0 = cx0 * c_px_stride, i1 = cx1 * c_px_stride;
            const float cbv = lerp2(cbp + (long)cy0 * c_stride, i0, i1, cdx) * (1.0f - cdy) +
                              lerp2(cbp + (long)cy1 * c_stride, i0, i1, cdx) * cdy;
            const float crv = lerp2(crp + (long)cy0 * c_stride, i0, i1, cdx) * (1.0f - cdy) +
                              lerp2(crp + (long)cy1 * c_stride, i0, i1, cdx) * cdy;

            const float yv = (yv0 - 16.0f) * kY;
            const float cb = cbv - 128.0f, cr = crv - 128.0f;
            float r, g, b;
            if (bt709) {
                r = yv + 1.792741f * cr;
                g = yv - 0.213249f * cb - 0.532909f * cr;
                b = yv + 2.112402f * cb;
            } else {
                r = yv + 1.596027f * cr;
                g = yv - 0.391762f * cb - 0.812968f * cr;
                b = yv + 2.017232f * cb;
            }
            const float rgb[3] = {fminf(fmaxf(r / 255.0f, 0.0f), 1.0f), fminf(fmaxf(g / 255.0f, 0.0f), 1.0f),
                                  fminf(fmaxf(b / 255.0f, 0.0f), 1.0f)};
            for (int c = 0; c < 3; ++c)
                out[((long)c * dst_h + y) * dst_w + x] = (rgb[c] - mean[c]) * isd[c];
        }
    }
}
