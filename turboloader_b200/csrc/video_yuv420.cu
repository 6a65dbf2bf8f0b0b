// Fused YUV 4:2:0 video transform for sm_100a: per output pixel, bilinear luma + bilinear
// chroma (MPEG siting: horizontally co-sited, vertically centred), video-range BT.601 / BT.709
// matrix, clip to [0,1], mean/std normalize, planar (T,3,H,W) fp32 or bf16 output; optionally a
// crop window + horizontal flip shared by all frames of a clip.  One launch covers every frame of
// the batch (the functions replaced launch once per frame or once per clip):
//   turboloader::cuda::video_yuv420_batch   src/cuda/cuda_transforms.cu:143-197, 367-409
//   turboloader::cuda::video_clip_yuv420    src/cuda/cuda_transforms.cu:207-268, 416-473
//
// Arithmetic: the kernels replaced are the only statement of this math; it is followed operation
// by operation with every multiply, add and divide rounded to fp32 separately (this library is
// built without FMA contraction), which is what the CPU oracle restates.  Bytes become floats
// without an integer conversion: fma(2^23 + b, w, -2^23 * w) is exactly RN(b * w).
//
// Work split: a CTA owns kVideoRows output rows of one frame; a thread owns one output column
// (columns beyond the block width wrap) and walks down the rows, so the horizontal taps and
// weights (luma and chroma) are worked out once per thread and the vertical ones once per CTA
// (a small table in shared memory).  A warp's stores are 32 consecutive outputs of one row.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdint>

#include "video_params.h"

namespace tlb {
namespace {

constexpr int kVideoRows = 8;  // output rows per CTA

struct RowTaps {
    int y0, y1;    // byte offsets of the two luma rows
    int c0, c1;    // byte offsets of the two chroma rows
    float dy, cdy;
    float idy, icdy;  // 1 - dy, 1 - cdy
};

__device__ __forceinline__ float byte_times(unsigned b, float w, float nw) {
    return __fmaf_rn(__uint_as_float(b | 0x4B000000u), w, nw);  // == RN(b * w); nw = -2^23 * w
}

template <int DTYPE>
__device__ __forceinline__ void put(void* out, long long idx, float v) {
    if constexpr (DTYPE == 0)
        static_cast<float*>(out)[idx] = v;
    else
        static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
}

template <int DTYPE>
__global__ void __launch_bounds__(256) yuv420_kernel(const __grid_constant__ VideoParams p) {
    __shared__ RowTaps taps[kVideoRows];
    const int t = blockIdx.y;                    // frame
    const int r0 = blockIdx.x * kVideoRows;      // first output row of this CTA
    const int rows = min(kVideoRows, p.dst_h - r0);
    const int W = p.dst_w, H = p.dst_h;
    const int cw = (p.src_w + 1) / 2, ch = (p.src_h + 1) / 2;
    const bool use_crop = p.crops != nullptr;
    float4 crop = make_float4(0.f, 0.f, 0.f, 0.f);
    bool flip = false;
    if (use_crop) {
        const int clip = p.clip_len > 0 ? t / p.clip_len : 0;
        crop = p.crops[clip];
        flip = p.flips ? p.flips[clip] != 0 : false;
    }

    if (threadIdx.x < rows) {
        const int y = r0 + threadIdx.x;
        float sy;
        if (use_crop) {
            sy = crop.y + __fdiv_rn(static_cast<float>(y) + 0.5f, static_cast<float>(H)) * crop.w - 0.5f;
            sy = fminf(fmaxf(sy, 0.0f), static_cast<float>(p.src_h - 1));
        } else {
            sy = fmaxf(0.0f, __fdiv_rn((static_cast<float>(y) + 0.5f) * static_cast<float>(p.src_h),
                                       static_cast<float>(H)) - 0.5f);
        }
        const int y0 = static_cast<int>(sy);
        const int y1 = min(y0 + 1, p.src_h - 1);
        const float cyf = fminf(fmaxf(sy * 0.5f - 0.25f, 0.0f), static_cast<float>(ch - 1));
        const int cy0 = static_cast<int>(cyf);
        const int cy1 = min(cy0 + 1, ch - 1);
        RowTaps rt;
        rt.y0 = y0 * p.y_stride;
        rt.y1 = y1 * p.y_stride;
        rt.c0 = cy0 * p.c_stride;
        rt.c1 = cy1 * p.c_stride;
        rt.dy = sy - static_cast<float>(y0);
        rt.cdy = cyf - static_cast<float>(cy0);
        rt.idy = 1.0f - rt.dy;
        rt.icdy = 1.0f - rt.cdy;
        taps[threadIdx.x] = rt;
    }
    const unsigned char* __restrict__ yp = p.planes[t];
    const unsigned char* __restrict__ cbp = p.planes[p.n + t];
    const unsigned char* __restrict__ crp = p.planes[2 * p.n + t];
    __syncthreads();

    const float kY = 255.0f / 219.0f;
    const float kRV = p.bt709 ? 1.792741f : 1.596027f;
    const float kGU = p.bt709 ? 0.213249f : 0.391762f;
    const float kGV = p.bt709 ? 0.532909f : 0.812968f;
    const float kBU = p.bt709 ? 2.112402f : 2.017232f;
    const float nm0 = p.mean[0], nm1 = p.mean[1], nm2 = p.mean[2];
    const float is0 = p.inv_std[0], is1 = p.inv_std[1], is2 = p.inv_std[2];
    const long long plane = static_cast<long long>(H) * W;
    const long long frame_base = static_cast<long long>(t) * 3 * plane;

    for (int x = threadIdx.x; x < W; x += blockDim.x) {
        float sx;
        if (use_crop) {
            const int ox = flip ? (W - 1 - x) : x;
            sx = crop.x + __fdiv_rn(static_cast<float>(ox) + 0.5f, static_cast<float>(W)) * crop.z - 0.5f;
            sx = fminf(fmaxf(sx, 0.0f), static_cast<float>(p.src_w - 1));
        } else {
            sx = fmaxf(0.0f, __fdiv_rn((static_cast<float>(x) + 0.5f) * static_cast<float>(p.src_w),
                                       static_cast<float>(W)) - 0.5f);
        }
        const int x0 = static_cast<int>(sx);
        const int x1 = min(x0 + 1, p.src_w - 1);
        const float dx = sx - static_cast<float>(x0);
        const float idx_ = 1.0f - dx;
        const float ndx = -8388608.0f * dx, nidx = -8388608.0f * idx_;
        const float cxf = fminf(fmaxf(sx * 0.5f, 0.0f), static_cast<float>(cw - 1));
        const int cx0 = static_cast<int>(cxf);
        const int cx1 = min(cx0 + 1, cw - 1);
        const float cdx = cxf - static_cast<float>(cx0);
        const float icdx = 1.0f - cdx;
        const float ncdx = -8388608.0f * cdx, nicdx = -8388608.0f * icdx;
        const int i0 = cx0 * p.c_px_stride, i1 = cx1 * p.c_px_stride;
        long long o = frame_base + static_cast<long long>(r0) * W + x;

#pragma unroll 2
        for (int r = 0; r < rows; ++r, o += W) {
            const RowTaps rt = taps[r];
            const unsigned char* ya = yp + rt.y0;
            const unsigned char* yb = yp + rt.y1;
            const unsigned a0 = __ldg(ya + x0), a1 = __ldg(ya + x1), b0 = __ldg(yb + x0), b1 = __ldg(yb + x1);
            const unsigned char* ua = cbp + rt.c0;
            const unsigned char* ub = cbp + rt.c1;
            const unsigned char* va = crp + rt.c0;
            const unsigned char* vb = crp + rt.c1;
            const unsigned u00 = __ldg(ua + i0), u01 = __ldg(ua + i1), u10 = __ldg(ub + i0), u11 = __ldg(ub + i1);
            const unsigned v00 = __ldg(va + i0), v01 = __ldg(va + i1), v10 = __ldg(vb + i0), v11 = __ldg(vb + i1);

            const float ytop = byte_times(a0, idx_, nidx) + byte_times(a1, dx, ndx);
            const float ybot = byte_times(b0, idx_, nidx) + byte_times(b1, dx, ndx);
            const float yv0 = ytop * rt.idy + ybot * rt.dy;
            const float cbv = (byte_times(u00, icdx, nicdx) + byte_times(u01, cdx, ncdx)) * rt.icdy +
                              (byte_times(u10, icdx, nicdx) + byte_times(u11, cdx, ncdx)) * rt.cdy;
            const float crv = (byte_times(v00, icdx, nicdx) + byte_times(v01, cdx, ncdx)) * rt.icdy +
                              (byte_times(v10, icdx, nicdx) + byte_times(v11, cdx, ncdx)) * rt.cdy;

            const float yv = (yv0 - 16.0f) * kY;
            const float cb = cbv - 128.0f, cr = crv - 128.0f;
            const float R = yv + kRV * cr;
            const float G = yv - kGU * cb - kGV * cr;
            const float B = yv + kBU * cb;
            const float r01 = fminf(fmaxf(__fdiv_rn(R, 255.0f), 0.0f), 1.0f);
            const float g01 = fminf(fmaxf(__fdiv_rn(G, 255.0f), 0.0f), 1.0f);
            const float b01 = fminf(fmaxf(__fdiv_rn(B, 255.0f), 0.0f), 1.0f);
            put<DTYPE>(p.out, o, (r01 - nm0) * is0);
            put<DTYPE>(p.out, o + plane, (g01 - nm1) * is1);
            put<DTYPE>(p.out, o + 2 * plane, (b01 - nm2) * is2);
        }
    }
}

std::atomic<unsigned long long> g_video_launches{0};

}  // namespace

int launch_video(const VideoParams& p, int out_dtype, void* stream) {
    const int threads = std::min(256, ((p.dst_w + 31) / 32) * 32);
    const dim3 grid(static_cast<unsigned>((p.dst_h + kVideoRows - 1) / kVideoRows), static_cast<unsigned>(p.n));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (out_dtype == 0)
        yuv420_kernel<0><<<grid, threads, 0, st>>>(p);
    else
        yuv420_kernel<1><<<grid, threads, 0, st>>>(p);
    g_video_launches.fetch_add(1, std::memory_order_relaxed);
    return static_cast<int>(cudaGetLastError());
}

unsigned long long video_launch_count() { return g_video_launches.load(std::memory_order_relaxed); }

}  // namespace tlb
