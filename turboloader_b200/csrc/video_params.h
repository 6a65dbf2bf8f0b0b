// Launch parameters of the fused YUV 4:2:0 video kernel (video_yuv420.cu), shared with the
// host C ABI (capi.cu).
#pragma once
#include <cuda_runtime.h>

namespace tlb {

struct VideoParams {
    const unsigned char* const* planes;  // DEVICE array of 3n plane addresses: [0,n) Y, [n,2n) Cb, [2n,3n) Cr
    const float4* crops;                 // DEVICE array, one window (x, y, w, h in source pixels) per clip;
                                         // nullptr selects whole-frame sampling
    const int* flips;                    // DEVICE array, one flag per clip (nullptr: no flip)
    int n;                               // frames
    int clip_len;                        // consecutive frames sharing one crops/flips entry (0: all n frames)
    int y_stride, c_stride, c_px_stride; // bytes; c_px_stride 1 = I420 planes, 2 = NV12 interleaved
    int src_w, src_h, dst_w, dst_h, bt709;
    float mean[3], inv_std[3];
    void* out;                           // (n, 3, dst_h, dst_w)
};

int launch_video(const VideoParams& p, int out_dtype, void* stream);  // returns a cudaError_t value
unsigned long long video_launch_count();

}  // namespace tlb
