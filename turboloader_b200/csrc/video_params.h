// Launch parameters of the fused YUV 4:2:0 video kernel (video_yuv420.cu), shared with the
// host C ABI (capi.cu).
#pragma once
#include <cuda_runtime.h>

namespace tlb {

// A batch of at most kVideoInlineFrames frames in at most kVideoInlineClips clips carries its
// address and crop tables inside the kernel's parameter block: no table upload precedes the
// launch, so consecutive launches are kernel-after-kernel in their stream (and may overlap head to
// tail when the caller allows it).  Larger batches upload the tables to device memory as before.
constexpr int kVideoInlineFrames = 256;
constexpr int kVideoInlineClips = 32;
struct VideoTables {
    const unsigned char* planes[3 * kVideoInlineFrames];  // [0,n) Y, [n,2n) Cb, [2n,3n) Cr
    float4 crops[kVideoInlineClips];
    int flips[kVideoInlineClips];
};

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
    float one;                           // 1.0f, passed at run time (see add_prod in video_yuv420.cu)
    void* out;                           // (n, 3, dst_h, dst_w)
    unsigned* status;                    // optional device word, OR-ed with 8 if a staging copy never completed
    int stage_rows;                      // set by launch_video: output rows per CTA of the staged kernel
    int direct_rows;                     // set by launch_video: output rows per CTA of the direct kernel (even, <= 32)
    int use_staged;                      // non-zero: use the shared-memory staged kernel when the frame fits
    int inline_tables;                   // non-zero: planes / crops / flips are read from `in` (direct kernel only)
    int has_crops, has_flips;            // with inline tables: which of them are given
    VideoTables in;
};

constexpr int kVideoStageMaxBytes = 200 * 1024;  // most dynamic shared memory the staged kernel may ask for

int prepare_video();                                           // once per device: shared-memory opt-in
// flags: kLaunchOverlap of fused_params.h or 0; returns a cudaError_t value
int launch_video(const VideoParams& p, int out_dtype, void* stream, unsigned flags);
unsigned long long video_launch_count();

}  // namespace tlb
