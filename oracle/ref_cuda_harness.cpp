// TEST / BENCHMARK INFRASTRUCTURE ONLY -- C wrappers around the UNMODIFIED reference GPU entry
// points (turboloader::cuda::*, src/cuda/cuda_transforms.hpp), so that the reference's own CUDA
// kernels, compiled for this GPU from the reference tree (oracle/Makefile target `refcuda`), can
// be run beside the sm_100a kernel: (a) as a second statement of the normalize/gather math and
// (b) as the "reference GPU kernels on the same box" timing.  Nothing in the package links this.
#include <cstdint>
#include <vector>

#include "src/cuda/cuda_transforms.hpp"

#define API extern "C" __attribute__((visibility("default")))

API int tlrefcuda_available() { return turboloader::cuda::available() ? 1 : 0; }

// normalize_resident_batch / normalize_resident_gather_batch (cuda_transforms.hpp:49-55):
// returns the device address of the library-owned (N,3,H,W) float32 result, 0 on error.
API uintptr_t tlrefcuda_normalize_resident(uintptr_t src_dev, int n, int h, int w, const float* mean,
                                           const float* std_) {
    return turboloader::cuda::normalize_resident_batch(src_dev, n, h, w, mean, std_);
}
API uintptr_t tlrefcuda_normalize_resident_gather(uintptr_t src_dev, uintptr_t sel_dev, int n, int h, int w,
                                                  const float* mean, const float* std_) {
    return turboloader::cuda::normalize_resident_gather_batch(src_dev, sel_dev, n, h, w, mean, std_);
}

// resize_normalize_batch / crop_resize_normalize_batch (cuda_transforms.hpp:41-42, 117-119): host
// images in, host float32 NCHW out (allocates, uploads, launches one kernel per image, downloads).
API int tlrefcuda_resize_normalize(const uint8_t* const* data, const int* ws, const int* hs, int n, int dst_h,
                                   int dst_w, const float* mean, const float* std_, float* out) {
    std::vector<turboloader::cuda::ImageRef> imgs(n);
    for (int i = 0; i < n; ++i) imgs[i] = {data[i], ws[i], hs[i]};
    return turboloader::cuda::resize_normalize_batch(imgs, dst_h, dst_w, mean, std_, out) ? 1 : 0;
}
API int tlrefcuda_crop_resize_normalize(const uint8_t* const* data, const int* ws, const int* hs,
                                        const float* crops_xywh, const int* flips, int n, int dst_h, int dst_w,
                                        const float* mean, const float* std_, float* out) {
    std::vector<turboloader::cuda::ImageRef> imgs(n);
    std::vector<turboloader::cuda::CropParams> cps(n);
    for (int i = 0; i < n; ++i) {
        imgs[i] = {data[i], ws[i], hs[i]};
        cps[i] = {crops_xywh[4 * i], crops_xywh[4 * i + 1], crops_xywh[4 * i + 2], crops_xywh[4 * i + 3], flips[i]};
    }
    return turboloader::cuda::crop_resize_normalize_batch(imgs, cps, dst_h, dst_w, mean, std_, out) ? 1 : 0;
}

// video_yuv420_batch / video_clip_yuv420 (cuda_transforms.hpp:65-81): n frames given as device
// plane addresses; returns the device address of the library-owned (n,3,dst_h,dst_w) float32
// result (valid until the next call), 0 on error.
API uintptr_t tlrefcuda_video_yuv420_batch(const uintptr_t* y, const uintptr_t* cb, const uintptr_t* cr, int n,
                                           int y_stride, int c_stride, int c_px_stride, int src_w, int src_h,
                                           int dst_h, int dst_w, int bt709, const float* mean, const float* std_) {
    std::vector<uintptr_t> vy(y, y + n), vcb(cb, cb + n), vcr(cr, cr + n);
    return turboloader::cuda::video_yuv420_batch(vy, vcb, vcr, y_stride, c_stride, c_px_stride, src_w, src_h, dst_h,
                                                 dst_w, bt709 != 0, mean, std_);
}
API uintptr_t tlrefcuda_video_clip_yuv420(const uintptr_t* y, const uintptr_t* cb, const uintptr_t* cr, int n,
                                          int y_stride, int c_stride, int c_px_stride, int src_w, int src_h,
                                          int dst_h, int dst_w, const float* crop, int flip, int bt709,
                                          const float* mean, const float* std_) {
    std::vector<uintptr_t> vy(y, y + n), vcb(cb, cb + n), vcr(cr, cr + n);
    return turboloader::cuda::video_clip_yuv420(vy, vcb, vcr, y_stride, c_stride, c_px_stride, src_w, src_h, dst_h,
                                                dst_w, crop, flip != 0, bt709 != 0, mean, std_);
}

// CudaStreamCore (cuda_transforms.hpp:100-112): dataset in pinned host memory streamed by K worker
// threads.  next returns the device address of the next ready (n,3,h,w) float32 batch, 0 at the end.
API void* tlrefcuda_stream_create(uintptr_t host_ptr, int n, int h, int w, int batch, const float* mean,
                                  const float* std_, int num_slots, int drop_last) {
    return new turboloader::cuda::CudaStreamCore(host_ptr, n, h, w, batch, mean, std_, num_slots, drop_last != 0);
}
API void tlrefcuda_stream_destroy(void* core) { delete static_cast<turboloader::cuda::CudaStreamCore*>(core); }
API int tlrefcuda_stream_num_batches(void* core) {
    return static_cast<turboloader::cuda::CudaStreamCore*>(core)->num_batches();
}
API void tlrefcuda_stream_begin_epoch(void* core) { static_cast<turboloader::cuda::CudaStreamCore*>(core)->begin_epoch(); }
API uintptr_t tlrefcuda_stream_next(void* core, int* out_n) {
    return static_cast<turboloader::cuda::CudaStreamCore*>(core)->next_batch(out_n);
}
