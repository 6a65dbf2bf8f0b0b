// Gather of crop rectangles from page-locked HOST memory into a packed device buffer, done by
// the GPU itself: when the caller's images live in pinned (device-mapped) host memory, the
// kernel below reads exactly the crop rows across PCIe with aligned 16-byte loads and writes
// them, row by row, into device memory with 16-byte-aligned row starts.  This replaces the
// host-side packing loop + one large H2D copy of the streaming entry point (TurboLoader's
// CudaStreamCore uploads whole pre-resized batches with cudaMemcpyAsync,
// src/cuda/cuda_transforms.cu:629-780; a crop gather has no counterpart there) and leaves the
// host with nothing to do per batch but fill a small table.  One cudaMemcpyAsync per crop row
// would be far too many calls, and no batched-copy API is used; a kernel is the gather.
#include <cuda_runtime.h>

#include <cstdint>

#include "host_gather.h"

namespace tlb {
namespace {

constexpr int kGatherThreads = 128;
constexpr int kRowsPerBlock = 16;

__device__ __forceinline__ uint4 ld16(const unsigned char* p) {
    return *reinterpret_cast<const uint4*>(p);
}

// out = bytes [s, s+16) of the 32-byte window (x ‖ y), 0 <= s < 16.
__device__ __forceinline__ uint4 window16(uint4 x, uint4 y, unsigned s) {
    const unsigned sh = (s & 3u) * 8u;
    uint32_t w0, w1, w2, w3, w4;
    switch (s >> 2) {  // uniform across the warp: s is a property of the row
        case 0: w0 = x.x; w1 = x.y; w2 = x.z; w3 = x.w; w4 = y.x; break;
        case 1: w0 = x.y; w1 = x.z; w2 = x.w; w3 = y.x; w4 = y.y; break;
        case 2: w0 = x.z; w1 = x.w; w2 = y.x; w3 = y.y; w4 = y.z; break;
        default: w0 = x.w; w1 = y.x; w2 = y.y; w3 = y.z; w4 = y.w; break;
    }
    return make_uint4(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh), __funnelshift_r(w2, w3, sh),
                      __funnelshift_r(w3, w4, sh));
}

__global__ void __launch_bounds__(kGatherThreads) gather_crops_kernel(const GatherItem* items, unsigned char* dst) {
    const GatherItem it = items[blockIdx.x];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned nchunks = it.dst_pitch >> 4;  // 16-byte chunks per packed row
    const unsigned row_end = min(it.rows, (blockIdx.y + 1) * kRowsPerBlock);
    for (unsigned r = blockIdx.y * kRowsPerBlock + warp; r < row_end; r += kGatherThreads / 32) {
        const unsigned char* src = reinterpret_cast<const unsigned char*>(it.src) + static_cast<size_t>(r) * it.src_pitch;
        const unsigned s = static_cast<unsigned>(reinterpret_cast<uintptr_t>(src) & 15u);
        const unsigned char* base = src - s;  // aligned start; the bytes before src share its 16-byte granule
        // Aligned chunks that hold at least one byte of the row: [0, last].
        const unsigned last = (s + it.row_bytes - 1) >> 4;
        unsigned char* out = dst + it.dst_off + static_cast<size_t>(r) * it.dst_pitch;
        for (unsigned c0 = 0; c0 < nchunks; c0 += 32) {
            const unsigned c = c0 + lane;
            // Each lane loads source chunk c once; chunk c+1 comes from the next lane (the last
            // lane of the group loads its own).  Chunks past the row's last granule are not read.
            uint4 x = make_uint4(0, 0, 0, 0), y = make_uint4(0, 0, 0, 0);
            if (c <= last) x = ld16(base + 16u * c);
            y.x = __shfl_down_sync(0xffffffffu, x.x, 1);
            y.y = __shfl_down_sync(0xffffffffu, x.y, 1);
            y.z = __shfl_down_sync(0xffffffffu, x.z, 1);
            y.w = __shfl_down_sync(0xffffffffu, x.w, 1);
            if (lane == 31) y = (c + 1 <= last) ? ld16(base + 16u * (c + 1)) : make_uint4(0, 0, 0, 0);
            if (c < nchunks) *reinterpret_cast<uint4*>(out + 16u * c) = window16(x, y, s);
        }
    }
}

}  // namespace

int launch_gather(const GatherItem* items_dev, int n, unsigned max_rows, unsigned char* dst, void* stream) {
    if (n <= 0) return 0;
    dim3 grid(static_cast<unsigned>(n), (max_rows + kRowsPerBlock - 1) / kRowsPerBlock);
    gather_crops_kernel<<<grid, kGatherThreads, 0, static_cast<cudaStream_t>(stream)>>>(items_dev, dst);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace tlb
