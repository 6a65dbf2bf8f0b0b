// Internal (not part of the C ABI): parameter block and launch plan shared by the
// host-side C ABI implementation and the sm_100a kernels.
#pragma once
#include <cstdint>

namespace tlb {

constexpr int kMaxNewRows = 32;    // one planner lane issues the copy of one new source row
constexpr int kMaxStrips = 8;      // compute warps per CTA
constexpr int kMaxTileRows = 128;  // output rows per CTA (row tables are sized for this)

// Launch geometry chosen on the host from sizes only (never from device data).
struct Plan {
    int tile_rows;    // output rows per CTA
    int tile_cols;    // output columns per CTA (multiple of strip_cols)
    int n_col_tiles;  // ceil(dst_w / tile_cols)
    int n_row_tiles;  // ceil(dst_h / tile_rows)
    int strips;       // compute warps; CTA size = 32 * (strips + 1)
    int cpl;          // output columns owned by one lane: c and c + 32 of a 64-column strip (2), or one (1)
    int pitch;        // bytes per staged raw row at the widest crop (multiple of 16)
    int smem_bytes;   // dynamic shared memory per CTA
    int vec_ok;       // 1: every 16-byte output chunk is aligned and whole (identity-size kernel only)
    long long grid;   // CTAs
};

struct FusedParams {
    const uint8_t* src;
    unsigned long long src_bytes;
    long long n_src;
    const long long* src_offsets;
    const int* src_sizes;
    int src_w, src_h;
    int n;
    const long long* sel;
    const int* boxes;
    int ubox[4];
    const uint8_t* flips;
    int dst_h, dst_w;
    void* out;
    long long* out_indices;
    const long long* labels_in;
    long long* labels_out;
    float mean[3];
    float inv_std[3];  // 1.0f / std formed on the host in fp32 (direct_batch_loader.hpp:57)
    float pre_scale;   // 1/255 when normalize_01 else 1
    float one;         // 1.0f, deliberately a run-time value (see add2_exact in the kernel)
    float neg_k_pre;   // -2^23 * pre_scale (exact: a power-of-two scaling)
    const float* jitter;  // [n][3] per-sample (brightness, contrast, saturation) factors, or NULL
    int per_image_region; // 1: images are separate allocations -- no load may leave the image itself
    unsigned int* status;
    Plan plan;
};

// Shared-memory layout: a fixed header followed by kNBuf raw staging buffers of Rr source rows
// each (filled by bulk async copies; the planner runs that many passes ahead).  Rr is derived per
// CTA from its own footprint width.
#ifndef TLB_NBUF
#define TLB_NBUF 3
#endif
constexpr int kNBuf = TLB_NBUF;    // raw staging buffers = passes the planner may run ahead (<= 4)
constexpr int kSlots = kNBuf + 1;  // pass records kept (a record outlives its raw buffer by one pass)
constexpr int kSmemFull = 0;       // kNBuf x 8 B mbarriers: raw buffer b filled (transaction count)
constexpr int kSmemEmpty = 32;     // kNBuf x 8 B mbarriers: raw buffer b consumed by every compute warp
constexpr int kSmemMeta = 64;      // kSlots x int4 {new source rows, output rows emitted before the first of them, last pass?, -}
constexpr int kSmemSrcRec = 256;   // kSlots x 32 x int2 {byte offset of a new source row in shared memory, output rows emitted after it}
constexpr int kSmemRowW = kSmemSrcRec + kSlots * 32 * 8;   // kMaxTileRows x float4 {wA, wA, wB, wB}: vertical weights of the two row buffers
constexpr int kSmemRowY = kSmemRowW + kMaxTileRows * 16;   // kMaxTileRows x int: y0, the upper source row (crop-local)
constexpr int kSmemVar = (kSmemRowY + kMaxTileRows * 4 + 127) & ~127;  // start of the raw buffers
static_assert(kNBuf >= 2 && kNBuf <= 4, "header slots are sized for at most 4 buffers");

inline __host__ __device__ int raw_rows_for(int var_bytes, int own_pitch) {
    const int r = var_bytes / (kNBuf * own_pitch);
    return r > kMaxNewRows ? kMaxNewRows : r;
}

// Launch flags (per call).
constexpr unsigned kLaunchOverlap = 1u;  // programmatic stream serialization: may start while the previous kernel drains

// Implemented in fused_transform.cu.  Returns a cudaError_t as int.
int launch_fused(const FusedParams& p, int out_dtype, int out_layout, void* stream, unsigned flags);
// One-time per-device opt-in to large dynamic shared memory; returns a cudaError_t as int.
int prepare_device();
unsigned long long launch_count();

// Implemented in normalize_copy.cu: the identity-size case (crop size == output size, uniform
// dataset, no per-sample boxes).  Returns a cudaError_t as int.
int launch_normalize_copy(const FusedParams& p, int out_dtype, int out_layout, void* stream, unsigned flags);
unsigned long long normalize_copy_launch_count();

}  // namespace tlb
