// Internal (not part of the C ABI): parameter block and launch plan shared by the
// host-side C ABI implementation and the sm_100a kernels.
#pragma once
#include <cstdint>

namespace tlb {

constexpr int kStripCols = 32;     // output columns owned by one compute warp
constexpr int kStripRowBytes = 400; // one h row of a strip: 3 x 32 floats + 16 B of bank stagger
constexpr int kMaxNewRows = 32;    // one planner lane issues the copy of one new source row
constexpr int kMaxTileCols = 256;  // output columns per CTA (8 strips)

// Launch geometry chosen on the host from sizes only (never from device data).
struct Plan {
    int tile_rows;    // output rows per CTA
    int tile_cols;    // output columns per CTA (multiple of 32, <= kMaxTileCols)
    int n_col_tiles;  // ceil(dst_w / tile_cols)
    int n_row_tiles;  // ceil(dst_h / tile_rows)
    int strips;       // compute warps = tile_cols / 32; CTA size = 32 * (strips + 1)
    int pitch;        // bytes per staged raw row at the widest crop (multiple of 16)
    int smem_bytes;   // dynamic shared memory per CTA
    int vec_ok;       // 1: every 16-byte output chunk is aligned and whole -> vector stores
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
    unsigned int* status;
    Plan plan;
};

// Shared-memory layout.  A fixed header is followed by a region the CTA carves up itself
// from its own footprint width: kNBuf raw staging buffers of Rr source rows each (filled by
// bulk async copies, the planner runs that many passes ahead) and, per 32-column strip, a ring of Rh = Rr + 2 rows
// of horizontally-interpolated fp32 values (kStripRowBytes each).
constexpr int kMaxTileRows = 64;   // output rows per CTA (row tables are sized for this)
#ifndef TLB_NBUF
#define TLB_NBUF 3
#endif
constexpr int kNBuf = TLB_NBUF;    // raw staging buffers = passes the planner may run ahead (<= 4)
constexpr int kSlots = kNBuf + 1;  // pass records kept (a record outlives its raw buffer by one pass)
constexpr int kSmemFull = 0;       // kNBuf x 8 B mbarriers: raw buffer b filled (transaction count)
constexpr int kSmemEmpty = 32;     // kNBuf x 8 B mbarriers: raw buffer b consumed by every compute warp
constexpr int kSmemMeta = 64;      // kSlots x int4 {output rows, new source rows, last pass?, first output row}
constexpr int kSmemRowOff = 256;   // kSlots x 32 x int2 {raw byte offset, ring byte offset} per new source row of a pass
constexpr int kSmemRowp = 256 + 1280;          // kMaxTileRows x float4 {ring byte offset of y0 row, of y1 row, dy, 1-dy}
constexpr int kSmemRowY = 256 + 1280 + 1024;   // kMaxTileRows x int2 {y0, y1} crop-local source rows
constexpr int kSmemVar = 256 + 1280 + 1024 + 512;  // = 3072, start of the carved region (128-byte multiple)
static_assert(kNBuf >= 2 && kNBuf <= 4 && kSlots * 256 <= 1280, "header slots are sized for at most 4 buffers");

inline __host__ __device__ int raw_rows_for(int var_bytes, int own_pitch, int strips) {
    const int hrow = strips * kStripRowBytes;
    int r = (var_bytes - 2 * hrow) / (kNBuf * own_pitch + hrow);
    return r > kMaxNewRows ? kMaxNewRows : r;
}

// Implemented in fused_transform.cu.  Returns a cudaError_t as int.
int launch_fused(const FusedParams& p, int out_dtype, int out_layout, void* stream, bool may_overlap);
// One-time per-device opt-in to large dynamic shared memory; returns a cudaError_t as int.
int prepare_device();
unsigned long long launch_count();
int set_launch_overlap(int enable);  // returns the previous setting

// Implemented in normalize_copy.cu: the identity-size case (crop size == output size, uniform
// dataset, no per-sample boxes).  Uses p.plan.vec_ok only.  Returns a cudaError_t as int.
int launch_normalize_copy(const FusedParams& p, int out_dtype, int out_layout, void* stream);
unsigned long long normalize_copy_launch_count();

}  // namespace tlb
