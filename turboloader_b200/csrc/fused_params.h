// Internal (not part of the C ABI): parameter block and launch plan shared by the
// host-side C ABI implementation and the sm_100a kernels.
#pragma once
#include <cstdint>

namespace tlb {

constexpr int kThreads = 256;      // threads per CTA
constexpr int kMaxStagedRows = 32; // one lane of warp 0 issues the copy of one staged row
constexpr int kMaxTileCols = 256;  // output columns per CTA (== kThreads: one column per thread)

// Launch geometry chosen on the host from sizes only (never from device data).
struct Plan {
    int tile_rows;    // output rows per CTA
    int tile_cols;    // output columns per CTA (multiple of 16, <= kMaxTileCols)
    int n_col_tiles;  // ceil(dst_w / tile_cols)
    int n_row_tiles;  // ceil(dst_h / tile_rows)
    int staged_rows;  // source rows staged in shared memory per pass (R), <= kMaxStagedRows
    int pitch;        // bytes per staged raw row (multiple of 16)
    int hpitch;       // floats per row of horizontally-interpolated values (3 * tile_cols)
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
    unsigned int* status;
    Plan plan;
};

// Shared-memory layout (byte offsets from the dynamic shared base), derived from the plan.
struct SmemLayout {
    int mbar;   // 16 B
    int colp;   // tile_cols * 16 B   per-column {off0, off1, dx, 1-dx}
    int rowp;   // 32 * 16 B          per-row    {slot0, slot1, dy, 1-dy}
    int rowsh;  // 32 * 4 B           byte phase of each staged row inside its slot
    int ctab;   // 48 * 4 B           NHWC normalize constants by channel phase
    int raw;    // staged_rows * pitch
    int hbuf;   // staged_rows * hpitch * 4
    int total;
};

inline __host__ __device__ SmemLayout smem_layout(int tile_cols, int staged_rows, int pitch, int hpitch) {
    SmemLayout L;
    L.mbar = 0;
    L.colp = 16;
    L.rowp = L.colp + tile_cols * 16;
    L.rowsh = L.rowp + 32 * 16;
    L.ctab = L.rowsh + 32 * 4;
    L.raw = L.ctab + 48 * 4;
    L.hbuf = L.raw + staged_rows * pitch;
    L.total = L.hbuf + staged_rows * hpitch * 4;
    return L;
}

// Implemented in fused_transform.cu.  Returns a cudaError_t as int.
int launch_fused(const FusedParams& p, int out_dtype, int out_layout, void* stream);
// One-time per-device opt-in to large dynamic shared memory; returns a cudaError_t as int.
int prepare_device();
unsigned long long launch_count();

}  // namespace tlb
