// Launch plan of the antialiased variant of the fused transform (antialias.cu), shared with the
// host C ABI (capi.cu).
#pragma once

namespace tlb {

struct FusedParams;

struct AAPlan {
    int xt, yt;        // most taps per output column / row any sample of the batch can have
    int tile_rows;     // output rows per CTA
    int tile_cols;     // output columns per CTA (multiple of 32, <= 256); one thread per column, or per two (pair)
    int n_row_tiles, n_col_tiles;
    int smem_bytes;
    int pair;          // 1: the packed two-columns-per-thread kernel (tile_cols / 2 threads per CTA)
    long long grid;
};

constexpr int kAAMaxSmem = 200 * 1024;

// Taps bound for a scale factor, with the reference's own expression
// (src/transforms/simd_utils.hpp:1947-1951): ceil(max(scale, 1) * 2) + 2.
int aa_max_taps(int src_dim, int dst_dim);
int prepare_antialias();  // once per device: shared-memory opt-in; returns a cudaError_t value
// flags: kLaunchOverlap of fused_params.h or 0
int launch_antialias(const FusedParams& p, const AAPlan& a, int out_dtype, int out_layout, void* stream, unsigned flags);
unsigned long long antialias_launch_count();

}  // namespace tlb
