// Antialiased (triangle filter) variant of the fused transform for sm_100a: crop -> separable
// triangle-filter resize whose support widens on downscale -> round half up to the 8-bit code ->
// flip -> normalize -> NCHW/NHWC fp32/bf16, one launch per batch.  It is the opt-in quality path
// of the reference (DirectBatchCore's `antialias` flag, src/pipeline/direct_batch_loader.hpp:229-231;
// filter: resize_triangle_antialias, src/transforms/simd_utils.hpp:1939-2014), which the reference
// itself implements in scalar code; results here are bit-identical to it:
//   * taps and weights per output index exactly as its `build` lambda (fp32 scale, support,
//     centre, floor/ceil bounds, w = max(0, 1 - |t|), sequential sum, division by the sum);
//   * horizontal pass first into fp32, vertical pass second, each a sequential fp32 sum of
//     separately rounded products, first tap first;
//   * code = (uint8)clamp(acc + 0.5f), then the same flip / normalize as the bilinear kernel.
//
// Work split: a CTA owns a tile of output rows x output columns of one sample; a thread owns one
// column of the RESIZED image for both passes, so the two passes need no synchronisation: the
// horizontal results of the source rows an output row taps sit in a shared-memory ring indexed by
// source row, written and read by the same thread.  Every source row of the tile's footprint is
// filtered horizontally once.  Column weights live in shared memory ([tap][column], conflict-free),
// row weights in a small per-tile table.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdint>

#include "antialias_params.h"
#include "fused_params.h"

namespace tlb {
namespace {

constexpr unsigned kBadIndex = 1u, kBadBox = 2u, kTooWide = 4u;

template <int DTYPE>
__device__ __forceinline__ void put(void* out, long long idx, float v) {
    if constexpr (DTYPE == 0)
        static_cast<float*>(out)[idx] = v;
    else
        static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
}

// simd_utils.hpp:1945-1975 for ONE output index: first tap, tap count, unnormalized weights
// written to w[k * stride], their sequential sum returned through `wsum`.
__device__ __forceinline__ void aa_taps(int i, int src_dim, float scale, float support, int max_taps, float* w,
                                        int stride, int& lo_out, int& n_out, float& wsum_out) {
    const float center = __fmul_rn(__fadd_rn(static_cast<float>(i), 0.5f), scale);
    int lo = static_cast<int>(floorf(__fsub_rn(center, support)));
    int hi = static_cast<int>(ceilf(__fadd_rn(center, support)));
    if (lo < 0) lo = 0;
    if (hi > src_dim) hi = src_dim;
    float wsum = 0.0f;
    int n = 0;
    for (int j = lo; j < hi && n < max_taps; ++j, ++n) {
        const float t = __fdiv_rn(__fsub_rn(__fadd_rn(static_cast<float>(j), 0.5f), center), support);
        float v = __fsub_rn(1.0f, fabsf(t));
        if (v < 0.0f) v = 0.0f;
        w[n * stride] = v;
        wsum = __fadd_rn(wsum, v);
    }
    lo_out = lo;
    n_out = n;
    wsum_out = wsum;
}

template <int DTYPE, int LAYOUT>
__global__ void __launch_bounds__(256) antialias_kernel(const __grid_constant__ FusedParams p,
                                                        const __grid_constant__ AAPlan a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x;
    const int TC = a.tile_cols, TR = a.tile_rows;
    float* const xw = reinterpret_cast<float*>(smem);                      // [xt][TC]
    float* const yw = xw + a.xt * TC;                                      // [TR][yt]
    int* const yl = reinterpret_cast<int*>(yw + TR * a.yt);                // [TR]
    int* const yc = yl + TR;                                               // [TR]
    float* const ring = reinterpret_cast<float*>(yc + TR);                 // [yt][3][TC]

    unsigned bid = blockIdx.x;
    const int ct = static_cast<int>(bid % static_cast<unsigned>(a.n_col_tiles));
    bid /= static_cast<unsigned>(a.n_col_tiles);
    const int rt = static_cast<int>(bid % static_cast<unsigned>(a.n_row_tiles));
    const int k = static_cast<int>(bid / static_cast<unsigned>(a.n_row_tiles));
    const int W = p.dst_w, H = p.dst_h;
    const int ty0 = rt * TR, ty1 = min(ty0 + TR, H);
    const int tx0 = ct * TC, tcw = min(TC, W - tx0);

    // ---- per-sample parameters (same rules as the bilinear kernel) ---------------------------
    const long long s = p.sel ? p.sel[k] : static_cast<long long>(k);
    unsigned bad = 0;
    if (s < 0 || s >= p.n_src) bad = kBadIndex;
    int iw = p.src_w, ih = p.src_h;
    long long img_off = 0;
    int cx = 0, cy = 0, cw = 0, ch = 0;
    if (!bad) {
        if (p.src_sizes) {
            iw = p.src_sizes[2 * s];
            ih = p.src_sizes[2 * s + 1];
        }
        img_off = p.src_offsets ? p.src_offsets[s] : s * (static_cast<long long>(iw) * ih * 3);
        if (p.boxes) {
            const int4 b = *reinterpret_cast<const int4*>(p.boxes + 4 * static_cast<long long>(k));
            cx = b.x; cy = b.y; cw = b.z; ch = b.w;
        } else if (p.ubox[2] > 0) {
            cx = p.ubox[0]; cy = p.ubox[1]; cw = p.ubox[2]; ch = p.ubox[3];
        } else {
            cw = iw; ch = ih;
        }
        const long long img_bytes = static_cast<long long>(iw) * ih * 3;
        if (iw <= 0 || ih <= 0 || cw <= 0 || ch <= 0 || cx < 0 || cy < 0 || cx > iw - cw || cy > ih - ch ||
            img_off < 0 || img_bytes > 0x7fffffffll ||
            static_cast<unsigned long long>(img_off) + img_bytes > p.src_bytes)
            bad = kBadBox;
    }
    const bool flip = p.flips ? (p.flips[k] != 0) : false;
    if (rt == 0 && ct == 0 && tid == 0) {
        if (p.out_indices) p.out_indices[k] = s;
        if (p.labels_out) p.labels_out[k] = (bad & kBadIndex) || !p.labels_in ? -1 : p.labels_in[s];
    }
    // simd_utils.hpp:1947-1951
    const float xscale = __fdiv_rn(static_cast<float>(cw), static_cast<float>(W > 0 ? W : 1));
    const float yscale = __fdiv_rn(static_cast<float>(ch), static_cast<float>(H > 0 ? H : 1));
    const float xsup = xscale > 1.0f ? xscale : 1.0f, ysup = yscale > 1.0f ? yscale : 1.0f;
    const int xmax = static_cast<int>(ceilf(__fmul_rn(xsup, 2.0f))) + 2;
    const int ymax = static_cast<int>(ceilf(__fmul_rn(ysup, 2.0f))) + 2;
    if (!bad && (xmax > a.xt || ymax > a.yt)) bad = kTooWide;  // the crop exceeds the bound the tables were sized for

    if (bad) {
        if (tid == 0 && p.status) atomicOr(p.status, bad);
        const int rows = ty1 - ty0;
        for (int i = tid; i < rows * tcw * 3; i += blockDim.x) {
            const int c = i % 3, x = (i / 3) % tcw, y = i / (3 * tcw);
            long long idx;
            if constexpr (LAYOUT == 0)
                idx = ((static_cast<long long>(k) * 3 + c) * H + (ty0 + y)) * W + tx0 + x;
            else
                idx = ((static_cast<long long>(k) * H + (ty0 + y)) * W + tx0 + x) * 3 + c;
            put<DTYPE>(p.out, idx, 0.0f);
        }
        return;
    }

    // ---- taps: one thread per column, one thread per tile row ---------------------------------
    int xlo = 0, xn = 0;
    const bool active = tid < tcw;
    if (active) {
        float wsum;
        aa_taps(tx0 + tid, cw, xscale, xsup, xmax, xw + tid, TC, xlo, xn, wsum);
        if (wsum > 0.0f)
            for (int q = 0; q < xn; ++q) xw[q * TC + tid] = __fdiv_rn(xw[q * TC + tid], wsum);
    }
    if (tid < ty1 - ty0) {
        float wsum;
        int lo, n;
        aa_taps(ty0 + tid, ch, yscale, ysup, ymax, yw + tid * a.yt, 1, lo, n, wsum);
        if (wsum > 0.0f)
            for (int q = 0; q < n; ++q) yw[tid * a.yt + q] = __fdiv_rn(yw[tid * a.yt + q], wsum);
        yl[tid] = lo;
        yc[tid] = n;
    }
    __syncthreads();
    if (!active) return;

    const unsigned char* const img = p.src + img_off;
    const unsigned char* const col = img + (static_cast<long long>(cy) * iw + cx + xlo) * 3;  // first tap, crop row 0
    const long long row_pitch = static_cast<long long>(iw) * 3;
    const int xr = tx0 + tid;                           // column of the RESIZED image
    const int xo = flip ? (W - 1 - xr) : xr;            // where it lands after the flip
    float* const myring = ring + tid;                   // [slot][c][TC] -> slot * 3 * TC + c * TC
    const int RR = a.yt;
    const float pre = p.pre_scale;
    const float m0 = p.mean[0], m1 = p.mean[1], m2 = p.mean[2];
    const float i0 = p.inv_std[0], i1 = p.inv_std[1], i2 = p.inv_std[2];

    // Ring slots advance with the source rows (slot = source row modulo RR, kept incrementally:
    // an integer modulo per tap was a third of the instructions of the first version).
    int next_src = yl[0];      // next source row to filter horizontally
    int next_slot = 0;         // ring slot of next_src
    int lo_prev = yl[0], lo_slot = 0;  // first tap row of the previous output row and its slot
    for (int r = 0; r < ty1 - ty0; ++r) {
        const int lo = yl[r], n = yc[r];
        lo_slot += lo - lo_prev;  // lo never decreases
        lo_prev = lo;
        while (lo_slot >= RR) lo_slot -= RR;
        // ---- horizontal pass for the source rows this output row adds ---------------------
        if (next_src < lo) {  // rows no output row of this tile taps
            next_slot += lo - next_src;
            next_src = lo;
            while (next_slot >= RR) next_slot -= RR;
        }
        for (; next_src < lo + n; ++next_src) {
            const unsigned char* sp = col + next_src * row_pitch;
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f;
            // w * (float)byte without an integer conversion: fma(2^23 + b, w, -2^23 * w) is exactly
            // RN(b * w), the product the reference forms.  Four taps per trip keep 12 loads in flight.
            for (int q0 = 0; q0 < xn; q0 += 4) {
                unsigned b[4][3];
                float w[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const bool on = q0 + u < xn;
                    w[u] = on ? xw[(q0 + u) * TC + tid] : 0.0f;
#pragma unroll
                    for (int c = 0; c < 3; ++c) b[u][c] = on ? static_cast<unsigned>(__ldg(sp + 3 * (q0 + u) + c)) : 0u;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (q0 + u < xn) {
                        const float nw = __fmul_rn(-8388608.0f, w[u]);
                        a0 = __fadd_rn(a0, __fmaf_rn(__uint_as_float(b[u][0] | 0x4B000000u), w[u], nw));
                        a1 = __fadd_rn(a1, __fmaf_rn(__uint_as_float(b[u][1] | 0x4B000000u), w[u], nw));
                        a2 = __fadd_rn(a2, __fmaf_rn(__uint_as_float(b[u][2] | 0x4B000000u), w[u], nw));
                    }
                }
            }
            float* slot = myring + next_slot * 3 * TC;
            slot[0] = a0;
            slot[TC] = a1;
            slot[2 * TC] = a2;
            if (++next_slot == RR) next_slot = 0;
        }
        // ---- vertical pass, rounding, normalize, store --------------------------------------
        float v0 = 0.0f, v1 = 0.0f, v2 = 0.0f;
        const float* wr = yw + r * a.yt;
        int vs = lo_slot;
        for (int q = 0; q < n; ++q) {
            const float w = wr[q];
            const float* slot = myring + vs * 3 * TC;
            if (++vs == RR) vs = 0;
            v0 = __fadd_rn(v0, __fmul_rn(w, slot[0]));
            v1 = __fadd_rn(v1, __fmul_rn(w, slot[TC]));
            v2 = __fadd_rn(v2, __fmul_rn(w, slot[2 * TC]));
        }
        // (uint8)max(0, min(255, acc + 0.5f))   simd_utils.hpp:2008-2009
        const float c0 = static_cast<float>(static_cast<int>(fmaxf(0.0f, fminf(255.0f, __fadd_rn(v0, 0.5f)))));
        const float c1 = static_cast<float>(static_cast<int>(fmaxf(0.0f, fminf(255.0f, __fadd_rn(v1, 0.5f)))));
        const float c2 = static_cast<float>(static_cast<int>(fmaxf(0.0f, fminf(255.0f, __fadd_rn(v2, 0.5f)))));
        const float o0 = __fmul_rn(__fsub_rn(__fmul_rn(c0, pre), m0), i0);
        const float o1 = __fmul_rn(__fsub_rn(__fmul_rn(c1, pre), m1), i1);
        const float o2 = __fmul_rn(__fsub_rn(__fmul_rn(c2, pre), m2), i2);
        const int y = ty0 + r;
        if constexpr (LAYOUT == 0) {
            const long long base = (static_cast<long long>(k) * 3 * H + y) * W + xo;
            const long long plane = static_cast<long long>(H) * W;
            put<DTYPE>(p.out, base, o0);
            put<DTYPE>(p.out, base + plane, o1);
            put<DTYPE>(p.out, base + 2 * plane, o2);
        } else {
            const long long base = ((static_cast<long long>(k) * H + y) * W + xo) * 3;
            put<DTYPE>(p.out, base, o0);
            put<DTYPE>(p.out, base + 1, o1);
            put<DTYPE>(p.out, base + 2, o2);
        }
    }
}

std::atomic<unsigned long long> g_aa_launches{0};

template <int DTYPE, int LAYOUT>
int launch_one(const FusedParams& p, const AAPlan& a, cudaStream_t st) {
    antialias_kernel<DTYPE, LAYOUT><<<static_cast<unsigned>(a.grid), a.tile_cols, a.smem_bytes, st>>>(p, a);
    g_aa_launches.fetch_add(1, std::memory_order_relaxed);
    return static_cast<int>(cudaGetLastError());
}

template <int DTYPE, int LAYOUT>
int opt_in() {
    return static_cast<int>(cudaFuncSetAttribute(antialias_kernel<DTYPE, LAYOUT>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, kAAMaxSmem));
}

}  // namespace

int aa_max_taps(int src_dim, int dst_dim) {
    const float scale = static_cast<float>(src_dim) / static_cast<float>(dst_dim > 0 ? dst_dim : 1);
    const float support = scale > 1.0f ? scale : 1.0f;
    return static_cast<int>(ceilf(support * 2.0f)) + 2;
}

int prepare_antialias() {
    int e = opt_in<0, 0>();
    if (!e) e = opt_in<0, 1>();
    if (!e) e = opt_in<1, 0>();
    if (!e) e = opt_in<1, 1>();
    return e;
}

int launch_antialias(const FusedParams& p, const AAPlan& a, int out_dtype, int out_layout, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (out_dtype == 0) return out_layout == 0 ? launch_one<0, 0>(p, a, st) : launch_one<0, 1>(p, a, st);
    return out_layout == 0 ? launch_one<1, 0>(p, a, st) : launch_one<1, 1>(p, a, st);
}

unsigned long long antialias_launch_count() { return g_aa_launches.load(std::memory_order_relaxed); }

}  // namespace tlb
