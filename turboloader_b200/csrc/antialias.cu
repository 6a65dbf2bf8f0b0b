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

// ---- packed form: two columns per thread ---------------------------------------------------------
// Same filter, same order of operations, organised like the bilinear kernel: a thread owns output
// columns t and t + TC/2 of the tile and carries them as the two halves of packed fp32 values, so
// every multiply and add of the filter is issued once per column PAIR.  Per horizontal tap and
// pair: six byte loads, six ORs (2^23 + byte), three packed FMAs for the products
// fma(2^23 + b, w, -2^23 w) == RN(b w) and three for the running sums (fma(prod, 1, acc), the exact
// packed add); the weights of the pair sit in shared memory as {wA, wB, -2^23 wA, -2^23 wB}.
// The tap loop has the SAMPLE's tap bound as its trip count for every column; a column with fewer
// taps gets zero weights in front or behind (adding +0 changes no bit), and its tap window is shifted
// left where it would leave the crop, so no load ever leaves the crop row.
__device__ __forceinline__ float2 aa_fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "mov.b64 rc, {%6, %7};\n\tfma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ float2 aa_mul2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "mul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float2 aa_add2_rz(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "add.rz.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}

struct PairCtx {
    void* out;
    const unsigned char* img;      // the sample's image
    unsigned row_pitch;            // bytes per image row
    unsigned offA, offB;           // byte offset (from img) of the first pixel of each column's tap window, crop row 0
    const float4* xw;              // this thread's weights: xw[q * xw_stride] = {wA, wB, -2^23 wA, -2^23 wB}
    int xw_stride;
    const float* yw;               // [rows][yt]
    const int* yl;
    const int* yc;
    int yt, rows;
    int slot_bytes;                // bytes between ring slots
    unsigned char* myring;         // this thread's 24 bytes of slot 0
    unsigned char* ring_end;       // ... of the slot past the last
    int nt;                        // horizontal taps of this sample
    float one, pre, nkpre;
    float nmean[3], inv_std[3];
    bool validB;
    long long oA, oB;              // element index of channel 0 of each column at tile row 0
    long long row_step, chan_step; // elements to the next output row / channel
};

// The words of one source row's tap window for one column: NW aligned 32-bit words starting at the
// word that holds the window's first byte, and the bit shift that realigns them.
template <int NW>
struct RowWords {
    unsigned w[NW];
    unsigned sh;
};

template <int NT, int NW>
__device__ __forceinline__ void load_window(const unsigned char* imga, unsigned g, RowWords<NW>& r) {
    // g = byte offset of the window from the 4-aligned `imga`.  Words 0..NW-2 always hold window bytes;
    // the last one may lie wholly behind the window (it then feeds only shifted-out bits), so its
    // address is clamped to the last word that does.
    const unsigned first = g & ~3u;
    const unsigned last = (g + 3u * NT - 1u) & ~3u;
    const unsigned* wp = reinterpret_cast<const unsigned*>(imga + first);
#pragma unroll
    for (int i = 0; i < NW - 1; ++i) r.w[i] = __ldg(wp + i);
    r.w[NW - 1] = __ldg(reinterpret_cast<const unsigned*>(imga + min(first + 4u * (NW - 1), last)));
    r.sh = (g & 3u) * 8u;
}

// Rows of one tile for a thread's column pair.  NT > 0: the sample has exactly NT horizontal taps;
// the tap loop is unrolled, the window is fetched as aligned words (bytes picked by PRMT straight
// into 2^23 + b) and the NEXT source row's words are requested before the current row is filtered,
// so their latency hides behind a row of arithmetic.  NT == 0: any tap count, byte loads.
template <int DTYPE, int NT>
__device__ __forceinline__ void pair_rows(const PairCtx& c) {
    constexpr int NS = (3 * NT + 3) / 4;   // words of window bytes
    constexpr int NW = NS + 1;             // ... plus the one the realignment may need
    const float2 one2 = make_float2(c.one, c.one);
    const float2 k2 = make_float2(8388608.0f, 8388608.0f);
    const float2 pre2 = make_float2(c.pre, c.pre), nkpre2 = make_float2(c.nkpre, c.nkpre);
    const int RR_bytes = static_cast<int>(c.ring_end - c.myring);
    const unsigned lowbits = static_cast<unsigned>(reinterpret_cast<unsigned long long>(c.img) & 3ull);
    const unsigned char* const imga = c.img - lowbits;
    const int last_src = c.yl[c.rows - 1] + c.yc[c.rows - 1];  // one past the last source row the tile taps

    int next_src = c.yl[0];               // next source row to filter horizontally
    unsigned char* next_slot = c.myring;  // its ring slot
    int lo_prev = c.yl[0];
    unsigned char* lo_slot = c.myring;    // slot of the first tap row of the current output row
    long long oA = c.oA, oB = c.oB;
    RowWords<NW> nxtA, nxtB;
    if constexpr (NT > 0) {
        load_window<NT, NW>(imga, lowbits + c.offA + static_cast<unsigned>(next_src) * c.row_pitch, nxtA);
        load_window<NT, NW>(imga, lowbits + c.offB + static_cast<unsigned>(next_src) * c.row_pitch, nxtB);
    }
    for (int r = 0; r < c.rows; ++r, oA += c.row_step, oB += c.row_step) {
        const int lo = c.yl[r], n = c.yc[r];
        lo_slot += (lo - lo_prev) * c.slot_bytes;  // lo never decreases, by less than a ring per step
        lo_prev = lo;
        if (lo_slot >= c.ring_end) lo_slot -= RR_bytes;
        if (next_src < lo) {  // rows no output row of this tile taps
            next_slot += (lo - next_src) * c.slot_bytes;
            next_src = lo;
            while (next_slot >= c.ring_end) next_slot -= RR_bytes;
            if constexpr (NT > 0) {
                load_window<NT, NW>(imga, lowbits + c.offA + static_cast<unsigned>(next_src) * c.row_pitch, nxtA);
                load_window<NT, NW>(imga, lowbits + c.offB + static_cast<unsigned>(next_src) * c.row_pitch, nxtB);
            }
        }
        // ---- horizontal pass for the source rows this output row adds -------------------------
        for (; next_src < lo + n; ++next_src) {
            float2 acc0 = make_float2(0.0f, 0.0f), acc1 = acc0, acc2 = acc0;
            if constexpr (NT > 0) {
                const RowWords<NW> curA = nxtA, curB = nxtB;
                if (next_src + 1 < last_src) {
                    const unsigned rowoff = static_cast<unsigned>(next_src + 1) * c.row_pitch + lowbits;
                    load_window<NT, NW>(imga, rowoff + c.offA, nxtA);
                    load_window<NT, NW>(imga, rowoff + c.offB, nxtB);
                }
                unsigned sA[NS], sB[NS];
#pragma unroll
                for (int i = 0; i < NS; ++i) {
                    sA[i] = __funnelshift_r(curA.w[i], curA.w[i + 1], curA.sh);
                    sB[i] = __funnelshift_r(curB.w[i], curB.w[i + 1], curB.sh);
                }
                const float4* wq = c.xw;
#pragma unroll
                for (int q = 0; q < NT; ++q, wq += c.xw_stride) {
                    const float4 w = *wq;
                    const float2 w2 = make_float2(w.x, w.y), nw2 = make_float2(w.z, w.w);
                    float2 px[3];
#pragma unroll
                    for (int ch = 0; ch < 3; ++ch) {
                        constexpr unsigned kHi = 0x4B000000u;
                        const int j = 3 * q + ch;
                        px[ch].x = __uint_as_float(__byte_perm(sA[j >> 2], kHi, 0x7440u | (j & 3)));
                        px[ch].y = __uint_as_float(__byte_perm(sB[j >> 2], kHi, 0x7440u | (j & 3)));
                    }
                    acc0 = aa_fma2(aa_fma2(px[0], w2, nw2), one2, acc0);
                    acc1 = aa_fma2(aa_fma2(px[1], w2, nw2), one2, acc1);
                    acc2 = aa_fma2(aa_fma2(px[2], w2, nw2), one2, acc2);
                }
            } else {
                const unsigned char* pa = c.img + c.offA + static_cast<unsigned long long>(next_src) * c.row_pitch;
                const unsigned char* pb = c.img + c.offB + static_cast<unsigned long long>(next_src) * c.row_pitch;
                const float4* wq = c.xw;
#pragma unroll 2
                for (int q = 0; q < c.nt; ++q, pa += 3, pb += 3, wq += c.xw_stride) {
                    const float4 w = *wq;
                    const float2 w2 = make_float2(w.x, w.y), nw2 = make_float2(w.z, w.w);
                    const unsigned a0 = __ldg(pa), a1 = __ldg(pa + 1), a2 = __ldg(pa + 2);
                    const unsigned b0 = __ldg(pb), b1 = __ldg(pb + 1), b2 = __ldg(pb + 2);
                    acc0 = aa_fma2(aa_fma2(make_float2(__uint_as_float(a0 | 0x4B000000u), __uint_as_float(b0 | 0x4B000000u)), w2, nw2), one2, acc0);
                    acc1 = aa_fma2(aa_fma2(make_float2(__uint_as_float(a1 | 0x4B000000u), __uint_as_float(b1 | 0x4B000000u)), w2, nw2), one2, acc1);
                    acc2 = aa_fma2(aa_fma2(make_float2(__uint_as_float(a2 | 0x4B000000u), __uint_as_float(b2 | 0x4B000000u)), w2, nw2), one2, acc2);
                }
            }
            float2* slot = reinterpret_cast<float2*>(next_slot);
            slot[0] = acc0;
            slot[1] = acc1;
            slot[2] = acc2;
            next_slot += c.slot_bytes;
            if (next_slot == c.ring_end) next_slot = c.myring;
        }
        // ---- vertical pass, rounding, normalize, store --------------------------------------
        float2 v0 = make_float2(0.0f, 0.0f), v1 = v0, v2 = v0;
        const float* wr = c.yw + r * c.yt;
        const unsigned char* vs = lo_slot;
        for (int q = 0; q < n; ++q) {
            const float w = wr[q];
            const float2 w2 = make_float2(w, w);
            const float2* slot = reinterpret_cast<const float2*>(vs);
            vs += c.slot_bytes;
            if (vs == c.ring_end) vs = c.myring;
            v0 = aa_fma2(aa_mul2(w2, slot[0]), one2, v0);
            v1 = aa_fma2(aa_mul2(w2, slot[1]), one2, v1);
            v2 = aa_fma2(aa_mul2(w2, slot[2]), one2, v2);
        }
        // (uint8)max(0, min(255, acc + 0.5f))   simd_utils.hpp:2008-2009.  acc >= 0 (weights and pixels are),
        // so only the upper clamp can act; the truncation is RZ(x + 2^23), and code * pre is
        // fma(2^23 + code, pre, -2^23 pre), exactly RN(code * pre).
        auto finish = [&](float2 v, int ch) {
            float2 t = aa_fma2(v, one2, make_float2(0.5f, 0.5f));
            t.x = fminf(t.x, 255.0f);
            t.y = fminf(t.y, 255.0f);
            const float2 x = aa_fma2(aa_add2_rz(t, k2), pre2, nkpre2);
            return aa_mul2(aa_fma2(x, one2, make_float2(c.nmean[ch], c.nmean[ch])), make_float2(c.inv_std[ch], c.inv_std[ch]));
        };
        const float2 o0 = finish(v0, 0), o1 = finish(v1, 1), o2 = finish(v2, 2);
        put<DTYPE>(c.out, oA, o0.x);
        put<DTYPE>(c.out, oA + c.chan_step, o1.x);
        put<DTYPE>(c.out, oA + 2 * c.chan_step, o2.x);
        if (c.validB) {
            put<DTYPE>(c.out, oB, o0.y);
            put<DTYPE>(c.out, oB + c.chan_step, o1.y);
            put<DTYPE>(c.out, oB + 2 * c.chan_step, o2.y);
        }
    }
}

template <int DTYPE, int LAYOUT>
__global__ void __launch_bounds__(128) antialias_pair_kernel(const __grid_constant__ FusedParams p,
                                                             const __grid_constant__ AAPlan a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x;
    const int TC = a.tile_cols, TR = a.tile_rows, HT = TC / 2;  // HT = threads per CTA
    float4* const xw4 = reinterpret_cast<float4*>(smem);                   // [xt][HT] {wA, wB, -2^23 wA, -2^23 wB}
    unsigned char* const ring = reinterpret_cast<unsigned char*>(xw4 + a.xt * HT);  // [yt][HT] x 24 B: three float2 per thread
    float* const scratch = reinterpret_cast<float*>(ring + a.yt * HT * 24);  // [xt][TC] unnormalized weights
    float* const yw = scratch + a.xt * TC;                                 // [TR][yt]
    int* const yl = reinterpret_cast<int*>(yw + TR * a.yt);                // [TR] first tap row
    int* const yc = yl + TR;                                               // [TR] tap count

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

    // ---- taps: each thread builds the tables of its two columns; one thread per tile row -------
    // nt = horizontal taps the loop runs for every column of this sample; a column's own taps sit at
    // positions [shift, shift + n) of that window, whose first pixel is lo - shift >= 0.
    const int nt = min(xmax, cw);
    const int colA = tid, colB = tid + HT;
    const bool validA = colA < tcw, validB = colB < tcw;
    int firstA = 0, firstB = 0;  // first pixel of each column's tap window (crop-local)
    {
        auto build = [&](int col, bool valid, int& first, int half) {
            int lo = 0, n = 0, shift = 0;
            float wsum = 0.0f;
            if (valid) {
                aa_taps(tx0 + col, cw, xscale, xsup, xmax, scratch + col, TC, lo, n, wsum);
                first = max(0, min(lo, cw - nt));
                shift = lo - first;
            }
            for (int q = 0; q < nt; ++q) {
                const int j = q - shift;
                float w = 0.0f;
                if (valid && j >= 0 && j < n) {
                    w = scratch[j * TC + col];
                    if (wsum > 0.0f) w = __fdiv_rn(w, wsum);
                }
                float* e = reinterpret_cast<float*>(xw4 + q * HT + tid);
                e[half] = w;
                e[2 + half] = __fmul_rn(-8388608.0f, w);
            }
        };
        build(colA, validA, firstA, 0);
        build(colB, validB, firstB, 1);
    }
    for (int r = tid; r < ty1 - ty0; r += blockDim.x) {
        float wsum;
        int lo, n;
        aa_taps(ty0 + r, ch, yscale, ysup, ymax, yw + r * a.yt, 1, lo, n, wsum);
        if (wsum > 0.0f)
            for (int q = 0; q < n; ++q) yw[r * a.yt + q] = __fdiv_rn(yw[r * a.yt + q], wsum);
        yl[r] = lo;
        yc[r] = n;
    }
    __syncthreads();
    if (!validA) return;

    PairCtx c;
    c.out = p.out;
    c.img = p.src + img_off;
    {
        // Ask L2 for the tile's whole source footprint now: every source row is a fresh DRAM line for
        // the thread that filters it, and the one-row register prefetch of the row loop covers an L2
        // hit, not a DRAM miss.  One request per 128-byte line that holds a byte some column taps.
        const int r0 = yl[0], r1 = yl[ty1 - ty0 - 1] + yc[ty1 - ty0 - 1];
        const float cl = __fmul_rn(static_cast<float>(tx0), xscale) - xsup - 1.0f;
        const float cr = __fmul_rn(static_cast<float>(tx0 + tcw), xscale) + xsup + 1.0f;
        const int x0 = max(0, min(cw - 1, static_cast<int>(cl))), x1 = max(x0 + 1, min(cw, static_cast<int>(cr) + 1));
        const unsigned long long rowb = reinterpret_cast<unsigned long long>(c.img) +
                                        (static_cast<unsigned long long>(cy) * iw + cx + x0) * 3;
        const unsigned span = static_cast<unsigned>(x1 - x0) * 3u;
        for (int rr = r0 + tid / 8; rr < r1; rr += blockDim.x / 8) {
            const unsigned long long b = rowb + static_cast<unsigned long long>(rr) * iw * 3;
            const unsigned long long e = b + span - 1;
            for (unsigned long long ln = (b & ~127ull) + 128ull * (tid & 7); ln <= e; ln += 128ull * 8)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(ln > b ? ln : b));
        }
    }
    c.row_pitch = static_cast<unsigned>(iw) * 3u;
    c.offA = static_cast<unsigned>((static_cast<long long>(cy) * iw + cx + firstA) * 3);
    c.offB = static_cast<unsigned>((static_cast<long long>(cy) * iw + cx + firstB) * 3);
    c.xw = xw4 + tid;
    c.xw_stride = HT;
    c.yw = yw;
    c.yl = yl;
    c.yc = yc;
    c.yt = a.yt;
    c.rows = ty1 - ty0;
    c.slot_bytes = HT * 24;
    c.myring = ring + tid * 24;
    c.ring_end = c.myring + a.yt * c.slot_bytes;
    c.nt = nt;
    c.one = p.one;
    c.pre = p.pre_scale;
    c.nkpre = p.neg_k_pre;
    for (int q = 0; q < 3; ++q) {
        c.nmean[q] = -p.mean[q];
        c.inv_std[q] = p.inv_std[q];
    }
    c.validB = validB;
    // where the two columns land after the flip, as element offsets of channel 0 at tile row 0
    const int xoA = flip ? (W - 1 - (tx0 + colA)) : tx0 + colA;
    const int xoB = flip ? (W - 1 - (tx0 + colB)) : tx0 + colB;
    if constexpr (LAYOUT == 0) {
        const long long base = (static_cast<long long>(k) * 3 * H + ty0) * W;
        c.oA = base + xoA;
        c.oB = base + xoB;
        c.row_step = W;
        c.chan_step = static_cast<long long>(H) * W;
    } else {
        const long long base = (static_cast<long long>(k) * H + ty0) * W;
        c.oA = (base + xoA) * 3;
        c.oB = (base + xoB) * 3;
        c.row_step = 3 * W;
        c.chan_step = 1;
    }
    // Word loads round the tap window out to 4-byte words; that must stay inside memory the caller
    // handed over: inside the image when images are separate allocations, inside the source range
    // otherwise.  A sample that cannot promise it takes the byte loads.
    const unsigned long long ia = reinterpret_cast<unsigned long long>(c.img);
    const unsigned long long ie = ia + static_cast<unsigned long long>(iw) * ih * 3;
    const unsigned long long sa = reinterpret_cast<unsigned long long>(p.src);
    const bool words_ok = p.per_image_region ? ((ia & 3) == 0 && (ie & 3) == 0)
                                             : ((ia & ~3ull) >= sa && ((ie + 3) & ~3ull) <= sa + p.src_bytes);
    switch (words_ok ? nt : 0) {
        case 1: pair_rows<DTYPE, 1>(c); break;
        case 2: pair_rows<DTYPE, 2>(c); break;
        case 3: pair_rows<DTYPE, 3>(c); break;
        case 4: pair_rows<DTYPE, 4>(c); break;
        case 5: pair_rows<DTYPE, 5>(c); break;
        case 6: pair_rows<DTYPE, 6>(c); break;
        case 7: pair_rows<DTYPE, 7>(c); break;
        case 8: pair_rows<DTYPE, 8>(c); break;
        default: pair_rows<DTYPE, 0>(c); break;
    }
}

std::atomic<unsigned long long> g_aa_launches{0};

template <int DTYPE, int LAYOUT>
int launch_one(const FusedParams& p, const AAPlan& a, cudaStream_t st) {
    if (a.pair)
        antialias_pair_kernel<DTYPE, LAYOUT><<<static_cast<unsigned>(a.grid), a.tile_cols / 2, a.smem_bytes, st>>>(p, a);
    else
        antialias_kernel<DTYPE, LAYOUT><<<static_cast<unsigned>(a.grid), a.tile_cols, a.smem_bytes, st>>>(p, a);
    g_aa_launches.fetch_add(1, std::memory_order_relaxed);
    return static_cast<int>(cudaGetLastError());
}

template <int DTYPE, int LAYOUT>
int opt_in() {
    int e = static_cast<int>(cudaFuncSetAttribute(antialias_kernel<DTYPE, LAYOUT>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, kAAMaxSmem));
    if (!e)
        e = static_cast<int>(cudaFuncSetAttribute(antialias_pair_kernel<DTYPE, LAYOUT>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, kAAMaxSmem));
    return e;
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
