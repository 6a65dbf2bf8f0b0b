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
// Two kernels compute it.  antialias_pair_kernel (the default) gives a thread TWO columns of the
// resized image in packed fp32, walks down the source rows a tile taps, drops the taps whose weight
// is exactly zero (bit-neutral), fetches tap windows as aligned words and asks for the next row and
// for the tile's whole footprint ahead of use; it is described where it is defined.
// antialias_kernel is the first, one-column form, kept as a cross-check (TLB_AA_ONE_COLUMN):
// a CTA owns a tile of output rows x output columns of one sample; a thread owns one column of the
// RESIZED image for both passes, so the two passes need no synchronisation: the horizontal results
// of the source rows an output row taps sit in a shared-memory ring indexed by source row, written
// and read by the same thread.  Every source row of the tile's footprint is filtered horizontally
// once.  Column weights live in shared memory ([tap][column], conflict-free), row weights in a small
// per-tile table.
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
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // see the packed kernel
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
// pair: six bytes picked out of realigned 32-bit words by PRMT straight into 2^23 + byte (byte loads
// for filters wider than the unrolled ones), three packed FMAs for the products
// fma(2^23 + b, w, -2^23 w) == RN(b w) and three for the running sums (fma(prod, 1, acc), the exact
// packed add); the weights of the pair sit in shared memory as {wA, wB, -2^23 wA, -2^23 wB}.
// The tap loop has the TILE's tap count (the most any of its columns kept after the zero-weight
// taps were dropped) as its trip count for every column; a column with fewer taps gets zero weights
// in front or behind (adding +0 changes no bit), and its tap window is shifted left where it would
// leave the crop, so no load ever leaves the crop row.
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

// Shared memory through 32-bit shared-window addresses: the ring and the tables are walked with
// 32-bit adds instead of 64-bit generic pointers.  All of these are `volatile`, which keeps a
// thread's ring stores and loads in program order.
__device__ __forceinline__ uint32_t aa_smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ float4 aa_lds_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float aa_lds_f(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ int2 aa_lds_i2(uint32_t addr) {
    int2 v;
    asm volatile("ld.shared.v2.s32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
template <int OFF>
__device__ __forceinline__ void aa_sts_f2(uint32_t addr, float2 v) {
    asm volatile("st.shared.v2.f32 [%0+%1], {%2, %3};" ::"r"(addr), "n"(OFF), "f"(v.x), "f"(v.y));
}
template <int OFF>
__device__ __forceinline__ float2 aa_lds_f2o(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2+%3];" : "=f"(v.x), "=f"(v.y) : "r"(addr), "n"(OFF));
    return v;
}

struct PairCtx {
    const unsigned char* img;      // the sample's image
    unsigned row_pitch;            // bytes per image row
    unsigned offA, offB;           // byte offset (from img) of the first pixel of each column's tap window, crop row 0
    uint32_t xw;                   // this thread's weights: float4 {wA, wB, -2^23 wA, -2^23 wB} every xw_stride bytes
    uint32_t xw_stride;
    uint32_t yw;                   // [rows][yt] floats
    uint32_t yrec;                 // [rows] int2 {last source row the output row taps, tap count}
    int yt, rows;
    int first_src, end_src;        // source rows the tile taps: [first_src, end_src)
    uint32_t ring;                 // this thread's 24 bytes of ring slot 0
    int slot_bytes;                // bytes between ring slots
    int slots;                     // ring slots (>= the most vertical taps)
    int nt;                        // horizontal taps of this sample
    float one, pre, nkpre;
    float nmean[3], inv_std[3];
    bool jit;                      // colour jitter (brightness jb, contrast jc, saturation js) before the normalize
    float jb, jc, js;
    bool validB;
    unsigned char* pA;             // channel 0 of column A at tile row 0
    long long dB;                  // bytes from column A to column B
    long long row_step, chan_step; // bytes to the next output row / channel
};

// The words of one source row's tap window for one column: aligned 32-bit words starting at the
// word that holds the window's first byte, and the bit shift that realigns them.  Sized for the
// widest unrolled filter; a narrower one uses the first words only.
constexpr int kAAUnrolledTaps = 8;
constexpr int kAAMaxWords = (3 * kAAUnrolledTaps + 3) / 4 + 1;
struct RowWords {
    unsigned w[kAAMaxWords];
    unsigned sh;
};

template <int NT>
__device__ __forceinline__ void load_window(const unsigned char* imga, unsigned g, RowWords& r) {
    // g = byte offset of the window from the 4-aligned `imga`.  Words 0..NS-1 always hold window
    // bytes; the last one is fetched only when the window reaches into it (otherwise it would feed
    // nothing but shifted-out bits, and might lie past the end of the image).
    constexpr int NS = (3 * NT + 3) / 4;
    const unsigned al = g & 3u;
    const unsigned* wp = reinterpret_cast<const unsigned*>(imga + (g - al));
#pragma unroll
    for (int i = 0; i < NS; ++i) r.w[i] = __ldg(wp + i);
    r.w[NS] = 0u;
    if (al + 3u * NT > 4u * NS) r.w[NS] = __ldg(wp + NS);
    r.sh = al * 8u;
}

template <int DTYPE>
__device__ __forceinline__ void put_at(unsigned char* ptr, float v) {
    if constexpr (DTYPE == 0)
        *reinterpret_cast<float*>(ptr) = v;
    else
        *reinterpret_cast<__nv_bfloat16*>(ptr) = __float2bfloat16_rn(v);
}

// The horizontal sums of one source row go to the thread's ring slot.
__device__ __forceinline__ void ring_store(uint32_t at, float2 c0, float2 c1, float2 c2) {
    aa_sts_f2<0>(at, c0);
    aa_sts_f2<8>(at, c1);
    aa_sts_f2<16>(at, c2);
}

// Horizontal pass of one source row for a column pair whose tile has exactly NT taps.  `a`, `b`
// hold the row's words on entry; they are realigned first, so that the same registers can take
// the NEXT row's words (requested here, a row of arithmetic ahead of their use).  The first tap
// starts the sums (0 + x is x), the others add to them in tap order.
template <int NT>
__device__ __forceinline__ void hrow_words(const PairCtx& c, const unsigned char* imga, unsigned gA, unsigned gB,
                                           int src, RowWords& a, RowWords& b, float2 one2, uint32_t ring_at) {
    constexpr int NS = (3 * NT + 3) / 4;
    unsigned sA[NS], sB[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        sA[i] = __funnelshift_r(a.w[i], a.w[i + 1], a.sh);
        sB[i] = __funnelshift_r(b.w[i], b.w[i + 1], b.sh);
    }
    if (src + 1 < c.end_src) {
        const unsigned rowoff = static_cast<unsigned>(src + 1) * c.row_pitch;
        load_window<NT>(imga, rowoff + gA, a);
        load_window<NT>(imga, rowoff + gB, b);
    }
    float2 acc0, acc1, acc2;
    uint32_t wq = c.xw;
#pragma unroll
    for (int q = 0; q < NT; ++q, wq += c.xw_stride) {
        const float4 w = aa_lds_f4(wq);
        const float2 w2 = make_float2(w.x, w.y), nw2 = make_float2(w.z, w.w);
        float2 px[3];
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) {
            constexpr unsigned kHi = 0x4B000000u;
            const int j = 3 * q + ch;
            px[ch].x = __uint_as_float(__byte_perm(sA[j >> 2], kHi, 0x7440u | (j & 3)));
            px[ch].y = __uint_as_float(__byte_perm(sB[j >> 2], kHi, 0x7440u | (j & 3)));
        }
        if (q == 0) {
            acc0 = aa_fma2(px[0], w2, nw2);
            acc1 = aa_fma2(px[1], w2, nw2);
            acc2 = aa_fma2(px[2], w2, nw2);
        } else {
            acc0 = aa_fma2(aa_fma2(px[0], w2, nw2), one2, acc0);
            acc1 = aa_fma2(aa_fma2(px[1], w2, nw2), one2, acc1);
            acc2 = aa_fma2(aa_fma2(px[2], w2, nw2), one2, acc2);
        }
    }
    ring_store(ring_at, acc0, acc1, acc2);
}

// ... any tap count, byte loads, nothing requested ahead.
__device__ __forceinline__ void hrow_bytes(const PairCtx& c, int src, float2 one2, uint32_t ring_at) {
    const unsigned char* pa = c.img + c.offA + static_cast<unsigned long long>(src) * c.row_pitch;
    const unsigned char* pb = c.img + c.offB + static_cast<unsigned long long>(src) * c.row_pitch;
    uint32_t wq = c.xw;
    float2 acc0 = make_float2(0.0f, 0.0f), acc1 = acc0, acc2 = acc0;
#pragma unroll 2
    for (int q = 0; q < c.nt; ++q, pa += 3, pb += 3, wq += c.xw_stride) {
        const float4 w = aa_lds_f4(wq);
        const float2 w2 = make_float2(w.x, w.y), nw2 = make_float2(w.z, w.w);
        const unsigned a0 = __ldg(pa), a1 = __ldg(pa + 1), a2 = __ldg(pa + 2);
        const unsigned b0 = __ldg(pb), b1 = __ldg(pb + 1), b2 = __ldg(pb + 2);
        acc0 = aa_fma2(aa_fma2(make_float2(__uint_as_float(a0 | 0x4B000000u), __uint_as_float(b0 | 0x4B000000u)), w2, nw2), one2, acc0);
        acc1 = aa_fma2(aa_fma2(make_float2(__uint_as_float(a1 | 0x4B000000u), __uint_as_float(b1 | 0x4B000000u)), w2, nw2), one2, acc1);
        acc2 = aa_fma2(aa_fma2(make_float2(__uint_as_float(a2 | 0x4B000000u), __uint_as_float(b2 | 0x4B000000u)), w2, nw2), one2, acc2);
    }
    ring_store(ring_at, acc0, acc1, acc2);
}

// Rows of one tile for a thread's column pair, as a walk down the SOURCE rows the tile taps: each
// is filtered horizontally into the thread's ring slot, then every output row whose last tap row it
// was is finished (vertical pass over the ring, rounding, normalize, store).  `mode` picks the
// horizontal pass: 1..kAAUnrolledTaps = that many taps, unrolled, window fetched as aligned words
// (bytes picked by PRMT straight into 2^23 + b); 0 = byte loads.  The choice is made per row by a
// CTA-uniform branch so that the vertical pass exists once in the kernel's code: with one copy per
// filter width the CTAs of a batch (whose samples differ in width) thrashed the instruction cache.
template <int DTYPE>
__device__ __forceinline__ void pair_rows(const PairCtx& c, const int mode) {
    const float2 one2 = make_float2(c.one, c.one);
    const float2 k2 = make_float2(8388608.0f, 8388608.0f);
    const float2 half2 = make_float2(0.5f, 0.5f);
    const float2 pre2 = make_float2(c.pre, c.pre), nkpre2 = make_float2(c.nkpre, c.nkpre);
    const unsigned lowbits = static_cast<unsigned>(reinterpret_cast<unsigned long long>(c.img) & 3ull);
    const unsigned char* const imga = c.img - lowbits;
    const unsigned gA = lowbits + c.offA, gB = lowbits + c.offB;

    int src = c.first_src;        // source row being filtered
    int slot = 0;                 // its ring slot, and the slot's byte offset
    int slot_off = 0;
    int r = 0;                    // next output row to finish
    int2 rec = aa_lds_i2(c.yrec); // {its last tap row, its tap count}
    uint32_t wrow = c.yw;         // its weights
    unsigned char* pA = c.pA;

    RowWords bufA, bufB;
#pragma unroll
    for (int i = 0; i < kAAMaxWords; ++i) bufA.w[i] = bufB.w[i] = 0u;
    bufA.sh = bufB.sh = 0u;
    {
        const unsigned rowoff = static_cast<unsigned>(src) * c.row_pitch;
        switch (mode) {
            case 1: load_window<1>(imga, rowoff + gA, bufA); load_window<1>(imga, rowoff + gB, bufB); break;
            case 2: load_window<2>(imga, rowoff + gA, bufA); load_window<2>(imga, rowoff + gB, bufB); break;
            case 3: load_window<3>(imga, rowoff + gA, bufA); load_window<3>(imga, rowoff + gB, bufB); break;
            case 4: load_window<4>(imga, rowoff + gA, bufA); load_window<4>(imga, rowoff + gB, bufB); break;
            case 5: load_window<5>(imga, rowoff + gA, bufA); load_window<5>(imga, rowoff + gB, bufB); break;
            case 6: load_window<6>(imga, rowoff + gA, bufA); load_window<6>(imga, rowoff + gB, bufB); break;
            case 7: load_window<7>(imga, rowoff + gA, bufA); load_window<7>(imga, rowoff + gB, bufB); break;
            case 8: load_window<8>(imga, rowoff + gA, bufA); load_window<8>(imga, rowoff + gB, bufB); break;
            default: break;
        }
    }
    for (;;) {
        // ---- horizontal pass of source row `src` into its ring slot (commonest widths first) -------
        const uint32_t ring_at = c.ring + slot_off;
        if (mode == 3) hrow_words<3>(c, imga, gA, gB, src, bufA, bufB, one2, ring_at);
        else if (mode == 2) hrow_words<2>(c, imga, gA, gB, src, bufA, bufB, one2, ring_at);
        else if (mode == 4) hrow_words<4>(c, imga, gA, gB, src, bufA, bufB, one2, ring_at);
        else if (mode == 5) hrow_words<5>(c, imga, gA, gB, src, bufA, bufB, one2, ring_at);
        else if (mode == 6) hrow_words<6>(c, imga, gA, gB, src, bufA, bufB, one2, ring_at);
        else if (mode == 7) hrow_words<7>(c, imga, gA, gB, src, bufA, bufB, one2, ring_at);
        else if (mode == 8) hrow_words<8>(c, imga, gA, gB, src, bufA, bufB, one2, ring_at);
        else if (mode == 1) hrow_words<1>(c, imga, gA, gB, src, bufA, bufB, one2, ring_at);
        else hrow_bytes(c, src, one2, ring_at);
        // ---- finish the output rows whose last tap row this was ----------------------------------
        while (rec.x <= src) {  // == for every table the tap rule can produce (last tap rows never decrease)
            const int n = rec.y;
            int lo_slot = slot - (n - 1);
            if (lo_slot < 0) lo_slot += c.slots;
            const int n1 = min(n, c.slots - lo_slot);   // taps before the ring wraps
            uint32_t vs = c.ring + lo_slot * c.slot_bytes;
            uint32_t wq = wrow;
            float2 v0, v1, v2;
            {   // the first tap starts the sums (0 + x is x)
                const float w = aa_lds_f(wq);
                const float2 w2 = make_float2(w, w);
                v0 = aa_mul2(w2, aa_lds_f2o<0>(vs));
                v1 = aa_mul2(w2, aa_lds_f2o<8>(vs));
                v2 = aa_mul2(w2, aa_lds_f2o<16>(vs));
            }
            auto tap = [&]() {
                wq += 4;
                vs += c.slot_bytes;
                const float w = aa_lds_f(wq);
                const float2 w2 = make_float2(w, w);
                const float2 s0 = aa_lds_f2o<0>(vs), s1 = aa_lds_f2o<8>(vs), s2 = aa_lds_f2o<16>(vs);
                v0 = aa_fma2(aa_mul2(w2, s0), one2, v0);
                v1 = aa_fma2(aa_mul2(w2, s1), one2, v1);
                v2 = aa_fma2(aa_mul2(w2, s2), one2, v2);
            };
            for (int q = 1; q < n1; ++q) tap();
            vs = c.ring - c.slot_bytes;
            for (int q = n1; q < n; ++q) tap();
            // (uint8)max(0, min(255, acc + 0.5f))   simd_utils.hpp:2008-2009.  acc >= 0 (weights and pixels
            // are), so only the upper clamp can act; the truncation is RZ(x + 2^23), and code * pre is
            // fma(2^23 + code, pre, -2^23 pre), exactly RN(code * pre).
            auto code01 = [&](float2 v) {
                float2 t = aa_fma2(v, one2, half2);
                t.x = fminf(t.x, 255.0f);
                t.y = fminf(t.y, 255.0f);
                return aa_fma2(aa_add2_rz(t, k2), pre2, nkpre2);
            };
            float2 x0 = code01(v0), x1 = code01(v1), x2 = code01(v2);
            if (c.jit) {
                // Colour jitter on rgb = code/255 in the order of the reference's train_transform shader
                // (src/metal/metal_transforms.mm:111-115), every operation rounded separately: brightness,
                // contrast about 0.5, saturation as lum + (rgb-lum)*s with lum = (0.299 r + 0.587 g) + 0.114 b,
                // clamp to [0,1].  Same sequence as in the bilinear kernel.
                auto jitter1 = [&](float& r, float& g, float& b) {
                    r = __fadd_rn(__fmul_rn(__fsub_rn(__fmul_rn(r, c.jb), 0.5f), c.jc), 0.5f);
                    g = __fadd_rn(__fmul_rn(__fsub_rn(__fmul_rn(g, c.jb), 0.5f), c.jc), 0.5f);
                    b = __fadd_rn(__fmul_rn(__fsub_rn(__fmul_rn(b, c.jb), 0.5f), c.jc), 0.5f);
                    const float lum = __fadd_rn(__fadd_rn(__fmul_rn(r, 0.299f), __fmul_rn(g, 0.587f)), __fmul_rn(b, 0.114f));
                    r = fminf(fmaxf(__fadd_rn(lum, __fmul_rn(__fsub_rn(r, lum), c.js)), 0.0f), 1.0f);
                    g = fminf(fmaxf(__fadd_rn(lum, __fmul_rn(__fsub_rn(g, lum), c.js)), 0.0f), 1.0f);
                    b = fminf(fmaxf(__fadd_rn(lum, __fmul_rn(__fsub_rn(b, lum), c.js)), 0.0f), 1.0f);
                };
                jitter1(x0.x, x1.x, x2.x);
                jitter1(x0.y, x1.y, x2.y);
            }
            auto normalize = [&](float2 x, int ch) {
                return aa_mul2(aa_fma2(x, one2, make_float2(c.nmean[ch], c.nmean[ch])),
                               make_float2(c.inv_std[ch], c.inv_std[ch]));
            };
            const float2 o0 = normalize(x0, 0), o1 = normalize(x1, 1), o2 = normalize(x2, 2);
            put_at<DTYPE>(pA, o0.x);
            put_at<DTYPE>(pA + c.chan_step, o1.x);
            put_at<DTYPE>(pA + 2 * c.chan_step, o2.x);
            if (c.validB) {
                unsigned char* const pB = pA + c.dB;
                put_at<DTYPE>(pB, o0.y);
                put_at<DTYPE>(pB + c.chan_step, o1.y);
                put_at<DTYPE>(pB + 2 * c.chan_step, o2.y);
            }
            ++r;
            pA += c.row_step;
            wrow += 4 * c.yt;
            rec = r < c.rows ? aa_lds_i2(c.yrec + 8 * r) : make_int2(0x7fffffff, 0);  // no row left: never matches
        }
        if (r >= c.rows) break;
        if (++src >= c.end_src) break;  // never walks past the rows the tile taps, whatever the tables say
        slot_off += c.slot_bytes;
        if (++slot == c.slots) slot = 0, slot_off = 0;
    }
}

template <int DTYPE, int LAYOUT>
__global__ void __launch_bounds__(128) antialias_pair_kernel(const __grid_constant__ FusedParams p,
                                                             const __grid_constant__ AAPlan a) {
    extern __shared__ __align__(16) unsigned char smem[];
    // Lets a launch made with programmatic stream serialization start behind this one as soon as
    // every CTA of this one has been scheduled; a no-op for any other launch.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int tid = threadIdx.x;
    const int TC = a.tile_cols, TR = a.tile_rows, HT = TC / 2;  // HT = threads per CTA
    float4* const xw4 = reinterpret_cast<float4*>(smem);                   // [xt][HT] {wA, wB, -2^23 wA, -2^23 wB}
    unsigned char* const ring = reinterpret_cast<unsigned char*>(xw4 + a.xt * HT);  // [yt][HT] x 24 B: three float2 per thread
    float* const scratch = reinterpret_cast<float*>(ring);                 // [xt][TC] unnormalized weights, dead before the ring is first written
    const int ring_or_scratch = max(a.yt * HT * 24, a.xt * TC * 4);
    int2* const yrec = reinterpret_cast<int2*>(ring + ring_or_scratch);     // [TR] {last tap row, tap count}
    float* const yw = reinterpret_cast<float*>(yrec + TR);                 // [TR][yt]

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
    // Taps whose weight is exactly zero are dropped from the front and the back of every table: the
    // reference multiplies them in, but w = +0 times a non-negative pixel is +0 and acc + (+0) is acc,
    // so the sums keep every bit.  The tap bounds lo = floor(c - s), hi = ceil(c + s) reach up to one
    // pixel past the filter's support on either side; without them a column has at most ceil(2 s)
    // taps instead of ceil(2 s) + 2 -- three instead of five for a mild downscale.
    // nt = taps the horizontal loop runs for every column of this tile (the most any of its columns
    // kept); a column's own taps sit at positions [shift, shift + n) of that window, whose first
    // pixel is lo - shift >= 0.
    __shared__ int s_nt;
    if (tid == 0) s_nt = 1;
    __syncthreads();
    const int colA = tid, colB = tid + HT;
    const bool validA = colA < tcw, validB = colB < tcw;
    struct ColTaps {
        int lo, n, z0;   // first kept tap (crop-local pixel), kept taps, dropped in front
        float wsum;
    } tA{0, 0, 0, 0.0f}, tB{0, 0, 0, 0.0f};
    {
        auto taps_of = [&](int col, ColTaps& t) {
            int lo, n;
            aa_taps(tx0 + col, cw, xscale, xsup, xmax, scratch + col, TC, lo, n, t.wsum);
            int z0 = 0, z1 = n;
            while (z0 < n - 1 && scratch[z0 * TC + col] == 0.0f) ++z0;
            while (z1 > z0 + 1 && scratch[(z1 - 1) * TC + col] == 0.0f) --z1;
            t.lo = lo + z0;
            t.n = z1 - z0;
            t.z0 = z0;
            atomicMax(&s_nt, t.n);
        };
        if (validA) taps_of(colA, tA);
        if (validB) taps_of(colB, tB);
    }
    for (int r = tid; r < ty1 - ty0; r += blockDim.x) {
        float wsum;
        int lo, n;
        float* const w = yw + r * a.yt;
        aa_taps(ty0 + r, ch, yscale, ysup, ymax, w, 1, lo, n, wsum);
        int z0 = 0, z1 = n;
        while (z0 < n - 1 && w[z0] == 0.0f) ++z0;
        while (z1 > z0 + 1 && w[z1 - 1] == 0.0f) --z1;
        for (int q = z0; q < z1; ++q) w[q - z0] = wsum > 0.0f ? __fdiv_rn(w[q], wsum) : w[q];
        yrec[r] = make_int2(lo + z1 - 1, z1 - z0);
    }
    __syncthreads();
    const int nt = s_nt;
    int firstA = 0, firstB = 0;  // first pixel of each column's tap window (crop-local)
    {
        auto fill = [&](int col, bool valid, const ColTaps& t, int& first, int half) {
            int shift = 0;
            if (valid) {
                first = max(0, min(t.lo, cw - nt));   // nt <= cw: no column keeps more taps than the crop has pixels
                shift = t.lo - first;
            }
            for (int q = 0; q < nt; ++q) {
                const int j = q - shift;
                float w = 0.0f;
                if (valid && j >= 0 && j < t.n) {
                    w = scratch[(j + t.z0) * TC + col];
                    if (t.wsum > 0.0f) w = __fdiv_rn(w, t.wsum);
                }
                float* e = reinterpret_cast<float*>(xw4 + q * HT + tid);
                e[half] = w;
                e[2 + half] = __fmul_rn(-8388608.0f, w);
            }
        };
        fill(colA, validA, tA, firstA, 0);
        fill(colB, validB, tB, firstB, 1);
    }
    __syncthreads();
    if (!validA) return;

    const int first_src = yrec[0].x - yrec[0].y + 1;
    const int end_src = yrec[ty1 - ty0 - 1].x + 1;
    PairCtx c;
    c.img = p.src + img_off;
    {
        // Ask L2 for the tile's whole source footprint now: every source row is a fresh DRAM line for
        // the thread that filters it, and the one-row register prefetch of the row loop covers an L2
        // hit, not a DRAM miss.  One request per 128-byte line that holds a byte some column taps.
        const float cl = __fmul_rn(static_cast<float>(tx0), xscale) - xsup - 1.0f;
        const float cr = __fmul_rn(static_cast<float>(tx0 + tcw), xscale) + xsup + 1.0f;
        const int x0 = max(0, min(cw - 1, static_cast<int>(cl))), x1 = max(x0 + 1, min(cw, static_cast<int>(cr) + 1));
        const unsigned long long rowb = reinterpret_cast<unsigned long long>(c.img) +
                                        (static_cast<unsigned long long>(cy) * iw + cx + x0) * 3;
        const unsigned span = static_cast<unsigned>(x1 - x0) * 3u;
        for (int rr = first_src + tid / 8; rr < end_src; rr += blockDim.x / 8) {
            const unsigned long long b = rowb + static_cast<unsigned long long>(rr) * iw * 3;
            const unsigned long long e = b + span - 1;
            for (unsigned long long ln = (b & ~127ull) + 128ull * (tid & 7); ln <= e; ln += 128ull * 8)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(ln > b ? ln : b));
        }
    }
    c.row_pitch = static_cast<unsigned>(iw) * 3u;
    c.offA = static_cast<unsigned>((static_cast<long long>(cy) * iw + cx + firstA) * 3);
    c.offB = static_cast<unsigned>((static_cast<long long>(cy) * iw + cx + firstB) * 3);
    c.xw = aa_smem_u32(xw4 + tid);
    c.xw_stride = static_cast<uint32_t>(HT) * 16u;
    c.yw = aa_smem_u32(yw);
    c.yrec = aa_smem_u32(yrec);
    c.yt = a.yt;
    c.rows = ty1 - ty0;
    c.first_src = first_src;
    c.end_src = end_src;
    c.ring = aa_smem_u32(ring + tid * 24);
    c.slot_bytes = HT * 24;
    c.slots = a.yt;
    c.nt = nt;
    c.one = p.one;
    c.pre = p.pre_scale;
    c.nkpre = p.neg_k_pre;
    for (int q = 0; q < 3; ++q) {
        c.nmean[q] = -p.mean[q];
        c.inv_std[q] = p.inv_std[q];
    }
    c.jit = p.jitter != nullptr;
    c.jb = c.jc = c.js = 1.0f;
    if (c.jit) {
        c.jb = p.jitter[3 * static_cast<long long>(k)];
        c.jc = p.jitter[3 * static_cast<long long>(k) + 1];
        c.js = p.jitter[3 * static_cast<long long>(k) + 2];
    }
    c.validB = validB;
    // where the two columns land after the flip
    const int xoA = flip ? (W - 1 - (tx0 + colA)) : tx0 + colA;
    const int xoB = flip ? (W - 1 - (tx0 + colB)) : tx0 + colB;
    constexpr int kElem = DTYPE == 0 ? 4 : 2;
    if constexpr (LAYOUT == 0) {
        c.pA = static_cast<unsigned char*>(p.out) + ((static_cast<long long>(k) * 3 * H + ty0) * W + xoA) * kElem;
        c.dB = static_cast<long long>(xoB - xoA) * kElem;
        c.row_step = static_cast<long long>(W) * kElem;
        c.chan_step = static_cast<long long>(H) * W * kElem;
    } else {
        c.pA = static_cast<unsigned char*>(p.out) + ((static_cast<long long>(k) * H + ty0) * W + xoA) * 3 * kElem;
        c.dB = static_cast<long long>(xoB - xoA) * 3 * kElem;
        c.row_step = static_cast<long long>(W) * 3 * kElem;
        c.chan_step = kElem;
    }
    // Word loads round the tap window out to 4-byte words; that must stay inside memory the caller
    // handed over: inside the image when images are separate allocations, inside the source range
    // otherwise.  A sample that cannot promise it takes the byte loads.
    const unsigned long long ia = reinterpret_cast<unsigned long long>(c.img);
    const unsigned long long ie = ia + static_cast<unsigned long long>(iw) * ih * 3;
    const unsigned long long sa = reinterpret_cast<unsigned long long>(p.src);
    const bool words_ok = p.per_image_region ? ((ia & 3) == 0 && (ie & 3) == 0)
                                             : ((ia & ~3ull) >= sa && ((ie + 3) & ~3ull) <= sa + p.src_bytes);
    pair_rows<DTYPE>(c, words_ok && nt <= kAAUnrolledTaps ? nt : 0);
}

std::atomic<unsigned long long> g_aa_launches{0};

template <int DTYPE, int LAYOUT>
int launch_one(const FusedParams& p, const AAPlan& a, cudaStream_t st, unsigned flags) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(a.grid));
    cfg.blockDim = dim3(static_cast<unsigned>(a.pair ? a.tile_cols / 2 : a.tile_cols));
    cfg.dynamicSmemBytes = static_cast<size_t>(a.smem_bytes);
    cfg.stream = st;
    // Same contract as the bilinear kernel's launch: with kLaunchOverlap the launch may start while
    // the kernel before it in the stream drains its last CTAs; it never waits on that kernel.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & kLaunchOverlap) ? 1 : 0;
    if (a.pair)
        cudaLaunchKernelEx(&cfg, antialias_pair_kernel<DTYPE, LAYOUT>, p, a);
    else
        cudaLaunchKernelEx(&cfg, antialias_kernel<DTYPE, LAYOUT>, p, a);
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

int launch_antialias(const FusedParams& p, const AAPlan& a, int out_dtype, int out_layout, void* stream, unsigned flags) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (out_dtype == 0) return out_layout == 0 ? launch_one<0, 0>(p, a, st, flags) : launch_one<0, 1>(p, a, st, flags);
    return out_layout == 0 ? launch_one<1, 0>(p, a, st, flags) : launch_one<1, 1>(p, a, st, flags);
}

unsigned long long antialias_launch_count() { return g_aa_launches.load(std::memory_order_relaxed); }

}  // namespace tlb
