// Fused YUV 4:2:0 video transform for sm_100a: per output pixel, bilinear luma + bilinear
// chroma (MPEG siting: horizontally co-sited, vertically centred), video-range BT.601 / BT.709
// matrix, clip to [0,1], mean/std normalize, planar (T,3,H,W) fp32 or bf16 output; optionally a
// crop window + horizontal flip shared by all frames of a clip.  One launch covers every frame of
// the batch (the functions replaced launch once per frame or once per clip):
//   turboloader::cuda::video_yuv420_batch   src/cuda/cuda_transforms.cu:143-197, 367-409
//   turboloader::cuda::video_clip_yuv420    src/cuda/cuda_transforms.cu:207-268, 416-473
//
// Arithmetic: the kernels replaced are the only statement of this math; it is followed operation
// by operation with every multiply, add and divide rounded to fp32 separately, which is what the
// CPU oracle restates.  Two output rows ride in the two lanes of the packed fp32 instructions;
// bytes become floats without an integer conversion (fma(2^23 + b, w, -2^23 * w) == RN(b * w));
// the division by 255 is a three-operation sequence that equals the IEEE quotient.
//
// Two kernels share that arithmetic:
//  * yuv420_direct_kernel (the default): per-thread byte loads of the taps straight from global
//    memory through L1, with the next row pair's lines prefetched.  A bilinear downscale taps only
//    part of the source, and this kernel reads only the sectors it taps.
//  * yuv420_staged_kernel (opt-in): a CTA owns a few output rows of one frame; one warp issues a
//    bulk asynchronous copy (cp.async.bulk, completion on an mbarrier) for every source row
//    segment the CTA needs -- two luma and two chroma rows per output row, clipped to the columns
//    the CTA's outputs tap -- and everybody then reads taps from shared memory.  Measured on the
//    benchmark's clip workload it is the slower of the two (one copy-then-compute phase per CTA,
//    no overlap inside the CTA), so it is not the default; it moves whole row segments, which
//    pays when nearly every source byte is tapped (resize factors near 1).
// A thread owns one output column and walks down the CTA's rows, so the horizontal taps and
// weights are worked out once per thread and the vertical ones once per CTA.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstdlib>

#include "fused_params.h"
#include "video_params.h"

namespace tlb {
namespace {

constexpr int kDirectRowsAlone = 12, kDirectRowsOverlap = 24;  // output rows per CTA of the direct kernel (processed as pairs)
constexpr int kStageMaxRows = 16;  // most output rows per CTA of the staged kernel
constexpr unsigned kVideoCopyTimeout = 8u;  // status bit: a bounded wait on the staging copies gave up

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

// Packed two-lane fp32 operations of sm_100; each lane rounds like the scalar instruction.
#define TLB_V2(name, op)                                                                              \
    __device__ __forceinline__ float2 name(float2 a, float2 b) {                                      \
        float2 d;                                                                                     \
        asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t" op      \
            " rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"                                              \
            : "=f"(d.x), "=f"(d.y)                                                                    \
            : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));                                                \
        return d;                                                                                     \
    }
TLB_V2(mul2, "mul.rn.f32x2")
TLB_V2(add2, "add.rn.f32x2")
#undef TLB_V2
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "mov.b64 rc, {%6, %7};\n\tfma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
// (RN(b0 * w.x), RN(b1 * w.y)) for two bytes without an integer conversion: OR-ing a byte into
// the mantissa of 2^23 gives the float 2^23 + b; with nw = -2^23 * w (exact),
// fma(2^23 + b, w, nw) evaluates b * w exactly and rounds once.
__device__ __forceinline__ float2 bytes_times(unsigned b0, unsigned b1, float2 w, float2 nw) {
    return fma2(f2(__uint_as_float(b0 | 0x4B000000u), __uint_as_float(b1 | 0x4B000000u)), w, nw);
}
// a + b where a is a product: issued as fma(a, one, b).  The assembler fuses a packed multiply
// that feeds a packed add into one FMA (observed even with contraction disabled), which would
// drop the product's own rounding; an FMA whose multiplicand is the finished product and whose
// multiplier is a 1.0f it cannot see through (a kernel parameter) cannot be fused any further.
// sign_one = +1 adds the product, -1 subtracts it (a * -1 is exact).
__device__ __forceinline__ float2 add_prod(float2 prod, float2 sign_one, float2 b) { return fma2(prod, sign_one, b); }

// x / 255 correctly rounded in three operations (q = x * r; e = x - q * 255 exactly, by FMA;
// q + e * r): equal to the IEEE quotient for every float with 2^-40 <= |x| <= 2^12 and for zero
// (checked exhaustively on the CPU against the division); channel values lie within +-1000.
__device__ __forceinline__ float2 div255(float2 x) {
    const float r = 1.0f / 255.0f;
    const float2 q = mul2(x, f2(r, r));
    const float2 e = fma2(q, f2(-255.0f, -255.0f), x);
    return fma2(e, f2(r, r), q);
}

template <int DTYPE>
__device__ __forceinline__ void put(void* out, long long idx, float v) {
    if constexpr (DTYPE == 0)
        static_cast<float*>(out)[idx] = v;
    else
        static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
}

// The 24 taps of a pair of output rows (index [h]: row r + h): luma upper/lower row (a, b),
// Cb and Cr upper/lower row (ua, ub, va, vb), left/right tap (0, 1).
struct Taps {
    unsigned a0[2], a1[2], b0[2], b1[2], ua0[2], ua1[2], ub0[2], ub1[2], va0[2], va1[2], vb0[2], vb1[2];
};
// Vertical weights of the pair, (row r, row r+1) in the two lanes.
struct PairWeights {
    float2 dy, idy, cdy, icdy;
};
// Per-column weights (both lanes equal) and launch constants, packed.
struct ColWeights {
    float2 wx, iwx, nwx, niwx, wc, iwc, nwc, niwc;
};
struct Consts {
    float2 kY, kRV, kGU, kGV, kBU, one, mone, m16, m128, nm0, nm1, nm2, is0, is1, is2;
};

__device__ __forceinline__ Consts make_consts(const VideoParams& p) {
    Consts c;
    const float ky = 255.0f / 219.0f;
    const float rv = p.bt709 ? 1.792741f : 1.596027f, gu = p.bt709 ? 0.213249f : 0.391762f;
    const float gv = p.bt709 ? 0.532909f : 0.812968f, bu = p.bt709 ? 2.112402f : 2.017232f;
    c.kY = f2(ky, ky); c.kRV = f2(rv, rv); c.kGU = f2(gu, gu); c.kGV = f2(gv, gv); c.kBU = f2(bu, bu);
    c.one = f2(p.one, p.one); c.mone = f2(-p.one, -p.one);
    c.m16 = f2(-16.0f, -16.0f); c.m128 = f2(-128.0f, -128.0f);
    c.nm0 = f2(-p.mean[0], -p.mean[0]); c.nm1 = f2(-p.mean[1], -p.mean[1]); c.nm2 = f2(-p.mean[2], -p.mean[2]);
    c.is0 = f2(p.inv_std[0], p.inv_std[0]); c.is1 = f2(p.inv_std[1], p.inv_std[1]); c.is2 = f2(p.inv_std[2], p.inv_std[2]);
    return c;
}

__device__ __forceinline__ ColWeights make_col(float dx, float cdx) {
    ColWeights w;
    const float idx = 1.0f - dx, icdx = 1.0f - cdx;
    w.wx = f2(dx, dx); w.iwx = f2(idx, idx);
    w.nwx = f2(-8388608.0f * dx, -8388608.0f * dx); w.niwx = f2(-8388608.0f * idx, -8388608.0f * idx);
    w.wc = f2(cdx, cdx); w.iwc = f2(icdx, icdx);
    w.nwc = f2(-8388608.0f * cdx, -8388608.0f * cdx); w.niwc = f2(-8388608.0f * icdx, -8388608.0f * icdx);
    return w;
}

// Output-row coordinates (cuda_transforms.cu:150-152 whole frame; :219-223 crop window).
__device__ __forceinline__ float src_y(const VideoParams& p, bool use_crop, float4 crop, int y) {
    if (use_crop) {
        const float sy = crop.y + __fdiv_rn(static_cast<float>(y) + 0.5f, static_cast<float>(p.dst_h)) * crop.w - 0.5f;
        return fminf(fmaxf(sy, 0.0f), static_cast<float>(p.src_h - 1));
    }
    return fmaxf(0.0f, __fdiv_rn((static_cast<float>(y) + 0.5f) * static_cast<float>(p.src_h),
                                 static_cast<float>(p.dst_h)) - 0.5f);
}
__device__ __forceinline__ float src_x(const VideoParams& p, bool use_crop, float4 crop, bool flip, int x) {
    if (use_crop) {
        const int ox = flip ? (p.dst_w - 1 - x) : x;
        const float sx = crop.x + __fdiv_rn(static_cast<float>(ox) + 0.5f, static_cast<float>(p.dst_w)) * crop.z - 0.5f;
        return fminf(fmaxf(sx, 0.0f), static_cast<float>(p.src_w - 1));
    }
    return fmaxf(0.0f, __fdiv_rn((static_cast<float>(x) + 0.5f) * static_cast<float>(p.src_w),
                                 static_cast<float>(p.dst_w)) - 0.5f);
}

// Blend, colour conversion, clip and normalize of one row pair; stores up to two rows.
template <int DTYPE>
__device__ __forceinline__ void convert_store(const Taps& k, const PairWeights& pw, const ColWeights& w, const Consts& c,
                                              void* out, long long o, long long plane, int W, bool second) {
    const float2 ytop = add2(bytes_times(k.a0[0], k.a0[1], w.iwx, w.niwx), bytes_times(k.a1[0], k.a1[1], w.wx, w.nwx));
    const float2 ybot = add2(bytes_times(k.b0[0], k.b0[1], w.iwx, w.niwx), bytes_times(k.b1[0], k.b1[1], w.wx, w.nwx));
    const float2 yv0 = add_prod(mul2(ytop, pw.idy), c.one, mul2(ybot, pw.dy));
    const float2 utop = add2(bytes_times(k.ua0[0], k.ua0[1], w.iwc, w.niwc), bytes_times(k.ua1[0], k.ua1[1], w.wc, w.nwc));
    const float2 ubot = add2(bytes_times(k.ub0[0], k.ub0[1], w.iwc, w.niwc), bytes_times(k.ub1[0], k.ub1[1], w.wc, w.nwc));
    const float2 cbv = add_prod(mul2(utop, pw.icdy), c.one, mul2(ubot, pw.cdy));
    const float2 vtop = add2(bytes_times(k.va0[0], k.va0[1], w.iwc, w.niwc), bytes_times(k.va1[0], k.va1[1], w.wc, w.nwc));
    const float2 vbot = add2(bytes_times(k.vb0[0], k.vb0[1], w.iwc, w.niwc), bytes_times(k.vb1[0], k.vb1[1], w.wc, w.nwc));
    const float2 crv = add_prod(mul2(vtop, pw.icdy), c.one, mul2(vbot, pw.cdy));

    const float2 yv = mul2(add2(yv0, c.m16), c.kY);
    const float2 cb = add2(cbv, c.m128), cr = add2(crv, c.m128);
    const float2 R = add_prod(mul2(c.kRV, cr), c.one, yv);                                        // yv + kRV*cr
    const float2 G = add_prod(mul2(c.kGV, cr), c.mone, add_prod(mul2(c.kGU, cb), c.mone, yv));  // (yv - kGU*cb) - kGV*cr
    const float2 B = add_prod(mul2(c.kBU, cb), c.one, yv);                                        // yv + kBU*cb
    float2 r01 = div255(R), g01 = div255(G), b01 = div255(B);
    r01 = f2(fminf(fmaxf(r01.x, 0.0f), 1.0f), fminf(fmaxf(r01.y, 0.0f), 1.0f));
    g01 = f2(fminf(fmaxf(g01.x, 0.0f), 1.0f), fminf(fmaxf(g01.y, 0.0f), 1.0f));
    b01 = f2(fminf(fmaxf(b01.x, 0.0f), 1.0f), fminf(fmaxf(b01.y, 0.0f), 1.0f));
    const float2 ro = mul2(add2(r01, c.nm0), c.is0);
    const float2 go = mul2(add2(g01, c.nm1), c.is1);
    const float2 bo = mul2(add2(b01, c.nm2), c.is2);
    put<DTYPE>(out, o, ro.x);
    put<DTYPE>(out, o + plane, go.x);
    put<DTYPE>(out, o + 2 * plane, bo.x);
    if (second) {
        put<DTYPE>(out, o + W, ro.y);
        put<DTYPE>(out, o + plane + W, go.y);
        put<DTYPE>(out, o + 2 * plane + W, bo.y);
    }
}

// ================= direct kernel: taps loaded from global memory ==========================
struct __align__(16) DirectPair {
    int ya[2], yb[2];  // byte offsets of the upper / lower luma row, for row r and row r+1
    int ca[2], cb[2];  // same for the chroma rows
    PairWeights w;
};

// Two horizontally adjacent taps of a row.  The right tap is the left one again at the right
// edge; its load is skipped there so that nothing beyond the row is touched.
__device__ __forceinline__ void taps_global(const unsigned char* p, int step, bool edge, unsigned& t0, unsigned& t1) {
    t0 = __ldg(p);
    t1 = t0;
    if (!edge) t1 = __ldg(p + step);
}

// Asks for the line of the next row pair's taps while the current pair is being converted: costs
// no register and no wait, and turns most of the next iteration's misses into hits (+6 %).
__device__ __forceinline__ void prefetch_line(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

template <int DTYPE, int ROWS>
__global__ void __launch_bounds__(256, 6) yuv420_direct_kernel(const __grid_constant__ VideoParams p) {
    __shared__ DirectPair pairs[ROWS / 2];
    // Lets a launch made with programmatic stream serialization start behind this one as soon as
    // every CTA of this one has been scheduled; a no-op for any other launch.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int t = blockIdx.y;                     // frame
    const int r0 = blockIdx.x * ROWS;             // first output row of this CTA
    const int rows = min(ROWS, p.dst_h - r0);
    const int W = p.dst_w, H = p.dst_h;
    const int cw = (p.src_w + 1) / 2, ch = (p.src_h + 1) / 2;
    // Tables in the parameter block (small batches) or in device memory: either way behind pointers
    // (the parameter is __grid_constant__, so its members have addresses).
    const bool inl = p.inline_tables != 0;
    const unsigned char* const* const planes = inl ? p.in.planes : p.planes;
    const float4* const crops = inl ? (p.has_crops ? p.in.crops : nullptr) : p.crops;
    const int* const flips = inl ? (p.has_flips ? p.in.flips : nullptr) : p.flips;
    const bool use_crop = crops != nullptr;
    float4 crop = make_float4(0.f, 0.f, 0.f, 0.f);
    bool flip = false;
    if (use_crop) {
        const int clip = p.clip_len > 0 ? t / p.clip_len : 0;
        crop = crops[clip];
        flip = flips ? flips[clip] != 0 : false;
    }
    if (threadIdx.x < ROWS) {  // a block has at least 32 threads
        // Rows past the end of the frame repeat the last row (their results are never stored).
        const int y = min(r0 + static_cast<int>(threadIdx.x), H - 1);
        const float sy = src_y(p, use_crop, crop, y);
        const int y0 = static_cast<int>(sy);
        const int y1 = min(y0 + 1, p.src_h - 1);
        const float cyf = fminf(fmaxf(sy * 0.5f - 0.25f, 0.0f), static_cast<float>(ch - 1));
        const int cy0 = static_cast<int>(cyf);
        const int cy1 = min(cy0 + 1, ch - 1);
        const float dy = sy - static_cast<float>(y0), cdy = cyf - static_cast<float>(cy0);
        DirectPair& pt = pairs[threadIdx.x >> 1];
        const int h = threadIdx.x & 1;
        pt.ya[h] = y0 * p.y_stride;
        pt.yb[h] = y1 * p.y_stride;
        pt.ca[h] = cy0 * p.c_stride;
        pt.cb[h] = cy1 * p.c_stride;
        (&pt.w.dy.x)[h] = dy;
        (&pt.w.idy.x)[h] = 1.0f - dy;
        (&pt.w.cdy.x)[h] = cdy;
        (&pt.w.icdy.x)[h] = 1.0f - cdy;
    }
    const unsigned char* __restrict__ yp = planes[t];
    const unsigned char* __restrict__ cbp = planes[p.n + t];
    const unsigned char* __restrict__ crp = planes[2 * p.n + t];
    __syncthreads();

    const Consts c = make_consts(p);
    const long long plane = static_cast<long long>(H) * W;
    const long long frame_base = static_cast<long long>(t) * 3 * plane;
    const int cstep = p.c_px_stride;
    for (int x = threadIdx.x; x < W; x += blockDim.x) {
        const float sx = src_x(p, use_crop, crop, flip, x);
        const int x0 = static_cast<int>(sx);
        const bool yedge = x0 + 1 > p.src_w - 1;
        const float cxf = fminf(fmaxf(sx * 0.5f, 0.0f), static_cast<float>(cw - 1));
        const int cx0 = static_cast<int>(cxf);
        const bool cedge = cx0 + 1 > cw - 1;
        const ColWeights w = make_col(sx - static_cast<float>(x0), cxf - static_cast<float>(cx0));
        const unsigned char* ycol = yp + x0;
        const unsigned char* ucol = cbp + cx0 * cstep;
        const unsigned char* vcol = crp + cx0 * cstep;
        long long o = frame_base + static_cast<long long>(r0) * W + x;
        for (int r = 0; r < rows; r += 2, o += 2 * W) {
            const DirectPair& q = pairs[r >> 1];
            if (r + 2 < rows) {
                const DirectPair& nx = pairs[(r >> 1) + 1];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    prefetch_line(ycol + nx.ya[h]);
                    prefetch_line(ycol + nx.yb[h]);
                    prefetch_line(ucol + nx.ca[h]);
                    prefetch_line(ucol + nx.cb[h]);
                    prefetch_line(vcol + nx.ca[h]);
                    prefetch_line(vcol + nx.cb[h]);
                }
            }
            Taps k;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                taps_global(ycol + q.ya[h], 1, yedge, k.a0[h], k.a1[h]);
                taps_global(ycol + q.yb[h], 1, yedge, k.b0[h], k.b1[h]);
                taps_global(ucol + q.ca[h], cstep, cedge, k.ua0[h], k.ua1[h]);
                taps_global(ucol + q.cb[h], cstep, cedge, k.ub0[h], k.ub1[h]);
                taps_global(vcol + q.ca[h], cstep, cedge, k.va0[h], k.va1[h]);
                taps_global(vcol + q.cb[h], cstep, cedge, k.vb0[h], k.vb1[h]);
            }
            convert_store<DTYPE>(k, q.w, w, c, p.out, o, plane, W, r + 1 < rows);
        }
    }
}

// ================= staged kernel: source row segments copied to shared memory first =======
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t mbar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(mbar), "r"(parity), "r"(1000000u)
        : "memory");
    return ok != 0;
}
// Bounded (about one second on the global timer): returns false if the copies never landed.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t mbar, uint32_t parity) {
    if (mbar_try_wait(mbar, parity)) return true;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (unsigned it = 0; it < (1u << 20); ++it) {
        if (mbar_try_wait(mbar, parity)) return true;
        if ((it & 15u) == 15u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (now - t0 > 1000000000ull) return false;
        }
    }
    return false;
}

// Shared-memory layout of the staged kernel: header (mbarrier, row table), then one slot per
// staged row segment.  A slot keeps the segment at the same offset modulo 16 as in global
// memory, so that the aligned middle of it can be moved by one bulk copy (16-byte granularity
// on both sides) and only its ragged first and last bytes by plain loads.
struct __align__(16) StageRow {
    int ya, yb;          // shared-memory byte offsets of the first luma tap column in the upper / lower row
    int ua, ub, va, vb;  // same for Cb and Cr
    float dy, idy, cdy, icdy;
    int pad[2];
};
constexpr int kStageBars = 8 * (kStageMaxRows / 2);  // one 8-byte mbarrier per pair of output rows
constexpr int kStageHeader = kStageBars + kStageMaxRows * static_cast<int>(sizeof(StageRow));

template <int DTYPE>
__global__ void __launch_bounds__(256, 5) yuv420_staged_kernel(const __grid_constant__ VideoParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    StageRow* const table = reinterpret_cast<StageRow*>(smem + kStageBars);
    const uint32_t mbar = smem_addr(smem);
    const int R = p.stage_rows;                   // output rows per CTA (even)
    const int t = blockIdx.y;                     // frame
    const int r0 = blockIdx.x * R;                // first output row of this CTA
    const int rows = min(R, p.dst_h - r0);
    const int W = p.dst_w, H = p.dst_h;
    const int cw = (p.src_w + 1) / 2, ch = (p.src_h + 1) / 2;
    const int cstep = p.c_px_stride;
    const bool use_crop = p.crops != nullptr;
    float4 crop = make_float4(0.f, 0.f, 0.f, 0.f);
    bool flip = false;
    if (use_crop) {
        const int clip = p.clip_len > 0 ? t / p.clip_len : 0;
        crop = p.crops[clip];
        flip = p.flips ? p.flips[clip] != 0 : false;
    }
    // Columns the CTA's outputs tap: sx is monotonic in the (possibly mirrored) output column.
    const float sx_a = src_x(p, use_crop, crop, flip, flip ? W - 1 : 0);
    const float sx_b = src_x(p, use_crop, crop, flip, flip ? 0 : W - 1);
    const int fx_lo = static_cast<int>(sx_a);
    const int fx_hi = min(static_cast<int>(sx_b) + 1, p.src_w - 1);
    const int cfx_lo = static_cast<int>(fminf(fmaxf(sx_a * 0.5f, 0.0f), static_cast<float>(cw - 1)));
    const int cfx_hi = min(static_cast<int>(fminf(fmaxf(sx_b * 0.5f, 0.0f), static_cast<float>(cw - 1))) + 1, cw - 1);
    const int ylen = fx_hi - fx_lo + 1;                       // bytes of a luma segment
    const int clen = (cfx_hi - cfx_lo) * cstep + 1;           // bytes of a chroma segment of ONE plane
    const unsigned char* const yp = p.planes[t];
    const unsigned char* const cbp = p.planes[p.n + t];
    const unsigned char* const crp = p.planes[2 * p.n + t];
    // NV12 / NV21: both chroma planes live interleaved in one buffer; stage it once.
    const bool shared_uv = cstep == 2 && (crp == cbp + 1 || cbp == crp + 1);
    const unsigned char* const uvp = crp < cbp ? crp : cbp;   // lower of the two addresses (shared_uv only)
    const int uvlen = clen + 1;
    const int ypitch = (ylen + 15 + 15) & ~15;
    const int cpitch = ((shared_uv ? uvlen : clen) + 15 + 15) & ~15;
    const int cslots = shared_uv ? 2 : 4;                     // chroma slots per output row
    const int row_bytes = 2 * ypitch + cslots * cpitch;
    unsigned char* const slots = smem + kStageHeader;

    // One mbarrier per PAIR of output rows: the pairs' copies are all issued up front and the
    // arithmetic on pair i starts as soon as its own rows have landed, while later pairs are
    // still in flight.
    const int npairs = (rows + 1) >> 1;
    if (threadIdx.x < npairs) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar + 8 * threadIdx.x), "r"(1u) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    {
        // ---- one thread per staged segment: row table entry + copy ---------------------------
        const int nseg = rows * (2 + cslots);
        for (int sgi = threadIdx.x; sgi < nseg; sgi += blockDim.x) {
            unsigned bytes = 0;
            unsigned long long lo = 0;
            uint32_t dst = 0;
            const uint32_t pbar = mbar + 8 * ((sgi / (2 + cslots)) >> 1);
            {
                const int j = sgi / (2 + cslots), kind = sgi % (2 + cslots);
                const int y = r0 + j;
                const float sy = src_y(p, use_crop, crop, y);
                const int y0 = static_cast<int>(sy);
                const int y1 = min(y0 + 1, p.src_h - 1);
                const float cyf = fminf(fmaxf(sy * 0.5f - 0.25f, 0.0f), static_cast<float>(ch - 1));
                const int cy0 = static_cast<int>(cyf);
                const int cy1 = min(cy0 + 1, ch - 1);
                unsigned long long a0, reg_lo, reg_hi;  // segment start; readable bytes of its plane
                int len, slot_off;
                if (kind < 2) {
                    reg_lo = reinterpret_cast<unsigned long long>(yp);
                    reg_hi = reg_lo + static_cast<unsigned long long>(p.src_h - 1) * p.y_stride + p.src_w;
                    a0 = reg_lo + static_cast<unsigned long long>(kind ? y1 : y0) * p.y_stride + fx_lo;
                    len = ylen;
                    slot_off = j * row_bytes + kind * ypitch;
                } else {
                    const int ck = kind - 2;                  // shared: 0 upper, 1 lower; else 0 Ua 1 Ub 2 Va 3 Vb
                    const int crow = (shared_uv ? ck : (ck & 1)) ? cy1 : cy0;
                    const unsigned char* base = shared_uv ? uvp : (ck < 2 ? cbp : crp);
                    reg_lo = reinterpret_cast<unsigned long long>(base);
                    reg_hi = reg_lo + static_cast<unsigned long long>(ch - 1) * p.c_stride + (cw - 1) * cstep + 1 +
                             (shared_uv ? 1 : 0);
                    a0 = reg_lo + static_cast<unsigned long long>(crow) * p.c_stride + cfx_lo * cstep;
                    len = shared_uv ? uvlen : clen;
                    slot_off = j * row_bytes + 2 * ypitch + ck * cpitch;
                }
                const unsigned long long a1 = a0 + len;
                const int phase = static_cast<int>(a0 & 15ull);
                unsigned char* slot = slots + slot_off;      // holds global bytes [a0 - phase, ...)
                // Copy whole 16-byte chunks around the segment, but never beyond the plane: only the
                // first and the last row of a plane can have a ragged edge, moved by plain loads.
                lo = a0 & ~15ull;
                if (lo < reg_lo) lo += 16;
                unsigned long long hi = (a1 + 15ull) & ~15ull;
                if (hi > reg_hi) hi = a1 & ~15ull;
                bytes = hi > lo ? static_cast<unsigned>(hi - lo) : 0u;
                dst = smem_addr(slot) + static_cast<uint32_t>(lo - (a0 - phase));
                const unsigned long long head_end = bytes ? (lo < a1 ? lo : a1) : a1;
                for (unsigned long long a = a0; a < head_end; ++a)
                    slot[phase + (a - a0)] = *reinterpret_cast<const unsigned char*>(a);
                if (bytes)
                    for (unsigned long long a = (hi > a0 ? hi : a0); a < a1; ++a)
                        slot[phase + (a - a0)] = *reinterpret_cast<const unsigned char*>(a);
                // table entry: the lane that stages a row's first segment also writes its weights
                StageRow& e = table[j];
                const int first = slot_off + phase + kStageHeader;
                if (kind == 0) {
                    e.ya = first;
                    e.dy = sy - static_cast<float>(y0);
                    e.idy = 1.0f - e.dy;
                    e.cdy = cyf - static_cast<float>(cy0);
                    e.icdy = 1.0f - e.cdy;
                } else if (kind == 1) {
                    e.yb = first;
                } else if (shared_uv) {
                    const int uo = first + (cbp > crp ? 1 : 0), vo = first + (crp > cbp ? 1 : 0);
                    if (kind == 2) { e.ua = uo; e.va = vo; } else { e.ub = uo; e.vb = vo; }
                } else {
                    (kind == 2 ? e.ua : kind == 3 ? e.ub : kind == 4 ? e.va : e.vb) = first;
                }
            }
            if (bytes) {
                // The byte count is added to the pair's barrier before the copy is issued; the
                // barrier's single arrival comes after every thread has done so (below).
                asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(pbar), "r"(bytes) : "memory");
                asm volatile(
                    "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                    "l"(lo), "r"(bytes), "r"(pbar)
                    : "memory");
            }
        }
    }
    // Per-column setup overlaps the copies.
    const Consts c = make_consts(p);
    const long long plane = static_cast<long long>(H) * W;
    const long long frame_base = static_cast<long long>(t) * 3 * plane;
    __syncthreads();  // row table, ragged bytes and every expected byte count are in place
    if (threadIdx.x < npairs)
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar + 8 * threadIdx.x) : "memory");
    // Each warp waits for a pair's rows once (the wait is uniform across the warp) and keeps a
    // bit per pair, since the column loop below may visit the pairs more than once.
    unsigned landed = 0;
    bool gave_up = false;

    for (int x = threadIdx.x; x < W; x += blockDim.x) {
        const float sx = src_x(p, use_crop, crop, flip, x);
        const int x0 = static_cast<int>(sx);
        const bool yedge = x0 + 1 > p.src_w - 1;
        const float cxf = fminf(fmaxf(sx * 0.5f, 0.0f), static_cast<float>(cw - 1));
        const int cx0 = static_cast<int>(cxf);
        const bool cedge = cx0 + 1 > cw - 1;
        const ColWeights w = make_col(sx - static_cast<float>(x0), cxf - static_cast<float>(cx0));
        const unsigned char* const ycol = smem + (x0 - fx_lo);
        const unsigned char* const ccol = smem + (cx0 - cfx_lo) * cstep;
        const int ystep = yedge ? 0 : 1, ccstep = cedge ? 0 : cstep;
        long long o = frame_base + static_cast<long long>(r0) * W + x;
        for (int r = 0; r < rows; r += 2, o += 2 * W) {
            if (!((landed >> (r >> 1)) & 1u)) {
                if (!mbar_wait_bounded(mbar + 8 * (r >> 1), 0u)) {
                    gave_up = true;
                    break;
                }
                landed |= 1u << (r >> 1);
            }
            Taps k;
            PairWeights pw;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const StageRow& e = table[min(r + h, rows - 1)];
                k.a0[h] = ycol[e.ya]; k.a1[h] = ycol[e.ya + ystep];
                k.b0[h] = ycol[e.yb]; k.b1[h] = ycol[e.yb + ystep];
                k.ua0[h] = ccol[e.ua]; k.ua1[h] = ccol[e.ua + ccstep];
                k.ub0[h] = ccol[e.ub]; k.ub1[h] = ccol[e.ub + ccstep];
                k.va0[h] = ccol[e.va]; k.va1[h] = ccol[e.va + ccstep];
                k.vb0[h] = ccol[e.vb]; k.vb1[h] = ccol[e.vb + ccstep];
                (&pw.dy.x)[h] = e.dy; (&pw.idy.x)[h] = e.idy; (&pw.cdy.x)[h] = e.cdy; (&pw.icdy.x)[h] = e.icdy;
            }
            convert_store<DTYPE>(k, pw, w, c, p.out, o, plane, W, r + 1 < rows);
        }
        if (gave_up) break;
    }
    if (gave_up) {
        // A copy did not land within the limit: report it, then give every copy of this CTA one
        // more bounded chance to finish before the shared memory it targets is released.
        if (p.status) atomicOr(p.status, kVideoCopyTimeout);
        for (int i = 0; i < npairs; ++i) mbar_wait_bounded(mbar + 8 * i, 0u);
    }
}

std::atomic<unsigned long long> g_video_launches{0};

template <int DTYPE>
int opt_in() {
    return static_cast<int>(cudaFuncSetAttribute(yuv420_staged_kernel<DTYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 kVideoStageMaxBytes));
}

}  // namespace

// Shared memory the staged kernel needs for `rows` output rows per CTA (an upper bound over all
// alignments: every segment is padded to a 16-byte multiple plus 16).
int video_stage_bytes(const VideoParams& p, int rows) {
    const int cw = (p.src_w + 1) / 2;
    const int ypitch = (p.src_w + 30) & ~15;
    const int cpitch_shared = ((cw - 1) * 2 + 2 + 30) & ~15, cpitch_split = ((cw - 1) * p.c_px_stride + 1 + 30) & ~15;
    const int chroma = std::max(2 * cpitch_shared, 4 * cpitch_split);
    return kStageHeader + rows * (2 * ypitch + chroma);
}

int prepare_video() {
    int e = opt_in<0>();
    if (!e) e = opt_in<1>();
    return e;
}

int launch_video(const VideoParams& pin, int out_dtype, void* stream, unsigned flags) {
    VideoParams p = pin;
    const int threads = std::min(256, ((p.dst_w + 31) / 32) * 32);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Rows per CTA of the staged kernel: as many (even, at most kStageMaxRows) as keep the staging
    // buffer near 40 KB, so that several CTAs share an SM and overlap copy with arithmetic.
    int rows = 0;
    if (p.use_staged && !p.inline_tables) {
        for (int r = kStageMaxRows; r >= 2; r -= 2) {
            if (video_stage_bytes(p, r) <= (r == 2 ? kVideoStageMaxBytes : 40 * 1024)) {
                rows = r;
                break;
            }
        }
    }
    if (rows) {
        p.stage_rows = rows;
        const int smem = video_stage_bytes(p, rows);
        const dim3 grid(static_cast<unsigned>((p.dst_h + rows - 1) / rows), static_cast<unsigned>(p.n));
        if (out_dtype == 0)
            yuv420_staged_kernel<0><<<grid, threads, smem, st>>>(p);
        else
            yuv420_staged_kernel<1><<<grid, threads, smem, st>>>(p);
    } else {
        // Rows per CTA (compile-time: two instantiations): a launch on its own finishes soonest with 12 (many small CTAs, short tail); when
        // launches overlap head to tail, 24 rows amortise a CTA's set-up better and the tail is covered
        // (measured on 128 frames 1280x720 -> 224x224: 8 / 12 / 16 / 24 rows = 2.69 / 2.72 / 2.62 / 2.42 M
        // frames/s serialized, 3.27 / 3.43 / 3.52 / 3.60 M overlapping).
        const bool tall = (flags & kLaunchOverlap) != 0;
        const int drows = tall ? kDirectRowsOverlap : kDirectRowsAlone;
        p.direct_rows = drows;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(static_cast<unsigned>((p.dst_h + drows - 1) / drows), static_cast<unsigned>(p.n));
        cfg.blockDim = dim3(static_cast<unsigned>(threads));
        cfg.stream = st;
        // Same contract as the image kernels: with kLaunchOverlap the launch may start while the
        // kernel before it in the stream drains its last CTAs; it never waits on that kernel.
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = (flags & kLaunchOverlap) ? 1 : 0;
        if (out_dtype == 0) {
            if (tall) cudaLaunchKernelEx(&cfg, yuv420_direct_kernel<0, kDirectRowsOverlap>, p);
            else cudaLaunchKernelEx(&cfg, yuv420_direct_kernel<0, kDirectRowsAlone>, p);
        } else {
            if (tall) cudaLaunchKernelEx(&cfg, yuv420_direct_kernel<1, kDirectRowsOverlap>, p);
            else cudaLaunchKernelEx(&cfg, yuv420_direct_kernel<1, kDirectRowsAlone>, p);
        }
    }
    g_video_launches.fetch_add(1, std::memory_order_relaxed);
    return static_cast<int>(cudaGetLastError());
}

unsigned long long video_launch_count() { return g_video_launches.load(std::memory_order_relaxed); }

}  // namespace tlb
