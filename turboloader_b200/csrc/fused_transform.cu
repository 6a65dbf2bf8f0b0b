// Fused crop -> hflip -> bilinear resize -> normalize -> layout/cast kernel for sm_100a.
//
// Replaces TurboLoader's per-image kernels resize_normalize_kernel /
// crop_resize_normalize_kernel (src/cuda/cuda_transforms.cu:35-80) and its
// one-thread-per-float normalize_nhwc_to_nchw_kernel / normalize_gather_kernel
// (src/cuda/cuda_transforms.cu:103-135) with ONE launch per batch.  The arithmetic
// is that of the CPU fused path, which is the parity target:
//   src/transforms/simd_utils.hpp:97-103     s = max(0, (i + 0.5) * (src/dst) - 0.5)
//   src/transforms/simd_utils.hpp:1897-1931  top/bot/val, clamp, TRUNCATE to a u8 code
//   src/transforms/simd_utils.hpp:2201-2222  (u8 * s - mean) * inv_std
//   src/pipeline/direct_batch_loader.hpp:219-243  coordinates are crop-local; the flip is
//                                                  applied to the RESIZED image
// Every multiply and add is a separately rounded fp32 operation (no FMA contraction),
// in the CPU path's order, so fp32 output is bit-identical to it.
//
// Structure of one CTA = one tile of `tile_rows` x `tile_cols` outputs of one sample.  One
// warp per 32-column strip computes; one more warp only plans and copies.  No CTA-wide barrier
// is used after the prologue: the warps meet through mbarriers only.
//   planner warp: walks down the tile in passes of at most Rr NEW source rows (rows the strips
//      do not hold yet).  One lane per output row looks up (y0, y1) in a per-tile row table; the
//      first and last rows are exchanged with warp shuffles to find the range of new rows.  It
//      issues one 1-D bulk async copy (cp.async.bulk, global -> this CTA's shared memory,
//      completion on a "full" mbarrier) per new source row, each rounded out to 16-byte
//      boundaries; bytes that cannot be reached on a 16-byte grid inside the readable region are
//      fetched with plain loads.  Raw rows are double buffered; a buffer is refilled once every
//      compute warp has arrived on its "empty" mbarrier.
//   compute warp, "H" step: every new source row is interpolated horizontally once,
//      h = p[x0]*(1-dx) + p[x1]*dx, into a ring of fp32 rows private to the strip.  Each lane owns
//      one output column for the whole tile and keeps its weights in registers.
//   compute warp, "V" step: each lane owns 4 (fp32) or 8 (bf16) adjacent pixels of the strip and
//      the warp covers 8 / 4 output rows at a time: v = h[y0]*(1-dy) + h[y1]*dy, truncate,
//      normalize, cast, three 16-byte stores per row.  The layout of a ring row (planar for
//      NCHW, interleaved for NHWC, rows staggered by 16 bytes) makes every input a
//      conflict-free 16-byte shared load.  The fp32 arithmetic uses the packed two-lane forms
//      (mul/fma .f32x2) of sm_100; they round each lane exactly like the scalar instructions.
// The bilinear blend is exactly separable in this order (top and bot depend on one
// source row each), so sharing h between neighbouring output rows changes no bit.
//
// No tensor-core instruction is used: there is no contraction in this operation.
// No cluster launch and no multicast form of any copy is used; every load reads the
// memory of the GPU the kernel runs on.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <type_traits>

#include "fused_params.h"

namespace tlb {
namespace {

#ifndef TLB_H_UNROLL
#define TLB_H_UNROLL 4
#endif
constexpr int kHUnroll = TLB_H_UNROLL;  // source rows in flight per lane in the H step

constexpr unsigned kDevBadIndex = 1u, kDevBadBox = 2u, kDevTooWide = 4u, kDevCopyTimeout = 8u;
constexpr unsigned kWaitLimit = 1u << 20;  // bounded mbarrier polling (each poll may suspend briefly)

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes)
                 : "memory");
}
// One poll.  The suspend-time hint lets the hardware park the warp until the phase completes
// (or the hint expires) instead of returning at once: a warp that waits does not burn issue
// slots re-polling -- with plain polls the waiting planner and compute warps executed more than
// a quarter of all instructions of the kernel.
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t mbar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(mbar), "r"(parity), "r"(1000000u)
        : "memory");
    return ok;
}
// Returns false if the phase did not complete within about one second of wall time (each
// poll may suspend the warp for a while, so the bound is kept on the global timer, not on
// the poll count).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t mbar, uint32_t parity) {
    if (mbar_try_wait(mbar, parity)) return true;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (unsigned it = 0; it < kWaitLimit; ++it) {
        if (mbar_try_wait(mbar, parity)) return true;
        if ((it & 15u) == 15u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (now - t0 > 1000000000ull) return false;
        }
    }
    return false;
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// 1-D bulk async copy global -> shared memory of the executing CTA; dst, src and bytes
// must be multiples of 16.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t mbar) {
    asm volatile(
        "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(mbar)
        : "memory");
}

// simd_utils.hpp:100-103, with each operation rounded separately.
__device__ __forceinline__ float src_coord(int i, float scale) {
    float s = __fsub_rn(__fmul_rn(__fadd_rn(static_cast<float>(i), 0.5f), scale), 0.5f);
    return s < 0.0f ? 0.0f : s;
}

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

// Packed two-lane fp32 multiply / add of sm_100 (mul.f32x2, add.f32x2) with explicit rounding.
// Each lane rounds like the scalar instruction.  CAUTION: the assembler was observed to
// contract a packed multiply feeding a packed add into one FMA even with explicit .rn and with
// fmad disabled (it flips ~1e-5 of the 8-bit codes and the last bit of most normalized
// values).  So wherever a product feeds a sum, the sum is done with the scalar __fadd_rn,
// which is never contracted; packed adds are used only where no product is an input.
#ifdef TLB_NO_PACKED
__device__ __forceinline__ float2 mul2_rn(float2 a, float2 b) { return make_float2(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y)); }
__device__ __forceinline__ float2 add2_rn(float2 a, float2 b) { return make_float2(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y)); }
__device__ __forceinline__ float2 add2_rz(float2 a, float2 b) { return make_float2(__fadd_rz(a.x, b.x), __fadd_rz(a.y, b.y)); }
#else
#define TLB_F32X2_OP(name, op)                                                                   \
    __device__ __forceinline__ float2 name(float2 a, float2 b) {                                 \
        float2 d;                                                                                \
        asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t" op    \
            " rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"                                         \
            : "=f"(d.x), "=f"(d.y)                                                               \
            : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));                                           \
        return d;                                                                                \
    }
TLB_F32X2_OP(mul2_rn, "mul.rn.f32x2")
TLB_F32X2_OP(add2_rn, "add.rn.f32x2")
TLB_F32X2_OP(add2_rz, "add.rz.f32x2")
#undef TLB_F32X2_OP
#endif
// Packed FMA.  Used only where the fused result is exactly the wanted singly-rounded product
// (see byte_product2).
__device__ __forceinline__ float2 fma2_rn(float2 a, float2 b, float2 c) {
#ifdef TLB_NO_PACKED
    return make_float2(__fmaf_rn(a.x, b.x, c.x), __fmaf_rn(a.y, b.y, c.y));
#endif
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "mov.b64 rc, {%6, %7};\n\tfma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
// (RN(b0 * w.x), RN(b1 * w.y)) for two bytes b0, b1 in [0,255] WITHOUT an integer-to-float
// conversion (those run at a fraction of the fp32 rate on this GPU and were the busiest pipe).
// OR-ing a byte into the mantissa of 2^23 gives the float 2^23 + b exactly; with
// negw = -2^23 * w (exact: a power-of-two scaling), fma(2^23 + b, w, negw) evaluates
// (2^23 + b)*w - 2^23*w = b*w exactly and rounds once, i.e. it IS RN(b*w), bit for bit
// (and +0 when b or w is 0, like the plain product of non-negative operands).
__device__ __forceinline__ float2 byte_product2(unsigned b0, unsigned b1, float2 w, float2 negw) {
    return fma2_rn(f2(__uint_as_float(b0 | 0x4B000000u), __uint_as_float(b1 | 0x4B000000u)), w, negw);
}
// Packed sum a + b where a is a packed product: issued as fma(a, one, b) with `one` = 1.0f
// held in a register the assembler cannot see through (it comes from the kernel parameters).
// a*1 is exact, so the result is RN(a + b) lane by lane; and because the instruction already
// is an FMA whose multiplicand is a finished (rounded) product, nothing can be contracted
// into it.  This is what a packed add of products would be if it were safe (see above).
__device__ __forceinline__ float2 add2_exact(float2 a, float2 b, float2 one) { return fma2_rn(a, one, b); }

template <int DTYPE>
struct OutT;
template <>
struct OutT<0> {
    static constexpr int V = 4;
};
template <>
struct OutT<1> {
    static constexpr int V = 8;
};

template <int DTYPE>
__device__ __forceinline__ void store_scalar(void* out, long long idx, float v) {
    if constexpr (DTYPE == 0)
        static_cast<float*>(out)[idx] = v;
    else
        static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
}

// One 16-byte store of V finished outputs (fp32: 4 values, bf16: 8 values rounded RNE).
template <int DTYPE>
__device__ __forceinline__ void store_chunk(char* ptr, const float2* v) {
    if constexpr (DTYPE == 0) {
        *reinterpret_cast<float4*>(ptr) = make_float4(v[0].x, v[0].y, v[1].x, v[1].y);
    } else {
        uint4 u;
        __nv_bfloat162 a = __float22bfloat162_rn(v[0]);
        __nv_bfloat162 b = __float22bfloat162_rn(v[1]);
        __nv_bfloat162 c = __float22bfloat162_rn(v[2]);
        __nv_bfloat162 d = __float22bfloat162_rn(v[3]);
        u.x = *reinterpret_cast<uint32_t*>(&a);
        u.y = *reinterpret_cast<uint32_t*>(&b);
        u.z = *reinterpret_cast<uint32_t*>(&c);
        u.w = *reinterpret_cast<uint32_t*>(&d);
        *reinterpret_cast<uint4*>(ptr) = u;
    }
}

// Two outputs at once: blend of the two source rows, truncation to the 8-bit code and
// normalization, each lane rounded exactly like the scalar sequence
//   v = a*(1-dy) + b*dy;  code = floor(v);  out = (code*pre - mean) * inv_std.
// floor(v) for 0 <= v < 2^22 without a float->int->float round trip: adding 2^23 with
// round-toward-zero drops the fraction, subtracting it back is exact.  The CPU path's clamp
// to [0,255] before its uint8 cast cannot change the code: v is a convex blend of values in
// [0,255], so 0 <= v < 256 always.
__device__ __forceinline__ float2 finish2(float2 a, float2 b, float2 idy, float2 dy, float2 pre, float2 neg_mean,
                                          float2 istd, float2 one) {
    const float2 k = f2(8388608.0f, 8388608.0f), nk = f2(-8388608.0f, -8388608.0f);
    float2 v = add2_exact(mul2_rn(a, idy), mul2_rn(b, dy), one);
    v = add2_rn(add2_rz(v, k), nk);                                        // floor(v)
    return mul2_rn(add2_exact(mul2_rn(v, pre), neg_mean, one), istd);  // x - m == x + (-m) bit for bit
}

// Plain (release) arrival on an mbarrier.
__device__ __forceinline__ void mbar_arrive(uint32_t mbar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar) : "memory");
}

// Everything the planner warp needs to plan a pass and issue its copies.
struct PassCtx {
    int ty0, ty1, iw, cx, cy, fx_lo, fw, Rr, Rh, pitch, rpi;
    bool pairs;  // vertical downscale steeper than 2x: output rows share no source row
    const unsigned char* img;
    unsigned long long reg_lo, reg_hi;
};

// Planner state carried from one pass to the next (uniform across the warp).
struct PassState {
    int yb;           // first output row of the next pass to plan
    int staged_last;  // last source row already present in the strips' rings (contiguous mode), or -1
    int index;        // number of passes planned so far
};

// Executed by all 32 lanes of the planner warp.  Plans the pass that starts at output row st.yb
// from the per-tile row table: one lane per output row; the first row's y0 and the last row's
// y1 are exchanged with warp shuffles to find the range of NEW source rows.  Writes the pass
// record into slot (index % kSlots) of the header and issues one bulk copy per new source row
// into raw buffer (index % kNBuf), completing on that buffer's "full" mbarrier.
__device__ __forceinline__ void plan_and_issue(const PassCtx& c, PassState& st, unsigned char* smem,
                                               unsigned char* raw, int lane) {
    const int slot3 = st.index % kSlots, buf = st.index % kNBuf;
    int4* meta = reinterpret_cast<int4*>(smem + kSmemMeta);
    int2* rowoff = reinterpret_cast<int2*>(smem + kSmemRowOff) + slot3 * 32;
    const int2* rowy = reinterpret_cast<const int2*>(smem + kSmemRowY);
    unsigned char* rawbuf = raw + buf * c.Rr * c.pitch;
    const uint32_t mbar = smem_addr(smem + kSmemFull + 8 * buf);
    const int yb = st.yb;

    const int y = yb + lane;
    const bool valid = y < c.ty1;
    const int2 yy = rowy[min(y, c.ty1 - 1) - c.ty0];  // {y0, y1} of this lane's output row
    int nrows, nnew, new_first = 0;
    if (c.pairs) {
        nrows = min(c.Rr >> 1, min(c.ty1 - yb, 32));
        if (nrows > c.rpi) nrows -= nrows % c.rpi;
        nnew = 2 * nrows;
    } else {
        const int first = __shfl_sync(0xffffffffu, yy.x, 0);
        new_first = max(first, st.staged_last + 1);
        // Output rows whose source rows fit among the Rr rows this pass may add form a prefix
        // (y1 is non-decreasing in y).
        const unsigned fits = __ballot_sync(0xffffffffu, valid && (yy.y - new_first + 1 <= c.Rr));
        nrows = __popc(fits);
        // Whole groups of `rpi` rows keep every lane of the V step busy; the tile's tail is exempt.
        if (nrows > c.rpi && yb + nrows < c.ty1) nrows -= nrows % c.rpi;
        const int last_y1 = __shfl_sync(0xffffffffu, yy.y, nrows - 1);
        nnew = max(last_y1 - new_first + 1, 0);
        st.staged_last = max(st.staged_last, last_y1);
    }
    const int ynext = yb + nrows;
    if (lane == 0) meta[slot3] = make_int4(nrows, nnew, ynext >= c.ty1 ? 1 : 0, yb);
    const int j = lane;  // new source row staged by this lane
    const int ya = __shfl_sync(0xffffffffu, yy.x, j >> 1);
    const int yc = __shfl_sync(0xffffffffu, yy.y, j >> 1);
    const int srow = c.pairs ? ((j & 1) ? yc : ya) : (new_first + j);
    // Ring position of a source row: its row number (contiguous mode) or its sequence number
    // 2*(y - ty0) + {0,1} (pairs mode), modulo the ring depth -- the same rule the row table uses.
    const int q0 = (c.pairs ? 2 * (yb - c.ty0) : new_first) % c.Rh;  // uniform
    int q = q0 + j;
    if (q >= c.Rh) q -= c.Rh;  // j < Rr < Rh
    unsigned bytes = 0;
    unsigned long long lo = 0, a0 = 0, a1 = 0, hi = 0;
    if (j < nnew) {
        const unsigned off = (static_cast<unsigned>(c.cy + srow) * c.iw + (c.cx + c.fx_lo)) * 3u;
        a0 = reinterpret_cast<unsigned long long>(c.img) + off;
        a1 = a0 + static_cast<unsigned>(c.fw) * 3u;
        lo = a0 & ~15ull;
        if (lo < c.reg_lo) lo += 16;               // region does not start on the 16-byte grid
        hi = (a1 + 15ull) & ~15ull;
        if (hi > c.reg_hi) hi = c.reg_hi & ~15ull;  // region does not end on the 16-byte grid
        bytes = hi > lo ? static_cast<unsigned>(hi - lo) : 0u;
        rowoff[j] = make_int2(j * c.pitch + static_cast<int>(a0 & 15ull), q * kStripRowBytes);
        // Ragged edges outside the 16-byte grid of the readable region (rare): plain loads, stored
        // before the arrival below so that the "full" barrier publishes them too.
        unsigned char* slot = rawbuf + j * c.pitch;
        const unsigned long long origin = a0 & ~15ull;  // global address of slot byte 0
        const unsigned long long head_end = bytes ? lo : a1;
        for (unsigned long long a = a0; a < head_end && a < a1; ++a)
            slot[a - origin] = *reinterpret_cast<const unsigned char*>(a);
        if (bytes)
            for (unsigned long long a = (hi > a0 ? hi : a0); a < a1; ++a)
                slot[a - origin] = *reinterpret_cast<const unsigned char*>(a);
    }
    unsigned total = bytes;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    fence_proxy_async();  // earlier generic reads of this staging buffer precede the new copies
    __syncwarp();         // the record and the row offsets are written before the arrival publishes them
    if (lane == 0) mbar_arrive_expect_tx(mbar, total);
    __syncwarp();
    if (j < nnew) {
        unsigned char* slot = rawbuf + j * c.pitch;
        const unsigned long long origin = a0 & ~15ull;  // global address of slot byte 0
        if (bytes) bulk_copy_g2s(smem_addr(slot + (lo - origin)), reinterpret_cast<const void*>(lo), bytes, mbar);
    }
    st.yb = ynext;
    st.index += 1;
}

template <int DTYPE, int LAYOUT>
__global__ void __launch_bounds__(32 * (kMaxTileCols / kStripCols + 1))
fused_transform_kernel(const __grid_constant__ FusedParams p) {
    constexpr int V = OutT<DTYPE>::V;       // outputs per 16-byte chunk
    constexpr int G = kStripCols / V;       // pixel groups per strip row (8 fp32, 4 bf16)
    constexpr int RPI = 32 / G;             // output rows one V step covers (4 fp32, 8 bf16)
    constexpr int ESZ = DTYPE == 0 ? 4 : 2;
    extern __shared__ __align__(128) unsigned char smem[];
    const Plan& pl = p.plan;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int strips = pl.strips;

    // A batch never reads what the previous launch of this kernel wrote, so the next launch in the
    // stream may start filling SMs as soon as every CTA of this one has been scheduled.  Only a
    // launch made with programmatic stream serialization reacts to this; otherwise it is a no-op.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- which tile of which sample ------------------------------------------------
    unsigned bid = blockIdx.x;
    const int ct = static_cast<int>(bid % static_cast<unsigned>(pl.n_col_tiles));
    bid /= static_cast<unsigned>(pl.n_col_tiles);
    const int rt = static_cast<int>(bid % static_cast<unsigned>(pl.n_row_tiles));
    const int k = static_cast<int>(bid / static_cast<unsigned>(pl.n_row_tiles));

    const int W = p.dst_w, H = p.dst_h;
    const int ty0 = rt * pl.tile_rows;
    const int ty1 = min(ty0 + pl.tile_rows, H);
    const int tx0 = ct * pl.tile_cols;
    const int tcw = min(pl.tile_cols, W - tx0);

    // ---- per-sample parameters (uniform across the CTA) -----------------------------
    const long long s = p.sel ? p.sel[k] : static_cast<long long>(k);
    unsigned bad = 0;
    if (s < 0 || s >= p.n_src) bad = kDevBadIndex;
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
            bad = kDevBadBox;
    }
    const bool flip = p.flips ? (p.flips[k] != 0) : false;

    if (rt == 0 && ct == 0 && tid == 0) {
        if (p.out_indices) p.out_indices[k] = s;
        if (p.labels_out) p.labels_out[k] = (bad & kDevBadIndex) || !p.labels_in ? -1 : p.labels_in[s];
    }

    const float xscale = __fdiv_rn(static_cast<float>(cw), static_cast<float>(W > 0 ? W : 1));
    const float yscale = __fdiv_rn(static_cast<float>(ch), static_cast<float>(H > 0 ? H : 1));
    // Source-column footprint of the tile: resized columns [oxa, oxb] (mirrored when flipped).
    const int oxa = flip ? (W - 1 - (tx0 + tcw - 1)) : tx0;
    const int oxb = flip ? (W - 1 - tx0) : (tx0 + tcw - 1);
    int fx_lo = 0, fw = 0, own_pitch = 16, Rr = 0;
    if (!bad) {
        fx_lo = min(static_cast<int>(src_coord(oxa, xscale)), cw - 1);
        const int hi0 = min(static_cast<int>(src_coord(oxb, xscale)), cw - 1);
        const int fx_hi = min(hi0 + 1, cw - 1);
        fw = fx_hi - fx_lo + 1;
        own_pitch = (fw * 3 + 30 + 15) & ~15;
        Rr = raw_rows_for(pl.smem_bytes - kSmemVar, own_pitch, strips);
        if (Rr < 2) bad = kDevTooWide;
    }

    if (bad) {
        // Defined behaviour for an invalid sample: zero-fill its tile, report, never trap.
        if (tid == 0 && p.status) atomicOr(p.status, bad);
        const int rows = ty1 - ty0;
        for (int i = tid; i < rows * tcw * 3; i += blockDim.x) {
            const int c = i % 3, x = (i / 3) % tcw, y = i / (3 * tcw);
            long long idx;
            if constexpr (LAYOUT == 0)
                idx = ((static_cast<long long>(k) * 3 + c) * H + (ty0 + y)) * W + tx0 + x;
            else
                idx = ((static_cast<long long>(k) * H + (ty0 + y)) * W + tx0 + x) * 3 + c;
            store_scalar<DTYPE>(p.out, idx, 0.0f);
        }
        return;
    }

    // ---- carve the variable part of shared memory for this tile's footprint ----------
    const int Rh = Rr + 2;  // ring depth: the new rows of a pass plus at most two carried rows
    unsigned char* raw = smem + kSmemVar;                    // kNBuf buffers of Rr x own_pitch bytes
    unsigned char* rings = raw + kNBuf * Rr * own_pitch;    // strips x Rh x kStripRowBytes
    const int4* meta = reinterpret_cast<const int4*>(smem + kSmemMeta);

    if (tid == 0) {
        for (int b = 0; b < kNBuf; ++b) {
            mbar_init(smem_addr(smem + kSmemFull + 8 * b), 1);
            mbar_init(smem_addr(smem + kSmemEmpty + 8 * b), strips);
        }
        fence_proxy_async();
    }
    // ---- row table of the tile: one thread per output row, once ------------------------
    const bool pairs = ch > 2 * H;  // steeper than 2x: every output row has its own two source rows
    if (tid < ty1 - ty0) {
        const int y = ty0 + tid;
        const float sy = src_coord(y, yscale);
        const int y0 = min(static_cast<int>(sy), ch - 1);
        const int y1 = min(y0 + 1, ch - 1);
        const float dy = __fsub_rn(sy, static_cast<float>(y0));
        // Ring slot of a source row: row number (or, in pairs mode, sequence number) modulo Rh.
        const int q0 = pairs ? 2 * tid : y0;
        const int q1 = pairs ? 2 * tid + 1 : y1;
        reinterpret_cast<float4*>(smem + kSmemRowp)[tid] =
            make_float4(__int_as_float((q0 % Rh) * kStripRowBytes), __int_as_float((q1 % Rh) * kStripRowBytes), dy,
                        __fsub_rn(1.0f, dy));
        reinterpret_cast<int2*>(smem + kSmemRowY)[tid] = make_int2(y0, y1);
    }
    __syncthreads();  // the only CTA-wide barrier: tables and mbarriers are ready

    if (warp == strips) {
        // ================= planner warp =================================================================
        PassCtx pc;
        pc.ty0 = ty0; pc.ty1 = ty1; pc.iw = iw; pc.cx = cx; pc.cy = cy;
        pc.fx_lo = fx_lo; pc.fw = fw; pc.Rr = Rr; pc.Rh = Rh; pc.pitch = own_pitch; pc.rpi = RPI;
        pc.pairs = pairs;
        pc.img = p.src + img_off;
        pc.reg_lo = reinterpret_cast<unsigned long long>(p.src);
        pc.reg_hi = pc.reg_lo + p.src_bytes;
        PassState st;
        st.yb = ty0; st.staged_last = -1; st.index = 0;
        for (int n = 0; n < kNBuf && st.yb < ty1; ++n) plan_and_issue(pc, st, smem, raw, lane);  // passes 0 .. kNBuf-1
        while (st.yb < ty1) {
            // Pass n reuses the raw buffer of pass n - kNBuf: wait until every compute warp has
            // finished reading that buffer.
            const int n = st.index;
            const uint32_t mb = smem_addr(smem + kSmemEmpty + 8 * (n % kNBuf));
            if (!mbar_wait_bounded(mb, static_cast<uint32_t>(n / kNBuf - 1) & 1u)) {
                if (lane == 0 && p.status) atomicOr(p.status, kDevCopyTimeout);
            }
            plan_and_issue(pc, st, smem, raw, lane);
        }
        return;
    }

    // ================= compute warps: one 32-column strip each ===========================================
    unsigned char* ring = rings + warp * Rh * kStripRowBytes;
    // ---- H step ownership: one output column per lane, weights in registers ---------
    const int hx = warp * kStripCols + lane;  // column inside the tile
    int off0 = 0, off1 = 0;
    float2 wx = f2(0.0f, 0.0f);                // (1-dx, dx)
    const bool h_active = hx < tcw;
    if (h_active) {
        const int x = tx0 + hx;
        const int ox = flip ? (W - 1 - x) : x;
        const float sx = src_coord(ox, xscale);
        const int x0 = min(static_cast<int>(sx), cw - 1);
        const int x1 = min(x0 + 1, cw - 1);
        const float dx = __fsub_rn(sx, static_cast<float>(x0));
        off0 = (x0 - fx_lo) * 3;
        off1 = (x1 - fx_lo) * 3;
        wx = f2(__fsub_rn(1.0f, dx), dx);
    }
    const float2 nwx = f2(__fmul_rn(-8388608.0f, wx.x), __fmul_rn(-8388608.0f, wx.y));
    // Ring row layout.  NCHW: three planes of 32 floats.  NHWC: 32 x 3 interleaved floats.
    float* const h_store = reinterpret_cast<float*>(ring) + (LAYOUT == 0 ? lane : 3 * lane);
    // ---- V step ownership: V adjacent pixels x RPI rows per step ------------------------
    const int vg = lane % G;
    const int vr = lane / G;
    const int px0 = warp * kStripCols + vg * V;  // first pixel of the group inside the tile
    const bool v_active = px0 < tcw;
    const bool v_full = pl.vec_ok && (px0 + V <= tcw);
    const float2 pre2 = f2(p.pre_scale, p.pre_scale);
    const float2 one2 = f2(p.one, p.one);
    long long obase;                              // element index of (row 0, this group) of the sample
    if constexpr (LAYOUT == 0)
        obase = static_cast<long long>(k) * 3 * H * W + tx0 + px0;
    else
        obase = (static_cast<long long>(k) * H * W + tx0 + px0) * 3;
    // Byte offset of this group's first 16-byte chunk inside a ring row (plane 0 for NCHW).
    const unsigned char* const h_load = ring + (LAYOUT == 0 ? vg * V * 4 : vg * V * 12);
    void* const outp = p.out;
    char* const obytes = static_cast<char*>(p.out) + obase * ESZ;
    const long long row_bytes = static_cast<long long>(W) * ESZ * (LAYOUT == 0 ? 1 : 3);
    const long long chan_bytes = static_cast<long long>(H) * W * ESZ;  // NCHW plane stride
    const float4* const rowp_tile = reinterpret_cast<const float4*>(smem + kSmemRowp);

    // One 16-byte chunk q of an output row: blend the two ring rows ra / rb, truncate, normalize.
    // NCHW: chunk q = channel q of the group's V pixels.  NHWC: chunk q = elements [q*V, q*V+V) of
    // the group's 3V interleaved elements (element e has channel e % 3).
    auto chunk = [&](const unsigned char* ra, const unsigned char* rb, float2 idy2, float2 dy2, auto qc, float2* v) {
        constexpr int q = decltype(qc)::value;
#pragma unroll
        for (int i = 0; i < V / 4; ++i) {
            constexpr int base = LAYOUT == 0 ? q * kStripCols * 4 : q * V * 4;
            const float4 a = *reinterpret_cast<const float4*>(ra + base + 16 * i);
            const float4 b = *reinterpret_cast<const float4*>(rb + base + 16 * i);
            const int c0 = LAYOUT == 0 ? q : (q * V + 4 * i + 0) % 3;
            const int c1 = LAYOUT == 0 ? q : (q * V + 4 * i + 1) % 3;
            const int c2 = LAYOUT == 0 ? q : (q * V + 4 * i + 2) % 3;
            const int c3 = LAYOUT == 0 ? q : (q * V + 4 * i + 3) % 3;
            v[2 * i] = finish2(f2(a.x, a.y), f2(b.x, b.y), idy2, dy2, pre2, f2(-p.mean[c0], -p.mean[c1]),
                               f2(p.inv_std[c0], p.inv_std[c1]), one2);
            v[2 * i + 1] = finish2(f2(a.z, a.w), f2(b.z, b.w), idy2, dy2, pre2, f2(-p.mean[c2], -p.mean[c3]),
                                   f2(p.inv_std[c2], p.inv_std[c3]), one2);
        }
    };

    for (int i = 0;; ++i) {
        // ---- wait for the raw rows of pass i ---------------------------------------------
        const int b = i % kNBuf;
        const uint32_t full = smem_addr(smem + kSmemFull + 8 * b);
        const uint32_t full_parity = static_cast<uint32_t>(i / kNBuf) & 1u;
        if (!mbar_wait_bounded(full, full_parity)) {
            // The copies did not land within the time limit.  Report it and give them one more
            // bounded chance; the warp then carries on (every later wait is bounded too).  The
            // status word marks the output invalid.
            if (lane == 0 && p.status) atomicOr(p.status, kDevCopyTimeout);
            mbar_wait_bounded(full, full_parity);
        }
        const int4 m = meta[i % kSlots];  // {output rows, new source rows, last?, first output row}

        // ---- H step: new source rows -> horizontally interpolated fp32 in the strip's ring ----
        if (h_active) {
            const unsigned char* rawb = raw + b * Rr * own_pitch;
            const int2* rowoff = reinterpret_cast<const int2*>(smem + kSmemRowOff) + (i % kSlots) * 32;
#pragma unroll kHUnroll
            for (int j = 0; j < m.y; ++j) {
                const int2 ro = rowoff[j];  // {raw byte offset of the row, byte offset of its ring slot}
                const unsigned char* q0 = rawb + off0 + ro.x;
                const unsigned char* q1 = rawb + off1 + ro.x;
                const float2 t0 = byte_product2(q0[0], q1[0], wx, nwx);
                const float2 t1 = byte_product2(q0[1], q1[1], wx, nwx);
                const float2 t2 = byte_product2(q0[2], q1[2], wx, nwx);
                float* h = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(h_store) + ro.y);
                if constexpr (LAYOUT == 0) {
                    h[0] = __fadd_rn(t0.x, t0.y);
                    h[kStripCols] = __fadd_rn(t1.x, t1.y);
                    h[2 * kStripCols] = __fadd_rn(t2.x, t2.y);
                } else {
                    h[0] = __fadd_rn(t0.x, t0.y);
                    h[1] = __fadd_rn(t1.x, t1.y);
                    h[2] = __fadd_rn(t2.x, t2.y);
                }
            }
        }
        __syncwarp();  // the strip's new h rows are visible to the whole warp; raw reads are done
        if (lane == 0) mbar_arrive(smem_addr(smem + kSmemEmpty + 8 * b));  // this warp is done with raw buffer b

        // ---- V step: blend, truncate, normalize, store --------------------------------------
        if (v_active) {
            const float4* rowp = rowp_tile + (m.w - ty0);
            if (v_full) {
                char* orow = obytes + (m.w + vr) * row_bytes;
                const long long ostep = RPI * row_bytes;
                for (int l = vr; l < m.x; l += RPI, orow += ostep) {
                    const float4 rp = rowp[l];  // {ring byte offset of y0 row, of y1 row, dy, 1-dy}
                    const float2 dy2 = f2(rp.z, rp.z), idy2 = f2(rp.w, rp.w);
                    const unsigned char* ra = h_load + __float_as_int(rp.x);
                    const unsigned char* rb = h_load + __float_as_int(rp.y);
                    float2 v[V / 2];
                    chunk(ra, rb, idy2, dy2, std::integral_constant<int, 0>{}, v);
                    store_chunk<DTYPE>(orow, v);
                    chunk(ra, rb, idy2, dy2, std::integral_constant<int, 1>{}, v);
                    store_chunk<DTYPE>(orow + (LAYOUT == 0 ? chan_bytes : 16), v);
                    chunk(ra, rb, idy2, dy2, std::integral_constant<int, 2>{}, v);
                    store_chunk<DTYPE>(orow + (LAYOUT == 0 ? 2 * chan_bytes : 32), v);
                }
            } else {
                // Ragged or unaligned rows: element-wise guarded stores.
                for (int l = vr; l < m.x; l += RPI) {
                    const float4 rp = rowp[l];
                    const float2 dy2 = f2(rp.z, rp.z), idy2 = f2(rp.w, rp.w);
                    const unsigned char* ra = h_load + __float_as_int(rp.x);
                    const unsigned char* rb = h_load + __float_as_int(rp.y);
                    const int y = m.w + l;
                    auto emit = [&](auto qc) {
                        constexpr int q = decltype(qc)::value;
                        float2 v[V / 2];
                        chunk(ra, rb, idy2, dy2, qc, v);
                        long long idx;
                        if constexpr (LAYOUT == 0)
                            idx = obase + static_cast<long long>((q * H + y) * W);
                        else
                            idx = obase + static_cast<long long>(y) * W * 3 + q * V;
#pragma unroll
                        for (int e = 0; e < V; ++e) {
                            const float val = (e & 1) ? v[e >> 1].y : v[e >> 1].x;
                            const bool in = LAYOUT == 0 ? (px0 + e < tcw) : (3 * px0 + q * V + e < 3 * tcw);
                            if (in) store_scalar<DTYPE>(outp, idx + e, val);
                        }
                    };
                    emit(std::integral_constant<int, 0>{});
                    emit(std::integral_constant<int, 1>{});
                    emit(std::integral_constant<int, 2>{});
                }
            }
        }
        if (m.z) break;
        __syncwarp();  // every lane has consumed pass i before the ring slots are rewritten
    }
}

std::atomic<unsigned long long> g_launches{0};
std::atomic<int> g_overlap{0};

template <int DTYPE, int LAYOUT>
int launch_one(const FusedParams& p, cudaStream_t st, bool may_overlap) {
    auto kern = fused_transform_kernel<DTYPE, LAYOUT>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(p.plan.grid));
    cfg.blockDim = dim3(32 * (p.plan.strips + 1));
    cfg.dynamicSmemBytes = static_cast<size_t>(p.plan.smem_bytes);
    cfg.stream = st;
    // Programmatic stream serialization: when the work directly before this launch in the stream
    // is a launch of this same kernel (which signals early, see the top of the kernel), this one
    // may begin while that one drains its last CTAs; the head and tail of back-to-back batches
    // then overlap instead of leaving SMs idle.  Behind a copy, a memset or a kernel that does not
    // signal early the usual stream order holds.  The caller opts in (tlb_set_launch_overlap)
    // because the kernel does not wait on its predecessor: see the header for the condition.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (may_overlap && g_overlap.load(std::memory_order_relaxed)) ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kern, p);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return static_cast<int>(cudaGetLastError());
}

template <int DTYPE, int LAYOUT>
int opt_in_smem() {
    return static_cast<int>(cudaFuncSetAttribute(fused_transform_kernel<DTYPE, LAYOUT>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
}

}  // namespace

int prepare_device() {
    int e = opt_in_smem<0, 0>();
    if (!e) e = opt_in_smem<0, 1>();
    if (!e) e = opt_in_smem<1, 0>();
    if (!e) e = opt_in_smem<1, 1>();
    return e;
}

int launch_fused(const FusedParams& p, int out_dtype, int out_layout, void* stream, bool may_overlap) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (out_dtype == 0) return out_layout == 0 ? launch_one<0, 0>(p, st, may_overlap) : launch_one<0, 1>(p, st, may_overlap);
    return out_layout == 0 ? launch_one<1, 0>(p, st, may_overlap) : launch_one<1, 1>(p, st, may_overlap);
}

int set_launch_overlap(int enable) { return g_overlap.exchange(enable ? 1 : 0, std::memory_order_relaxed); }

unsigned long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

}  // namespace tlb
