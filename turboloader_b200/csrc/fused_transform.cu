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
// Structure of one CTA = one tile of `tile_rows` x `tile_cols` outputs of one sample,
// processed in passes of at most R staged source rows (R is what fits in shared memory
// for this tile's own footprint width):
//   1. warp 0 plans the pass: one lane per output row computes (y0, y1, dy); the first and
//      last rows are exchanged with warp shuffles to find the contiguous range of source
//      rows (or, for a >2x vertical downscale, the exact (y0, y1) pairs).  It then issues
//      one 1-D bulk async copy (cp.async.bulk, global -> this CTA's shared memory,
//      completion on an mbarrier) per source row, each rounded out to 16-byte boundaries.
//      Bytes that cannot be reached on a 16-byte grid inside the readable region are
//      fetched with plain loads.  Raw rows are double buffered: the copies of pass i+1
//      are in flight while pass i is computed.
//   2. "H" phase: every staged row is interpolated horizontally once,
//      h = p[x0]*(1-dx) + p[x1]*dx, into fp32 in shared memory.  Each thread owns one
//      output column for the whole tile and keeps its weights in registers.
//   3. "V" phase: each thread owns a group of 4 (fp32) or 8 (bf16) adjacent pixels and
//      walks down the rows of the pass: v = h[y0]*(1-dy) + h[y1]*dy, truncate, normalize,
//      cast, three 16-byte stores per row.  The layout of h in shared memory (planar for
//      NCHW, interleaved for NHWC) makes every input a 16-byte shared load.  The fp32
//      arithmetic uses the packed two-lane forms (mul/add .f32x2) of sm_100; they round
//      each lane exactly like the scalar instructions.
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

#include "fused_params.h"

namespace tlb {
namespace {

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
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t mbar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(mbar), "r"(parity)
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
// Sum of two packed products, lane by lane, with scalar adds (see the caution above).
__device__ __forceinline__ float2 add2_of_products(float2 a, float2 b) {
    return f2(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y));
}

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

// One 16-byte store of V consecutive output elements starting at element index idx.
template <int DTYPE>
__device__ __forceinline__ void store_chunk(void* out, long long idx, const float2* v) {
    if constexpr (DTYPE == 0) {
        *reinterpret_cast<float4*>(static_cast<float*>(out) + idx) = make_float4(v[0].x, v[0].y, v[1].x, v[1].y);
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
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out) + idx) = u;
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
                                          float2 istd) {
    const float2 k = f2(8388608.0f, 8388608.0f), nk = f2(-8388608.0f, -8388608.0f);
    float2 v = add2_of_products(mul2_rn(a, idy), mul2_rn(b, dy));
    v = add2_rn(add2_rz(v, k), nk);                                          // floor(v)
    return mul2_rn(add2_of_products(mul2_rn(v, pre), neg_mean), istd);  // x - m == x + (-m) bit for bit
}

// Everything warp 0 needs to plan a pass and issue its copies.
struct PassCtx {
    int ty1, H, ch, iw, cx, cy, fx_lo, fw, R, pitch, hp;
    float yscale;
    const unsigned char* img;
    unsigned long long reg_lo, reg_hi;
};

// Executed by all 32 lanes of warp 0.  Plans the pass that starts at output row yb, writes
// its row tables into the `buf` half of the header and issues the bulk copies into rawbuf.
__device__ __forceinline__ void plan_and_issue(const PassCtx& c, int yb, int buf, unsigned char* smem,
                                               unsigned char* rawbuf, int lane) {
    int4* meta = reinterpret_cast<int4*>(smem + kSmemMeta);
    float4* rowp = reinterpret_cast<float4*>(smem + kSmemRowp) + buf * 32;
    int* rowoff = reinterpret_cast<int*>(smem + kSmemRowOff) + buf * 32;
    const uint32_t mbar = smem_addr(smem + kSmemMbar + 8 * buf);

    const int y = yb + lane;
    const float sy = src_coord(min(y, c.H - 1), c.yscale);
    const int y0 = min(static_cast<int>(sy), c.ch - 1);
    const int y1 = min(y0 + 1, c.ch - 1);
    const float dy = __fsub_rn(sy, static_cast<float>(y0));
    const int first = __shfl_sync(0xffffffffu, y0, 0);
    // Contiguous staging: source rows first .. y1 of the last output row that still fits in R.
    const unsigned fits = __ballot_sync(0xffffffffu, (y < c.ty1) && (y1 - first + 1 <= c.R));
    int nrows = __popc(fits);  // the fitting rows form a prefix: y1 is non-decreasing in y
    const int npair = min(c.R >> 1, c.ty1 - yb);
    const bool pairs = nrows < npair;  // steep downscale: stage exactly (y0, y1) per output row
    if (pairs) nrows = npair;
    const int last_y1 = __shfl_sync(0xffffffffu, y1, nrows - 1);
    const int nstaged = pairs ? 2 * nrows : (last_y1 - first + 1);
    if (lane == 0) meta[buf] = make_int4(nrows, nstaged, 0, 0);
    if (lane < nrows) {
        const int s0 = pairs ? 2 * lane : (y0 - first);
        const int s1 = pairs ? 2 * lane + 1 : (y1 - first);
        rowp[lane] = make_float4(__int_as_float(s0 * c.hp), __int_as_float(s1 * c.hp), dy, __fsub_rn(1.0f, dy));
    }
    const int j = lane;  // slot staged by this lane
    const int ya = __shfl_sync(0xffffffffu, y0, j >> 1);
    const int yc = __shfl_sync(0xffffffffu, y1, j >> 1);
    const int srow = pairs ? ((j & 1) ? yc : ya) : (first + j);
    unsigned bytes = 0;
    unsigned long long lo = 0, a0 = 0, a1 = 0, hi = 0;
    if (j < nstaged) {
        a0 = reinterpret_cast<unsigned long long>(c.img) +
             (static_cast<unsigned long long>(c.cy + srow) * c.iw + (c.cx + c.fx_lo)) * 3ull;
        a1 = a0 + static_cast<unsigned long long>(c.fw) * 3ull;
        lo = a0 & ~15ull;
        if (lo < c.reg_lo) lo += 16;               // region does not start on the 16-byte grid
        hi = (a1 + 15ull) & ~15ull;
        if (hi > c.reg_hi) hi = c.reg_hi & ~15ull;  // region does not end on the 16-byte grid
        bytes = hi > lo ? static_cast<unsigned>(hi - lo) : 0u;
        rowoff[j] = j * c.pitch + static_cast<int>(a0 & 15ull);
    }
    unsigned total = bytes;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    fence_proxy_async();  // earlier generic reads of this staging buffer precede the new copies
    if (lane == 0) mbar_arrive_expect_tx(mbar, total);
    __syncwarp();
    if (j < nstaged) {
        unsigned char* slot = rawbuf + j * c.pitch;
        const unsigned long long origin = a0 & ~15ull;  // global address of slot byte 0
        if (bytes) bulk_copy_g2s(smem_addr(slot + (lo - origin)), reinterpret_cast<const void*>(lo), bytes, mbar);
        // Ragged edges outside the 16-byte grid of the readable region (rare).
        const unsigned long long head_end = bytes ? lo : a1;
        for (unsigned long long a = a0; a < head_end && a < a1; ++a)
            slot[a - origin] = *reinterpret_cast<const unsigned char*>(a);
        if (bytes)
            for (unsigned long long a = (hi > a0 ? hi : a0); a < a1; ++a)
                slot[a - origin] = *reinterpret_cast<const unsigned char*>(a);
    }
}

template <int DTYPE, int LAYOUT>
__global__ void __launch_bounds__(kMaxThreads, 3) fused_transform_kernel(const __grid_constant__ FusedParams p) {
    constexpr int V = OutT<DTYPE>::V;
    extern __shared__ __align__(128) unsigned char smem[];
    const Plan& pl = p.plan;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;

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
            img_off < 0 || static_cast<unsigned long long>(img_off) + img_bytes > p.src_bytes)
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
    int fx_lo = 0, fw = 0, own_pitch = 16, R = 0;
    const int var_bytes = pl.smem_bytes - kSmemVar;
    if (!bad) {
        fx_lo = min(static_cast<int>(src_coord(oxa, xscale)), cw - 1);
        const int hi0 = min(static_cast<int>(src_coord(oxb, xscale)), cw - 1);
        const int fx_hi = min(hi0 + 1, cw - 1);
        fw = fx_hi - fx_lo + 1;
        own_pitch = (fw * 3 + 30 + 15) & ~15;
        R = staged_rows_for(var_bytes, own_pitch, pl.hpitch);
        if (R < 2) bad = kDevTooWide;
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
    const int hp = pl.hpitch, tcp = pl.tile_cols;
    unsigned char* raw0 = smem + kSmemVar;
    unsigned char* raw1 = raw0 + R * own_pitch;
    float* hbuf = reinterpret_cast<float*>(raw1 + R * own_pitch);
    const int4* meta = reinterpret_cast<const int4*>(smem + kSmemMeta);

    // ---- H-phase ownership: one output column per thread, weights in registers -------
    const int hx = tid % tcp;          // column inside the tile
    const int hg = tid / tcp;          // row group of this thread
    const int hgroups = blockDim.x / tcp;
    int off0 = 0, off1 = 0;
    float2 wx = f2(0.0f, 0.0f);        // (1-dx, dx)
    if (hx < tcw) {
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
    // ---- V-phase ownership: V adjacent pixels, three 16-byte chunks per row ------------
    const int gp = tcp / V;            // pixel groups per tile row
    const int vg = tid % gp;
    const int vr = tid / gp;
    const int vgroups = blockDim.x / gp;
    const int px0 = vg * V;            // first pixel of the group inside the tile
    const bool v_active = px0 < tcw;
    const bool v_full = pl.vec_ok && (px0 + V <= tcw);
    const float2 pre2 = f2(p.pre_scale, p.pre_scale);
    long long obase;                    // element index of (row 0, this group) of the sample
    if constexpr (LAYOUT == 0)
        obase = static_cast<long long>(k) * 3 * H * W + tx0 + px0;
    else
        obase = (static_cast<long long>(k) * H * W + tx0 + px0) * 3;

    if (tid == 0) {
        mbar_init(smem_addr(smem + kSmemMbar), 1);
        mbar_init(smem_addr(smem + kSmemMbar + 8), 1);
        fence_proxy_async();
    }
    __syncthreads();

    PassCtx pc;
    pc.ty1 = ty1; pc.H = H; pc.ch = ch; pc.iw = iw; pc.cx = cx; pc.cy = cy; pc.fx_lo = fx_lo; pc.fw = fw;
    pc.R = R; pc.pitch = own_pitch; pc.hp = hp; pc.yscale = yscale;
    pc.img = p.src + img_off;
    pc.reg_lo = reinterpret_cast<unsigned long long>(p.src);
    pc.reg_hi = pc.reg_lo + p.src_bytes;

    if (warp == 0) plan_and_issue(pc, ty0, 0, smem, raw0, lane);

    void* const outp = p.out;
    uint32_t phases = 0;  // bit b = parity to wait for on mbarrier b
    int buf = 0;
    for (int yb = ty0; yb < ty1;) {
        __syncthreads();  // tables of this pass visible; previous V phase done with hbuf and rowp[buf^1]
        const int4 m = meta[buf];
        const int nrows = m.x, nstaged = m.y;
        const int ynext = yb + nrows;
        unsigned char* rawbuf = buf ? raw1 : raw0;
        if (warp == 0 && ynext < ty1) plan_and_issue(pc, ynext, buf ^ 1, smem, buf ? raw0 : raw1, lane);
        const uint32_t mbar = smem_addr(smem + kSmemMbar + 8 * buf);
        if (!mbar_wait_bounded(mbar, (phases >> buf) & 1u)) {
            // The copies did not land within the polling limit.  Report it and give them one more
            // bounded chance; the CTA then carries on (every later wait is bounded too) so that no
            // thread leaves while others sit at a barrier.  The status word marks the output invalid.
            if (p.status) atomicOr(p.status, kDevCopyTimeout);
            mbar_wait_bounded(mbar, (phases >> buf) & 1u);
        }
        phases ^= 1u << buf;

        // ---- H phase: staged rows -> horizontally interpolated fp32 ---------------------
        if (hx < tcw) {
            const int* rowoff = reinterpret_cast<const int*>(smem + kSmemRowOff) + buf * 32;
            for (int j = hg; j < nstaged; j += hgroups) {
                const unsigned char* row = rawbuf + rowoff[j];
                const unsigned char* q0 = row + off0;
                const unsigned char* q1 = row + off1;
                const float2 t0 = mul2_rn(f2(static_cast<float>(q0[0]), static_cast<float>(q1[0])), wx);
                const float2 t1 = mul2_rn(f2(static_cast<float>(q0[1]), static_cast<float>(q1[1])), wx);
                const float2 t2 = mul2_rn(f2(static_cast<float>(q0[2]), static_cast<float>(q1[2])), wx);
                float* h = hbuf + j * hp;
                if constexpr (LAYOUT == 0) {
                    h[hx] = __fadd_rn(t0.x, t0.y);
                    h[tcp + hx] = __fadd_rn(t1.x, t1.y);
                    h[2 * tcp + hx] = __fadd_rn(t2.x, t2.y);
                } else {
                    h[3 * hx] = __fadd_rn(t0.x, t0.y);
                    h[3 * hx + 1] = __fadd_rn(t1.x, t1.y);
                    h[3 * hx + 2] = __fadd_rn(t2.x, t2.y);
                }
            }
        }
        __syncthreads();

        // ---- V phase --------------------------------------------------------------------
        if (v_active) {
            const float4* rowp = reinterpret_cast<const float4*>(smem + kSmemRowp) + buf * 32;
            for (int l = vr; l < nrows; l += vgroups) {
                const float4 rp = rowp[l];
                const float2 dy2 = f2(rp.z, rp.z), idy2 = f2(rp.w, rp.w);
                const int y = yb + l;
#pragma unroll
                for (int q = 0; q < 3; ++q) {
                    // NCHW: chunk q = channel q of the group's V pixels.  NHWC: chunk q = elements
                    // [q*V, q*V+V) of the group's 3V interleaved elements (element e has channel e % 3).
                    const int hoff = LAYOUT == 0 ? (q * tcp + px0) : (3 * px0 + q * V);
                    const float* ha = hbuf + __float_as_int(rp.x) + hoff;
                    const float* hb = hbuf + __float_as_int(rp.y) + hoff;
                    float2 v[V / 2];
#pragma unroll
                    for (int i = 0; i < V / 4; ++i) {
                        const float4 a = *reinterpret_cast<const float4*>(ha + 4 * i);
                        const float4 b = *reinterpret_cast<const float4*>(hb + 4 * i);
                        const int c0 = LAYOUT == 0 ? q : (q * V + 4 * i + 0) % 3;
                        const int c1 = LAYOUT == 0 ? q : (q * V + 4 * i + 1) % 3;
                        const int c2 = LAYOUT == 0 ? q : (q * V + 4 * i + 2) % 3;
                        const int c3 = LAYOUT == 0 ? q : (q * V + 4 * i + 3) % 3;
                        v[2 * i] = finish2(f2(a.x, a.y), f2(b.x, b.y), idy2, dy2, pre2, f2(-p.mean[c0], -p.mean[c1]),
                                           f2(p.inv_std[c0], p.inv_std[c1]));
                        v[2 * i + 1] = finish2(f2(a.z, a.w), f2(b.z, b.w), idy2, dy2, pre2,
                                               f2(-p.mean[c2], -p.mean[c3]), f2(p.inv_std[c2], p.inv_std[c3]));
                    }
                    long long idx;
                    if constexpr (LAYOUT == 0)
                        idx = obase + static_cast<long long>((q * H + y) * W);
                    else
                        idx = obase + static_cast<long long>(y) * W * 3 + q * V;
                    if (v_full) {
                        store_chunk<DTYPE>(outp, idx, v);
                    } else {
#pragma unroll
                        for (int i = 0; i < V; ++i) {
                            const float val = (i & 1) ? v[i >> 1].y : v[i >> 1].x;
                            const bool in = LAYOUT == 0 ? (px0 + i < tcw) : (3 * px0 + q * V + i < 3 * tcw);
                            if (in) store_scalar<DTYPE>(outp, idx + i, val);
                        }
                    }
                }
            }
        }
        yb = ynext;
        buf ^= 1;
    }
}

std::atomic<unsigned long long> g_launches{0};

template <int DTYPE, int LAYOUT>
int launch_one(const FusedParams& p, cudaStream_t st) {
    auto kern = fused_transform_kernel<DTYPE, LAYOUT>;
    kern<<<static_cast<unsigned>(p.plan.grid), p.plan.threads, p.plan.smem_bytes, st>>>(p);
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

int launch_fused(const FusedParams& p, int out_dtype, int out_layout, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (out_dtype == 0) return out_layout == 0 ? launch_one<0, 0>(p, st) : launch_one<0, 1>(p, st);
    return out_layout == 0 ? launch_one<1, 0>(p, st) : launch_one<1, 1>(p, st);
}

unsigned long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

}  // namespace tlb
