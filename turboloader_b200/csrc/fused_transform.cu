// Fused crop -> hflip -> bilinear resize -> (colour jitter) -> normalize -> layout/cast kernel
// for sm_100a.
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
// warp per strip of 32*CPL output columns computes; one more warp only plans and copies.  No
// CTA-wide barrier is used after the prologue: the warps meet through mbarriers only.
//   planner warp: walks down the tile in passes of at most Rr NEW source rows (rows the compute
//      warps have not consumed yet).  One lane per output row looks up (y0, y1) in a per-tile row
//      table; the first and last rows are exchanged with warp shuffles to find the range of new
//      rows.  It issues one 1-D bulk async copy (cp.async.bulk, global -> this CTA's shared
//      memory, completion on a "full" mbarrier) per new source row, each rounded out to 16-byte
//      boundaries; bytes that cannot be reached on a 16-byte grid inside the readable region are
//      fetched with plain loads.  kNBuf raw buffers let it run that many passes ahead; a buffer is
//      refilled once every compute warp has arrived on its "empty" mbarrier.
//   compute warp: each lane owns output columns c and c + 32 of the strip (CPL = 2; offsets and
//      weights of their source columns stay in registers) and walks DOWN the tile, consuming the
//      staged source rows in order.  It keeps the horizontally interpolated values
//      h = p[x0]*(1-dx) + p[x1]*dx of the two most recent source rows in two register buffers; a
//      new source row costs one "H step" (six byte loads per column from the staged row, into the
//      buffer that holds the older row), and every output row that is complete after it one
//      "V step": v = hA*wA + hB*wB, truncate, normalize, cast, store.  Nothing but the staged bytes
//      ever goes through shared memory: the blend is exactly separable in this order (top and bot
//      depend on one source row each), so reusing h between neighbouring output rows changes no
//      bit.  Across a warp each store covers 32 adjacent pixels.  The fp32 arithmetic uses the
//      packed two-lane forms (fma/mul/add .f32x2) of sm_100 with the two columns of a lane
//      (CPL = 2) or two channels (CPL = 1) in the two halves; they round each half exactly like
//      the scalar instructions.
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
// slots re-polling.
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
// Hardware named barriers (1..15) between the compute warps and the planner warp of one CTA: a
// compute warp signals "done with raw buffer b" without blocking, the planner blocks (issuing
// nothing) until all of them have.  Like __syncthreads, this waits only for warps of the same CTA,
// all of which always get there: their own waits on asynchronous copies are bounded.
// The barrier number is an immediate (one barrier per raw buffer): with a run-time number the
// compiler reserves all 16 barriers for the CTA, which caps the CTAs per SM.
__device__ __forceinline__ void named_arrive(int buf, int threads) {
    if (buf == 0)
        asm volatile("bar.arrive 1, %0;" ::"r"(threads) : "memory");
    else if (buf == 1)
        asm volatile("bar.arrive 2, %0;" ::"r"(threads) : "memory");
    else if (buf == 2)
        asm volatile("bar.arrive 3, %0;" ::"r"(threads) : "memory");
    else
        asm volatile("bar.arrive 4, %0;" ::"r"(threads) : "memory");
}
__device__ __forceinline__ void named_sync(int buf, int threads) {
    if (buf == 0)
        asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
    else if (buf == 1)
        asm volatile("bar.sync 2, %0;" ::"r"(threads) : "memory");
    else if (buf == 2)
        asm volatile("bar.sync 3, %0;" ::"r"(threads) : "memory");
    else
        asm volatile("bar.sync 4, %0;" ::"r"(threads) : "memory");
}
// Shared-memory loads by 32-bit shared-window address (no 64-bit generic pointer arithmetic in
// the inner loops).
template <int IMM>
__device__ __forceinline__ unsigned lds_u8(uint32_t addr) {
    unsigned v;
    asm volatile("ld.shared.u8 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(IMM));
    return v;
}
__device__ __forceinline__ float4 lds_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ int2 lds_i2(uint32_t addr) {
    int2 v;
    asm volatile("ld.shared.v2.s32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ int4 lds_i4(uint32_t addr) {
    int4 v;
    asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// simd_utils.hpp:100-103, with each operation rounded separately.
__device__ __forceinline__ float src_coord(int i, float scale) {
    float s = __fsub_rn(__fmul_rn(__fadd_rn(static_cast<float>(i), 0.5f), scale), 0.5f);
    return s < 0.0f ? 0.0f : s;
}

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

// Packed two-lane fp32 multiply / add of sm_100 (mul.f32x2, add.f32x2) with explicit rounding.
// Each half rounds like the scalar instruction.  CAUTION: the assembler was observed to
// contract a packed multiply feeding a packed add into one FMA even with explicit .rn and with
// fmad disabled (it flips ~1e-5 of the 8-bit codes and the last bit of most normalized
// values).  So wherever a product feeds a sum, the sum is issued through add2_exact below;
// the plain packed add is used only where no product is an input.
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
TLB_F32X2_OP(add2_rz, "add.rz.f32x2")
#undef TLB_F32X2_OP
// Packed FMA.  Used only where the fused result is exactly the wanted singly-rounded value
// (byte_product2, add2_exact).
__device__ __forceinline__ float2 fma2_rn(float2 a, float2 b, float2 c) {
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
// a*1 is exact, so the result is RN(a + b) half by half; and because the instruction already
// is an FMA whose multiplicand is a finished (rounded) product, nothing can be contracted
// into it.
__device__ __forceinline__ float2 add2_exact(float2 a, float2 b, float2 one) { return fma2_rn(a, one, b); }

// (x - mean) * inv_std for x = code*pre;  x - m == x + (-m) bit for bit.  floor(v) for 0 <= v < 2^22
// needs no float->int->float round trip: adding 2^23 with round-toward-zero drops the fraction.  The
// CPU path's clamp to [0,255] before its uint8 cast cannot change the code: v is a convex blend of
// values in [0,255], so 0 <= v < 256 always.
__device__ __forceinline__ float2 normalize2(float2 x, float2 neg_mean, float2 istd, float2 one) {
    return mul2_rn(add2_exact(x, neg_mean, one), istd);
}

template <int DTYPE>
__device__ __forceinline__ void store_scalar(void* out, long long idx, float v) {
    if constexpr (DTYPE == 0)
        static_cast<float*>(out)[idx] = v;
    else
        static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
}
template <int DTYPE>
__device__ __forceinline__ void store1(char* ptr, float v) {
    if constexpr (DTYPE == 0)
        *reinterpret_cast<float*>(ptr) = v;
    else
        *reinterpret_cast<__nv_bfloat16*>(ptr) = __float2bfloat16_rn(v);
}
// Everything the planner warp needs to plan a pass and issue its copies.
struct PassCtx {
    int ty0, ty1, iw, cx, cy, ch, fx_lo, fw, Rr, pitch;
    bool pairs;  // vertical downscale steeper than 2x: output rows share no source row
    const unsigned char* img;
    unsigned long long reg_lo, reg_hi;
};

// Planner state carried from one pass to the next (uniform across the warp).
struct PassState {
    int yb;           // first output row of the next pass to plan
    int staged_last;  // last virtual source row already handed to the compute warps (contiguous mode), or -1
    int index;        // number of passes planned so far
};

// Executed by all 32 lanes of the planner warp.  Plans the pass that starts at output row st.yb
// from the per-tile row table, one lane per output row.  Output row y blends source rows y0 and
// y0 + 1; row y0 + 1 may be the "virtual" row ch, which stands for a second copy of row ch - 1
// (the bottom clamp), so that every output row needs two consecutive rows and the compute warps
// need no special case.  In contiguous mode the virtual rows of a tile are staged consecutively,
// each exactly once; the first row's y0 and the last row's y0 + 1 are exchanged with warp
// shuffles to find the range of NEW rows.  The pass record {new rows, output rows to emit before
// the first new row, last pass?} goes to slot (index % kSlots) of the header, together with one
// record per new row {its byte offset in shared memory, output rows to emit once it has been
// consumed}; one bulk copy per new row goes into raw buffer (index % kNBuf), completing on that
// buffer's "full" mbarrier.
__device__ __forceinline__ void plan_and_issue(const PassCtx& c, PassState& st, unsigned char* smem, int lane) {
    const int slot = st.index % kSlots, buf = st.index % kNBuf;
    int4* meta = reinterpret_cast<int4*>(smem + kSmemMeta);
    int2* srcrec = reinterpret_cast<int2*>(smem + kSmemSrcRec) + slot * 32;
    const int* rowy = reinterpret_cast<const int*>(smem + kSmemRowY);
    const int buf_off = kSmemVar + buf * c.Rr * c.pitch;
    const uint32_t mbar = smem_addr(smem + kSmemFull + 8 * buf);
    const int yb = st.yb;

    const int y = yb + lane;
    const bool valid = y < c.ty1;
    const int y0 = rowy[min(y, c.ty1 - 1) - c.ty0];
    const int y1v = y0 + 1;  // second (possibly virtual) source row of this lane's output row
    int nrows, nnew, new_first = 0, jlast;
    if (c.pairs) {
        nrows = min(c.Rr >> 1, min(c.ty1 - yb, 32));
        nnew = 2 * nrows;
        jlast = 2 * lane + 1;
    } else {
        const int first = __shfl_sync(0xffffffffu, y0, 0);
        new_first = max(first, st.staged_last + 1);
        // Output rows whose rows fit among the Rr rows this pass may add form a prefix (y0 is
        // non-decreasing in y); the first row always fits (it needs at most two new rows).
        const unsigned fits = __ballot_sync(0xffffffffu, valid && (y1v - new_first + 1 <= c.Rr));
        nrows = __popc(fits);
        const int last_y1v = __shfl_sync(0xffffffffu, y1v, nrows - 1);
        nnew = max(last_y1v - new_first + 1, 0);
        st.staged_last = max(st.staged_last, last_y1v);
        jlast = y1v - new_first;  // negative: both rows were consumed in an earlier pass
    }
    const bool in_pass = lane < nrows;
    const unsigned pre_mask = __ballot_sync(0xffffffffu, in_pass && jlast < 0);
    const int ynext = yb + nrows;
    if (lane == 0) meta[slot] = make_int4(nnew, __popc(pre_mask), ynext >= c.ty1 ? 1 : 0, 0);
    // Output rows that become ready after new row j: lanes with the same jlast form a group.
    const unsigned grp = __match_any_sync(0xffffffffu, (in_pass && jlast >= 0) ? jlast : 64 + lane);

    const int j = lane;  // new source row staged by this lane
    const int ya = __shfl_sync(0xffffffffu, y0, j >> 1);
    const int srow = c.pairs ? ya + (j & 1) : min(new_first + j, c.ch - 1);
    unsigned bytes = 0;
    unsigned long long lo = 0, a0 = 0, a1 = 0, hi = 0;
    unsigned char* row = smem + buf_off + j * c.pitch;
    if (j < nnew) {
        const unsigned off = (static_cast<unsigned>(c.cy + srow) * c.iw + (c.cx + c.fx_lo)) * 3u;
        a0 = reinterpret_cast<unsigned long long>(c.img) + off;
        a1 = a0 + static_cast<unsigned>(c.fw) * 3u;
        lo = a0 & ~15ull;
        if (lo < c.reg_lo) lo += 16;               // region does not start on the 16-byte grid
        hi = (a1 + 15ull) & ~15ull;
        if (hi > c.reg_hi) hi = c.reg_hi & ~15ull;  // region does not end on the 16-byte grid
        bytes = hi > lo ? static_cast<unsigned>(hi - lo) : 0u;
        srcrec[j] = make_int2(buf_off + j * c.pitch + static_cast<int>(a0 & 15ull), 0);
        // Ragged edges outside the 16-byte grid of the readable region (rare): plain loads, stored
        // before the arrival below so that the "full" barrier publishes them too.
        const unsigned long long origin = a0 & ~15ull;  // global address of row byte 0
        const unsigned long long head_end = bytes ? lo : a1;
        for (unsigned long long a = a0; a < head_end && a < a1; ++a)
            row[a - origin] = *reinterpret_cast<const unsigned char*>(a);
        if (bytes)
            for (unsigned long long a = (hi > a0 ? hi : a0); a < a1; ++a)
                row[a - origin] = *reinterpret_cast<const unsigned char*>(a);
    }
    __syncwarp();  // the per-row records exist before the group leaders add their counts
    if (in_pass && jlast >= 0 && (__ffs(grp) - 1) == lane) srcrec[jlast].y = __popc(grp);
    unsigned total = bytes;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    fence_proxy_async();  // earlier generic reads of this staging buffer precede the new copies
    __syncwarp();         // the records are written before the arrival publishes them
    if (lane == 0) mbar_arrive_expect_tx(mbar, total);
    __syncwarp();
    if (j < nnew && bytes) {
        const unsigned long long origin = a0 & ~15ull;
        bulk_copy_g2s(smem_addr(row + (lo - origin)), reinterpret_cast<const void*>(lo), bytes, mbar);
    }
    st.yb = ynext;
    st.index += 1;
}

#ifndef TLB_MIN_CTAS
#define TLB_MIN_CTAS 3
#endif

template <int DTYPE, int LAYOUT, int CPL, bool JIT>
__global__ void __launch_bounds__(32 * (kMaxStrips + 1), TLB_MIN_CTAS)
fused_transform_kernel(const __grid_constant__ FusedParams p) {
    constexpr int ESZ = DTYPE == 0 ? 4 : 2;
    constexpr int NP = CPL == 2 ? 3 : 2;  // packed pairs per lane: (colA, colB) x 3 channels, or (c0, c1), (c2, c2)
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
        Rr = raw_rows_for(pl.smem_bytes - kSmemVar, own_pitch);
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

    if (tid == 0) {
        for (int b = 0; b < kNBuf; ++b) mbar_init(smem_addr(smem + kSmemFull + 8 * b), 1);
        fence_proxy_async();
    }
    // ---- row table of the tile, once ---------------------------------------------------
    // Output row y blends source rows y0 and y0 + 1 (see plan_and_issue for the virtual bottom
    // row).  The compute warps keep the two most recent rows in two register buffers A and B and
    // write the n-th row they consume (n = 0, 1, ... from the top of the tile) into buffer n & 1, so
    // which buffer holds the row of weight dy is known here: the table stores the weight OF EACH
    // BUFFER, and the blend a*(1-dy) + b*dy (a sum, so its order is free) needs no case split.
    // Pairs mode (steeper than 2x): every output row consumes two fresh rows, y0 + 1 always lands in B.
    const bool pairs = ch > 2 * H;
    const int kbase = min(static_cast<int>(src_coord(ty0, yscale)), ch - 1);  // first row the tile consumes
    for (int r = tid; r < ty1 - ty0; r += blockDim.x) {
        const float sy = src_coord(ty0 + r, yscale);
        const int y0 = min(static_cast<int>(sy), ch - 1);
        const float dy = __fsub_rn(sy, static_cast<float>(y0));
        const float idy = __fsub_rn(1.0f, dy);
        const bool new_in_b = pairs || (((y0 + 1 - kbase) & 1) != 0);
        const float wa = new_in_b ? idy : dy, wb = new_in_b ? dy : idy;
        reinterpret_cast<float4*>(smem + kSmemRowW)[r] = make_float4(wa, wa, wb, wb);
        reinterpret_cast<int*>(smem + kSmemRowY)[r] = y0;
    }
    __syncthreads();  // the only CTA-wide barrier: tables and mbarriers are ready

    if (warp == strips) {
        // ================= planner warp =================================================================
        PassCtx pc;
        pc.ty0 = ty0; pc.ty1 = ty1; pc.iw = iw; pc.cx = cx; pc.cy = cy; pc.ch = ch;
        pc.fx_lo = fx_lo; pc.fw = fw; pc.Rr = Rr; pc.pitch = own_pitch;
        pc.pairs = pairs;
        pc.img = p.src + img_off;
        // Readable region for the 16-byte round-out of the row copies: the whole source buffer, or,
        // when the images are separate allocations, the image itself.
        if (p.per_image_region) {
            pc.reg_lo = reinterpret_cast<unsigned long long>(pc.img);
            pc.reg_hi = pc.reg_lo + static_cast<unsigned long long>(iw) * ih * 3ull;
        } else {
            pc.reg_lo = reinterpret_cast<unsigned long long>(p.src);
            pc.reg_hi = pc.reg_lo + p.src_bytes;
        }
        PassState st;
        st.yb = ty0; st.staged_last = -1; st.index = 0;
        const int cta_threads = 32 * (strips + 1);
        for (int n = 0; n < kNBuf && st.yb < ty1; ++n) plan_and_issue(pc, st, smem, lane);  // passes 0 .. kNBuf-1
        int released = 0;  // passes whose raw buffer the compute warps have handed back
        while (st.yb < ty1) {
            // Pass n reuses the raw buffer of pass n - kNBuf: block until every compute warp has
            // finished reading that buffer.
            named_sync(released % kNBuf, cta_threads);
            ++released;
            plan_and_issue(pc, st, smem, lane);
        }
        // Match the remaining hand-backs, so that no barrier is left half-way when the CTA retires.
        for (; released < st.index; ++released) named_sync(released % kNBuf, cta_threads);
        return;
    }

    // ================= compute warps: one strip each ======================================================
    // ---- column ownership: lane l owns columns l and l + 32 of the strip (CPL = 2) --------------
    // Neighbouring lanes read neighbouring source pixels, so the byte loads of a warp fall into
    // distinct banks, and a warp's store covers 32 adjacent pixels.
    const int colA = warp * (32 * CPL) + lane;  // inside the tile
    const int colB = colA + 32;
    const bool validA = colA < tcw;
    const bool validB = CPL == 2 && colB < tcw;
    int offA0 = 0, offA1 = 0, offB0 = 0, offB1 = 0;  // byte offsets of the source pixels inside a staged row
    float2 W0 = f2(0.0f, 0.0f), W1 = f2(0.0f, 0.0f);  // (1-dx) and dx of the lane's pairs
    {
        auto column = [&](int hx, int& o0, int& o1, float& w0, float& w1) {
            const int x = tx0 + hx;
            const int ox = flip ? (W - 1 - x) : x;
            const float sx = src_coord(ox, xscale);
            const int x0 = min(static_cast<int>(sx), cw - 1);
            const int x1 = min(x0 + 1, cw - 1);
            const float dx = __fsub_rn(sx, static_cast<float>(x0));
            o0 = (x0 - fx_lo) * 3;
            o1 = (x1 - fx_lo) * 3;
            w0 = __fsub_rn(1.0f, dx);
            w1 = dx;
        };
        if (validA) column(colA, offA0, offA1, W0.x, W1.x);
        if constexpr (CPL == 2) {
            if (validB) column(colB, offB0, offB1, W0.y, W1.y);
        } else {
            W0.y = W0.x;
            W1.y = W1.x;
        }
    }
    const float2 NW0 = f2(__fmul_rn(-8388608.0f, W0.x), __fmul_rn(-8388608.0f, W0.y));
    const float2 NW1 = f2(__fmul_rn(-8388608.0f, W1.x), __fmul_rn(-8388608.0f, W1.y));
    const float2 one2 = f2(p.one, p.one);
    const float2 pre2 = f2(p.pre_scale, p.pre_scale);
    const float2 nkpre2 = f2(p.neg_k_pre, p.neg_k_pre);
    const float2 k2 = f2(8388608.0f, 8388608.0f);
    // Normalization constants of the NP pairs.
    float2 nmean2[NP], istd2[NP];
    if constexpr (CPL == 2) {
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            nmean2[c] = f2(-p.mean[c], -p.mean[c]);
            istd2[c] = f2(p.inv_std[c], p.inv_std[c]);
        }
    } else {
        nmean2[0] = f2(-p.mean[0], -p.mean[1]);
        nmean2[1] = f2(-p.mean[2], -p.mean[2]);
        istd2[0] = f2(p.inv_std[0], p.inv_std[1]);
        istd2[1] = f2(p.inv_std[2], p.inv_std[2]);
    }
    // Colour jitter factors of this sample (uniform across the CTA).
    float jb = 1.0f, jc = 1.0f, js = 1.0f;
    if constexpr (JIT) {
        jb = p.jitter[3 * static_cast<long long>(k)];
        jc = p.jitter[3 * static_cast<long long>(k) + 1];
        js = p.jitter[3 * static_cast<long long>(k) + 2];
    }

    // ---- output addressing: one pointer per channel plane (NCHW) or one in all (NHWC) ----------
    long long obase;  // element index of (row ty0, column A) of the sample
    if constexpr (LAYOUT == 0)
        obase = (static_cast<long long>(k) * 3 * H + ty0) * W + tx0 + colA;
    else
        obase = ((static_cast<long long>(k) * H + ty0) * W + tx0 + colA) * 3;
    char* o0 = static_cast<char*>(p.out) + obase * ESZ;
    const long long row_bytes = static_cast<long long>(W) * ESZ * (LAYOUT == 0 ? 1 : 3);
    const long long chan_bytes = static_cast<long long>(H) * W * ESZ;  // NCHW plane stride
    char* o1 = o0 + chan_bytes;
    char* o2 = o1 + chan_bytes;
    constexpr int kColB = LAYOUT == 0 ? 32 * ESZ : 96 * ESZ;  // byte distance of column B's pixel
    const uint32_t smem_base = smem_addr(smem);
    uint32_t roww = smem_base + kSmemRowW;  // next output row's weights

    float2 hA[NP], hB[NP];
#pragma unroll
    for (int i = 0; i < NP; ++i) hA[i] = hB[i] = f2(0.0f, 0.0f);

    // H step: one staged source row (shared-window address) -> the lane's horizontally interpolated values.
    auto hstep = [&](uint32_t row, float2* h) {
        const uint32_t a0 = row + offA0, a1 = row + offA1;
        if constexpr (CPL == 2) {
            const uint32_t b0 = row + offB0, b1 = row + offB1;
            h[0] = add2_exact(byte_product2(lds_u8<0>(a0), lds_u8<0>(b0), W0, NW0),
                              byte_product2(lds_u8<0>(a1), lds_u8<0>(b1), W1, NW1), one2);
            h[1] = add2_exact(byte_product2(lds_u8<1>(a0), lds_u8<1>(b0), W0, NW0),
                              byte_product2(lds_u8<1>(a1), lds_u8<1>(b1), W1, NW1), one2);
            h[2] = add2_exact(byte_product2(lds_u8<2>(a0), lds_u8<2>(b0), W0, NW0),
                              byte_product2(lds_u8<2>(a1), lds_u8<2>(b1), W1, NW1), one2);
        } else {
            const unsigned p0 = lds_u8<0>(a0), p1 = lds_u8<1>(a0), p2 = lds_u8<2>(a0);
            const unsigned q0 = lds_u8<0>(a1), q1 = lds_u8<1>(a1), q2 = lds_u8<2>(a1);
            h[0] = add2_exact(byte_product2(p0, p1, W0, NW0), byte_product2(q0, q1, W1, NW1), one2);
            h[1] = add2_exact(byte_product2(p2, p2, W0, NW0), byte_product2(q2, q2, W1, NW1), one2);
        }
    };

    // One output row: blend the two row buffers with the row's weights, truncate, (jitter,) normalize,
    // store.  Lanes without a column compute on zeros and only skip the stores.
    auto vrow = [&](const float4 w) {  // {wA, wA, wB, wB}
        const float2 wa2 = f2(w.x, w.y), wb2 = f2(w.z, w.w);
        float2 v[NP];
#pragma unroll
        for (int q = 0; q < NP; ++q) {
            // v = a*(1-dy) + b*dy;  code = floor(v) as RZ(v + 2^23) - 2^23;  x = code*pre.  The last two
            // steps are one fma((2^23 + code), pre, -2^23*pre): exact product, one rounding.
            const float2 blend = add2_exact(mul2_rn(hA[q], wa2), mul2_rn(hB[q], wb2), one2);
            v[q] = fma2_rn(add2_rz(blend, k2), pre2, nkpre2);
        }
        if constexpr (JIT) {
            // Colour jitter on rgb = code/255 in the order of the reference's train_transform shader
            // (src/metal/metal_transforms.mm:111-115), every operation rounded separately: brightness,
            // contrast about 0.5, saturation as lum + (rgb-lum)*s with lum = (0.299 r + 0.587 g) + 0.114 b,
            // clamp to [0,1].
            float r[CPL][3];
#pragma unroll
            for (int e = 0; e < CPL; ++e) {
                if constexpr (CPL == 2) {
                    r[e][0] = e ? v[0].y : v[0].x;
                    r[e][1] = e ? v[1].y : v[1].x;
                    r[e][2] = e ? v[2].y : v[2].x;
                } else {
                    r[e][0] = v[0].x; r[e][1] = v[0].y; r[e][2] = v[1].x;
                }
#pragma unroll
                for (int c = 0; c < 3; ++c) {
                    float x = __fmul_rn(r[e][c], jb);
                    x = __fadd_rn(__fmul_rn(__fsub_rn(x, 0.5f), jc), 0.5f);
                    r[e][c] = x;
                }
                const float lum = __fadd_rn(__fadd_rn(__fmul_rn(r[e][0], 0.299f), __fmul_rn(r[e][1], 0.587f)),
                                            __fmul_rn(r[e][2], 0.114f));
#pragma unroll
                for (int c = 0; c < 3; ++c) {
                    float x = __fadd_rn(lum, __fmul_rn(__fsub_rn(r[e][c], lum), js));
                    r[e][c] = fminf(fmaxf(x, 0.0f), 1.0f);
                }
            }
            if constexpr (CPL == 2) {
#pragma unroll
                for (int c = 0; c < 3; ++c) v[c] = f2(r[0][c], r[1][c]);
            } else {
                v[0] = f2(r[0][0], r[0][1]);
                v[1] = f2(r[0][2], r[0][2]);
            }
        }
#pragma unroll
        for (int q = 0; q < NP; ++q) v[q] = normalize2(v[q], nmean2[q], istd2[q], one2);
        // ---- store: per channel the warp covers 32 adjacent pixels (twice for CPL = 2) ----
        if constexpr (CPL == 2) {
            if constexpr (LAYOUT == 0) {
                if (validA) {
                    store1<DTYPE>(o0, v[0].x);
                    store1<DTYPE>(o1, v[1].x);
                    store1<DTYPE>(o2, v[2].x);
                }
                if (validB) {
                    store1<DTYPE>(o0 + kColB, v[0].y);
                    store1<DTYPE>(o1 + kColB, v[1].y);
                    store1<DTYPE>(o2 + kColB, v[2].y);
                }
            } else {
                if (validA) {
                    store1<DTYPE>(o0, v[0].x);
                    store1<DTYPE>(o0 + ESZ, v[1].x);
                    store1<DTYPE>(o0 + 2 * ESZ, v[2].x);
                }
                if (validB) {
                    store1<DTYPE>(o0 + kColB, v[0].y);
                    store1<DTYPE>(o0 + kColB + ESZ, v[1].y);
                    store1<DTYPE>(o0 + kColB + 2 * ESZ, v[2].y);
                }
            }
        } else if (validA) {
            if constexpr (LAYOUT == 0) {
                store1<DTYPE>(o0, v[0].x);
                store1<DTYPE>(o1, v[0].y);
                store1<DTYPE>(o2, v[1].x);
            } else {
                store1<DTYPE>(o0, v[0].x);
                store1<DTYPE>(o0 + ESZ, v[0].y);
                store1<DTYPE>(o0 + 2 * ESZ, v[1].x);
            }
        }
        o0 += row_bytes;
        if constexpr (LAYOUT == 0) {
            o1 += row_bytes;
            o2 += row_bytes;
        }
    };

    const int cta_threads = 32 * (strips + 1);
    bool next_in_b = false;  // buffer the next consumed row goes to (uniform across the warp)
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
        const int slot = i % kSlots;
        const int4 m = lds_i4(smem_base + kSmemMeta + 16 * slot);  // {new source rows, output rows before the first, last?, -}
        uint32_t srcrec = smem_base + kSmemSrcRec + slot * 256;
        const uint32_t srcend = srcrec + 8 * m.x;

        for (int emit = m.y; emit > 0; --emit, roww += 16) vrow(lds_f4(roww));  // rows whose source rows came earlier
        while (srcrec != srcend) {
            const int2 rec = lds_i2(srcrec);  // {byte offset of the staged row, output rows ready after it}
            srcrec += 8;
            if (next_in_b)
                hstep(smem_base + rec.x, hB);
            else
                hstep(smem_base + rec.x, hA);
            next_in_b = !next_in_b;
            for (int emit = rec.y; emit > 0; --emit, roww += 16) vrow(lds_f4(roww));
        }
        __syncwarp();                      // every lane is done reading raw buffer b
        named_arrive(b, cta_threads);      // hand it back to the planner
        if (m.z) break;
    }
}

std::atomic<unsigned long long> g_launches{0};

template <int DTYPE, int LAYOUT, int CPL, bool JIT>
int launch_one(const FusedParams& p, cudaStream_t st, unsigned flags) {
    auto kern = fused_transform_kernel<DTYPE, LAYOUT, CPL, JIT>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(p.plan.grid));
    cfg.blockDim = dim3(32 * (p.plan.strips + 1));
    cfg.dynamicSmemBytes = static_cast<size_t>(p.plan.smem_bytes);
    cfg.stream = st;
    // Programmatic stream serialization: when the work directly before this launch in the stream
    // is a launch of this same kernel (which signals early, see the top of the kernel), this one
    // may begin while that one drains its last CTAs; the head and tail of back-to-back batches
    // then overlap instead of leaving SMs idle.  Behind a copy, a memset or a kernel that does not
    // signal early the usual stream order holds.  Requested per call, because the kernel does not
    // wait on its predecessor.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & kLaunchOverlap) ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kern, p);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return static_cast<int>(cudaGetLastError());
}

template <int DTYPE, int LAYOUT, int CPL, bool JIT>
int opt_in_smem() {
    return static_cast<int>(cudaFuncSetAttribute(fused_transform_kernel<DTYPE, LAYOUT, CPL, JIT>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
}

template <int DTYPE, int LAYOUT>
int launch_dl(const FusedParams& p, cudaStream_t st, unsigned flags) {
    const bool jit = p.jitter != nullptr;
    if (p.plan.cpl == 2)
        return jit ? launch_one<DTYPE, LAYOUT, 2, true>(p, st, flags) : launch_one<DTYPE, LAYOUT, 2, false>(p, st, flags);
    return jit ? launch_one<DTYPE, LAYOUT, 1, true>(p, st, flags) : launch_one<DTYPE, LAYOUT, 1, false>(p, st, flags);
}

template <int DTYPE, int LAYOUT>
int opt_in_dl() {
    int e = opt_in_smem<DTYPE, LAYOUT, 1, false>();
    if (!e) e = opt_in_smem<DTYPE, LAYOUT, 1, true>();
    if (!e) e = opt_in_smem<DTYPE, LAYOUT, 2, false>();
    if (!e) e = opt_in_smem<DTYPE, LAYOUT, 2, true>();
    return e;
}

}  // namespace

int prepare_device() {
    int e = opt_in_dl<0, 0>();
    if (!e) e = opt_in_dl<0, 1>();
    if (!e) e = opt_in_dl<1, 0>();
    if (!e) e = opt_in_dl<1, 1>();
    return e;
}

int launch_fused(const FusedParams& p, int out_dtype, int out_layout, void* stream, unsigned flags) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (out_dtype == 0) return out_layout == 0 ? launch_dl<0, 0>(p, st, flags) : launch_dl<0, 1>(p, st, flags);
    return out_layout == 0 ? launch_dl<1, 0>(p, st, flags) : launch_dl<1, 1>(p, st, flags);
}

unsigned long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

}  // namespace tlb
