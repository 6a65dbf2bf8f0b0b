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
// Structure of one CTA (256 threads) = one tile of `tile_rows` x `tile_cols` outputs of
// one sample, processed in passes of at most R staged source rows:
//   1. warp 0 works out which source rows the pass needs (one lane per output row, the
//      first/last row exchanged with warp shuffles) and issues one 1-D bulk async copy
//      (cp.async.bulk, global -> this CTA's shared memory, completion on an mbarrier)
//      per source row, each rounded out to 16-byte boundaries.  Bytes that cannot be
//      reached on a 16-byte grid inside the readable region are fetched with plain loads.
//   2. "H" phase: every staged row is interpolated horizontally once,
//      h = p[x0]*(1-dx) + p[x1]*dx, into fp32 in shared memory.  Column weights are
//      computed once per tile (one column per thread) and kept in shared memory.
//   3. "V" phase: each thread produces one 16-byte output chunk at a time:
//      v = h[y0]*(1-dy) + h[y1]*dy, truncate, normalize, cast, one 16-byte store.
//      The layout of h in shared memory (planar for NCHW, interleaved for NHWC) makes
//      the inputs of a chunk two 16-byte shared loads per source row.
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
// Returns false if the phase did not complete within the polling limit.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t mbar, uint32_t parity) {
    for (unsigned it = 0; it < kWaitLimit; ++it)
        if (mbar_try_wait(mbar, parity)) return true;
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

// floor(v) for 0 <= v < 2^22 without a float->int->float round trip: adding 2^23 with
// round-toward-zero drops the fraction, subtracting it back is exact.  The CPU path's
// clamp to [0,255] before the uint8 cast cannot change the code: v is a convex blend of
// values in [0,255], so v < 256 and v >= 0 always.
__device__ __forceinline__ float trunc_code(float v) {
    return __fsub_rn(__fadd_rz(v, 8388608.0f), 8388608.0f);
}

__device__ __forceinline__ float blend(float a, float wa, float b, float wb) {
    return __fadd_rn(__fmul_rn(a, wa), __fmul_rn(b, wb));
}

__device__ __forceinline__ float normalize(float code, float pre, float mean, float inv_std) {
    return __fmul_rn(__fsub_rn(__fmul_rn(code, pre), mean), inv_std);
}

template <int DTYPE>
struct OutT;
template <>
struct OutT<0> {
    using type = float;
    static constexpr int V = 4;
};
template <>
struct OutT<1> {
    using type = __nv_bfloat16;
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
__device__ __forceinline__ void store_chunk(void* out, long long idx, const float* v) {
    if constexpr (DTYPE == 0) {
        *reinterpret_cast<float4*>(static_cast<float*>(out) + idx) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
        __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
        __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]);
        __nv_bfloat162 d = __floats2bfloat162_rn(v[6], v[7]);
        uint4 u;
        u.x = *reinterpret_cast<uint32_t*>(&a);
        u.y = *reinterpret_cast<uint32_t*>(&b);
        u.z = *reinterpret_cast<uint32_t*>(&c);
        u.w = *reinterpret_cast<uint32_t*>(&d);
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out) + idx) = u;
    }
}

template <int DTYPE, int LAYOUT>
__global__ void __launch_bounds__(kThreads) fused_transform_kernel(const __grid_constant__ FusedParams p) {
    constexpr int V = OutT<DTYPE>::V;
    extern __shared__ __align__(128) unsigned char smem[];
    const Plan& pl = p.plan;
    const SmemLayout L = smem_layout(pl.tile_cols, pl.staged_rows, pl.pitch, pl.hpitch);
    float4* colp = reinterpret_cast<float4*>(smem + L.colp);
    float4* rowp = reinterpret_cast<float4*>(smem + L.rowp);
    int* rowsh = reinterpret_cast<int*>(smem + L.rowsh);
    float* ctab = reinterpret_cast<float*>(smem + L.ctab);
    unsigned char* raw = smem + L.raw;
    float* hbuf = reinterpret_cast<float*>(smem + L.hbuf);
    const uint32_t mbar = smem_addr(smem + L.mbar);

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

    // ---- column weights: one output column per thread, once per tile ----------------
    const float xscale = __fdiv_rn(static_cast<float>(cw), static_cast<float>(W > 0 ? W : 1));
    const float yscale = __fdiv_rn(static_cast<float>(ch), static_cast<float>(H > 0 ? H : 1));
    // Source-column footprint of the tile: resized columns [oxa, oxb] (mirrored when flipped).
    const int oxa = flip ? (W - 1 - (tx0 + tcw - 1)) : tx0;
    const int oxb = flip ? (W - 1 - tx0) : (tx0 + tcw - 1);
    int fx_lo = 0, fw = 0;
    if (!bad) {
        fx_lo = min(static_cast<int>(src_coord(oxa, xscale)), cw - 1);
        const int hi0 = min(static_cast<int>(src_coord(oxb, xscale)), cw - 1);
        const int fx_hi = min(hi0 + 1, cw - 1);
        fw = fx_hi - fx_lo + 1;
        if (fw * 3 + 30 > pl.pitch) bad = kDevTooWide;
    }

    if (bad) {
        // Defined behaviour for an invalid sample: zero-fill its tile, report, never trap.
        if (tid == 0 && p.status) atomicOr(p.status, bad);
        const int rows = ty1 - ty0;
        for (int i = tid; i < rows * tcw * 3; i += kThreads) {
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

    if (tid < tcw) {
        const int x = tx0 + tid;
        const int ox = flip ? (W - 1 - x) : x;
        const float sx = src_coord(ox, xscale);
        const int x0 = min(static_cast<int>(sx), cw - 1);
        const int x1 = min(x0 + 1, cw - 1);
        const float dx = __fsub_rn(sx, static_cast<float>(x0));
        colp[tid] = make_float4(__int_as_float((x0 - fx_lo) * 3), __int_as_float((x1 - fx_lo) * 3), dx,
                                __fsub_rn(1.0f, dx));
    }
    if (LAYOUT == 1 && tid < 48) {
        // NHWC chunks start at channel phase ph = (first element index) % 3; element i of the
        // chunk has channel (ph + i) % 3.  ctab[ph*16 + i] = mean, ctab[ph*16 + 8 + i] = inv_std.
        const int ph = tid >> 4, i = tid & 7, c = (ph + i) % 3;
        ctab[tid] = (tid & 8) ? p.inv_std[c] : p.mean[c];
    }
    if (tid == 0) {
        mbar_init(mbar, 1);
        fence_proxy_async();
    }
    __syncthreads();

    const int R = pl.staged_rows;
    const int hp = pl.hpitch;
    const int tcp = pl.tile_cols;
    const unsigned char* img = p.src + img_off;
    const unsigned long long reg_lo = reinterpret_cast<unsigned long long>(p.src);
    const unsigned long long reg_hi = reg_lo + p.src_bytes;
    void* const outp = p.out;
    uint32_t parity = 0;

    for (int yb = ty0; yb < ty1;) {
        // ---- rows of this pass: lane l of every warp looks at output row yb + l -------
        const int y = yb + lane;
        const float sy = src_coord(min(y, H - 1), yscale);
        const int y0 = min(static_cast<int>(sy), ch - 1);
        const int y1 = min(y0 + 1, ch - 1);
        const float dy = __fsub_rn(sy, static_cast<float>(y0));
        const int first = __shfl_sync(0xffffffffu, y0, 0);
        // Contiguous staging: rows first .. y1 of the last output row that still fits in R.
        const unsigned fits = __ballot_sync(0xffffffffu, (y < ty1) && (y1 - first + 1 <= R));
        int nrows = __popc(fits);  // the fitting rows form a prefix: y1 is non-decreasing in y
        const int npair = min(R >> 1, ty1 - yb);
        const bool pairs = nrows < npair;  // steep downscale: stage exactly (y0, y1) per row
        if (pairs) nrows = npair;
        const int last_y1 = __shfl_sync(0xffffffffu, y1, nrows - 1);
        const int nstaged = pairs ? 2 * nrows : (last_y1 - first + 1);

        if (warp == 0) {
            if (lane < nrows) {
                const int s0 = pairs ? 2 * lane : (y0 - first);
                const int s1 = pairs ? 2 * lane + 1 : (y1 - first);
                rowp[lane] = make_float4(__int_as_float(s0), __int_as_float(s1), dy, __fsub_rn(1.0f, dy));
            }
            // Source row staged in slot j (one slot per lane).
            const int j = lane;
            int srow;
            if (pairs) {
                const int ya = __shfl_sync(0xffffffffu, y0, j >> 1);
                const int yb1 = __shfl_sync(0xffffffffu, y1, j >> 1);
                srow = (j & 1) ? yb1 : ya;
            } else {
                srow = first + j;
            }
            unsigned bytes = 0;
            unsigned long long lo = 0, a0 = 0, a1 = 0, hi = 0;
            if (j < nstaged) {
                a0 = reinterpret_cast<unsigned long long>(img) +
                     (static_cast<unsigned long long>(cy + srow) * iw + (cx + fx_lo)) * 3ull;
                a1 = a0 + static_cast<unsigned long long>(fw) * 3ull;
                lo = a0 & ~15ull;
                if (lo < reg_lo) lo += 16;           // region does not start on the 16-byte grid
                hi = (a1 + 15ull) & ~15ull;
                if (hi > reg_hi) hi = reg_hi & ~15ull;  // region does not end on the 16-byte grid
                bytes = hi > lo ? static_cast<unsigned>(hi - lo) : 0u;
                rowsh[j] = static_cast<int>(a0 & 15ull);
            }
            unsigned total = bytes;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
            fence_proxy_async();  // earlier generic reads of the staging buffer precede the new copies
            if (lane == 0) mbar_arrive_expect_tx(mbar, total);
            __syncwarp();
            if (j < nstaged) {
                unsigned char* slot = raw + j * pl.pitch;
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
        __syncthreads();  // rowp / rowsh / ragged bytes visible
        if (!mbar_wait_bounded(mbar, parity)) {
            if (tid == 0 && p.status) atomicOr(p.status, kDevCopyTimeout);
            mbar_wait_bounded(mbar, parity);  // give in-flight copies a second bounded chance to land
            return;
        }
        parity ^= 1u;

        // ---- H phase: staged rows -> horizontally interpolated fp32 ---------------------
        {
            int j = tid / tcw;
            int t = tid - j * tcw;
            while (j < nstaged) {
                const float4 cp = colp[t];
                const unsigned char* row = raw + j * pl.pitch + rowsh[j];
                const unsigned char* q0 = row + __float_as_int(cp.x);
                const unsigned char* q1 = row + __float_as_int(cp.y);
                const float h0 = blend(static_cast<float>(q0[0]), cp.w, static_cast<float>(q1[0]), cp.z);
                const float h1 = blend(static_cast<float>(q0[1]), cp.w, static_cast<float>(q1[1]), cp.z);
                const float h2 = blend(static_cast<float>(q0[2]), cp.w, static_cast<float>(q1[2]), cp.z);
                float* h = hbuf + j * hp;
                if constexpr (LAYOUT == 0) {
                    h[t] = h0;
                    h[tcp + t] = h1;
                    h[2 * tcp + t] = h2;
                } else {
                    h[3 * t] = h0;
                    h[3 * t + 1] = h1;
                    h[3 * t + 2] = h2;
                }
                t += kThreads;
                while (t >= tcw) {
                    t -= tcw;
                    ++j;
                }
            }
        }
        __syncthreads();

        // ---- V phase: one 16-byte output chunk per step ----------------------------------
        if constexpr (LAYOUT == 0) {
            const int G = (tcw + V - 1) / V;  // chunks per channel row
            const int U = 3 * G;              // chunks per output row
            int l = tid / U;
            int u = tid - l * U;
            const long long sample_base = static_cast<long long>(k) * 3 * H * W;
            while (l < nrows) {
                const int c = (u >= 2 * G) ? 2 : ((u >= G) ? 1 : 0);
                const int g = u - c * G;
                const float4 rp = rowp[l];
                const float* ha = hbuf + __float_as_int(rp.x) * hp + c * tcp + g * V;
                const float* hb = hbuf + __float_as_int(rp.y) * hp + c * tcp + g * V;
                const float mean = c == 0 ? p.mean[0] : (c == 1 ? p.mean[1] : p.mean[2]);
                const float istd = c == 0 ? p.inv_std[0] : (c == 1 ? p.inv_std[1] : p.inv_std[2]);
                float v[V];
#pragma unroll
                for (int q = 0; q < V / 4; ++q) {
                    const float4 a = *reinterpret_cast<const float4*>(ha + 4 * q);
                    const float4 b = *reinterpret_cast<const float4*>(hb + 4 * q);
                    v[4 * q + 0] = normalize(trunc_code(blend(a.x, rp.w, b.x, rp.z)), p.pre_scale, mean, istd);
                    v[4 * q + 1] = normalize(trunc_code(blend(a.y, rp.w, b.y, rp.z)), p.pre_scale, mean, istd);
                    v[4 * q + 2] = normalize(trunc_code(blend(a.z, rp.w, b.z, rp.z)), p.pre_scale, mean, istd);
                    v[4 * q + 3] = normalize(trunc_code(blend(a.w, rp.w, b.w, rp.z)), p.pre_scale, mean, istd);
                }
                const long long idx = sample_base + (static_cast<long long>(c) * H + (yb + l)) * W + tx0 + g * V;
                if (pl.vec_ok && g * V + V <= tcw) {
                    store_chunk<DTYPE>(outp, idx, v);
                } else {
#pragma unroll
                    for (int i = 0; i < V; ++i)
                        if (g * V + i < tcw) store_scalar<DTYPE>(outp, idx + i, v[i]);
                }
                u += kThreads;
                while (u >= U) {
                    u -= U;
                    ++l;
                }
            }
        } else {
            const int E = 3 * tcw;            // interleaved elements per output row of the tile
            const int G = (E + V - 1) / V;    // chunks per output row
            int l = tid / G;
            int g = tid - l * G;
            while (l < nrows) {
                const float4 rp = rowp[l];
                const float* ha = hbuf + __float_as_int(rp.x) * hp + g * V;
                const float* hb = hbuf + __float_as_int(rp.y) * hp + g * V;
                const int ph = (g * V) % 3;
                const float* cm = ctab + ph * 16;
                float v[V];
#pragma unroll
                for (int q = 0; q < V / 4; ++q) {
                    const float4 a = *reinterpret_cast<const float4*>(ha + 4 * q);
                    const float4 b = *reinterpret_cast<const float4*>(hb + 4 * q);
                    const float4 m = *reinterpret_cast<const float4*>(cm + 4 * q);
                    const float4 is = *reinterpret_cast<const float4*>(cm + 8 + 4 * q);
                    v[4 * q + 0] = normalize(trunc_code(blend(a.x, rp.w, b.x, rp.z)), p.pre_scale, m.x, is.x);
                    v[4 * q + 1] = normalize(trunc_code(blend(a.y, rp.w, b.y, rp.z)), p.pre_scale, m.y, is.y);
                    v[4 * q + 2] = normalize(trunc_code(blend(a.z, rp.w, b.z, rp.z)), p.pre_scale, m.z, is.z);
                    v[4 * q + 3] = normalize(trunc_code(blend(a.w, rp.w, b.w, rp.z)), p.pre_scale, m.w, is.w);
                }
                const long long idx =
                    ((static_cast<long long>(k) * H + (yb + l)) * W + tx0) * 3 + static_cast<long long>(g) * V;
                if (pl.vec_ok && g * V + V <= E) {
                    store_chunk<DTYPE>(outp, idx, v);
                } else {
#pragma unroll
                    for (int i = 0; i < V; ++i)
                        if (g * V + i < E) store_scalar<DTYPE>(outp, idx + i, v[i]);
                }
                g += kThreads;
                while (g >= G) {
                    g -= G;
                    ++l;
                }
            }
        }
        yb += nrows;
        if (yb < ty1) __syncthreads();  // staging buffers are reused by the next pass
    }
}

std::atomic<unsigned long long> g_launches{0};

template <int DTYPE, int LAYOUT>
int launch_one(const FusedParams& p, cudaStream_t st) {
    auto kern = fused_transform_kernel<DTYPE, LAYOUT>;
    kern<<<static_cast<unsigned>(p.plan.grid), kThreads, p.plan.smem_bytes, st>>>(p);
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
