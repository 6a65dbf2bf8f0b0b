// Host side of the C ABI declared in include/turboloader_b200.h: argument validation,
// launch planning, the library-owned staging/param/output rings and the host-image
// convenience forms.  C++20, CUDA runtime only; no torch or pybind types appear here.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/turboloader_b200.h"
#include "fused_params.h"
#include "video_params.h"
#include "antialias_params.h"
#include "host_gather.h"

namespace {

thread_local std::string t_err;
std::atomic<unsigned long long> g_extra_launches{0};  // kernels other than the fused transform

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    t_err = buf;
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    return fail(TLB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define TLB_CUDA(call)                                      \
    do {                                                    \
        cudaError_t e__ = (call);                           \
        if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
    } while (0)

inline int round_up(int v, int m) { return (v + m - 1) / m * m; }

int env_int(const char* name, int dflt) {
    const char* s = std::getenv(name);
    if (!s || !*s) return dflt;
    return std::atoi(s);
}

// ---- per-device state ---------------------------------------------------------------
struct Buffer {
    void* host = nullptr;   // pinned
    void* dev = nullptr;
    size_t cap = 0;
    cudaEvent_t done = nullptr;  // recorded after the last upload from `host`
    bool pending = false;
};

struct DeviceState {
    std::mutex mu;
    std::mutex prep_mu;  // separate from mu: the resident forms hold mu while they launch
    std::atomic<bool> prepared{false};
    Buffer params[4];  // ring for host-supplied per-sample tables
    int params_next = 0;
    Buffer images[2];  // ring for host-image batches (pixels + tables)
    int images_next = 0;
    void* out_ring[4] = {nullptr, nullptr, nullptr, nullptr};  // legacy pointer-returning forms
    size_t out_cap[4] = {0, 0, 0, 0};
    int out_next = 0;
    void* video_out[2] = {nullptr, nullptr};  // pointer-returning video forms: valid until the next call
    size_t video_cap[2] = {0, 0};
    int video_next = 0;
    void* sync_out = nullptr;  // device result of the synchronous host-image forms
    size_t sync_out_cap = 0;
    cudaStream_t stream = nullptr;  // private stream of the synchronous forms
    // Idle prefetch streams and events of finished epoch pipelines, kept for the next one: creating
    // and destroying four streams and nine events per epoch cost 0.45 ms of a 5 ms epoch.
    std::mutex pool_mu;
    std::vector<cudaStream_t> idle_streams;
    std::vector<cudaEvent_t> idle_events;
};

constexpr int kMaxDevices = 64;
DeviceState g_dev[kMaxDevices];

int current_device(int* dev) {
    cudaError_t e = cudaGetDevice(dev);
    if (e != cudaSuccess) return fail(TLB_ERR_NO_DEVICE, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (*dev < 0 || *dev >= kMaxDevices) return fail(TLB_ERR_NO_DEVICE, "device ordinal %d unsupported", *dev);
    return TLB_OK;
}

int ensure_prepared(DeviceState& st) {
    if (st.prepared.load(std::memory_order_acquire)) return TLB_OK;
    std::lock_guard<std::mutex> lk(st.prep_mu);
    if (st.prepared.load(std::memory_order_acquire)) return TLB_OK;
    cudaError_t e = static_cast<cudaError_t>(tlb::prepare_device());
    if (e == cudaSuccess) e = static_cast<cudaError_t>(tlb::prepare_video());
    if (e == cudaSuccess) e = static_cast<cudaError_t>(tlb::prepare_antialias());
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(max dynamic shared memory)");
    st.prepared.store(true, std::memory_order_release);
    return TLB_OK;
}

int grow(Buffer& b, size_t need) {
    if (b.pending) {  // the previous upload from this pinned buffer must have left the host
        TLB_CUDA(cudaEventSynchronize(b.done));
        b.pending = false;
    }
    if (need <= b.cap) return TLB_OK;
    size_t cap = std::max<size_t>(need + need / 4, 1 << 16);
    if (b.host) cudaFreeHost(b.host);
    if (b.dev) cudaFree(b.dev);
    b.host = b.dev = nullptr;
    b.cap = 0;
    TLB_CUDA(cudaMallocHost(&b.host, cap));
    TLB_CUDA(cudaMalloc(&b.dev, cap));
    if (!b.done) TLB_CUDA(cudaEventCreateWithFlags(&b.done, cudaEventDisableTiming));
    b.cap = cap;
    return TLB_OK;
}

// ---- planning ------------------------------------------------------------------------
// `streaming`: the launch is one of a stream of back-to-back batches (TLB_FLAG_LAUNCH_OVERLAP, or
// the epoch pipeline): taller tiles halve the per-tile set-up, and the longer tail of a launch is
// covered by the head of the next one.  A launch on its own finishes sooner with the shorter tiles.
int make_plan(const tlb_transform_desc& d, int max_crop_w, tlb::Plan& pl, bool streaming = false) {
    const int W = d.dst_w, H = d.dst_h;
    const int esz = d.out_dtype == TLB_F32 ? 4 : 2;
    const bool base_ok = (reinterpret_cast<uintptr_t>(d.out) & 15u) == 0;
    // Two columns per lane (c and c + 32 of a 64-column strip) unless the output is narrower than
    // one such strip.
    pl.cpl = W > 32 ? 2 : 1;
    if (const int forced = env_int("TLB_CPL", 0); forced == 1) pl.cpl = 1;
    const int strip_cols = 32 * pl.cpl;
    const int max_cols = tlb::kMaxStrips * strip_cols;
    pl.n_col_tiles = (W + max_cols - 1) / max_cols;
    pl.tile_cols = std::min(max_cols, round_up((W + pl.n_col_tiles - 1) / pl.n_col_tiles, strip_cols));
    pl.n_col_tiles = (W + pl.tile_cols - 1) / pl.tile_cols;
    pl.strips = pl.tile_cols / strip_cols;  // one compute warp per strip
    // Row tiles of equal height, at most TLB_TILE_ROWS (default 64, or 128 when streaming) rows each.
    const int max_rows = std::clamp(env_int("TLB_TILE_ROWS", streaming ? 128 : 64), 1, tlb::kMaxTileRows);
    pl.n_row_tiles = (H + max_rows - 1) / max_rows;
    pl.tile_rows = (H + pl.n_row_tiles - 1) / pl.n_row_tiles;
    pl.n_row_tiles = (H + pl.tile_rows - 1) / pl.tile_rows;
    // Widest source footprint of one column tile (crop-local columns) -> worst-case row pitch.
    long long fw = std::min<long long>(max_crop_w, (static_cast<long long>(pl.tile_cols) * max_crop_w + W - 1) / W + 3);
    pl.pitch = round_up(static_cast<int>(fw) * 3 + 30, 16);
    // Shared memory: kNBuf raw buffers of Rr rows; a CTA derives Rr from its own (usually narrower)
    // footprint pitch.  Default: room for TLB_RAW_ROWS (8) rows of the widest crop per buffer.
    const int want_rows = std::clamp(env_int("TLB_RAW_ROWS", 8), 2, tlb::kMaxNewRows);
    int var = want_rows * tlb::kNBuf * pl.pitch;
    if (const int budget = env_int("TLB_SMEM_BUDGET", 0); budget > 0)
        var = std::clamp(budget - tlb::kSmemVar, 2 * tlb::kNBuf * pl.pitch, tlb::kMaxNewRows * tlb::kNBuf * pl.pitch);
    pl.smem_bytes = tlb::kSmemVar + var;
    if (pl.smem_bytes > 227 * 1024) {
        pl.smem_bytes = 227 * 1024;
        if (tlb::raw_rows_for(pl.smem_bytes - tlb::kSmemVar, pl.pitch) < 2)
            return fail(TLB_ERR_TOO_WIDE, "crop width %d does not fit the shared-memory staging buffers", max_crop_w);
    }
    const int V = 16 / esz;
    if (d.out_layout == TLB_NCHW)
        pl.vec_ok = base_ok && (W % V == 0);
    else
        pl.vec_ok = base_ok && ((3ll * W * esz) % 16 == 0);
    pl.grid = static_cast<long long>(d.n) * pl.n_row_tiles * pl.n_col_tiles;
    if (pl.grid > 0x7fffffffll) return fail(TLB_ERR_INVALID_ARG, "batch needs %lld CTAs (limit 2^31-1)", pl.grid);
    return TLB_OK;
}

int check_common(const tlb_transform_desc* d) {
    if (!d) return fail(TLB_ERR_INVALID_ARG, "desc is NULL");
    if (d->n < 0) return fail(TLB_ERR_INVALID_ARG, "n = %d is negative", d->n);
    if (d->dst_h <= 0 || d->dst_w <= 0) return fail(TLB_ERR_INVALID_ARG, "dst size %dx%d must be positive", d->dst_w, d->dst_h);
    if (3ll * d->dst_h * d->dst_w > 0x3fffffffll) return fail(TLB_ERR_INVALID_ARG, "dst size %dx%d too large", d->dst_w, d->dst_h);
    if (d->out_dtype != TLB_F32 && d->out_dtype != TLB_BF16) return fail(TLB_ERR_INVALID_ARG, "unknown out_dtype %d", d->out_dtype);
    if (d->out_layout != TLB_NCHW && d->out_layout != TLB_NHWC) return fail(TLB_ERR_INVALID_ARG, "unknown out_layout %d", d->out_layout);
    if (d->n == 0) return TLB_OK;
    if (!d->src || !d->out) return fail(TLB_ERR_INVALID_ARG, "src and out must be non-NULL");
    if (d->n_src <= 0) return fail(TLB_ERR_INVALID_ARG, "n_src = %lld must be positive", static_cast<long long>(d->n_src));
    if (!d->src_sizes && (d->src_w <= 0 || d->src_h <= 0))
        return fail(TLB_ERR_INVALID_ARG, "uniform source size %dx%d must be positive", d->src_w, d->src_h);
    if (!d->sel && d->n > d->n_src) return fail(TLB_ERR_BAD_INDEX, "n = %d exceeds n_src = %lld without a gather index", d->n, static_cast<long long>(d->n_src));
    for (int c = 0; c < 3; ++c)
        if (!(d->std[c] != 0.0f)) return fail(TLB_ERR_INVALID_ARG, "std[%d] must be non-zero", c);
    if (d->labels_out && !d->labels_in) return fail(TLB_ERR_INVALID_ARG, "labels_out given without labels_in");
    if (d->jitter && !d->normalize_01)
        return fail(TLB_ERR_INVALID_ARG, "colour jitter works on rgb in [0,1]: it needs normalize_01 = 1 (mean/std in [0,1] units)");
    if (d->flags & ~static_cast<uint32_t>(TLB_FLAG_LAUNCH_OVERLAP)) return fail(TLB_ERR_INVALID_ARG, "unknown bits in flags: 0x%x", d->flags);
    if (!d->boxes && d->uniform_box[2] != 0) {
        const int* b = d->uniform_box;
        if (b[2] < 0 || b[3] <= 0 || b[0] < 0 || b[1] < 0) return fail(TLB_ERR_BAD_BOX, "uniform box (%d,%d,%d,%d) invalid", b[0], b[1], b[2], b[3]);
        if (!d->src_sizes && (b[0] > d->src_w - b[2] || b[1] > d->src_h - b[3]))
            return fail(TLB_ERR_BAD_BOX, "uniform box (%d,%d,%d,%d) leaves the %dx%d image", b[0], b[1], b[2], b[3], d->src_w, d->src_h);
    }
    return TLB_OK;
}

void fill_params(const tlb_transform_desc& d, tlb::FusedParams& p) {
    p.src = d.src;
    p.src_bytes = d.src_bytes;
    p.n_src = d.n_src;
    p.src_offsets = reinterpret_cast<const long long*>(d.src_offsets);
    p.src_sizes = d.src_sizes;
    p.src_w = d.src_w;
    p.src_h = d.src_h;
    p.n = d.n;
    p.sel = reinterpret_cast<const long long*>(d.sel);
    p.boxes = d.boxes;
    for (int i = 0; i < 4; ++i) p.ubox[i] = d.uniform_box[i];
    p.flips = d.flips;
    p.dst_h = d.dst_h;
    p.dst_w = d.dst_w;
    p.out = d.out;
    p.out_indices = reinterpret_cast<long long*>(d.out_indices);
    p.labels_in = reinterpret_cast<const long long*>(d.labels_in);
    p.labels_out = reinterpret_cast<long long*>(d.labels_out);
    for (int c = 0; c < 3; ++c) {
        p.mean[c] = d.mean[c];
        p.inv_std[c] = 1.0f / d.std[c];
    }
    p.pre_scale = d.normalize_01 ? (1.0f / 255.0f) : 1.0f;
    p.one = 1.0f;
    p.neg_k_pre = -8388608.0f * p.pre_scale;
    p.jitter = d.jitter;
    p.status = d.status;
}

int derive_max_crop_w(const tlb_transform_desc& d) {
    if (d.max_crop_w > 0) return d.max_crop_w;
    if (!d.boxes && d.uniform_box[2] > 0) return d.uniform_box[2];
    return d.src_w;
}

// `honour_flags`: only tlb_fused_transform, whose inputs the caller staged itself, passes the
// descriptor's launch flags on (TLB_FLAG_LAUNCH_OVERLAP); every other entry point stages inputs in
// the stream just before the kernel and launches in full stream order.
int launch_desc(const tlb_transform_desc& d, int max_crop_w, void* stream, bool honour_flags = false,
                bool per_image_region = false, bool streaming = false) {
    int dev;
    if (int rc = current_device(&dev)) return rc;
    if (int rc = ensure_prepared(g_dev[dev])) return rc;
    tlb::FusedParams p{};
    fill_params(d, p);
    p.per_image_region = per_image_region ? 1 : 0;
    if (d.antialias) {
        // Opt-in triangle filter: its own kernel; tap tables are sized from the largest crop.
        int max_crop_h = d.max_crop_h;
        if (max_crop_h <= 0) max_crop_h = (!d.boxes && d.uniform_box[2] > 0) ? d.uniform_box[3] : d.src_h;
        if (max_crop_h <= 0) return fail(TLB_ERR_INVALID_ARG, "antialias: max_crop_h (or src_h) is required");
        tlb::AAPlan a{};
        a.xt = tlb::aa_max_taps(max_crop_w, d.dst_w);
        a.yt = tlb::aa_max_taps(max_crop_h, d.dst_h);
        // The packed kernel gives a thread two columns (tile_cols / 2 threads per CTA); its tables
        // take 3x the column weights of the one-column kernel, so very wide filters get narrower tiles.
        static const bool one_col = std::getenv("TLB_AA_ONE_COLUMN") != nullptr;
        a.pair = one_col ? 0 : 1;
        if (!a.pair && d.jitter) return fail(TLB_ERR_INVALID_ARG, "colour jitter needs the packed antialias kernel (TLB_AA_ONE_COLUMN is set)");
        // Row tiles of equal height: at most 32 rows for a launch on its own (more CTAs, shorter tail),
        // at most 64 for one of a stream of overlapping launches (the next launch covers the tail, and
        // the per-tile tables are built half as often).
        static const int aa_rows = env_int("TLB_AA_TILE_ROWS", 0);
        const bool overlapping = streaming || (honour_flags && (d.flags & TLB_FLAG_LAUNCH_OVERLAP));
        const int max_rows = std::min(std::max(aa_rows > 0 ? aa_rows : (overlapping ? 64 : 32), 1), d.dst_h);
        a.n_row_tiles = (d.dst_h + max_rows - 1) / max_rows;
        a.tile_rows = (d.dst_h + a.n_row_tiles - 1) / a.n_row_tiles;
        a.n_row_tiles = (d.dst_h + a.tile_rows - 1) / a.tile_rows;
        a.tile_cols = std::min(256, round_up(d.dst_w, 32));
        for (;;) {
            // one column: weights [xt][cols], ring [yt][3][cols]; pair: weights [xt][cols/2] x 16 B, then
            // the ring sharing its bytes with the [xt][cols] table the weights are normalized from
            const int xw_words = (a.pair ? 2 : 1) * a.xt * a.tile_cols;
            const int ring_words = a.pair ? std::max(a.yt * 3, a.xt) * a.tile_cols : a.yt * 3 * a.tile_cols;
            a.smem_bytes = 4 * (xw_words + a.tile_rows * a.yt + 2 * a.tile_rows + ring_words);
            if (a.smem_bytes <= tlb::kAAMaxSmem || a.tile_cols <= 32) break;
            a.tile_cols = round_up(a.tile_cols / 2, 32);
        }
        a.n_col_tiles = (d.dst_w + a.tile_cols - 1) / a.tile_cols;
        if (a.smem_bytes > tlb::kAAMaxSmem)
            return fail(TLB_ERR_TOO_LARGE, "antialias: a %d-tap filter does not fit the shared-memory tables", std::max(a.xt, a.yt));
        a.grid = static_cast<long long>(d.n) * a.n_row_tiles * a.n_col_tiles;
        if (a.grid > 0x7fffffffll) return fail(TLB_ERR_TOO_LARGE, "antialias: too many tiles for one launch");
        const unsigned aflags = (honour_flags && (d.flags & TLB_FLAG_LAUNCH_OVERLAP)) ? tlb::kLaunchOverlap : 0u;
        cudaError_t e = static_cast<cudaError_t>(tlb::launch_antialias(p, a, d.out_dtype, d.out_layout, stream, aflags));
        if (e != cudaSuccess) return cuda_fail(e, "antialias_kernel launch");
        return TLB_OK;
    }
    if (honour_flags && (d.flags & TLB_FLAG_LAUNCH_OVERLAP)) streaming = true;
    if (int rc = make_plan(d, max_crop_w, p.plan, streaming)) return rc;
    const unsigned lflags = (honour_flags && (d.flags & TLB_FLAG_LAUNCH_OVERLAP)) ? tlb::kLaunchOverlap : 0u;
    // Identity size (no resampling) on a uniform dataset: a plain streaming kernel does the job.
    const bool uniform = !d.boxes && !d.src_sizes && !d.src_offsets;
    const int cw = d.uniform_box[2] > 0 ? d.uniform_box[2] : d.src_w;
    const int ch = d.uniform_box[2] > 0 ? d.uniform_box[3] : d.src_h;
    if (uniform && !d.jitter && cw == d.dst_w && ch == d.dst_h && env_int("TLB_IDENTITY_FAST", 1) != 0) {
        cudaError_t ce = static_cast<cudaError_t>(tlb::launch_normalize_copy(p, d.out_dtype, d.out_layout, stream, lflags));
        if (ce != cudaSuccess) return cuda_fail(ce, "normalize_copy_kernel launch");
        return TLB_OK;
    }
    cudaError_t e = static_cast<cudaError_t>(tlb::launch_fused(p, d.out_dtype, d.out_layout, stream, lflags));
    if (e != cudaSuccess) return cuda_fail(e, "fused_transform_kernel launch");
    return TLB_OK;
}

// ---- small persistent worker pool for host-side packing ---------------------------------
class Pool {
public:
    static Pool& get() {
        static Pool p;
        return p;
    }
    void run(size_t n, const std::function<void(size_t)>& fn) {
        if (n == 0) return;
        if (workers_.empty() || n == 1) {
            for (size_t i = 0; i < n; ++i) fn(i);
            return;
        }
        std::lock_guard<std::mutex> serial(run_mu_);
        {
            std::lock_guard<std::mutex> lk(mu_);
            fn_ = &fn;
            n_ = n;
            next_.store(0);
            busy_ = workers_.size();
            ++epoch_;
        }
        cv_.notify_all();
        drain();
        std::unique_lock<std::mutex> lk(mu_);
        done_cv_.wait(lk, [this] { return busy_ == 0; });
    }

private:
    Pool() {
        unsigned hc = std::thread::hardware_concurrency();
        unsigned want = std::min<unsigned>(hc > 1 ? hc - 1 : 0, 31);
        int cap = env_int("TLB_PACK_THREADS", 0);
        if (cap > 0) want = std::min<unsigned>(want, cap - 1);
        for (unsigned i = 0; i < want; ++i) workers_.emplace_back([this] { loop(); });
    }
    ~Pool() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stop_ = true;
        }
        cv_.notify_all();
        for (auto& t : workers_) t.join();
    }
    void drain() {
        for (;;) {
            size_t i = next_.fetch_add(1);
            if (i >= n_) break;
            (*fn_)(i);
        }
    }
    void loop() {
        unsigned long long seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return stop_ || epoch_ != seen; });
                if (stop_) return;
                seen = epoch_;
            }
            drain();
            std::lock_guard<std::mutex> lk(mu_);
            if (--busy_ == 0) done_cv_.notify_one();
        }
    }
    std::vector<std::thread> workers_;
    std::mutex run_mu_, mu_;
    std::condition_variable cv_, done_cv_;
    const std::function<void(size_t)>* fn_ = nullptr;
    size_t n_ = 0, busy_ = 0;
    std::atomic<size_t> next_{0};
    unsigned long long epoch_ = 0;
    bool stop_ = false;
};

struct IntBox {
    int x, y, w, h, flip;
};

int to_int_boxes(const tlb_image_ref* imgs, const tlb_crop_params* crops, int n, std::vector<IntBox>& out) {
    out.resize(n);
    for (int i = 0; i < n; ++i) {
        if (!imgs[i].data || imgs[i].w <= 0 || imgs[i].h <= 0)
            return fail(TLB_ERR_INVALID_ARG, "image %d: NULL data or non-positive size", i);
        IntBox b{0, 0, imgs[i].w, imgs[i].h, 0};
        if (crops) {
            const tlb_crop_params& c = crops[i];
            if (c.x != std::floor(c.x) || c.y != std::floor(c.y) || c.w != std::floor(c.w) || c.h != std::floor(c.h))
                return fail(TLB_ERR_INVALID_ARG, "crop %d: (%g,%g,%g,%g) must be whole pixels", i, c.x, c.y, c.w, c.h);
            b = IntBox{static_cast<int>(c.x), static_cast<int>(c.y), static_cast<int>(c.w), static_cast<int>(c.h), c.flip != 0};
            if (b.w <= 0 || b.h <= 0 || b.x < 0 || b.y < 0 || b.x > imgs[i].w - b.w || b.y > imgs[i].h - b.h)
                return fail(TLB_ERR_BAD_BOX, "crop %d: (%d,%d,%d,%d) leaves the %dx%d image", i, b.x, b.y, b.w, b.h, imgs[i].w, imgs[i].h);
        }
        out[i] = b;
    }
    return TLB_OK;
}

// Packs the crop rectangle of every host image (rows of cw*3 bytes, 16-byte aligned starts)
// plus the per-sample tables into one pinned buffer and uploads and launches it chunk by chunk.
bool allocation_range(const void* p, unsigned long long* base_out, size_t* size_out);

int host_images_to_device(const tlb_image_ref* imgs, const tlb_crop_params* crops, int n, int dst_h, int dst_w,
                          const float mean[3], const float std_[3], int normalize_01, void* out_dev, int out_dtype,
                          int out_layout, uint32_t* status_dev, cudaStream_t stream) {
    if (n <= 0) return fail(TLB_ERR_INVALID_ARG, "empty image list");
    if (!imgs || !mean || !std_ || !out_dev) return fail(TLB_ERR_INVALID_ARG, "NULL argument");
    int dev;
    if (int rc = current_device(&dev)) return rc;
    DeviceState& st = g_dev[dev];
    std::vector<IntBox> boxes;
    if (int rc = to_int_boxes(imgs, crops, n, boxes)) return rc;

    // ---- pinned sources: let the GPU gather the crop rows itself --------------------------------
    // When every image lies in page-locked, device-mapped host memory, no host packing is needed:
    // a small kernel reads exactly the crop rows across PCIe (host_gather.cu) into the device
    // half of the staging buffer, and the fused kernel follows on the same stream.
    if (env_int("TLB_HOST_GATHER", 1) != 0) {
        std::vector<tlb::GatherItem> items(n);
        bool mapped = true;
        size_t gpix = 0;
        unsigned max_rows = 1;
        int gmax_cw = 1;
        // An image that lies inside the mapped allocation found for the one before it needs no
        // query of its own: a decoded batch usually sits in one or a few page-locked buffers, and
        // one driver query per image was a twentieth of the whole call.
        unsigned long long known_lo = 0, known_hi = 0, known_delta = 0;  // host range; device - host address
        for (int i = 0; i < n && mapped; ++i) {
            const unsigned long long hp = reinterpret_cast<unsigned long long>(imgs[i].data);
            const unsigned long long img_bytes = static_cast<unsigned long long>(imgs[i].w) * imgs[i].h * 3ull;
            unsigned long long dp;
            if (hp >= known_lo && hp + img_bytes <= known_hi) {
                dp = hp + known_delta;
            } else {
                cudaPointerAttributes attr{};
                if (cudaPointerGetAttributes(&attr, imgs[i].data) != cudaSuccess) {
                    cudaGetLastError();
                    mapped = false;
                    break;
                }
                if ((attr.type != cudaMemoryTypeHost && attr.type != cudaMemoryTypeManaged) || !attr.devicePointer) {
                    mapped = false;
                    break;
                }
                dp = reinterpret_cast<unsigned long long>(attr.devicePointer);
                unsigned long long base = 0;
                size_t size = 0;
                known_lo = known_hi = 0;
                if (attr.type == cudaMemoryTypeHost && allocation_range(attr.devicePointer, &base, &size)) {
                    known_delta = dp - hp;
                    known_lo = base - known_delta;
                    known_hi = known_lo + size;
                }
            }
            const IntBox& b = boxes[i];
            const unsigned wpad = (static_cast<unsigned>(b.w) + 15u) & ~15u;  // packed row = whole pixels, 16-byte multiple
            items[i].src = dp + (static_cast<unsigned long long>(b.y) * imgs[i].w + b.x) * 3ull;
            items[i].dst_off = gpix;
            items[i].src_pitch = static_cast<unsigned>(imgs[i].w) * 3u;
            items[i].row_bytes = static_cast<unsigned>(b.w) * 3u;
            items[i].rows = static_cast<unsigned>(b.h);
            items[i].dst_pitch = wpad * 3u;
            gpix += static_cast<size_t>(wpad) * 3u * b.h;
            max_rows = std::max(max_rows, static_cast<unsigned>(b.h));
            gmax_cw = std::max(gmax_cw, b.w);
        }
        if (mapped && env_int("TLB_HOST_DIRECT", 1) != 0) {
            // Default: no staging at all.  The fused kernel's planner warps pull exactly the crop rows
            // they need out of the mapped host images with the same bulk copies they use on device
            // memory, so the transform runs at the rate the rows cross PCIe and the packed copy of the
            // crops in device memory (written, then read once) never exists.  The images are separate
            // host allocations: one base (the lowest address) plus offsets, and the kernel is told that
            // no load may leave an image.  Only the four small tables are uploaded.
            unsigned long long lo = ~0ull, hi = 0;
            int max_w = 1, max_h = 1;
            for (int i = 0; i < n; ++i) {
                const unsigned long long a = items[i].src - (static_cast<unsigned long long>(boxes[i].y) * imgs[i].w + boxes[i].x) * 3ull;
                lo = std::min(lo, a);
                hi = std::max(hi, a + static_cast<unsigned long long>(imgs[i].w) * imgs[i].h * 3ull);
                max_w = std::max(max_w, imgs[i].w);
                max_h = std::max(max_h, imgs[i].h);
            }
            const size_t box_tab = 0;
            const size_t off_tab = box_tab + 16 * size_t(n);
            const size_t size_tab = off_tab + 8 * size_t(n);
            const size_t flip_tab = size_tab + 8 * size_t(n);
            const size_t tab_bytes = flip_tab + size_t(n);
            std::unique_lock<std::mutex> lk(st.mu);
            Buffer& buf = st.params[st.params_next];
            st.params_next = (st.params_next + 1) % 4;
            if (int rc = grow(buf, tab_bytes)) return rc;
            lk.unlock();
            auto* hb = static_cast<unsigned char*>(buf.host);
            auto* db = static_cast<unsigned char*>(buf.dev);
            auto* h_box = reinterpret_cast<int*>(hb + box_tab);
            auto* h_off = reinterpret_cast<long long*>(hb + off_tab);
            auto* h_size = reinterpret_cast<int*>(hb + size_tab);
            for (int i = 0; i < n; ++i) {
                h_box[4 * i] = boxes[i].x;
                h_box[4 * i + 1] = boxes[i].y;
                h_box[4 * i + 2] = boxes[i].w;
                h_box[4 * i + 3] = boxes[i].h;
                const unsigned long long a = items[i].src - (static_cast<unsigned long long>(boxes[i].y) * imgs[i].w + boxes[i].x) * 3ull;
                h_off[i] = static_cast<long long>(a - lo);
                h_size[2 * i] = imgs[i].w;
                h_size[2 * i + 1] = imgs[i].h;
                hb[flip_tab + i] = static_cast<unsigned char>(boxes[i].flip);
            }
            TLB_CUDA(cudaMemcpyAsync(db, hb, tab_bytes, cudaMemcpyHostToDevice, stream));
            tlb_transform_desc d{};
            d.src = reinterpret_cast<const uint8_t*>(lo);
            d.src_bytes = hi - lo;
            d.n_src = n;
            d.src_offsets = reinterpret_cast<const int64_t*>(db + off_tab);
            d.src_sizes = reinterpret_cast<const int32_t*>(db + size_tab);
            d.src_w = max_w;
            d.src_h = max_h;
            d.n = n;
            d.boxes = reinterpret_cast<const int32_t*>(db + box_tab);
            d.flips = db + flip_tab;
            d.dst_h = dst_h;
            d.dst_w = dst_w;
            d.out = out_dev;
            d.out_dtype = out_dtype;
            d.out_layout = out_layout;
            for (int ch = 0; ch < 3; ++ch) {
                d.mean[ch] = mean[ch];
                d.std[ch] = std_[ch];
            }
            d.normalize_01 = normalize_01;
            d.max_crop_w = gmax_cw;
            d.status = status_dev;
            int rc = check_common(&d);
            if (rc == TLB_OK) rc = launch_desc(d, gmax_cw, stream, false, /*per_image_region=*/true);
            TLB_CUDA(cudaEventRecord(buf.done, stream));
            buf.pending = true;
            return rc;
        }
        if (mapped) {
            // TLB_HOST_DIRECT=0: a gather kernel packs the crop rows into device memory first.
            // Buffer layout: host half holds [boxes | offsets | sizes | flips | gather items]; the device
            // half holds the same tables followed by the gathered pixels.
            const size_t box_tab = 0;
            const size_t off_tab = box_tab + 16 * size_t(n);
            const size_t size_tab = off_tab + 8 * size_t(n);
            const size_t flip_tab = size_tab + 8 * size_t(n);
            const size_t item_tab = (flip_tab + n + 15) & ~static_cast<size_t>(15);
            const size_t tab_bytes = item_tab + sizeof(tlb::GatherItem) * size_t(n);
            const size_t pix_base = (tab_bytes + 255) & ~static_cast<size_t>(255);
            std::unique_lock<std::mutex> lk(st.mu);
            Buffer& buf = st.images[st.images_next];
            st.images_next ^= 1;
            if (int rc = grow(buf, pix_base + gpix)) return rc;
            lk.unlock();
            auto* hb = static_cast<unsigned char*>(buf.host);
            auto* db = static_cast<unsigned char*>(buf.dev);
            auto* h_box = reinterpret_cast<int*>(hb + box_tab);
            auto* h_off = reinterpret_cast<long long*>(hb + off_tab);
            auto* h_size = reinterpret_cast<int*>(hb + size_tab);
            for (int i = 0; i < n; ++i) {
                h_box[4 * i] = 0;
                h_box[4 * i + 1] = 0;
                h_box[4 * i + 2] = boxes[i].w;
                h_box[4 * i + 3] = boxes[i].h;
                h_off[i] = static_cast<long long>(items[i].dst_off);
                h_size[2 * i] = static_cast<int>(items[i].dst_pitch / 3u);
                h_size[2 * i + 1] = boxes[i].h;
                hb[flip_tab + i] = static_cast<unsigned char>(boxes[i].flip);
            }
            std::memcpy(hb + item_tab, items.data(), sizeof(tlb::GatherItem) * size_t(n));
            TLB_CUDA(cudaMemcpyAsync(db, hb, tab_bytes, cudaMemcpyHostToDevice, stream));
            cudaError_t ge = static_cast<cudaError_t>(tlb::launch_gather(
                reinterpret_cast<const tlb::GatherItem*>(db + item_tab), n, max_rows, db + pix_base, stream));
            if (ge != cudaSuccess) return cuda_fail(ge, "gather_crops_kernel launch");
            g_extra_launches.fetch_add(1, std::memory_order_relaxed);
            tlb_transform_desc d{};
            d.src = db + pix_base;
            d.src_bytes = gpix;
            d.n_src = n;
            d.src_offsets = reinterpret_cast<const int64_t*>(db + off_tab);
            d.src_sizes = reinterpret_cast<const int32_t*>(db + size_tab);
            d.n = n;
            d.boxes = reinterpret_cast<const int32_t*>(db + box_tab);
            d.flips = db + flip_tab;
            d.dst_h = dst_h;
            d.dst_w = dst_w;
            d.out = out_dev;
            d.out_dtype = out_dtype;
            d.out_layout = out_layout;
            for (int ch = 0; ch < 3; ++ch) {
                d.mean[ch] = mean[ch];
                d.std[ch] = std_[ch];
            }
            d.normalize_01 = normalize_01;
            d.max_crop_w = gmax_cw;
            d.status = status_dev;
            int rc = check_common(&d);
            if (rc == TLB_OK) rc = launch_desc(d, gmax_cw, stream);
            TLB_CUDA(cudaEventRecord(buf.done, stream));
            buf.pending = true;
            return rc;
        }
    }

    std::vector<long long> offs(n);
    size_t pix = 0;
    int max_cw = 1;
    for (int i = 0; i < n; ++i) {
        offs[i] = static_cast<long long>(pix);
        pix += (static_cast<size_t>(boxes[i].w) * boxes[i].h * 3 + 15) & ~static_cast<size_t>(15);
        max_cw = std::max(max_cw, boxes[i].w);
    }
    // Buffer layout: [boxes | offsets | sizes | flips | pixels].  The tables go up first, then the
    // batch is cut into chunks: while the DMA engine uploads chunk c the host threads pack chunk
    // c+1, and each chunk's kernel starts as soon as its own pixels have landed.
    const size_t box_tab = 0;                          // int32 boxes[n][4] (16-byte aligned per sample)
    const size_t off_tab = box_tab + 16 * size_t(n);   // int64 offsets[n]
    const size_t size_tab = off_tab + 8 * size_t(n);   // int32 sizes[n][2]
    const size_t flip_tab = size_tab + 8 * size_t(n);  // u8 flips[n]
    const size_t pix_base = (flip_tab + n + 255) & ~static_cast<size_t>(255);
    const size_t total = pix_base + pix;

    std::unique_lock<std::mutex> lk(st.mu);
    Buffer& buf = st.images[st.images_next];
    st.images_next ^= 1;
    if (int rc = grow(buf, total)) return rc;
    lk.unlock();

    auto* base = static_cast<unsigned char*>(buf.host);
    auto* h_off = reinterpret_cast<long long*>(base + off_tab);
    auto* h_size = reinterpret_cast<int*>(base + size_tab);
    auto* h_box = reinterpret_cast<int*>(base + box_tab);
    auto* h_flip = base + flip_tab;
    for (int i = 0; i < n; ++i) {
        h_off[i] = offs[i];
        h_size[2 * i] = boxes[i].w;
        h_size[2 * i + 1] = boxes[i].h;
        h_box[4 * i] = 0;
        h_box[4 * i + 1] = 0;
        h_box[4 * i + 2] = boxes[i].w;
        h_box[4 * i + 3] = boxes[i].h;
        h_flip[i] = static_cast<unsigned char>(boxes[i].flip);
    }
    auto* dbase = static_cast<unsigned char*>(buf.dev);
    TLB_CUDA(cudaMemcpyAsync(dbase, base, flip_tab + n, cudaMemcpyHostToDevice, stream));

    tlb_transform_desc d{};
    d.src = dbase + pix_base;
    d.src_bytes = pix;
    d.dst_h = dst_h;
    d.dst_w = dst_w;
    d.out_dtype = out_dtype;
    d.out_layout = out_layout;
    for (int c = 0; c < 3; ++c) {
        d.mean[c] = mean[c];
        d.std[c] = std_[c];
    }
    d.normalize_01 = normalize_01;
    d.max_crop_w = max_cw;
    d.status = status_dev;
    const size_t out_stride = static_cast<size_t>(3) * dst_h * dst_w * (out_dtype == TLB_F32 ? 4 : 2);

    const size_t chunk_bytes = static_cast<size_t>(std::max(1, env_int("TLB_H2D_CHUNK_MB", 8))) << 20;
    int rc = TLB_OK;
    for (int i0 = 0; i0 < n && rc == TLB_OK;) {
        int i1 = i0;
        const size_t start = static_cast<size_t>(offs[i0]);
        size_t end = start;
        while (i1 < n && (i1 == i0 || end - start < chunk_bytes)) {
            end = static_cast<size_t>(offs[i1]) +
                  ((static_cast<size_t>(boxes[i1].w) * boxes[i1].h * 3 + 15) & ~static_cast<size_t>(15));
            ++i1;
        }
        Pool::get().run(static_cast<size_t>(i1 - i0), [&](size_t j) {
            const size_t i = static_cast<size_t>(i0) + j;
            const IntBox& b = boxes[i];
            const unsigned char* s = imgs[i].data + (static_cast<size_t>(b.y) * imgs[i].w + b.x) * 3;
            unsigned char* dst = base + pix_base + offs[i];
            const size_t row = static_cast<size_t>(b.w) * 3, pitch = static_cast<size_t>(imgs[i].w) * 3;
            if (b.w == imgs[i].w) {
                std::memcpy(dst, s, row * b.h);
            } else {
                for (int y = 0; y < b.h; ++y) std::memcpy(dst + y * row, s + y * pitch, row);
            }
        });
        TLB_CUDA(cudaMemcpyAsync(dbase + pix_base + start, base + pix_base + start, end - start,
                                 cudaMemcpyHostToDevice, stream));
        // Samples i0 .. i1-1: their images are dataset entries 0 .. (i1-i0)-1 of the shifted tables.
        d.n = i1 - i0;
        d.n_src = i1 - i0;
        d.src_offsets = reinterpret_cast<const int64_t*>(dbase + off_tab) + i0;
        d.src_sizes = reinterpret_cast<const int32_t*>(dbase + size_tab) + 2 * i0;
        d.boxes = reinterpret_cast<const int32_t*>(dbase + box_tab) + 4 * i0;
        d.flips = dbase + flip_tab + i0;
        d.out = static_cast<unsigned char*>(out_dev) + static_cast<size_t>(i0) * out_stride;
        rc = check_common(&d);
        if (rc == TLB_OK) rc = launch_desc(d, max_cw, stream);
        i0 = i1;
    }
    // The buffer pair is reusable once the last kernel that reads the device half has finished.
    TLB_CUDA(cudaEventRecord(buf.done, stream));
    buf.pending = true;
    return rc;
}

int sync_host_form(const tlb_image_ref* imgs, const tlb_crop_params* crops, int n, int dst_h, int dst_w,
                   const float mean[3], const float std_[3], float* out_host) {
    if (!out_host) return fail(TLB_ERR_INVALID_ARG, "out is NULL");
    if (n <= 0 || dst_h <= 0 || dst_w <= 0) return fail(TLB_ERR_INVALID_ARG, "empty batch or non-positive size");
    int dev;
    if (int rc = current_device(&dev)) return rc;
    DeviceState& st = g_dev[dev];
    const size_t bytes = static_cast<size_t>(n) * 3 * dst_h * dst_w * sizeof(float);
    {
        std::lock_guard<std::mutex> lk(st.mu);
        if (!st.stream) TLB_CUDA(cudaStreamCreateWithFlags(&st.stream, cudaStreamNonBlocking));
        if (bytes > st.sync_out_cap) {
            if (st.sync_out) cudaFree(st.sync_out);
            st.sync_out = nullptr;
            st.sync_out_cap = 0;
            TLB_CUDA(cudaMalloc(&st.sync_out, bytes));
            st.sync_out_cap = bytes;
        }
    }
    if (int rc = host_images_to_device(imgs, crops, n, dst_h, dst_w, mean, std_, 1, st.sync_out, TLB_F32, TLB_NCHW,
                                       nullptr, st.stream))
        return rc;
    TLB_CUDA(cudaMemcpyAsync(out_host, st.sync_out, bytes, cudaMemcpyDeviceToHost, st.stream));
    TLB_CUDA(cudaStreamSynchronize(st.stream));
    return TLB_OK;
}

// Bytes that are readable from `p` to the end of the device allocation that contains it (the
// driver's cuMemGetAddressRange, reached through the runtime's entry-point lookup so that the
// library needs no link-time dependency on the driver).  Returns false when the driver cannot
// tell (not an allocation of the current context).
bool allocation_range(const void* p, unsigned long long* base_out, size_t* size_out) {
    using Fn = int (*)(unsigned long long*, size_t*, unsigned long long);
    static Fn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            sym = nullptr;
        }
        return reinterpret_cast<Fn>(sym);
    }();
    if (!fn) return false;
    unsigned long long base = 0;
    size_t size = 0;
    const unsigned long long a = reinterpret_cast<unsigned long long>(p);
    if (fn(&base, &size, a) != 0 || a < base || a >= base + size) return false;
    *base_out = base;
    *size_out = size;
    return true;
}

bool readable_extent(const void* p, size_t* bytes) {
    unsigned long long base = 0;
    size_t size = 0;
    if (!allocation_range(p, &base, &size)) return false;
    *bytes = static_cast<size_t>(base + size - reinterpret_cast<unsigned long long>(p));
    return true;
}

// Output slot of the pointer-returning forms: a 4-deep ring of library-owned device buffers.
int ring_slot(DeviceState& st, size_t bytes, void** out, int* slot_out) {
    const int slot = st.out_next;
    if (bytes > st.out_cap[slot]) {
        if (st.out_ring[slot]) cudaFree(st.out_ring[slot]);
        st.out_ring[slot] = nullptr;
        st.out_cap[slot] = 0;
        TLB_CUDA(cudaMalloc(&st.out_ring[slot], bytes));
        st.out_cap[slot] = bytes;
    }
    *out = st.out_ring[slot];
    *slot_out = slot;
    return TLB_OK;
}

uintptr_t resident_form(uintptr_t src_dev, uintptr_t sel_dev, bool gather, int n, int h, int w, const float mean[3],
                        const float std_[3]) {
    if (!src_dev || (gather && !sel_dev) || n <= 0 || h <= 0 || w <= 0 || !mean || !std_) {
        fail(TLB_ERR_INVALID_ARG, "resident normalize: NULL pointer or non-positive size");
        return 0;
    }
    int dev;
    if (current_device(&dev)) return 0;
    DeviceState& st = g_dev[dev];
    std::lock_guard<std::mutex> lk(st.mu);
    if (!st.stream && cudaStreamCreateWithFlags(&st.stream, cudaStreamNonBlocking) != cudaSuccess) {
        fail(TLB_ERR_CUDA, "cudaStreamCreate failed");
        return 0;
    }
    const size_t bytes = static_cast<size_t>(n) * 3 * h * w * sizeof(float);
    void* out = nullptr;
    int slot = 0;
    if (ring_slot(st, bytes, &out, &slot)) return 0;
    tlb_transform_desc d{};
    d.src = reinterpret_cast<const uint8_t*>(src_dev);
    // Without a gather the batch is the first n images at src_dev.  With one, this legacy signature
    // does not say how many images the dataset holds: the bound is the end of the device allocation
    // that contains src_dev (asked from the driver), so an index beyond it is reported
    // (TLB_DEV_BAD_INDEX, sample zero-filled) instead of read, and no row copy is rounded out past it.
    // Only when the driver cannot name the allocation are indices trusted, as in the function replaced.
    const size_t img_bytes = static_cast<size_t>(h) * w * 3;
    if (gather) {
        size_t extent = 0;
        if (readable_extent(d.src, &extent) && extent >= img_bytes) {
            d.n_src = static_cast<int64_t>(extent / img_bytes);
            d.src_bytes = static_cast<uint64_t>(d.n_src) * img_bytes;
        } else {
            d.n_src = 1ll << 40;
            d.src_bytes = ~0ull >> 1;
        }
    } else {
        d.n_src = n;
        d.src_bytes = static_cast<uint64_t>(n) * img_bytes;
    }
    d.src_w = w;
    d.src_h = h;
    d.n = n;
    d.sel = gather ? reinterpret_cast<const int64_t*>(sel_dev) : nullptr;
    d.dst_h = h;
    d.dst_w = w;
    d.out = out;
    d.out_dtype = TLB_F32;
    d.out_layout = TLB_NCHW;
    for (int c = 0; c < 3; ++c) {
        d.mean[c] = mean[c];
        d.std[c] = std_[c];
    }
    d.normalize_01 = 1;
    if (check_common(&d)) return 0;
    if (launch_desc(d, w, st.stream)) return 0;
    cudaError_t e = cudaStreamSynchronize(st.stream);
    if (e != cudaSuccess) {
        cuda_fail(e, "resident normalize");
        return 0;
    }
    st.out_next = (slot + 1) % 4;
    return reinterpret_cast<uintptr_t>(out);
}

// resize_normalize_device_batch: already-decoded images in SEPARATE device allocations.
uintptr_t device_images_form(const uintptr_t* d_imgs, const int32_t* ws, const int32_t* hs, int n, int dst_h, int dst_w,
                             const float mean[3], const float std_[3]) {
    if (!d_imgs || !ws || !hs || n <= 0 || dst_h <= 0 || dst_w <= 0 || !mean || !std_) {
        fail(TLB_ERR_INVALID_ARG, "resize_normalize_device_batch: NULL pointer, empty list or non-positive size");
        return 0;
    }
    int dev;
    if (current_device(&dev)) return 0;
    DeviceState& st = g_dev[dev];
    // One base + non-negative offsets: the lowest address is the base.  Every image is checked
    // against the device allocation that holds it, and the kernel is told that images are separate
    // regions, so that no load (not even the 16-byte round-out of a row copy) leaves an image.
    uintptr_t lo = ~static_cast<uintptr_t>(0), hi = 0;
    int max_w = 1;
    for (int i = 0; i < n; ++i) {
        if (!d_imgs[i] || ws[i] <= 0 || hs[i] <= 0 || static_cast<long long>(ws[i]) * hs[i] * 3 > 0x7fffffffll) {
            fail(TLB_ERR_INVALID_ARG, "resize_normalize_device_batch: image %d has a NULL address or a bad size", i);
            return 0;
        }
        const size_t bytes = static_cast<size_t>(ws[i]) * hs[i] * 3;
        size_t extent = 0;
        if (readable_extent(reinterpret_cast<const void*>(d_imgs[i]), &extent) && extent < bytes) {
            fail(TLB_ERR_BAD_INDEX, "resize_normalize_device_batch: image %d (%dx%d) does not fit its device allocation", i, ws[i], hs[i]);
            return 0;
        }
        lo = std::min(lo, d_imgs[i]);
        hi = std::max(hi, d_imgs[i] + bytes);
        max_w = std::max(max_w, ws[i]);
    }
    std::unique_lock<std::mutex> lk(st.mu);
    if (!st.stream && cudaStreamCreateWithFlags(&st.stream, cudaStreamNonBlocking) != cudaSuccess) {
        fail(TLB_ERR_CUDA, "cudaStreamCreate failed");
        return 0;
    }
    void* out = nullptr;
    int slot = 0;
    if (ring_slot(st, static_cast<size_t>(n) * 3 * dst_h * dst_w * sizeof(float), &out, &slot)) return 0;
    Buffer& buf = st.params[st.params_next];
    st.params_next = (st.params_next + 1) % 4;
    if (grow(buf, 16 * static_cast<size_t>(n))) return 0;
    auto* h_off = static_cast<long long*>(buf.host);
    auto* h_size = reinterpret_cast<int*>(static_cast<unsigned char*>(buf.host) + 8 * static_cast<size_t>(n));
    for (int i = 0; i < n; ++i) {
        h_off[i] = static_cast<long long>(d_imgs[i] - lo);
        h_size[2 * i] = ws[i];
        h_size[2 * i + 1] = hs[i];
    }
    if (cudaMemcpyAsync(buf.dev, buf.host, 16 * static_cast<size_t>(n), cudaMemcpyHostToDevice, st.stream) != cudaSuccess) {
        cuda_fail(cudaGetLastError(), "resize_normalize_device_batch: table upload");
        return 0;
    }
    tlb_transform_desc d{};
    d.src = reinterpret_cast<const uint8_t*>(lo);
    d.src_bytes = hi - lo;
    d.n_src = n;
    d.src_offsets = static_cast<const int64_t*>(buf.dev);
    d.src_sizes = reinterpret_cast<const int32_t*>(static_cast<unsigned char*>(buf.dev) + 8 * static_cast<size_t>(n));
    d.src_w = max_w;
    d.n = n;
    d.dst_h = dst_h;
    d.dst_w = dst_w;
    d.out = out;
    d.out_dtype = TLB_F32;
    d.out_layout = TLB_NCHW;
    for (int c = 0; c < 3; ++c) {
        d.mean[c] = mean[c];
        d.std[c] = std_[c];
    }
    d.normalize_01 = 1;
    d.max_crop_w = max_w;
    if (check_common(&d)) return 0;
    if (launch_desc(d, max_w, st.stream, false, /*per_image_region=*/true)) return 0;
    cudaError_t e = cudaStreamSynchronize(st.stream);  // also makes the pinned table buffer reusable
    if (e != cudaSuccess) {
        cuda_fail(e, "resize_normalize_device_batch");
        return 0;
    }
    st.out_next = (slot + 1) % 4;
    return reinterpret_cast<uintptr_t>(out);
}

}  // namespace

extern "C" {

int tlb_available(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return 0;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return 0;
    return major == 10 ? 1 : 0;  // the kernels are built for sm_100a only
}

int tlb_device_name(int device, char* buf, size_t cap) {
    if (!buf || cap == 0) return fail(TLB_ERR_INVALID_ARG, "buf is NULL or empty");
    buf[0] = 0;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(TLB_ERR_NO_DEVICE, "cudaGetDeviceProperties(%d): %s", device, cudaGetErrorString(e));
    }
    std::snprintf(buf, cap, "%s", prop.name);
    return TLB_OK;
}

const char* tlb_version(void) { return "turboloader_b200 0.1 (sm_100a)"; }

const char* tlb_last_error(void) { return t_err.c_str(); }

int tlb_fused_transform(const tlb_transform_desc* desc, void* stream) {
    if (int rc = check_common(desc)) return rc;
    if (desc->n == 0) return TLB_OK;
    const int mcw = derive_max_crop_w(*desc);
    if (mcw <= 0)
        return fail(TLB_ERR_INVALID_ARG, "max_crop_w is required when sizes and boxes are per-sample device tables");
    return launch_desc(*desc, mcw, stream, /*honour_flags=*/true);
}

int tlb_fused_transform_host_params(const tlb_transform_desc* desc, void* stream) {
    if (int rc = check_common(desc)) return rc;
    const tlb_transform_desc& d = *desc;
    if (d.n == 0) return TLB_OK;
    const int n = d.n;
    // ---- validate on the host -----------------------------------------------------------
    int max_cw = 0;
    for (int k = 0; k < n; ++k) {
        const long long s = d.sel ? d.sel[k] : k;
        if (s < 0 || s >= d.n_src) return fail(TLB_ERR_BAD_INDEX, "sample %d: gather index %lld outside [0, %lld)", k, s, static_cast<long long>(d.n_src));
        const int iw = d.src_sizes ? d.src_sizes[2 * s] : d.src_w;
        const int ih = d.src_sizes ? d.src_sizes[2 * s + 1] : d.src_h;
        int x = 0, y = 0, w = iw, h = ih;
        if (d.boxes) {
            x = d.boxes[4 * k]; y = d.boxes[4 * k + 1]; w = d.boxes[4 * k + 2]; h = d.boxes[4 * k + 3];
        } else if (d.uniform_box[2] > 0) {
            x = d.uniform_box[0]; y = d.uniform_box[1]; w = d.uniform_box[2]; h = d.uniform_box[3];
        }
        if (iw <= 0 || ih <= 0 || w <= 0 || h <= 0 || x < 0 || y < 0 || x > iw - w || y > ih - h)
            return fail(TLB_ERR_BAD_BOX, "sample %d: box (%d,%d,%d,%d) leaves the %dx%d image", k, x, y, w, h, iw, ih);
        const long long off = d.src_offsets ? d.src_offsets[s] : s * (static_cast<long long>(iw) * ih * 3);
        if (off < 0 || static_cast<unsigned long long>(off) + static_cast<unsigned long long>(iw) * ih * 3 > d.src_bytes)
            return fail(TLB_ERR_BAD_INDEX, "sample %d: image %lld lies outside the %llu readable bytes", k, s, static_cast<unsigned long long>(d.src_bytes));
        max_cw = std::max(max_cw, w);
    }
    // ---- upload the tables ---------------------------------------------------------------
    int dev;
    if (int rc = current_device(&dev)) return rc;
    DeviceState& st = g_dev[dev];
    const size_t ns = static_cast<size_t>(d.n_src);
    size_t off_sel = 0, off_box = 0, off_flip = 0, off_offs = 0, off_sizes = 0, total = 0;
    auto reserve = [&](size_t bytes) { size_t o = total; total = (total + bytes + 15) & ~static_cast<size_t>(15); return o; };
    if (d.sel) off_sel = reserve(8 * size_t(n));
    if (d.boxes) off_box = reserve(16 * size_t(n));
    if (d.flips) off_flip = reserve(size_t(n));
    if (d.src_offsets) off_offs = reserve(8 * ns);
    if (d.src_sizes) off_sizes = reserve(8 * ns);
    tlb_transform_desc dd = d;
    if (total) {
        std::unique_lock<std::mutex> lk(st.mu);
        Buffer& buf = st.params[st.params_next];
        st.params_next = (st.params_next + 1) % 4;
        if (int rc = grow(buf, total)) return rc;
        lk.unlock();
        auto* hb = static_cast<unsigned char*>(buf.host);
        auto* db = static_cast<unsigned char*>(buf.dev);
        if (d.sel) { std::memcpy(hb + off_sel, d.sel, 8 * size_t(n)); dd.sel = reinterpret_cast<const int64_t*>(db + off_sel); }
        if (d.boxes) { std::memcpy(hb + off_box, d.boxes, 16 * size_t(n)); dd.boxes = reinterpret_cast<const int32_t*>(db + off_box); }
        if (d.flips) { std::memcpy(hb + off_flip, d.flips, size_t(n)); dd.flips = db + off_flip; }
        if (d.src_offsets) { std::memcpy(hb + off_offs, d.src_offsets, 8 * ns); dd.src_offsets = reinterpret_cast<const int64_t*>(db + off_offs); }
        if (d.src_sizes) { std::memcpy(hb + off_sizes, d.src_sizes, 8 * ns); dd.src_sizes = reinterpret_cast<const int32_t*>(db + off_sizes); }
        cudaStream_t cs = static_cast<cudaStream_t>(stream);
        TLB_CUDA(cudaMemcpyAsync(buf.dev, buf.host, total, cudaMemcpyHostToDevice, cs));
        const int rc = launch_desc(dd, max_cw, stream);
        // Reusable once the kernel that reads the device half has finished.
        TLB_CUDA(cudaEventRecord(buf.done, cs));
        buf.pending = true;
        return rc;
    }
    return launch_desc(dd, max_cw, stream);
}

int tlb_resize_normalize_batch(const tlb_image_ref* imgs, int32_t n, int32_t dst_h, int32_t dst_w, const float mean[3],
                               const float std_[3], float* out_host) {
    return sync_host_form(imgs, nullptr, n, dst_h, dst_w, mean, std_, out_host);
}

int tlb_crop_resize_normalize_batch(const tlb_image_ref* imgs, const tlb_crop_params* crops, int32_t n, int32_t dst_h,
                                    int32_t dst_w, const float mean[3], const float std_[3], float* out_host) {
    if (!crops) return fail(TLB_ERR_INVALID_ARG, "crops is NULL");
    return sync_host_form(imgs, crops, n, dst_h, dst_w, mean, std_, out_host);
}

int tlb_crop_resize_normalize_to_device(const tlb_image_ref* imgs, const tlb_crop_params* crops, int32_t n,
                                        int32_t dst_h, int32_t dst_w, const float mean[3], const float std_[3],
                                        int32_t normalize_01, void* out_dev, int32_t out_dtype, int32_t out_layout,
                                        uint32_t* status_dev, void* stream) {
    if (dst_h <= 0 || dst_w <= 0) return fail(TLB_ERR_INVALID_ARG, "dst size must be positive");
    return host_images_to_device(imgs, crops, n, dst_h, dst_w, mean, std_, normalize_01, out_dev, out_dtype, out_layout,
                                 status_dev, static_cast<cudaStream_t>(stream));
}

uintptr_t tlb_normalize_resident_batch(uintptr_t src_dev, int32_t n, int32_t h, int32_t w, const float mean[3],
                                       const float std_[3]) {
    return resident_form(src_dev, 0, false, n, h, w, mean, std_);
}

uintptr_t tlb_normalize_resident_gather_batch(uintptr_t src_dev, uintptr_t sel_dev, int32_t n, int32_t h, int32_t w,
                                              const float mean[3], const float std_[3]) {
    return resident_form(src_dev, sel_dev, true, n, h, w, mean, std_);
}

uintptr_t tlb_resize_normalize_device_batch(const uintptr_t* d_imgs, const int32_t* ws, const int32_t* hs, int32_t n,
                                            int32_t dst_h, int32_t dst_w, const float mean[3], const float std_[3]) {
    return device_images_form(d_imgs, ws, hs, n, dst_h, dst_w, mean, std_);
}

int tlb_fused_plan(const tlb_transform_desc* desc, int32_t* grid, int32_t* block, int32_t* smem_bytes,
                   int32_t* tile_rows, int32_t* tile_cols) {
    if (int rc = check_common(desc)) return rc;
    const int mcw = derive_max_crop_w(*desc);
    if (mcw <= 0) return fail(TLB_ERR_INVALID_ARG, "max_crop_w is required");
    tlb::Plan pl{};
    if (int rc = make_plan(*desc, mcw, pl, (desc->flags & TLB_FLAG_LAUNCH_OVERLAP) != 0)) return rc;
    if (grid) *grid = static_cast<int32_t>(pl.grid);
    if (block) *block = 32 * (pl.strips + 1);
    if (smem_bytes) *smem_bytes = pl.smem_bytes;
    if (tile_rows) *tile_rows = pl.tile_rows;
    if (tile_cols) *tile_cols = pl.tile_cols;
    return TLB_OK;
}

uint64_t tlb_launch_count(void) {
    return tlb::launch_count() + tlb::video_launch_count() + tlb::antialias_launch_count() + tlb::normalize_copy_launch_count() +
           g_extra_launches.load(std::memory_order_relaxed);
}

}  // extern "C"

// ---- allocation-free host-image entry point ------------------------------------------------
// Some callers may not allocate when they call us: a loader thread inside a process whose
// device memory is already fully committed to a training pool, a host that forbids
// allocation after start-up, a GPU shared under a fixed memory budget.  For them the device
// staging that tlb_crop_resize_normalize_to_device takes from a growable ring lives here in
// one fixed array of the library image, and the tables are built in a fixed host buffer.
namespace {

// Device scratch shared by every call on a device; it keeps the last call's bytes.  In host
// code this name is only a handle for the symbol, not a device address: the address each
// device gave the array is looked up once with cudaGetSymbolAddress (below) and passed to the
// kernel as its source pointer.
static __device__ __align__(256) unsigned char g_static_scratch[TLB_STATIC_SCRATCH_BYTES];

unsigned char* g_static_addr[kMaxDevices] = {};  // device address of g_static_scratch, per device
std::mutex g_static_mu;

// Fixed host-side staging for the per-sample tables (no heap use on the success path).
struct StaticTables {
    long long offs[TLB_STATIC_MAX_SAMPLES];
    int sizes[2 * TLB_STATIC_MAX_SAMPLES];
    int boxes[4 * TLB_STATIC_MAX_SAMPLES];
    unsigned char flips[TLB_STATIC_MAX_SAMPLES];
    IntBox rect[TLB_STATIC_MAX_SAMPLES];
};
StaticTables g_static_tables;

// First use on a device, with that device current: find where the array lives there.
int static_scratch_address(int dev, unsigned char** out) {
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_addr[dev]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        g_static_addr[dev] = static_cast<unsigned char*>(ptr);
    }
    *out = g_static_addr[dev];
    return TLB_OK;
}

}  // namespace

extern "C" {

int tlb_crop_resize_normalize_to_device_static(const tlb_image_ref* imgs, const tlb_crop_params* crops, int32_t n,
                                               int32_t dst_h, int32_t dst_w, const float mean[3],
                                               const float std_[3], int32_t normalize_01, void* out_dev,
                                               int32_t out_dtype, int32_t out_layout, uint32_t* status_dev,
                                               void* stream) {
    if (n <= 0) return fail(TLB_ERR_INVALID_ARG, "empty image list");
    if (!imgs || !mean || !std_ || !out_dev) return fail(TLB_ERR_INVALID_ARG, "NULL argument");
    if (dst_h <= 0 || dst_w <= 0) return fail(TLB_ERR_INVALID_ARG, "dst size must be positive");
    if (n > TLB_STATIC_MAX_SAMPLES)
        return fail(TLB_ERR_TOO_LARGE, "n = %d exceeds the %d samples the allocation-free entry point supports", n,
                    TLB_STATIC_MAX_SAMPLES);
    // One call at a time fills the shared host table buffer: the lock is held until the tables have
    // been handed to the copy engine (uploads from pageable host memory are staged before
    // cudaMemcpyAsync returns), so two host threads driving two different GPUs do not mix tables.
    static std::mutex tables_mu;
    std::lock_guard<std::mutex> tables_lock(tables_mu);
    StaticTables& t = g_static_tables;
    // ---- validate every crop on the host and lay the packed crops out ------------------------
    size_t pix = 0;
    int max_cw = 1;
    for (int i = 0; i < n; ++i) {
        if (!imgs[i].data || imgs[i].w <= 0 || imgs[i].h <= 0)
            return fail(TLB_ERR_INVALID_ARG, "image %d: NULL data or non-positive size", i);
        IntBox b{0, 0, imgs[i].w, imgs[i].h, 0};
        if (crops) {
            const tlb_crop_params& c = crops[i];
            if (c.x != std::floor(c.x) || c.y != std::floor(c.y) || c.w != std::floor(c.w) || c.h != std::floor(c.h))
                return fail(TLB_ERR_INVALID_ARG, "crop %d: (%g,%g,%g,%g) must be whole pixels", i, c.x, c.y, c.w, c.h);
            b = IntBox{static_cast<int>(c.x), static_cast<int>(c.y), static_cast<int>(c.w), static_cast<int>(c.h), c.flip != 0};
            if (b.w <= 0 || b.h <= 0 || b.x < 0 || b.y < 0 || b.x > imgs[i].w - b.w || b.y > imgs[i].h - b.h)
                return fail(TLB_ERR_BAD_BOX, "crop %d: (%d,%d,%d,%d) leaves the %dx%d image", i, b.x, b.y, b.w, b.h, imgs[i].w, imgs[i].h);
        }
        t.rect[i] = b;
        t.offs[i] = static_cast<long long>(pix);
        t.sizes[2 * i] = b.w;
        t.sizes[2 * i + 1] = b.h;
        t.boxes[4 * i] = 0;
        t.boxes[4 * i + 1] = 0;
        t.boxes[4 * i + 2] = b.w;
        t.boxes[4 * i + 3] = b.h;
        t.flips[i] = static_cast<unsigned char>(b.flip);
        pix += (static_cast<size_t>(b.w) * b.h * 3 + 15) & ~static_cast<size_t>(15);
        max_cw = std::max(max_cw, b.w);
    }
    const size_t off_tab = pix;                        // int64 offsets[n]
    const size_t size_tab = off_tab + 8 * size_t(n);   // int32 sizes[n][2]
    const size_t box_tab = size_tab + 8 * size_t(n);   // int32 boxes[n][4]
    const size_t flip_tab = box_tab + 16 * size_t(n);  // u8 flips[n]
    const size_t total = (flip_tab + n + 15) & ~static_cast<size_t>(15);
    if (total > TLB_STATIC_SCRATCH_BYTES)
        return fail(TLB_ERR_TOO_LARGE,
                    "batch needs %zu bytes of device staging; the allocation-free entry point has %u (use "
                    "tlb_crop_resize_normalize_to_device or split the batch)",
                    total, static_cast<unsigned>(TLB_STATIC_SCRATCH_BYTES));
    // ---- one-time set-up on this device (no allocation: address look-up + kernel attributes) --
    int dev;
    if (int rc = current_device(&dev)) return rc;
    unsigned char* base = nullptr;
    if (int rc = static_scratch_address(dev, &base)) return rc;
    if (int rc = ensure_prepared(g_dev[dev])) return rc;
    // ---- copy the crop rectangles straight from the caller's memory, then the tables ----------
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    for (int i = 0; i < n; ++i) {
        const IntBox& b = t.rect[i];
        const unsigned char* src = imgs[i].data + (static_cast<size_t>(b.y) * imgs[i].w + b.x) * 3;
        TLB_CUDA(cudaMemcpy2DAsync(base + t.offs[i], static_cast<size_t>(b.w) * 3, src, static_cast<size_t>(imgs[i].w) * 3,
                                   static_cast<size_t>(b.w) * 3, static_cast<size_t>(b.h), cudaMemcpyHostToDevice, cs));
    }
    TLB_CUDA(cudaMemcpyAsync(base + off_tab, t.offs, 8 * size_t(n), cudaMemcpyHostToDevice, cs));
    TLB_CUDA(cudaMemcpyAsync(base + size_tab, t.sizes, 8 * size_t(n), cudaMemcpyHostToDevice, cs));
    TLB_CUDA(cudaMemcpyAsync(base + box_tab, t.boxes, 16 * size_t(n), cudaMemcpyHostToDevice, cs));
    TLB_CUDA(cudaMemcpyAsync(base + flip_tab, t.flips, size_t(n), cudaMemcpyHostToDevice, cs));

    tlb_transform_desc d{};
    d.src = base;
    d.src_bytes = pix;
    d.n_src = n;
    d.src_offsets = reinterpret_cast<const int64_t*>(base + off_tab);
    d.src_sizes = reinterpret_cast<const int32_t*>(base + size_tab);
    d.n = n;
    d.boxes = reinterpret_cast<const int32_t*>(base + box_tab);
    d.flips = base + flip_tab;
    d.dst_h = dst_h;
    d.dst_w = dst_w;
    d.out = out_dev;
    d.out_dtype = out_dtype;
    d.out_layout = out_layout;
    for (int c = 0; c < 3; ++c) {
        d.mean[c] = mean[c];
        d.std[c] = std_[c];
    }
    d.normalize_01 = normalize_01;
    d.max_crop_w = max_cw;
    d.status = status_dev;
    if (int rc = check_common(&d)) return rc;
    return launch_desc(d, max_cw, stream);
}

}  // extern "C"

namespace {

// ---- YUV 4:2:0 video ------------------------------------------------------------------------
int check_video(const tlb_video_desc* d) {
    if (!d) return fail(TLB_ERR_INVALID_ARG, "video descriptor is NULL");
    if (d->n < 0) return fail(TLB_ERR_INVALID_ARG, "n < 0");
    if (d->n == 0) return TLB_OK;
    if (!d->y_ptrs || !d->cb_ptrs || !d->cr_ptrs || !d->out)
        return fail(TLB_ERR_INVALID_ARG, "video: a plane address array or the output is NULL");
    if (d->src_w <= 0 || d->src_h <= 0 || d->dst_w <= 0 || d->dst_h <= 0)
        return fail(TLB_ERR_INVALID_ARG, "video: non-positive frame or output size");
    if (d->c_px_stride != 1 && d->c_px_stride != 2)
        return fail(TLB_ERR_INVALID_ARG, "video: c_px_stride must be 1 (I420) or 2 (NV12)");
    if (d->y_stride < d->src_w || d->c_stride < ((d->src_w + 1) / 2 - 1) * d->c_px_stride + 1)
        return fail(TLB_ERR_INVALID_ARG, "video: a row stride is shorter than the row");
    if (static_cast<long long>(d->y_stride) * d->src_h > 0x7fffffffll)
        return fail(TLB_ERR_TOO_LARGE, "video: a plane exceeds 2 GiB");
    if (d->out_dtype != TLB_F32 && d->out_dtype != TLB_BF16) return fail(TLB_ERR_INVALID_ARG, "video: bad out_dtype");
    if (d->clip_len < 0) return fail(TLB_ERR_INVALID_ARG, "video: clip_len < 0");
    if (d->n > 65535) return fail(TLB_ERR_TOO_LARGE, "video: at most 65535 frames per call");
    for (int c = 0; c < 3; ++c)
        if (!(d->std[c] != 0.0f) || !std::isfinite(d->std[c]) || !std::isfinite(d->mean[c]))
            return fail(TLB_ERR_INVALID_ARG, "video: std must be finite and non-zero, mean finite");
    for (int i = 0; i < d->n; ++i)
        if (!d->y_ptrs[i] || !d->cb_ptrs[i] || !d->cr_ptrs[i])
            return fail(TLB_ERR_INVALID_ARG, "video: frame %d has a NULL plane address", i);
    if (d->flags & ~static_cast<uint32_t>(TLB_FLAG_LAUNCH_OVERLAP)) return fail(TLB_ERR_INVALID_ARG, "video: unknown bits in flags: 0x%x", d->flags);
    if (d->crops) {
        const int clips = d->clip_len > 0 ? (d->n + d->clip_len - 1) / d->clip_len : 1;
        for (int i = 0; i < 4 * clips; ++i)
            if (!std::isfinite(d->crops[i])) return fail(TLB_ERR_BAD_BOX, "video: a crop window is not finite");
    }
    return TLB_OK;
}

int video_enqueue(const tlb_video_desc& d, void* stream) {
    int dev;
    if (int rc = current_device(&dev)) return rc;
    DeviceState& st = g_dev[dev];
    if (int rc = ensure_prepared(st)) return rc;
    const size_t n = static_cast<size_t>(d.n);
    const size_t clips = d.crops ? (d.clip_len > 0 ? (n + d.clip_len - 1) / d.clip_len : 1) : 0;
    const bool staged = env_int("TLB_VIDEO_STAGED", 0) != 0;
    if (!staged && n <= static_cast<size_t>(tlb::kVideoInlineFrames) && clips <= static_cast<size_t>(tlb::kVideoInlineClips) &&
        env_int("TLB_VIDEO_INLINE_TABLES", 1) != 0) {
        // Small batch: the tables travel in the parameter block; nothing is uploaded, no staging
        // buffer is touched, and the launch follows the previous one in its stream directly.
        static thread_local tlb::VideoParams p;  // ~7 KB: kept off the stack
        p = tlb::VideoParams{};
        p.inline_tables = 1;
        for (size_t i = 0; i < n; ++i) {
            p.in.planes[i] = reinterpret_cast<const unsigned char*>(d.y_ptrs[i]);
            p.in.planes[n + i] = reinterpret_cast<const unsigned char*>(d.cb_ptrs[i]);
            p.in.planes[2 * n + i] = reinterpret_cast<const unsigned char*>(d.cr_ptrs[i]);
        }
        p.has_crops = clips ? 1 : 0;
        p.has_flips = (clips && d.flips) ? 1 : 0;
        for (size_t i = 0; i < clips; ++i) {
            p.in.crops[i] = make_float4(d.crops[4 * i], d.crops[4 * i + 1], d.crops[4 * i + 2], d.crops[4 * i + 3]);
            p.in.flips[i] = d.flips ? (d.flips[i] != 0) : 0;
        }
        p.n = d.n;
        p.clip_len = d.clip_len;
        p.y_stride = d.y_stride; p.c_stride = d.c_stride; p.c_px_stride = d.c_px_stride;
        p.src_w = d.src_w; p.src_h = d.src_h; p.dst_w = d.dst_w; p.dst_h = d.dst_h;
        p.bt709 = d.bt709 ? 1 : 0;
        for (int c = 0; c < 3; ++c) {
            p.mean[c] = d.mean[c];
            p.inv_std[c] = 1.0f / d.std[c];  // cuda_transforms.cu:392 computes the reciprocal on the host, in fp32
        }
        p.one = 1.0f;
        p.out = d.out;
        p.status = d.status;
        const unsigned lflags = (d.flags & TLB_FLAG_LAUNCH_OVERLAP) ? tlb::kLaunchOverlap : 0u;
        cudaError_t e = static_cast<cudaError_t>(tlb::launch_video(p, d.out_dtype, stream, lflags));
        if (e != cudaSuccess) return cuda_fail(e, "yuv420_kernel launch");
        return TLB_OK;
    }
    const size_t off_crop = (3 * n * sizeof(void*) + 15) & ~static_cast<size_t>(15);
    const size_t off_flip = off_crop + clips * 16;
    const size_t total = off_flip + clips * 4;
    std::unique_lock<std::mutex> lk(st.mu);
    Buffer& buf = st.params[st.params_next];
    st.params_next = (st.params_next + 1) % 4;
    if (int rc = grow(buf, total)) return rc;
    lk.unlock();
    auto* hb = static_cast<unsigned char*>(buf.host);
    auto* db = static_cast<unsigned char*>(buf.dev);
    auto* hp = reinterpret_cast<uintptr_t*>(hb);
    for (size_t i = 0; i < n; ++i) {
        hp[i] = d.y_ptrs[i];
        hp[n + i] = d.cb_ptrs[i];
        hp[2 * n + i] = d.cr_ptrs[i];
    }
    if (clips) {
        std::memcpy(hb + off_crop, d.crops, clips * 16);
        auto* hf = reinterpret_cast<int*>(hb + off_flip);
        for (size_t i = 0; i < clips; ++i) hf[i] = d.flips ? (d.flips[i] != 0) : 0;
    }
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    TLB_CUDA(cudaMemcpyAsync(buf.dev, buf.host, total, cudaMemcpyHostToDevice, cs));
    tlb::VideoParams p{};
    p.planes = reinterpret_cast<const unsigned char* const*>(db);
    p.crops = clips ? reinterpret_cast<const float4*>(db + off_crop) : nullptr;
    p.flips = clips ? reinterpret_cast<const int*>(db + off_flip) : nullptr;
    p.n = d.n;
    p.clip_len = d.clip_len;
    p.y_stride = d.y_stride; p.c_stride = d.c_stride; p.c_px_stride = d.c_px_stride;
    p.src_w = d.src_w; p.src_h = d.src_h; p.dst_w = d.dst_w; p.dst_h = d.dst_h;
    p.bt709 = d.bt709 ? 1 : 0;
    for (int c = 0; c < 3; ++c) {
        p.mean[c] = d.mean[c];
        p.inv_std[c] = 1.0f / d.std[c];  // cuda_transforms.cu:392 computes the reciprocal on the host, in fp32
    }
    p.one = 1.0f;
    p.out = d.out;
    p.status = d.status;
    p.use_staged = staged ? 1 : 0;
    cudaError_t e = static_cast<cudaError_t>(tlb::launch_video(p, d.out_dtype, stream, 0u));
    TLB_CUDA(cudaEventRecord(buf.done, cs));
    buf.pending = true;
    if (e != cudaSuccess) return cuda_fail(e, "yuv420_kernel launch");
    return TLB_OK;
}

uintptr_t video_pointer_form(tlb_video_desc d) {
    d.out = reinterpret_cast<void*>(1);  // placeholder so that validation sees a non-NULL output
    d.out_dtype = TLB_F32;
    if (d.n <= 0) {
        fail(TLB_ERR_INVALID_ARG, "video: no frames");
        return 0;
    }
    if (check_video(&d)) return 0;
    int dev;
    if (current_device(&dev)) return 0;
    DeviceState& st = g_dev[dev];
    void* out;
    {
        std::lock_guard<std::mutex> lk(st.mu);
        if (!st.stream && cudaStreamCreateWithFlags(&st.stream, cudaStreamNonBlocking) != cudaSuccess) {
            fail(TLB_ERR_CUDA, "cudaStreamCreate failed");
            return 0;
        }
        const size_t bytes = static_cast<size_t>(d.n) * 3 * d.dst_h * d.dst_w * sizeof(float);
        st.video_next ^= 1;
        const int slot = st.video_next;
        if (bytes > st.video_cap[slot]) {
            if (st.video_out[slot]) cudaFree(st.video_out[slot]);
            st.video_out[slot] = nullptr;
            st.video_cap[slot] = 0;
            cudaError_t e = cudaMalloc(&st.video_out[slot], bytes);
            if (e != cudaSuccess) {
                cuda_fail(e, "cudaMalloc(video output)");
                return 0;
            }
            st.video_cap[slot] = bytes;
        }
        out = st.video_out[slot];
    }
    d.out = out;
    if (video_enqueue(d, st.stream)) return 0;
    cudaError_t e = cudaStreamSynchronize(st.stream);
    if (e != cudaSuccess) {
        cuda_fail(e, "cudaStreamSynchronize(video)");
        return 0;
    }
    return reinterpret_cast<uintptr_t>(out);
}

}  // namespace

extern "C" {

int tlb_video_yuv420(const tlb_video_desc* desc, void* stream) {
    if (int rc = check_video(desc)) return rc;
    if (desc->n == 0) return TLB_OK;
    return video_enqueue(*desc, stream);
}

uintptr_t tlb_video_yuv420_batch(const uintptr_t* y_ptrs, const uintptr_t* cb_ptrs, const uintptr_t* cr_ptrs,
                                 int32_t n, int32_t y_stride, int32_t c_stride, int32_t c_px_stride, int32_t src_w,
                                 int32_t src_h, int32_t dst_h, int32_t dst_w, int32_t bt709, const float mean[3],
                                 const float std_[3]) {
    if (!mean || !std_) {
        fail(TLB_ERR_INVALID_ARG, "video: mean/std is NULL");
        return 0;
    }
    tlb_video_desc d{};
    d.y_ptrs = y_ptrs; d.cb_ptrs = cb_ptrs; d.cr_ptrs = cr_ptrs; d.n = n;
    d.y_stride = y_stride; d.c_stride = c_stride; d.c_px_stride = c_px_stride;
    d.src_w = src_w; d.src_h = src_h; d.dst_h = dst_h; d.dst_w = dst_w; d.bt709 = bt709;
    for (int c = 0; c < 3; ++c) { d.mean[c] = mean[c]; d.std[c] = std_[c]; }
    return video_pointer_form(d);
}

uintptr_t tlb_video_clip_yuv420(const uintptr_t* y_ptrs, const uintptr_t* cb_ptrs, const uintptr_t* cr_ptrs, int32_t n,
                                int32_t y_stride, int32_t c_stride, int32_t c_px_stride, int32_t src_w, int32_t src_h,
                                int32_t dst_h, int32_t dst_w, const float crop[4], int32_t flip, int32_t bt709,
                                const float mean[3], const float std_[3]) {
    if (!mean || !std_ || !crop) {
        fail(TLB_ERR_INVALID_ARG, "video: mean/std/crop is NULL");
        return 0;
    }
    tlb_video_desc d{};
    d.y_ptrs = y_ptrs; d.cb_ptrs = cb_ptrs; d.cr_ptrs = cr_ptrs; d.n = n;
    d.y_stride = y_stride; d.c_stride = c_stride; d.c_px_stride = c_px_stride;
    d.src_w = src_w; d.src_h = src_h; d.dst_h = dst_h; d.dst_w = dst_w; d.bt709 = bt709;
    d.crops = crop;
    d.flips = &flip;
    d.clip_len = 0;
    for (int c = 0; c < 3; ++c) { d.mean[c] = mean[c]; d.std[c] = std_[c]; }
    return video_pointer_form(d);
}

}  // extern "C"

// ---- streaming core: datasets larger than device memory ------------------------------------
// Replaces CudaStreamCore (src/cuda/cuda_transforms.cu:629-780): the uint8 dataset stays in
// (pinned) host memory and is streamed batch by batch.  The reference drives K slots with K worker
// threads that block on their own streams; here nothing blocks and there are no threads: a slot is
// a device staging buffer + output buffer + stream, one contiguous asynchronous copy and one fused
// kernel are enqueued per batch, K-1 batches ahead of the consumer, and a batch is handed over
// either by an event the consumer's stream waits on (no host synchronisation at all) or, without
// a consumer stream, by waiting for that event on the host as the reference does.
struct tlb_stream_core {
    int dev = 0;
    const uint8_t* host = nullptr;
    int64_t n = 0;
    int h = 0, w = 0, batch = 0, slots = 0;
    int out_h = 0, out_w = 0;
    int crop[4] = {0, 0, 0, 0};
    bool drop_last = true;
    int out_dtype = TLB_F32, out_layout = TLB_NCHW;
    float mean[3] = {0, 0, 0}, std_[3] = {1, 1, 1};
    int64_t n_batches = 0;
    int64_t enqueued = 0;  // batches enqueued this epoch
    int64_t returned = 0;  // batches handed to the consumer this epoch
    std::vector<void*> d_in, d_out;
    std::vector<cudaStream_t> streams;
    std::vector<cudaEvent_t> ready;   // slot's kernel finished
    cudaEvent_t consumed = nullptr;   // consumer stream's position at the latest next() call
    uint32_t* status = nullptr;       // device word
};

namespace {

int stream_enqueue(tlb_stream_core* c, void* consumer_stream) {
    const int64_t b = c->enqueued;
    const int slot = static_cast<int>(b % c->slots);
    const int64_t first = b * c->batch;
    const int nb = static_cast<int>(std::min<int64_t>(c->batch, c->n - first));
    cudaStream_t st = c->streams[slot];
    // The slot's previous output may still be in use by work the consumer enqueued before this
    // call: order this slot's stream behind the consumer stream's current position.
    if (consumer_stream) {
        TLB_CUDA(cudaEventRecord(c->consumed, static_cast<cudaStream_t>(consumer_stream)));
        TLB_CUDA(cudaStreamWaitEvent(st, c->consumed, 0));
    }
    const size_t img = static_cast<size_t>(c->h) * c->w * 3;
    TLB_CUDA(cudaMemcpyAsync(c->d_in[slot], c->host + first * img, nb * img, cudaMemcpyHostToDevice, st));
    tlb_transform_desc d{};
    d.src = static_cast<const uint8_t*>(c->d_in[slot]);
    d.src_bytes = nb * img;
    d.n_src = nb;
    d.src_w = c->w;
    d.src_h = c->h;
    d.n = nb;
    for (int i = 0; i < 4; ++i) d.uniform_box[i] = c->crop[i];
    d.dst_h = c->out_h;
    d.dst_w = c->out_w;
    d.out = c->d_out[slot];
    d.out_dtype = c->out_dtype;
    d.out_layout = c->out_layout;
    for (int i = 0; i < 3; ++i) {
        d.mean[i] = c->mean[i];
        d.std[i] = c->std_[i];
    }
    d.normalize_01 = 1;
    d.status = c->status;
    if (int rc = tlb_fused_transform(&d, st)) return rc;
    TLB_CUDA(cudaEventRecord(c->ready[slot], st));
    c->enqueued = b + 1;
    return TLB_OK;
}

void stream_free(tlb_stream_core* c) {
    if (!c) return;
    for (void* p : c->d_in) if (p) cudaFree(p);
    for (void* p : c->d_out) if (p) cudaFree(p);
    for (cudaEvent_t e : c->ready) if (e) cudaEventDestroy(e);
    for (cudaStream_t s : c->streams) if (s) cudaStreamDestroy(s);
    if (c->consumed) cudaEventDestroy(c->consumed);
    if (c->status) cudaFree(c->status);
    delete c;
}

}  // namespace

extern "C" {

tlb_stream_core* tlb_stream_create(const uint8_t* host_images, int64_t n, int32_t h, int32_t w, int32_t batch,
                                   const float mean[3], const float std_[3], int32_t slots, int32_t drop_last,
                                   const int32_t crop_box[4], int32_t out_h, int32_t out_w, int32_t out_dtype,
                                   int32_t out_layout) {
    if (!host_images || n <= 0 || h <= 0 || w <= 0 || batch <= 0 || !mean || !std_) {
        fail(TLB_ERR_INVALID_ARG, "stream: NULL pointer or non-positive size");
        return nullptr;
    }
    if ((out_dtype != TLB_F32 && out_dtype != TLB_BF16) || (out_layout != TLB_NCHW && out_layout != TLB_NHWC)) {
        fail(TLB_ERR_INVALID_ARG, "stream: unknown output dtype or layout");
        return nullptr;
    }
    int dev;
    if (current_device(&dev)) return nullptr;
    auto* c = new tlb_stream_core;
    c->dev = dev;
    c->host = host_images;
    c->n = n; c->h = h; c->w = w; c->batch = batch;
    c->slots = std::clamp(static_cast<int>(slots), 2, 16);
    c->drop_last = drop_last != 0;
    c->out_dtype = out_dtype; c->out_layout = out_layout;
    if (crop_box && crop_box[2] > 0) {
        for (int i = 0; i < 4; ++i) c->crop[i] = crop_box[i];
        if (crop_box[0] < 0 || crop_box[1] < 0 || crop_box[3] <= 0 || crop_box[0] > w - crop_box[2] ||
            crop_box[1] > h - crop_box[3]) {
            fail(TLB_ERR_BAD_BOX, "stream: crop box leaves the %dx%d images", w, h);
            delete c;
            return nullptr;
        }
    }
    const int cw = c->crop[2] > 0 ? c->crop[2] : w, chh = c->crop[2] > 0 ? c->crop[3] : h;
    c->out_h = out_h > 0 ? out_h : chh;
    c->out_w = out_w > 0 ? out_w : cw;
    for (int i = 0; i < 3; ++i) { c->mean[i] = mean[i]; c->std_[i] = std_[i]; }
    c->n_batches = c->drop_last ? n / batch : (n + batch - 1) / batch;
    const size_t in_bytes = static_cast<size_t>(batch) * h * w * 3;
    const size_t out_bytes = static_cast<size_t>(batch) * 3 * c->out_h * c->out_w * (out_dtype == TLB_F32 ? 4 : 2);
    c->d_in.assign(c->slots, nullptr);
    c->d_out.assign(c->slots, nullptr);
    c->streams.assign(c->slots, nullptr);
    c->ready.assign(c->slots, nullptr);
    bool ok = cudaMalloc(reinterpret_cast<void**>(&c->status), 4) == cudaSuccess && cudaMemset(c->status, 0, 4) == cudaSuccess &&
              cudaEventCreateWithFlags(&c->consumed, cudaEventDisableTiming) == cudaSuccess;
    for (int s = 0; ok && s < c->slots; ++s) {
        ok = cudaMalloc(&c->d_in[s], in_bytes) == cudaSuccess && cudaMalloc(&c->d_out[s], out_bytes) == cudaSuccess &&
             cudaStreamCreateWithFlags(&c->streams[s], cudaStreamNonBlocking) == cudaSuccess &&
             cudaEventCreateWithFlags(&c->ready[s], cudaEventDisableTiming) == cudaSuccess;
    }
    if (!ok) {
        cuda_fail(cudaGetLastError(), "stream: allocating the slots");
        stream_free(c);
        return nullptr;
    }
    return c;
}

void tlb_stream_destroy(tlb_stream_core* core) {
    if (!core) return;
    cudaSetDevice(core->dev);
    for (cudaStream_t s : core->streams) if (s) cudaStreamSynchronize(s);
    stream_free(core);
}

int64_t tlb_stream_num_batches(const tlb_stream_core* core) { return core ? core->n_batches : -1; }

int tlb_stream_begin_epoch(tlb_stream_core* core, void* consumer_stream) {
    if (!core) return fail(TLB_ERR_INVALID_ARG, "stream: core is NULL");
    TLB_CUDA(cudaSetDevice(core->dev));
    // Batches of an abandoned epoch may still be in flight; their slots are reused in stream order.
    core->enqueued = 0;
    core->returned = 0;
    const int64_t ahead = std::min<int64_t>(core->slots - 1, core->n_batches);
    for (int64_t i = 0; i < ahead; ++i)
        if (int rc = stream_enqueue(core, consumer_stream)) return rc;
    return TLB_OK;
}

int tlb_stream_next(tlb_stream_core* core, uintptr_t* out_dev, int32_t* out_n, void* consumer_stream) {
    if (!core || !out_dev || !out_n) return fail(TLB_ERR_INVALID_ARG, "stream: NULL argument");
    *out_dev = 0;
    *out_n = 0;
    if (core->returned >= core->n_batches) return TLB_OK;  // end of epoch
    TLB_CUDA(cudaSetDevice(core->dev));
    // Keep slots-1 batches enqueued beyond the ones already handed out.  The slot refilled here is
    // the one handed out two calls ago: a batch stays valid until the second next call.
    if (core->enqueued < core->n_batches && core->enqueued - core->returned < core->slots - 1)
        if (int rc = stream_enqueue(core, consumer_stream)) return rc;
    const int64_t b = core->returned;
    const int slot = static_cast<int>(b % core->slots);
    if (consumer_stream)
        TLB_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(consumer_stream), core->ready[slot], 0));
    else
        TLB_CUDA(cudaEventSynchronize(core->ready[slot]));
    *out_dev = reinterpret_cast<uintptr_t>(core->d_out[slot]);
    *out_n = static_cast<int32_t>(std::min<int64_t>(core->batch, core->n - b * core->batch));
    core->returned = b + 1;
    return TLB_OK;
}

int tlb_stream_status(tlb_stream_core* core, uint32_t* out_status) {
    if (!core || !out_status) return fail(TLB_ERR_INVALID_ARG, "stream: NULL argument");
    TLB_CUDA(cudaSetDevice(core->dev));
    for (cudaStream_t s : core->streams) TLB_CUDA(cudaStreamSynchronize(s));
    TLB_CUDA(cudaMemcpy(out_status, core->status, 4, cudaMemcpyDeviceToHost));
    return TLB_OK;
}

}  // extern "C"

// ---- resident epochs ---------------------------------------------------------------------------
// Replaces the per-batch call + synchronise loop of the reference's resident loader
// (turboloader/cuda_loader.py:512-535) by a prefetching pipeline on library-owned streams.
struct tlb_epoch {
    int dev = 0;
    tlb_transform_desc first{};
    int max_crop_w = 0;
    int64_t total = 0, n_batches = 0;
    int64_t enqueued = 0, returned = 0;
    int ring = 0, ahead = 0;
    int64_t out_slot = 0, idx_slot = 0, label_slot = 0;
    std::vector<cudaStream_t> streams;  // batch b runs on streams[b % size]: consecutive batches are independent
    cudaEvent_t consumed = nullptr;
    std::vector<cudaEvent_t> ready;
};

namespace {

int epoch_enqueue(tlb_epoch* e, void* consumer_stream) {
    const int64_t b = e->enqueued;
    const int64_t pos = b * e->first.n;
    const int slot = static_cast<int>(b % e->ring);
    cudaStream_t st = e->streams[static_cast<size_t>(b % static_cast<int64_t>(e->streams.size()))];
    // The slot about to be overwritten was handed out ring batches ago and its validity has run out:
    // order this launch behind everything the consumer has enqueued so far.
    TLB_CUDA(cudaEventRecord(e->consumed, static_cast<cudaStream_t>(consumer_stream)));
    TLB_CUDA(cudaStreamWaitEvent(st, e->consumed, 0));
    tlb_transform_desc d = e->first;
    d.n = static_cast<int32_t>(std::min<int64_t>(e->first.n, e->total - pos));
    if (d.sel) {
        d.sel += pos;
    } else {  // sequential: the batch is a contiguous slice of the uniform dataset
        const uint64_t img = static_cast<uint64_t>(d.src_w) * d.src_h * 3;
        d.src += pos * img;
        d.src_bytes = static_cast<uint64_t>(d.n) * img;
        d.n_src = d.n;
        if (d.labels_in) d.labels_in += pos;
    }
    if (d.boxes) d.boxes += 4 * pos;
    if (d.flips) d.flips += pos;
    if (d.jitter) d.jitter += 3 * pos;
    d.out = static_cast<char*>(d.out) + slot * e->out_slot;
    if (d.out_indices) d.out_indices = reinterpret_cast<int64_t*>(reinterpret_cast<char*>(d.out_indices) + slot * e->idx_slot);
    if (d.labels_out) d.labels_out = reinterpret_cast<int64_t*>(reinterpret_cast<char*>(d.labels_out) + slot * e->label_slot);
    d.flags = 0;
    if (int rc = launch_desc(d, e->max_crop_w, st, false, false, /*streaming=*/true)) return rc;
    TLB_CUDA(cudaEventRecord(e->ready[slot], st));
    e->enqueued = b + 1;
    return TLB_OK;
}

}  // namespace

extern "C" {

tlb_epoch* tlb_epoch_create(const tlb_transform_desc* first, int64_t total, int32_t drop_last, int64_t start_batch,
                            int32_t ring, int32_t ahead, int64_t out_slot_bytes, int64_t index_slot_bytes,
                            int64_t label_slot_bytes) {
    if (check_common(first)) return nullptr;
    if (first->n <= 0 || total <= 0 || start_batch < 0) {
        fail(TLB_ERR_INVALID_ARG, "epoch: batch size, total and start_batch must be positive / non-negative");
        return nullptr;
    }
    if (ahead < 1 || ring < ahead + 2) {
        fail(TLB_ERR_INVALID_ARG, "epoch: need ahead >= 1 and ring >= ahead + 2 (got ring %d, ahead %d)", ring, ahead);
        return nullptr;
    }
    if (!first->sel && (first->src_offsets || first->src_sizes)) {
        fail(TLB_ERR_INVALID_ARG, "epoch: reading the dataset in order needs the uniform layout (or pass sel)");
        return nullptr;
    }
    if (!first->sel && static_cast<int64_t>(first->n_src) < total) {
        fail(TLB_ERR_BAD_INDEX, "epoch: total = %lld exceeds n_src = %lld", static_cast<long long>(total), static_cast<long long>(first->n_src));
        return nullptr;
    }
    if (out_slot_bytes <= 0 || (first->out_indices && index_slot_bytes <= 0) || (first->labels_out && label_slot_bytes <= 0)) {
        fail(TLB_ERR_INVALID_ARG, "epoch: slot strides must be positive");
        return nullptr;
    }
    const int mcw = derive_max_crop_w(*first);
    if (mcw <= 0) {
        fail(TLB_ERR_INVALID_ARG, "epoch: max_crop_w is required when sizes and boxes are per-sample device tables");
        return nullptr;
    }
    int dev;
    if (current_device(&dev)) return nullptr;
    auto* e = new tlb_epoch;
    e->dev = dev;
    e->first = *first;
    e->max_crop_w = mcw;
    e->total = total;
    e->n_batches = drop_last ? total / first->n : (total + first->n - 1) / first->n;
    e->enqueued = e->returned = std::min<int64_t>(start_batch, e->n_batches);
    e->ring = ring; e->ahead = ahead;
    e->out_slot = out_slot_bytes; e->idx_slot = index_slot_bytes; e->label_slot = label_slot_bytes;
    e->ready.assign(ring, nullptr);
    e->streams.assign(static_cast<size_t>(std::min(ahead + 1, 4)), nullptr);
    DeviceState& ds = g_dev[dev];
    auto take_event = [&](cudaEvent_t* ev) {
        {
            std::lock_guard<std::mutex> lk(ds.pool_mu);
            if (!ds.idle_events.empty()) {
                *ev = ds.idle_events.back();
                ds.idle_events.pop_back();
                return true;
            }
        }
        return cudaEventCreateWithFlags(ev, cudaEventDisableTiming) == cudaSuccess;
    };
    auto take_stream = [&](cudaStream_t* st) {
        {
            std::lock_guard<std::mutex> lk(ds.pool_mu);
            if (!ds.idle_streams.empty()) {
                *st = ds.idle_streams.back();
                ds.idle_streams.pop_back();
                return true;
            }
        }
        return cudaStreamCreateWithFlags(st, cudaStreamNonBlocking) == cudaSuccess;
    };
    bool ok = take_event(&e->consumed);
    for (auto& st : e->streams) ok = ok && take_stream(&st);
    for (int i = 0; ok && i < ring; ++i) ok = take_event(&e->ready[i]);
    if (!ok) {
        cuda_fail(cudaGetLastError(), "epoch: creating the prefetch streams and events");
        tlb_epoch_destroy(e);
        return nullptr;
    }
    return e;
}

int tlb_epoch_next(tlb_epoch* e, int64_t* batch, int32_t* n, int32_t* slot, void* consumer_stream) {
    if (!e || !batch || !n || !slot) return fail(TLB_ERR_INVALID_ARG, "epoch: NULL argument");
    *n = 0;
    if (e->returned >= e->n_batches) return TLB_OK;  // epoch finished
    TLB_CUDA(cudaSetDevice(e->dev));
    // Keep `ahead` batches in flight beyond the one handed out now.  Batch q overwrites the slot of
    // batch q - ring; with q <= returned + ahead and ring >= ahead + 2 that batch was handed out at
    // least two calls ago, i.e. its validity (ring - ahead - 1 further calls) has run out.
    const int64_t want = std::min<int64_t>(e->n_batches, e->returned + 1 + e->ahead);
    while (e->enqueued < want)
        if (int rc = epoch_enqueue(e, consumer_stream)) return rc;
    const int64_t b = e->returned;
    const int s = static_cast<int>(b % e->ring);
    TLB_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(consumer_stream), e->ready[s], 0));
    *batch = b;
    *n = static_cast<int32_t>(std::min<int64_t>(e->first.n, e->total - b * e->first.n));
    *slot = s;
    e->returned = b + 1;
    return TLB_OK;
}

void tlb_epoch_destroy(tlb_epoch* e) {
    if (!e) return;
    cudaSetDevice(e->dev);
    // The streams are idle once synchronised, and an event may be recorded anew at any time: both go
    // back to the device's pool (bounded; what does not fit is destroyed).
    constexpr size_t kMaxIdleStreams = 16, kMaxIdleEvents = 128;
    DeviceState* ds = (e->dev >= 0 && e->dev < kMaxDevices) ? &g_dev[e->dev] : nullptr;
    for (cudaStream_t st : e->streams)
        if (st) {
            cudaStreamSynchronize(st);
            bool kept = false;
            if (ds) {
                std::lock_guard<std::mutex> lk(ds->pool_mu);
                if (ds->idle_streams.size() < kMaxIdleStreams) {
                    ds->idle_streams.push_back(st);
                    kept = true;
                }
            }
            if (!kept) cudaStreamDestroy(st);
        }
    auto give_event = [&](cudaEvent_t ev) {
        if (!ev) return;
        if (ds) {
            std::lock_guard<std::mutex> lk(ds->pool_mu);
            if (ds->idle_events.size() < kMaxIdleEvents) {
                ds->idle_events.push_back(ev);
                return;
            }
        }
        cudaEventDestroy(ev);
    };
    for (cudaEvent_t ev : e->ready) give_event(ev);
    give_event(e->consumed);
    delete e;
}

}  // extern "C"
