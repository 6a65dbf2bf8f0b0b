/*
 * turboloader_b200 -- C ABI of the B200 (sm_100a) fused image-transform path.
 *
 * One fused operation replaces TurboLoader's GPU transform entry points:
 *
 *   per-sample crop box -> horizontal flip -> bilinear resize (half-pixel centres,
 *   result truncated to an 8-bit code as the CPU path does) -> per-channel
 *   mean/std normalize -> HWC->NCHW (or NHWC) -> fp32 or bf16,
 *   optionally gathering the source image through a device index array.
 *
 * Every function is plain C: raw pointers, sizes, int status codes.  No torch
 * or pybind types cross this boundary.  Work is enqueued on the caller's
 * stream and the call returns without synchronising unless stated otherwise.
 * Citations name the TurboLoader interface each entry point stands in for
 * (paths inside the TurboLoader tree).
 */
#ifndef TURBOLOADER_B200_H
#define TURBOLOADER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TLB_API __attribute__((visibility("default")))

/* ---- status codes (0 = ok) -------------------------------------------------------- */
enum {
    TLB_OK = 0,
    TLB_ERR_INVALID_ARG = 1,   /* null pointer, non-positive size, unknown enum           */
    TLB_ERR_BAD_BOX = 2,       /* a crop box leaves its image (host-validated calls)       */
    TLB_ERR_BAD_INDEX = 3,     /* a gather index is outside [0, n_src)                     */
    TLB_ERR_TOO_WIDE = 4,      /* crop wider than the staging capacity (see max_crop_w)    */
    TLB_ERR_CUDA = 5,          /* a CUDA runtime call failed; see tlb_last_error()         */
    TLB_ERR_NO_DEVICE = 6,     /* no CUDA device / not an sm_100 device                    */
    TLB_ERR_TOO_LARGE = 7,     /* size beyond a fixed capacity (allocation-free entry)     */
};

/* Bits of the optional device status word written by the kernel (never traps). */
enum {
    TLB_DEV_BAD_INDEX = 1u,    /* sample skipped (output zero-filled): gather index invalid */
    TLB_DEV_BAD_BOX = 2u,      /* sample skipped (output zero-filled): box leaves the image */
    TLB_DEV_TOO_WIDE = 4u,     /* sample skipped (output zero-filled): crop exceeds staging */
    TLB_DEV_COPY_TIMEOUT = 8u, /* a bounded wait on an async copy gave up                   */
};

enum { TLB_F32 = 0, TLB_BF16 = 1 };
enum { TLB_NCHW = 0, TLB_NHWC = 1 };

/*
 * Descriptor of one fused batch.  All pointers are DEVICE pointers unless the
 * field says otherwise.  "Dataset image" = an image stored in `src`; "sample"
 * = one output slot of this batch.  Sample k reads dataset image
 * s = sel ? sel[k] : k.
 */
typedef struct tlb_transform_desc {
    /* -- source pixels: uint8, HWC, RGB, tightly packed rows ------------------------ */
    const uint8_t* src;        /* base of the readable region                              */
    uint64_t src_bytes;        /* readable bytes at src (no load ever leaves this range)   */
    int64_t n_src;             /* number of dataset images described below                 */
    const int64_t* src_offsets;/* [n_src] byte offset of each image, or NULL: uniform      */
                               /*   layout, image s at s * src_h * src_w * 3               */
    const int32_t* src_sizes;  /* [n_src][2] (w, h) per image, or NULL: all src_w x src_h  */
    int32_t src_w, src_h;      /* uniform size (used when src_sizes == NULL)               */

    /* -- per-sample parameters ------------------------------------------------------- */
    int32_t n;                 /* samples in this batch                                    */
    const int64_t* sel;        /* [n] gather indices into the dataset, or NULL             */
    const int32_t* boxes;      /* [n][4] crop (x, y, w, h) in source pixels, or NULL       */
    int32_t uniform_box[4];    /* used when boxes == NULL; w == 0 means the whole image    */
    const uint8_t* flips;      /* [n] non-zero = mirror the RESIZED image, or NULL         */

    /* -- output ---------------------------------------------------------------------- */
    int32_t dst_h, dst_w;
    void* out;                 /* n*3*dst_h*dst_w elements                                 */
    int32_t out_dtype;         /* TLB_F32 | TLB_BF16 (bf16 = RNE of the fp32 result)       */
    int32_t out_layout;        /* TLB_NCHW | TLB_NHWC                                      */
    int64_t* out_indices;      /* [n] receives s for every sample (bit-exact), or NULL     */
    const int64_t* labels_in;  /* [n_src] per-dataset-image labels, or NULL                */
    int64_t* labels_out;       /* [n] receives labels_in[s], or NULL                       */

    /* -- normalization: (u8 * (normalize_01 ? 1/255 : 1) - mean[c]) * (1.0f / std[c]) -- */
    float mean[3];
    float std[3];
    int32_t normalize_01;

    /* -- capacity hint ---------------------------------------------------------------- */
    int32_t max_crop_w;        /* upper bound of any crop width in this batch; 0 = derive  */
                               /*   (uniform box width, else src_w, which must then be set */
                               /*   to the widest image)                                   */
    uint32_t* status;          /* device word OR-ed with TLB_DEV_* bits, or NULL           */

    /* -- resize filter ---------------------------------------------------------------- */
    int32_t antialias;         /* 0: bilinear (above).  1: the reference's opt-in triangle  */
                               /*   filter whose support widens on downscale, rounded half  */
                               /*   up (DirectBatchCore antialias=true,                     */
                               /*   src/transforms/simd_utils.hpp:1939-2014)                */
    int32_t max_crop_h;        /* antialias only: upper bound of any crop height; 0 = derive */
                               /*   (uniform box height, else src_h = the tallest image)    */

    /* -- colour jitter (train_transform, src/metal/metal_transforms.mm:83-116) ---------- */
    const float* jitter;       /* [n][3] per-sample (brightness, contrast, saturation), or   */
                               /*   NULL.  Applied to rgb = code/255 between the 8-bit code  */
                               /*   and the normalize, in the shader's order (:111-115):     */
                               /*   rgb*=b; rgb=(rgb-0.5)*c+0.5; lum=(0.299r+0.587g)+0.114b; */
                               /*   rgb=lum+(rgb-lum)*s; clamp to [0,1].  Every operation is */
                               /*   rounded separately.  Needs normalize_01 = 1; works with  */
                               /*   either filter.                                           */

    /* -- launch flags (tlb_fused_transform only; the other entry points ignore them) ---- */
    uint32_t flags;            /* OR of TLB_FLAG_*                                           */
} tlb_transform_desc;

/* TLB_FLAG_LAUNCH_OVERLAP: launch with programmatic stream serialization.  When the work directly
 * before this call in its stream is another launch of this library's transform kernels (bilinear,
 * antialiased, identity-size, video), this one may start while that one drains its last CTAs, so
 * consecutive batches leave no SM idle between them.  The kernel does
 * not wait for its predecessor; by setting the flag the caller states that a KERNEL placed directly
 * before this call in the same stream neither writes this call's inputs (pixels, tables) nor reads
 * or writes its outputs.  Copies, memsets and event waits always keep full stream order.  A stream
 * that carries only this library's launches, each into its own output buffer -- a loader's prefetch
 * stream handing batches over by events -- meets the condition.  The choice is per call: a launch
 * without the flag is never affected by other callers' launches.  No counterpart in the reference
 * (its loaders synchronise after every batch). */
#define TLB_FLAG_LAUNCH_OVERLAP 1u

/* ---- capability ----------------------------------------------------------------------
 * Replace turboloader::cuda::available / device_name
 * (src/cuda/cuda_transforms.hpp:19-22, src/cuda/cuda_transforms.cu:270-286). */
TLB_API int tlb_available(void);
TLB_API int tlb_device_name(int device, char* buf, size_t cap);
TLB_API const char* tlb_version(void);
/* Message of the last failing call on this thread ("" when none). */
TLB_API const char* tlb_last_error(void);

/* ---- the fused operation ---------------------------------------------------------------
 * Replaces the kernels and launch loops behind
 *   turboloader::cuda::resize_normalize_batch          (cuda_transforms.hpp:41-42,  .cu:288-314)
 *   turboloader::cuda::crop_resize_normalize_batch     (cuda_transforms.hpp:117-119, .cu:316-347)
 *   turboloader::cuda::normalize_resident_batch        (cuda_transforms.hpp:49-50,  .cu:475-507)
 *   turboloader::cuda::normalize_resident_gather_batch (cuda_transforms.hpp:54-55,  .cu:511-544)
 * (resize_normalize_device_batch has its own entry point below: its images are separate allocations)
 * with ONE launch per batch on `stream` (a cudaStream_t passed as void*; NULL =
 * the legacy default stream), on the current device, with no synchronisation and
 * no allocation.  Parameters that live on the device cannot be checked by the
 * host: the kernel checks them, zero-fills an invalid sample and reports
 * through desc->status. */
TLB_API int tlb_fused_transform(const tlb_transform_desc* desc, void* stream);

/* Same operation, with the per-sample tables given as HOST arrays.  Boxes and
 * indices are validated on the host first (TLB_ERR_BAD_BOX / TLB_ERR_BAD_INDEX,
 * nothing is launched), then copied to a library-owned device ring on `stream`.
 * In `desc`, sel / boxes / flips / src_offsets / src_sizes are HOST pointers here;
 * src, out, out_indices, labels_* and status stay device pointers.  May allocate
 * (ring growth) on first use. */
TLB_API int tlb_fused_transform_host_params(const tlb_transform_desc* desc, void* stream);

/* ---- host-image convenience forms (synchronous, like the functions they replace) ----- */
typedef struct tlb_image_ref {  /* turboloader::cuda::ImageRef, cuda_transforms.hpp:25-29 */
    const uint8_t* data;        /* HOST pointer, HWC uint8 RGB */
    int32_t w, h;
} tlb_image_ref;

typedef struct tlb_crop_params { /* turboloader::cuda::CropParams, cuda_transforms.hpp:32-38 */
    float x, y, w, h;            /* must be whole numbers: the parity target is the CPU  */
    int32_t flip;                /* path, whose crop rects are integers                   */
} tlb_crop_params;

/* resize_normalize_batch (cuda_transforms.hpp:41-42): N host images -> host fp32
 * NCHW [n,3,dst_h,dst_w]; mean/std in [0,1] units.  Uploads, runs, downloads, syncs. */
TLB_API int tlb_resize_normalize_batch(const tlb_image_ref* imgs, int32_t n, int32_t dst_h,
                                       int32_t dst_w, const float mean[3], const float std_[3],
                                       float* out_host);
/* crop_resize_normalize_batch (cuda_transforms.hpp:117-119). */
TLB_API int tlb_crop_resize_normalize_batch(const tlb_image_ref* imgs, const tlb_crop_params* crops,
                                            int32_t n, int32_t dst_h, int32_t dst_w,
                                            const float mean[3], const float std_[3], float* out_host);

/* Host images in, DEVICE batch out, on `stream`, without synchronising.  When every image
 * lies in page-locked, device-mapped host memory the fused kernel reads the crop rows
 * straight out of the host images across PCIe (nothing is staged; the images must stay
 * valid and unchanged until the work on `stream` has finished).  Otherwise the crop rows
 * are packed into a pinned staging ring and uploaded first.  `out_dev` takes the batch
 * in the given dtype/layout.  The streaming counterpart of CudaStreamCore's H2D + kernel
 * slot (cuda_transforms.cu:629-780) for the crop/resize path. */
TLB_API int tlb_crop_resize_normalize_to_device(const tlb_image_ref* imgs, const tlb_crop_params* crops,
                                                int32_t n, int32_t dst_h, int32_t dst_w,
                                                const float mean[3], const float std_[3],
                                                int32_t normalize_01, void* out_dev, int32_t out_dtype,
                                                int32_t out_layout, uint32_t* status_dev, void* stream);

/* Allocation-free form of tlb_crop_resize_normalize_to_device.  It has no counterpart in
 * the reference.  It exists for callers that are not allowed to allocate device or pinned
 * memory at the point of the call -- a loader thread running inside a training process whose
 * memory pool is already sized to the GPU, a real-time or embedded host that forbids
 * allocation after start-up, a process sharing the GPU under a fixed memory budget.  This entry
 * point calls no cudaMalloc / cudaMallocHost / cudaFree and no allocating library routine: the
 * packed crop pixels and the per-sample tables are staged in one fixed device array that lives
 * in the library image (TLB_STATIC_SCRATCH_BYTES, held by every GPU that loads the library
 * until the process exits), and the host pixels are copied straight from the caller's memory.
 *
 * Limits: n <= TLB_STATIC_MAX_SAMPLES, and the packed crops (each crop's w*h*3 bytes rounded up
 * to 16) plus 33 bytes of tables per sample must fit TLB_STATIC_SCRATCH_BYTES; otherwise
 * TLB_ERR_TOO_LARGE is returned and nothing is enqueued.
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and
 * opts the kernels in to large shared memory; make that first call outside any stream capture.
 * Every call on a device uses the same array: it keeps the previous call's bytes (nothing in it
 * needs to start at zero -- each call overwrites what it reads), and two calls whose GPU work
 * overlaps (different streams, or concurrent host threads on one device) race on it.  Issue the
 * calls of one device on one stream, one host thread at a time.  The per-sample tables are built in
 * one fixed host buffer of the library; a lock serialises that step across all host threads, so
 * threads that drive different GPUs may call concurrently.  Same arguments and results as
 * tlb_crop_resize_normalize_to_device. */
#define TLB_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
#define TLB_STATIC_MAX_SAMPLES 4096
TLB_API int tlb_crop_resize_normalize_to_device_static(const tlb_image_ref* imgs, const tlb_crop_params* crops,
                                                       int32_t n, int32_t dst_h, int32_t dst_w,
                                                       const float mean[3], const float std_[3],
                                                       int32_t normalize_01, void* out_dev, int32_t out_dtype,
                                                       int32_t out_layout, uint32_t* status_dev, void* stream);

/* ---- resident-dataset forms returning a library-owned device pointer -------------------
 * normalize_resident_batch / normalize_resident_gather_batch
 * (cuda_transforms.hpp:49-55): src_dev = [N,H,W,3] uint8 on the device; returns the
 * device address of an [N,3,H,W] fp32 batch from a 4-deep ring (valid until the
 * 4th-next call), or 0 on error.  Synchronises its stream before returning, as the
 * functions it replaces do. */
TLB_API uintptr_t tlb_normalize_resident_batch(uintptr_t src_dev, int32_t n, int32_t h, int32_t w,
                                               const float mean[3], const float std_[3]);
TLB_API uintptr_t tlb_normalize_resident_gather_batch(uintptr_t src_dev, uintptr_t sel_dev, int32_t n,
                                                      int32_t h, int32_t w, const float mean[3],
                                                      const float std_[3]);

/* resize_normalize_device_batch (cuda_transforms.hpp:141-144, .cu:1008-1046): n ALREADY-DECODED
 * images given as device addresses d_imgs[i] of tightly packed ws[i] x hs[i] x 3 uint8 pixels, each
 * in its own device allocation (e.g. the outputs of an external GPU decoder), read in place ->
 * device address of the [n,3,dst_h,dst_w] fp32 batch in the same 4-deep ring (valid until the
 * 4th-next call of a pointer-returning form), or 0 on error.  Synchronises its stream before
 * returning, as the function it replaces does.  One launch for the whole list; every image is
 * checked against the allocation that holds it and no load leaves an image. */
TLB_API uintptr_t tlb_resize_normalize_device_batch(const uintptr_t* d_imgs, const int32_t* ws, const int32_t* hs,
                                                    int32_t n, int32_t dst_h, int32_t dst_w, const float mean[3],
                                                    const float std_[3]);

/* ---- YUV 4:2:0 video frames ----------------------------------------------------------------
 * Replaces turboloader::cuda::video_yuv420_batch and video_clip_yuv420
 * (src/cuda/cuda_transforms.hpp:65-81; kernels src/cuda/cuda_transforms.cu:143-268): decoded
 * frames given as DEVICE plane addresses -> YUV->RGB (video range, BT.601 or BT.709), bilinear
 * resize with MPEG chroma siting, clip to [0,1], normalize, planar (n,3,dst_h,dst_w) output.
 * c_px_stride 1 = I420 (separate Cb / Cr planes), 2 = NV12 (cr address = cb address + 1 in one
 * interleaved plane).  Strides are shared by all frames.  One kernel launch per call, whatever n. */
typedef struct tlb_video_desc {
    const uintptr_t* y_ptrs;  /* HOST arrays of n device addresses each */
    const uintptr_t* cb_ptrs;
    const uintptr_t* cr_ptrs;
    int32_t n;                /* frames */
    int32_t y_stride;         /* bytes between luma rows (>= src_w) */
    int32_t c_stride;         /* bytes between chroma rows */
    int32_t c_px_stride;      /* 1 or 2 */
    int32_t src_w, src_h;
    int32_t dst_h, dst_w;
    const float* crops;       /* HOST, (x, y, w, h) in source pixels per clip; NULL = whole-frame
                                 resize (the video_yuv420_batch sampling rule) */
    const int32_t* flips;     /* HOST, one per clip, or NULL (only read when crops != NULL) */
    int32_t clip_len;         /* consecutive frames sharing one crops/flips entry; 0 = all n */
    int32_t bt709;            /* 0: BT.601 matrix, 1: BT.709 */
    float mean[3];
    float std[3];             /* (rgb01 - mean) * (1.0f / std) */
    void* out;                /* DEVICE, caller-allocated (n,3,dst_h,dst_w) */
    int32_t out_dtype;        /* TLB_F32 / TLB_BF16 */
    uint32_t* status;         /* DEVICE word OR-ed with TLB_DEV_COPY_TIMEOUT if a bounded wait gave up; or NULL */
    uint32_t flags;           /* OR of TLB_FLAG_*: TLB_FLAG_LAUNCH_OVERLAP as for the image kernels (it takes
                                 effect for batches of at most 256 frames in at most 32 clips, whose tables
                                 travel in the kernel's parameter block instead of being uploaded first) */
} tlb_video_desc;

/* Asynchronous form on the caller's stream: one launch, no synchronisation.  The small address /
 * crop tables ride in the kernel's parameters (up to 256 frames in 32 clips) or are uploaded
 * through a pinned ring first (larger batches). */
TLB_API int tlb_video_yuv420(const tlb_video_desc* desc, void* stream);
/* The reference's two pointer-returning forms, same arguments and lifetime rule: the result is
 * a library-owned float32 (n,3,dst_h,dst_w) device buffer, double-buffered, valid until the next
 * call of either function; the call synchronises; returns 0 on error. */
TLB_API uintptr_t tlb_video_yuv420_batch(const uintptr_t* y_ptrs, const uintptr_t* cb_ptrs,
                                         const uintptr_t* cr_ptrs, int32_t n, int32_t y_stride,
                                         int32_t c_stride, int32_t c_px_stride, int32_t src_w,
                                         int32_t src_h, int32_t dst_h, int32_t dst_w, int32_t bt709,
                                         const float mean[3], const float std_[3]);
TLB_API uintptr_t tlb_video_clip_yuv420(const uintptr_t* y_ptrs, const uintptr_t* cb_ptrs,
                                        const uintptr_t* cr_ptrs, int32_t n, int32_t y_stride,
                                        int32_t c_stride, int32_t c_px_stride, int32_t src_w,
                                        int32_t src_h, int32_t dst_h, int32_t dst_w,
                                        const float crop[4], int32_t flip, int32_t bt709,
                                        const float mean[3], const float std_[3]);

/* ---- streaming core: datasets larger than device memory -------------------------------------
 * Replaces CudaStreamCore (src/cuda/cuda_transforms.cu:629-780; Python turboloader/cuda_loader.py:
 * 538-674): n uint8 HWC images of one size stay in host memory (pinned, for the copies to overlap)
 * and are streamed in index order, `slots`-1 batches ahead: per batch one asynchronous copy and one
 * fused kernel on the slot's own stream.  No worker threads and no host synchronisation when a
 * consumer stream is given.  crop_box (x,y,w,h; NULL or w<=0: whole image) and out_h/out_w (0: the
 * crop size) select a centre-crop / resize fused into the same kernel. */
typedef struct tlb_stream_core tlb_stream_core;
TLB_API tlb_stream_core* tlb_stream_create(const uint8_t* host_images, int64_t n, int32_t h, int32_t w,
                                           int32_t batch, const float mean[3], const float std_[3],
                                           int32_t slots, int32_t drop_last, const int32_t crop_box[4],
                                           int32_t out_h, int32_t out_w, int32_t out_dtype,
                                           int32_t out_layout);   /* NULL on error */
TLB_API void tlb_stream_destroy(tlb_stream_core* core);
TLB_API int64_t tlb_stream_num_batches(const tlb_stream_core* core);
/* Starts an epoch: enqueues the first slots-1 batches.  consumer_stream (may be NULL): the stream
 * on which batches of the previous epoch were used; the slots are reused behind its position. */
TLB_API int tlb_stream_begin_epoch(tlb_stream_core* core, void* consumer_stream);
/* Next batch in index order: *out_dev = device address of (n,3,out_h,out_w) [or NHWC], *out_n = n;
 * *out_n = 0 at the end of the epoch.  With consumer_stream != NULL nothing blocks: that stream is
 * made to wait for the batch, and slots are refilled only behind the work already enqueued on it.
 * With NULL the call waits on the host until the batch is complete (the reference's behaviour).
 * The batch stays valid until the second next call. */
TLB_API int tlb_stream_next(tlb_stream_core* core, uintptr_t* out_dev, int32_t* out_n, void* consumer_stream);
/* Drains the slots and returns the OR of the device status bits seen so far. */
TLB_API int tlb_stream_status(tlb_stream_core* core, uint32_t* out_status);

/* ---- resident epochs: one call per batch, no per-batch set-up on the host --------------------
 * The batch loop of the resident loader (turboloader/cuda_loader.py:512-535: one
 * normalize_resident(_gather)_batch call and one synchronisation per batch) as a pipeline: the
 * library owns a few prefetch streams and a ring of `ring` output slots in caller-allocated memory,
 * keeps `ahead` batches enqueued beyond the one being handed out, and hands a batch over by making
 * the consumer's stream wait for it -- the host never blocks.  Consecutive batches are enqueued on
 * different streams (they never depend on one another), so the head of one batch fills the SMs
 * that the tail of the previous one leaves idle.
 *
 * `first` describes batch 0 of the epoch exactly as tlb_fused_transform would take it: n = the
 * batch size; sel / boxes / flips / jitter (if given) point at epoch position 0 of tables that
 * cover the whole epoch; out / out_indices / labels_out point at slot 0.  Batch b reads the tables
 * at position b * n and writes slot b % ring (slots are out_slot_bytes, index_slot_bytes and
 * label_slot_bytes apart).  With sel == NULL the dataset is read in order: batch b starts at image
 * b * n of `first->src` (uniform layout only).  The last batch is short unless drop_last.
 * A batch stays valid until `ring - ahead - 1` further tlb_epoch_next calls have been made. */
typedef struct tlb_epoch tlb_epoch;
TLB_API tlb_epoch* tlb_epoch_create(const tlb_transform_desc* first, int64_t total, int32_t drop_last,
                                    int64_t start_batch, int32_t ring, int32_t ahead,
                                    int64_t out_slot_bytes, int64_t index_slot_bytes,
                                    int64_t label_slot_bytes);       /* NULL on error */
/* Next batch: *batch = its number in the epoch, *n = its samples (0: epoch finished), *slot = the
 * ring slot that holds it.  consumer_stream (a cudaStream_t as void*, NULL = legacy default stream)
 * is made to wait for the batch; slots are refilled only behind the work already enqueued on it. */
TLB_API int tlb_epoch_next(tlb_epoch* e, int64_t* batch, int32_t* n, int32_t* slot, void* consumer_stream);
TLB_API void tlb_epoch_destroy(tlb_epoch* e);

/* ---- introspection ---------------------------------------------------------------------
 * Launch geometry the fused kernel would use for `desc` (for tests and the
 * benchmark's launch/byte accounting).  Any out pointer may be NULL. */
TLB_API int tlb_fused_plan(const tlb_transform_desc* desc, int32_t* grid, int32_t* block,
                           int32_t* smem_bytes, int32_t* tile_rows, int32_t* tile_cols);
/* Number of kernels this library has launched in this process (all entry points). */
TLB_API uint64_t tlb_launch_count(void);

/* ---- shard index math (host only, no CUDA) ---------------------------------------------
 * kind 0/1/2 = ContiguousSharding / InterleavedSharding / HashBasedSharding
 * (src/distributed/sharding_strategies.hpp:150-316).  Returns the shard size (or -1
 * for world == 0 / rank >= world) and writes min(size, cap) indices. */
TLB_API int64_t tlb_shard_indices(int32_t kind, int64_t total, int64_t world, int64_t rank,
                                  int64_t* out, int64_t cap);
/* DistributedSampler::get_indices (src/distributed/distributed_dataloader.hpp:111-149). */
TLB_API int64_t tlb_sampler_indices(int64_t total, int32_t world, int32_t rank, int32_t shuffle,
                                    uint64_t seed, uint64_t epoch, int32_t drop_last, int64_t* out,
                                    int64_t cap);
/* DirectBatchCore::build_order (src/pipeline/direct_batch_loader.hpp:116-135). */
TLB_API int64_t tlb_direct_order(int64_t total, int32_t shuffle, int32_t seed, int32_t epoch,
                                 int32_t distributed, int32_t rank, int32_t world, int64_t* out,
                                 int64_t cap);

/* RandomResizedCrop(scale (0.08,1), ratio (3/4,4/3)) + flip sampler of the direct-batch loader
 * (DirectBatchCore::pick_crop, src/pipeline/direct_batch_loader.hpp:141-178), host only.
 * sizes_wh = n x (w, h) of the images the rects are drawn on; indices = n sample indices (NULL:
 * 0..n-1) that seed each sample's generator together with seed and epoch.  Writes n integer
 * rects (x, y, w, h) and, if flips_out != NULL, n flags.  Returns n, or a negative value for bad
 * arguments. */
TLB_API int64_t tlb_pick_crops(int32_t seed, int32_t epoch, const int64_t* indices, const int32_t* sizes_wh,
                               int64_t n, float hflip_prob, int32_t* boxes_out, uint8_t* flips_out);

#ifdef __cplusplus
}
#endif
#endif /* TURBOLOADER_B200_H */
