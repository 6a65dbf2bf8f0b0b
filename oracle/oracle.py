"""TEST INFRASTRUCTURE ONLY: ctypes front end of the CPU parity oracle.

Two implementations sit behind the same call:

* ``port``  -- ``oracle/libtl_oracle.so``, the plain-C restatement in ``fused_ref.c``
  (built by ``make -C oracle port``; needs only gcc).
* ``ref``   -- ``oracle/_ref/libtl_ref_<flavour>.so``, the TurboLoader headers themselves
  compiled in place from the reference tree (``make -C oracle ref``).  Flavours:
  ``parity`` (no FMA contraction; what parity is pinned to), ``avx2fma`` and ``avx512``
  (timed CPU baselines).

Only tests, the smoke check and the benchmark's CPU legs may import this module; the
package itself never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
# The reference tree: $TLB_REFERENCE_ROOT, else a checkout named "reference" beside this repository.
REF_ROOT = os.environ.get("TLB_REFERENCE_ROOT") or os.path.normpath(os.path.join(HERE, "..", "..", "reference"))
PORT_SO = os.path.join(HERE, "libtl_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")

_u8p = C.POINTER(C.c_uint8)
_i64p = C.POINTER(C.c_int64)
_i32p = C.POINTER(C.c_int32)
_f32p = C.POINTER(C.c_float)

_libs: dict[str, C.CDLL] = {}


def build_port(force: bool = False) -> str:
    """Compile the C restatement if it is missing (gcc only, no reference tree needed)."""
    srcs = [os.path.join(HERE, "fused_ref.c"), os.path.join(HERE, "video_ref.c")]
    if force or not os.path.exists(PORT_SO) or os.path.getmtime(PORT_SO) < max(os.path.getmtime(s) for s in srcs):
        subprocess.check_call(["make", "-C", HERE, "port"], stdout=subprocess.DEVNULL)
    return PORT_SO


def build_ref(ref_root: str = REF_ROOT) -> bool:
    """Compile the reference headers in place; returns False when the tree is absent."""
    if not os.path.isdir(os.path.join(ref_root, "src", "transforms")):
        return False
    subprocess.check_call(["make", "-C", HERE, "ref", f"REF={ref_root}"], stdout=subprocess.DEVNULL)
    return True


def _cpu_flags() -> set[str]:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def ref_available(flavour: str = "parity") -> bool:
    path = os.path.join(REF_DIR, f"libtl_ref_{flavour}.so")
    if not os.path.exists(path):
        return False
    flags = _cpu_flags()
    need = {"parity": {"avx2"}, "avx2fma": {"avx2", "fma"},
            "avx512": {"avx2", "fma", "avx512f", "avx512bw", "avx512vl", "avx512dq"}}[flavour]
    return need <= flags


def _load(impl: str) -> C.CDLL:
    if impl in _libs:
        return _libs[impl]
    if impl == "port":
        lib = C.CDLL(build_port())
        lib.tlo_fused_batch.restype = C.c_int
        lib.tlo_fused_batch.argtypes = [_u8p, _i64p, _i32p, C.c_int64, _i64p, _i32p, _u8p, C.c_int,
                                        C.c_int, C.c_int, _f32p, _f32p, C.c_int, _f32p]
        lib.tlo_fused_batch_aa.restype = C.c_int
        lib.tlo_fused_batch_aa.argtypes = lib.tlo_fused_batch.argtypes + [C.c_int]
        lib.tlo_fused_batch_jitter.restype = C.c_int
        lib.tlo_fused_batch_jitter.argtypes = [_u8p, _i64p, _i32p, C.c_int64, _i64p, _i32p, _u8p, C.c_int,
                                               C.c_int, C.c_int, _f32p, _f32p, _f32p, _f32p]
        lib.tlo_fused_batch_aa_jitter.restype = C.c_int
        lib.tlo_fused_batch_aa_jitter.argtypes = lib.tlo_fused_batch_jitter.argtypes
        lib.tlo_resize_bilinear_u8.restype = None
        lib.tlo_resize_bilinear_u8.argtypes = [_u8p, _u8p, C.c_int, C.c_int, C.c_int, C.c_int]
        lib.tlo_f32_to_bf16_array.restype = None
        lib.tlo_f32_to_bf16_array.argtypes = [_f32p, C.POINTER(C.c_uint16), C.c_size_t]
        lib.tlo_nchw_to_nhwc.restype = None
        lib.tlo_nchw_to_nhwc.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int]
        lib.tlo_yuv420_frame.restype = None
        lib.tlo_yuv420_frame.argtypes = [_u8p, _u8p, _u8p] + [C.c_int] * 8 + [_f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p]
    else:
        flavour = impl.split("-", 1)[1] if "-" in impl else "parity"
        if not ref_available(flavour):
            raise FileNotFoundError(f"reference harness flavour {flavour!r} is not usable on this host")
        lib = C.CDLL(os.path.join(REF_DIR, f"libtl_ref_{flavour}.so"))
        lib.tlref_fused_batch.restype = C.c_int
        lib.tlref_fused_batch.argtypes = [_u8p, _i64p, _i32p, C.c_int64, _i64p, _i32p, _u8p, C.c_int,
                                          C.c_int, C.c_int, _f32p, _f32p, C.c_int, _f32p, C.c_int]
        lib.tlref_fused_batch_aa.restype = C.c_int
        lib.tlref_fused_batch_aa.argtypes = lib.tlref_fused_batch.argtypes + [C.c_int]
        lib.tlref_resize_bilinear.restype = None
        lib.tlref_resize_bilinear.argtypes = [_u8p, _u8p, C.c_int, C.c_int, C.c_int, C.c_int]
        lib.tlref_threads.restype = C.c_int
        lib.tlref_simd_branch.restype = C.c_char_p
        lib.tlref_shard_indices.restype = C.c_int64
        lib.tlref_shard_indices.argtypes = [C.c_int, C.c_int64, C.c_int64, C.c_int64, _i64p, C.c_int64]
        lib.tlref_sampler_indices.restype = C.c_int64
        lib.tlref_sampler_indices.argtypes = [C.c_int64, C.c_int, C.c_int, C.c_int, C.c_uint64,
                                              C.c_uint64, C.c_int, _i64p, C.c_int64]
    _libs[impl] = lib
    return lib


def _ptr(a, ty):
    return a.ctypes.data_as(ty) if a is not None else None


def fused_batch(src, offsets, sizes, sel, boxes, flips, dst_h, dst_w, mean, std, normalize_01=True,
                impl="port", threads=1, out=None, antialias=False, jitter=None):
    """fp32 NCHW result of crop -> bilinear(u8, truncating) -> flip -> normalize.

    ``src`` packed uint8, ``offsets`` int64[n_src], ``sizes`` int32[n_src,2] as (w,h),
    ``sel`` int64[n] or None, ``boxes`` int32[n,4] (x,y,w,h) or None, ``flips`` uint8[n] or None.
    ``jitter`` float32[n,3] (brightness, contrast, saturation) applies the colour jitter of the
    reference's train_transform shader between the 8-bit code and the normalize (C restatement
    only; needs ``normalize_01``).  Raises IndexError naming the first invalid sample.
    """
    src = np.ascontiguousarray(src, dtype=np.uint8).reshape(-1)
    offsets = np.ascontiguousarray(offsets, dtype=np.int64)
    sizes = np.ascontiguousarray(sizes, dtype=np.int32).reshape(-1, 2)
    n_src = sizes.shape[0]
    sel = None if sel is None else np.ascontiguousarray(sel, dtype=np.int64)
    boxes = None if boxes is None else np.ascontiguousarray(boxes, dtype=np.int32).reshape(-1, 4)
    flips = None if flips is None else np.ascontiguousarray(flips, dtype=np.uint8)
    n = len(sel) if sel is not None else (len(boxes) if boxes is not None else n_src)
    mean = np.asarray(mean, dtype=np.float32)
    std = np.asarray(std, dtype=np.float32)
    if out is None:
        out = np.empty((n, 3, dst_h, dst_w), dtype=np.float32)
    lib = _load(impl)
    args = [_ptr(src, _u8p), _ptr(offsets, _i64p), _ptr(sizes, _i32p), n_src, _ptr(sel, _i64p),
            _ptr(boxes, _i32p), _ptr(flips, _u8p), n, dst_h, dst_w, _ptr(mean, _f32p),
            _ptr(std, _f32p), int(bool(normalize_01)), _ptr(out, _f32p)]
    if jitter is not None:
        if impl != "port" or not normalize_01:
            raise ValueError("jitter: C restatement only, normalize_01")
        jitter = np.ascontiguousarray(jitter, dtype=np.float32).reshape(n, 3)
        fn = lib.tlo_fused_batch_aa_jitter if antialias else lib.tlo_fused_batch_jitter
        rc = fn(*args[:12], _ptr(jitter, _f32p), _ptr(out, _f32p))
    elif antialias:
        rc = (lib.tlo_fused_batch_aa(*args, 1) if impl == "port"
              else lib.tlref_fused_batch_aa(*args, int(threads), 1))
    else:
        rc = lib.tlo_fused_batch(*args) if impl == "port" else lib.tlref_fused_batch(*args, int(threads))
    if rc != 0:
        raise IndexError(f"sample {-rc - 1}: index or crop box out of range")
    return out


def resize_bilinear_u8(img, dst_h, dst_w, impl="port"):
    img = np.ascontiguousarray(img, dtype=np.uint8)
    sh, sw = img.shape[:2]
    out = np.empty((dst_h, dst_w, 3), dtype=np.uint8)
    lib = _load(impl)
    fn = lib.tlo_resize_bilinear_u8 if impl == "port" else lib.tlref_resize_bilinear
    fn(_ptr(img, _u8p), _ptr(out, _u8p), sw, sh, dst_w, dst_h)
    return out


def bf16_bits(x):
    """Round-to-nearest-even bf16 bit patterns (uint16) of an fp32 array."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    _load("port").tlo_f32_to_bf16_array(_ptr(x, _f32p), out.ctypes.data_as(C.POINTER(C.c_uint16)), x.size)
    return out


def nchw_to_nhwc(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, c, h, w = x.shape
    assert c == 3
    out = np.empty((n, h, w, 3), dtype=np.float32)
    _load("port").tlo_nchw_to_nhwc(_ptr(x, _f32p), _ptr(out, _f32p), n, h, w)
    return out


def ref_threads(flavour="parity"):
    return int(_load(f"ref-{flavour}").tlref_threads())


def ref_branch(flavour="parity"):
    return _load(f"ref-{flavour}").tlref_simd_branch().decode()


# ---- sharding (reference index math through the compiled headers) -----------------------

def ref_shard_indices(kind, total, world, rank):
    lib = _load("ref-parity")
    out = np.empty(max(int(total), 1), dtype=np.int64)
    k = lib.tlref_shard_indices(int(kind), int(total), int(world), int(rank), _ptr(out, _i64p), out.size)
    if k < 0:
        raise ValueError("reference constructor rejected the arguments")
    return out[:k].copy()


def ref_sampler_indices(total, world, rank, shuffle, seed, epoch, drop_last):
    lib = _load("ref-parity")
    out = np.empty(int(total) + int(world) + 1, dtype=np.int64)
    k = lib.tlref_sampler_indices(int(total), int(world), int(rank), int(shuffle), int(seed), int(epoch),
                                  int(drop_last), _ptr(out, _i64p), out.size)
    if k < 0:
        raise ValueError("reference constructor rejected the arguments")
    return out[:k].copy()


def ref_direct_order(total, shuffle, seed, epoch, distributed, rank, world):
    """Epoch order from DirectBatchCore::build_order, by running the compiled class over `total`
    one-pixel samples."""
    imgs = [np.zeros((1, 1, 3), np.uint8)] * int(total)
    core = RefDirectBatchCore(imgs, 1, 1, 1, shuffle=bool(shuffle), seed=int(seed), distributed=bool(distributed),
                              world_rank=int(rank), world_size=int(world))
    core.begin_epoch(int(epoch))
    return core.order()


# ---- the reference's DirectBatchCore itself (oracle/_ref/libtl_ref_dbc.so) ---------------------

REF_DBC_SO = os.path.join(REF_DIR, "libtl_ref_dbc.so")


def build_ref_dbc(ref_root: str = REF_ROOT) -> bool:
    if not os.path.isfile(os.path.join(ref_root, "src", "pipeline", "direct_batch_loader.hpp")):
        return False
    subprocess.check_call(["make", "-C", HERE, "refdbc", f"REF={ref_root}"], stdout=subprocess.DEVNULL)
    return True


def ref_dbc():
    """ctypes handle of the compiled DirectBatchCore harness, or None when it was not built."""
    if "dbc" not in _libs:
        if not os.path.exists(REF_DBC_SO) or "avx2" not in _cpu_flags():
            return None
        lib = C.CDLL(REF_DBC_SO)
        lib.tlref_dbc_create.restype = C.c_void_p
        lib.tlref_dbc_create.argtypes = [_u8p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _f32p, _f32p,
                                         C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                         C.c_float]
        lib.tlref_dbc_destroy.restype = None
        lib.tlref_dbc_destroy.argtypes = [C.c_void_p]
        lib.tlref_dbc_num_samples.restype = C.c_int64
        lib.tlref_dbc_num_samples.argtypes = [C.c_void_p]
        lib.tlref_dbc_begin_epoch.restype = None
        lib.tlref_dbc_begin_epoch.argtypes = [C.c_void_p, C.c_int, C.c_int64]
        lib.tlref_dbc_next.restype = C.c_int
        lib.tlref_dbc_next.argtypes = [C.c_void_p, _i64p, _f32p]
        lib.tlref_dbc_order.restype = C.c_int64
        lib.tlref_dbc_order.argtypes = [C.c_void_p, _i64p, C.c_int64]
        lib.tlref_dbc_pick_crops.restype = None
        lib.tlref_dbc_pick_crops.argtypes = [C.c_void_p, _i32p, _i64p, C.c_int64, _i32p]
        lib.tlref_dbc_decode_failures.restype = C.c_int64
        lib.tlref_dbc_decode_failures.argtypes = [C.c_void_p]
        _libs["dbc"] = lib
    return _libs["dbc"]


def raw8_tar(images) -> np.ndarray:
    """An in-memory ustar archive with one "RAW8" sample (header + HWC RGB pixels, the container the
    stand-in decoder of the DirectBatchCore harness reads) per image, named 000000.jpg, 000001.jpg ..."""
    import io
    import tarfile

    buf = io.BytesIO()
    with tarfile.open(fileobj=buf, mode="w", format=tarfile.USTAR_FORMAT) as tf:
        for i, im in enumerate(images):
            im = np.ascontiguousarray(im, dtype=np.uint8)
            h, w = im.shape[:2]
            payload = b"RAW8" + np.array([w, h], dtype="<i4").tobytes() + im.tobytes()
            info = tarfile.TarInfo(f"{i:06d}.jpg")
            info.size = len(payload)
            tf.addfile(info, io.BytesIO(payload))
    return np.frombuffer(buf.getvalue(), dtype=np.uint8).copy()


class RefDirectBatchCore:
    """The reference's DirectBatchCore (unmodified, compiled in place) over an in-memory archive of
    pre-decoded images.  Same constructor arguments as the C++ class
    (src/pipeline/direct_batch_loader.hpp:34-41)."""

    def __init__(self, images, batch_size, target_h, target_w, *, chw=True, normalize_01=True, mean=None, std=None,
                 shuffle=False, seed=0, distributed=False, world_rank=0, world_size=1, drop_last=False,
                 antialias=False, train_aug=False, hflip_prob=0.5):
        self._lib = ref_dbc()
        if self._lib is None:
            raise FileNotFoundError("the DirectBatchCore harness (oracle/_ref/libtl_ref_dbc.so) is not built")
        tar = raw8_tar(images)
        m = None if mean is None else np.asarray(mean, np.float32)
        s = None if std is None else np.asarray(std, np.float32)
        self._h = self._lib.tlref_dbc_create(_ptr(tar, _u8p), tar.size, int(batch_size), int(target_h), int(target_w),
                                             int(chw), int(normalize_01), _ptr(m, _f32p), _ptr(s, _f32p), int(shuffle),
                                             int(seed), int(distributed), int(world_rank), int(world_size),
                                             int(drop_last), int(antialias), int(train_aug), float(hflip_prob))
        if not self._h:
            raise RuntimeError("DirectBatchCore constructor failed")
        self.batch_size, self.h, self.w, self.chw = int(batch_size), int(target_h), int(target_w), bool(chw)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.tlref_dbc_destroy(self._h)
            self._h = None

    def num_samples(self):
        return int(self._lib.tlref_dbc_num_samples(self._h))

    def begin_epoch(self, epoch, start_batch=0):
        self._lib.tlref_dbc_begin_epoch(self._h, int(epoch), int(start_batch))

    def order(self):
        out = np.empty(1 << 20, np.int64)
        k = self._lib.tlref_dbc_order(self._h, _ptr(out, _i64p), out.size)
        return out[:k].copy()

    def next(self):
        """(indices int64[bs], float32 batch) or None at the end of the epoch."""
        idx = np.empty(self.batch_size, np.int64)
        shape = (self.batch_size, 3, self.h, self.w) if self.chw else (self.batch_size, self.h, self.w, 3)
        out = np.empty(shape, np.float32)
        bs = self._lib.tlref_dbc_next(self._h, _ptr(idx, _i64p), _ptr(out, _f32p))
        if bs == 0:
            return None
        return idx[:bs].copy(), out[:bs].copy()

    def pick_crops(self, sizes_wh, indices):
        """int32[n,5] (x, y, w, h, flip) from DirectBatchCore::pick_crop for the current epoch."""
        sizes = np.ascontiguousarray(sizes_wh, np.int32).reshape(-1, 2)
        idx = np.ascontiguousarray(indices, np.int64)
        out = np.empty((len(idx), 5), np.int32)
        self._lib.tlref_dbc_pick_crops(self._h, _ptr(sizes, _i32p), _ptr(idx, _i64p), len(idx), _ptr(out, _i32p))
        return out

    def decode_failures(self):
        return int(self._lib.tlref_dbc_decode_failures(self._h))


# ---- the reference's own CUDA kernels, compiled in place (oracle/_ref/libtl_ref_cuda.so) ---------

REF_CUDA_SO = os.path.join(REF_DIR, "libtl_ref_cuda.so")
REF_CUDA_NOFMA_SO = os.path.join(REF_DIR, "libtl_ref_cuda_nofma.so")  # same sources, --fmad=false
_ref_cuda = {}


def build_ref_cuda(ref_root: str = REF_ROOT) -> bool:
    if not os.path.isfile(os.path.join(ref_root, "src", "cuda", "cuda_transforms.cu")):
        return False
    subprocess.check_call(["make", "-C", HERE, "refcuda", f"REF={ref_root}"], stdout=subprocess.DEVNULL)
    return True


def ref_cuda(nofma: bool = False):
    """ctypes handle of the reference GPU entry points, or None when the library is absent.
    ``nofma`` selects the build without FMA contraction (every fp32 operation rounds separately)."""
    path = REF_CUDA_NOFMA_SO if nofma else REF_CUDA_SO
    if path not in _ref_cuda:
        if not os.path.exists(path):
            return None
        lib = C.CDLL(path)
        lib.tlrefcuda_available.restype = C.c_int
        lib.tlrefcuda_normalize_resident.restype = C.c_size_t
        lib.tlrefcuda_normalize_resident.argtypes = [C.c_size_t, C.c_int, C.c_int, C.c_int, _f32p, _f32p]
        lib.tlrefcuda_normalize_resident_gather.restype = C.c_size_t
        lib.tlrefcuda_normalize_resident_gather.argtypes = [C.c_size_t, C.c_size_t, C.c_int, C.c_int, C.c_int, _f32p, _f32p]
        pp = C.POINTER(C.c_void_p)
        lib.tlrefcuda_resize_normalize.restype = C.c_int
        lib.tlrefcuda_resize_normalize.argtypes = [pp, _i32p, _i32p, C.c_int, C.c_int, C.c_int, _f32p, _f32p, _f32p]
        lib.tlrefcuda_crop_resize_normalize.restype = C.c_int
        lib.tlrefcuda_crop_resize_normalize.argtypes = [pp, _i32p, _i32p, _f32p, _i32p, C.c_int, C.c_int, C.c_int, _f32p,
                                                        _f32p, _f32p]
        up = C.POINTER(C.c_size_t)
        lib.tlrefcuda_video_yuv420_batch.restype = C.c_size_t
        lib.tlrefcuda_video_yuv420_batch.argtypes = [up, up, up] + [C.c_int] * 9 + [_f32p, _f32p]
        lib.tlrefcuda_video_clip_yuv420.restype = C.c_size_t
        lib.tlrefcuda_video_clip_yuv420.argtypes = [up, up, up] + [C.c_int] * 8 + [_f32p, C.c_int, C.c_int, _f32p, _f32p]
        lib.tlrefcuda_stream_create.restype = C.c_void_p
        lib.tlrefcuda_stream_create.argtypes = [C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int, _f32p, _f32p, C.c_int, C.c_int]
        lib.tlrefcuda_stream_destroy.restype = None
        lib.tlrefcuda_stream_destroy.argtypes = [C.c_void_p]
        lib.tlrefcuda_stream_num_batches.restype = C.c_int
        lib.tlrefcuda_stream_num_batches.argtypes = [C.c_void_p]
        lib.tlrefcuda_stream_begin_epoch.restype = None
        lib.tlrefcuda_stream_begin_epoch.argtypes = [C.c_void_p]
        lib.tlrefcuda_stream_next.restype = C.c_size_t
        lib.tlrefcuda_stream_next.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
        _ref_cuda[path] = lib
    return _ref_cuda[path]


def ref_cuda_video(y_ptrs, cb_ptrs, cr_ptrs, y_stride, c_stride, c_px_stride, src_w, src_h, dst_h, dst_w, mean, std,
                   crop=None, flip=False, bt709=False, nofma=False):
    """The reference's video_yuv420_batch (crop None) / video_clip_yuv420 on device plane addresses;
    returns the device address of its (n,3,dst_h,dst_w) float32 result (valid until its next call)."""
    lib = ref_cuda(nofma)
    n = len(y_ptrs)
    arrs = [(C.c_size_t * n)(*[int(p) for p in ps]) for ps in (y_ptrs, cb_ptrs, cr_ptrs)]
    mean = np.asarray(mean, dtype=np.float32)
    std = np.asarray(std, dtype=np.float32)
    if crop is None:
        out = lib.tlrefcuda_video_yuv420_batch(*arrs, n, y_stride, c_stride, c_px_stride, src_w, src_h, dst_h, dst_w,
                                               int(bool(bt709)), _ptr(mean, _f32p), _ptr(std, _f32p))
    else:
        cr = np.asarray(crop, dtype=np.float32)
        out = lib.tlrefcuda_video_clip_yuv420(*arrs, n, y_stride, c_stride, c_px_stride, src_w, src_h, dst_h, dst_w,
                                              _ptr(cr, _f32p), int(bool(flip)), int(bool(bt709)), _ptr(mean, _f32p),
                                              _ptr(std, _f32p))
    if not out:
        raise RuntimeError("reference video call failed")
    return int(out)


def yuv420_frame(y, cb, cr, c_px_stride, src_w, src_h, dst_h, dst_w, mean, std, crop=None, flip=False, bt709=False,
                 y_stride=None, c_stride=None):
    """CPU restatement (oracle/video_ref.c) of the fused YUV 4:2:0 transform for ONE frame:
    ``y``, ``cb``, ``cr`` are uint8 arrays holding the planes (for NV12 pass the interleaved plane as
    ``cb`` and ``cb.reshape(-1)[1:]`` as ``cr``); returns float32 (3, dst_h, dst_w)."""
    lib = _load("port")
    y_stride = y.strides[0] if y_stride is None else y_stride
    c_stride = cb.strides[0] if c_stride is None else c_stride
    mean = np.asarray(mean, dtype=np.float32)
    std = np.asarray(std, dtype=np.float32)
    cw = np.zeros(4, np.float32) if crop is None else np.asarray(crop, dtype=np.float32)
    out = np.empty((3, dst_h, dst_w), dtype=np.float32)
    lib.tlo_yuv420_frame(y.ctypes.data_as(_u8p), cb.ctypes.data_as(_u8p), cr.ctypes.data_as(_u8p), int(y_stride),
                         int(c_stride), int(c_px_stride), src_w, src_h, dst_w, dst_h, 0 if crop is None else 1,
                         _ptr(cw, _f32p), int(bool(flip)), int(bool(bt709)), _ptr(mean, _f32p), _ptr(std, _f32p),
                         _ptr(out, _f32p))
    return out


def ref_cuda_crop_resize_normalize(images, crops_xywh, flips, dst_h, dst_w, mean, std):
    """The reference's crop_resize_normalize_batch on host images -> host float32 NCHW."""
    lib = ref_cuda()
    n = len(images)
    holds = [np.ascontiguousarray(im, dtype=np.uint8) for im in images]
    ptrs = (C.c_void_p * n)(*[h.ctypes.data for h in holds])
    ws = np.array([h.shape[1] for h in holds], dtype=np.int32)
    hs = np.array([h.shape[0] for h in holds], dtype=np.int32)
    mean = np.asarray(mean, dtype=np.float32)
    std = np.asarray(std, dtype=np.float32)
    out = np.empty((n, 3, dst_h, dst_w), dtype=np.float32)
    if crops_xywh is None:
        ok = lib.tlrefcuda_resize_normalize(ptrs, _ptr(ws, _i32p), _ptr(hs, _i32p), n, dst_h, dst_w, _ptr(mean, _f32p),
                                            _ptr(std, _f32p), _ptr(out, _f32p))
    else:
        cr = np.ascontiguousarray(crops_xywh, dtype=np.float32)
        fl = np.ascontiguousarray(flips, dtype=np.int32)
        ok = lib.tlrefcuda_crop_resize_normalize(ptrs, _ptr(ws, _i32p), _ptr(hs, _i32p), _ptr(cr, _f32p), _ptr(fl, _i32p), n,
                                                 dst_h, dst_w, _ptr(mean, _f32p), _ptr(std, _f32p), _ptr(out, _f32p))
    if not ok:
        raise RuntimeError("reference CUDA call failed")
    return out
