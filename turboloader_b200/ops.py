"""Python-facing operators: the names and argument meaning of TurboLoader's ``cuda_*``
bindings (src/python/turboloader_bindings.cpp:1623-1753) over the B200 C ABI, plus the
general ``fused_transform`` the loaders use.  torch appears only to allocate device
memory and to name the current stream; every computation happens inside the C-ABI
library.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi

IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)


def cuda_available() -> bool:
    """True if the library loads and the current device is an sm_100 GPU
    (``turboloader.cuda_available``, turboloader_bindings.cpp:1627)."""
    return bool(_capi.load().tlb_available())


def cuda_device_name(device: int = 0) -> str:
    """Device name or '' (``turboloader.cuda_device_name``, turboloader_bindings.cpp:1629)."""
    buf = C.create_string_buffer(256)
    if _capi.load().tlb_device_name(int(device), buf, 256) != 0:
        return ""
    return buf.value.decode()


def _addr_array(ptrs):
    arr = (C.c_size_t * len(ptrs))(*[int(p) for p in ptrs])
    return arr


def cuda_video_yuv420_batch(y_ptrs, cb_ptrs, cr_ptrs, y_stride, c_stride, c_px_stride, src_w, src_h, dst_h, dst_w,
                            bt709=False, mean=IMAGENET_MEAN, std=IMAGENET_STD) -> int:
    """Decoded YUV 4:2:0 frames (lists of device plane addresses) -> device address of a library-owned
    (n, 3, dst_h, dst_w) float32 batch, valid until the next video call (same name, arguments and
    lifetime as TurboLoader's binding, src/python/turboloader_bindings.cpp:1686-1709)."""
    n = len(y_ptrs)
    if not (len(cb_ptrs) == len(cr_ptrs) == n):
        raise ValueError("y_ptrs, cb_ptrs and cr_ptrs must have the same length")
    out = _capi.load().tlb_video_yuv420_batch(_addr_array(y_ptrs), _addr_array(cb_ptrs), _addr_array(cr_ptrs), n,
                                              int(y_stride), int(c_stride), int(c_px_stride), int(src_w), int(src_h),
                                              int(dst_h), int(dst_w), int(bool(bt709)), _capi.f3(mean), _capi.f3(std))
    if not out:
        raise RuntimeError("cuda_video_yuv420_batch failed: " + _capi.load().tlb_last_error().decode(errors="replace"))
    return int(out)


def cuda_video_clip_yuv420(y_ptrs, cb_ptrs, cr_ptrs, y_stride, c_stride, c_px_stride, src_w, src_h, dst_h, dst_w,
                           crop, flip=False, bt709=False, mean=IMAGENET_MEAN, std=IMAGENET_STD) -> int:
    """One (T, 3, dst_h, dst_w) float32 clip from T decoded frames with the SAME crop window
    (x, y, w, h in source pixels) and flip for every frame (turboloader_bindings.cpp:1711-1734)."""
    n = len(y_ptrs)
    if not (len(cb_ptrs) == len(cr_ptrs) == n):
        raise ValueError("y_ptrs, cb_ptrs and cr_ptrs must have the same length")
    c4 = (C.c_float * 4)(*[float(v) for v in crop])
    out = _capi.load().tlb_video_clip_yuv420(_addr_array(y_ptrs), _addr_array(cb_ptrs), _addr_array(cr_ptrs), n,
                                             int(y_stride), int(c_stride), int(c_px_stride), int(src_w), int(src_h),
                                             int(dst_h), int(dst_w), c4, int(bool(flip)), int(bool(bt709)),
                                             _capi.f3(mean), _capi.f3(std))
    if not out:
        raise RuntimeError("cuda_video_clip_yuv420 failed: " + _capi.load().tlb_last_error().decode(errors="replace"))
    return int(out)


def make_video_desc(y_ptrs, cb_ptrs, cr_ptrs, *, y_stride, c_stride, c_px_stride, src_w, src_h, out, crops=None,
                    flips=None, clip_len=0, bt709=False, mean=IMAGENET_MEAN, std=IMAGENET_STD, status=None,
                    launch_overlap=False):
    """Fill a ``tlb_video_desc``; the returned struct keeps its host arrays alive (``_keep``) and can
    be enqueued any number of times with ``enqueue_video``.  ``launch_overlap`` sets
    ``TLB_FLAG_LAUNCH_OVERLAP`` (the caller states that the kernel before this one in the stream
    neither writes this call's frames nor touches its output)."""
    import numpy as np
    import torch

    n = len(y_ptrs)
    if not (len(cb_ptrs) == len(cr_ptrs) == n):
        raise ValueError("y_ptrs, cb_ptrs and cr_ptrs must have the same length")
    d = _capi.VideoDesc()
    keep = [_addr_array(y_ptrs), _addr_array(cb_ptrs), _addr_array(cr_ptrs)]
    d.y_ptrs, d.cb_ptrs, d.cr_ptrs = [C.cast(a, C.c_void_p) for a in keep]
    d.n = n
    d.y_stride, d.c_stride, d.c_px_stride = int(y_stride), int(c_stride), int(c_px_stride)
    d.src_w, d.src_h = int(src_w), int(src_h)
    if out.dim() != 4 or out.shape[0] != n or out.shape[1] != 3 or not out.is_contiguous():
        raise ValueError("out must be a contiguous (n, 3, dst_h, dst_w) CUDA tensor")
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("out must be float32 or bfloat16")
    d.dst_h, d.dst_w = int(out.shape[2]), int(out.shape[3])
    if crops is not None:
        cr = np.ascontiguousarray(crops, dtype=np.float32).reshape(-1, 4)
        fl = np.zeros(len(cr), np.int32) if flips is None else np.ascontiguousarray(flips, dtype=np.int32)
        keep += [cr, fl]
        d.crops, d.flips = cr.ctypes.data, fl.ctypes.data
    d.clip_len = int(clip_len)
    d.bt709 = int(bool(bt709))
    d.mean, d.std = _capi.f3(mean), _capi.f3(std)
    d.out = out.data_ptr()
    d.out_dtype = _capi.TLB_F32 if out.dtype == torch.float32 else _capi.TLB_BF16
    if status is not None:
        d.status = _dev_ptr(status, torch.int32, "status")
    d.flags = _capi.FLAG_LAUNCH_OVERLAP if launch_overlap else 0
    d._keep = keep + [out, status]
    return d


def enqueue_video(desc, stream_ptr) -> None:
    """``tlb_video_yuv420`` on a raw stream handle (int)."""
    _capi.check(_capi.load().tlb_video_yuv420(C.byref(desc), C.c_void_p(stream_ptr)))


def video_yuv420(y_ptrs, cb_ptrs, cr_ptrs, *, out, stream=None, **kw):
    """Asynchronous form (``tlb_video_yuv420``): ``out`` is a caller-allocated CUDA tensor
    (n, 3, dst_h, dst_w), float32 or bfloat16; ``crops`` an (n_clips, 4) array of windows shared by
    ``clip_len`` consecutive frames each (None: whole-frame resize).  Keyword arguments as
    ``make_video_desc``."""
    import torch

    d = make_video_desc(y_ptrs, cb_ptrs, cr_ptrs, out=out, **kw)
    st = stream if stream is not None else torch.cuda.current_stream(out.device)
    with torch.cuda.device(out.device):
        enqueue_video(d, st.cuda_stream)
    return out


def launch_count() -> int:
    return int(_capi.load().tlb_launch_count())


def _image_refs(images):
    holds, refs = [], (_capi.ImageRef * len(images))()
    for i, im in enumerate(images):
        a = np.ascontiguousarray(im, dtype=np.uint8)
        if a.ndim != 3 or a.shape[2] != 3:
            raise RuntimeError("each image must be HxWx3 uint8 (RGB)")
        holds.append(a)
        refs[i].data = a.ctypes.data
        refs[i].w = a.shape[1]
        refs[i].h = a.shape[0]
    return holds, refs


def _crop_params(crops, flips, n):
    crops = np.ascontiguousarray(crops, dtype=np.float32)
    flips = np.ascontiguousarray(flips, dtype=np.int32)
    if crops.ndim != 2 or crops.shape != (n, 4):
        raise RuntimeError("crops must have shape (N, 4): x, y, w, h in src pixels")
    if flips.ndim != 1 or flips.shape[0] != n:
        raise RuntimeError("flips must have shape (N,)")
    arr = (_capi.CropParams * n)()
    for i in range(n):
        arr[i].x, arr[i].y, arr[i].w, arr[i].h = (float(v) for v in crops[i])
        arr[i].flip = int(flips[i])
    return arr


def cuda_resize_normalize(images, dst_h, dst_w, mean=IMAGENET_MEAN, std=IMAGENET_STD):
    """List of HWC uint8 RGB arrays -> host float32 ``(N, 3, dst_h, dst_w)``
    (``turboloader.cuda_resize_normalize``, turboloader_bindings.cpp:1631-1664)."""
    images = list(images)
    if not images:
        raise RuntimeError("cuda_resize_normalize: empty image list")
    holds, refs = _image_refs(images)
    out = np.empty((len(images), 3, int(dst_h), int(dst_w)), dtype=np.float32)
    _capi.check(_capi.load().tlb_resize_normalize_batch(refs, len(images), int(dst_h), int(dst_w), _capi.f3(mean),
                                                        _capi.f3(std), out.ctypes.data))
    del holds
    return out


def cuda_crop_resize_normalize(images, crops, flips, dst_h, dst_w, mean=IMAGENET_MEAN, std=IMAGENET_STD):
    """Fused crop + flip + resize + normalize of host images -> host float32 NCHW.  Same
    arguments as the reference's ``metal_crop_resize_normalize`` binding
    (turboloader_bindings.cpp:1326-1363); the CUDA twin exists in the reference
    (src/cuda/cuda_transforms.hpp:117-119) but is not bound there.  Crop values must be
    whole pixels: results follow the CPU fused path, whose crop rects are integers."""
    images = list(images)
    if not images:
        raise RuntimeError("cuda_crop_resize_normalize: empty image list")
    holds, refs = _image_refs(images)
    cps = _crop_params(crops, flips, len(images))
    out = np.empty((len(images), 3, int(dst_h), int(dst_w)), dtype=np.float32)
    _capi.check(_capi.load().tlb_crop_resize_normalize_batch(refs, cps, len(images), int(dst_h), int(dst_w),
                                                             _capi.f3(mean), _capi.f3(std), out.ctypes.data))
    del holds
    return out


def cuda_normalize_resident(src_dev, N, H, W, mean=IMAGENET_MEAN, std=IMAGENET_STD) -> int:
    """Device ``[N,H,W,3]`` uint8 at address ``src_dev`` -> device address (int) of the
    ``[N,3,H,W]`` float32 batch, valid until the 4th-next call
    (``turboloader.cuda_normalize_resident``, turboloader_bindings.cpp:1665-1684)."""
    ptr = _capi.load().tlb_normalize_resident_batch(int(src_dev), int(N), int(H), int(W), _capi.f3(mean),
                                                    _capi.f3(std))
    if not ptr:
        raise RuntimeError("cuda_normalize_resident failed: " + _capi.load().tlb_last_error().decode())
    return int(ptr)


def cuda_normalize_resident_gather(src_dev, sel_dev, N, H, W, mean=IMAGENET_MEAN, std=IMAGENET_STD) -> int:
    """Like ``cuda_normalize_resident`` but sample n reads dataset image ``sel_dev[n]``
    (device int64) (``turboloader.cuda_normalize_resident_gather``,
    turboloader_bindings.cpp:1736-1753)."""
    ptr = _capi.load().tlb_normalize_resident_gather_batch(int(src_dev), int(sel_dev), int(N), int(H), int(W),
                                                           _capi.f3(mean), _capi.f3(std))
    if not ptr:
        raise RuntimeError("cuda_normalize_resident_gather failed: " + _capi.load().tlb_last_error().decode())
    return int(ptr)


def cuda_resize_normalize_from_device(ptrs, ws, hs, dst_h, dst_w, mean=IMAGENET_MEAN, std=IMAGENET_STD) -> int:
    """ALREADY-DECODED device images (device addresses ``ptrs`` of HWC uint8 RGB pixels with sizes
    ``ws`` x ``hs``, each in its own allocation, e.g. the outputs of a GPU decoder) -> device address
    (int) of the ``(N, 3, dst_h, dst_w)`` float32 batch, valid until the 4th-next call
    (``turboloader.cuda_resize_normalize_from_device``, turboloader_bindings.cpp:1900-1918)."""
    n = len(ptrs)
    if not (len(ws) == len(hs) == n) or n == 0:
        raise RuntimeError("cuda_resize_normalize_from_device: ptrs, ws and hs must be equally long and non-empty")
    wa = (C.c_int32 * n)(*[int(v) for v in ws])
    ha = (C.c_int32 * n)(*[int(v) for v in hs])
    out = _capi.load().tlb_resize_normalize_device_batch(_addr_array(ptrs), wa, ha, n, int(dst_h), int(dst_w),
                                                         _capi.f3(mean), _capi.f3(std))
    if not out:
        raise RuntimeError("cuda_resize_normalize_from_device failed: " +
                           _capi.load().tlb_last_error().decode(errors="replace"))
    return int(out)


# ---- the general device-resident call ---------------------------------------------------------

def _dev_ptr(t, dtype, what):
    import torch

    if t is None:
        return None
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError(f"{what} must be a CUDA tensor")
    if t.dtype != dtype:
        raise TypeError(f"{what} must have dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{what} must be contiguous")
    return t.data_ptr()


def make_desc(src, *, n, dst_h, dst_w, out, src_w=0, src_h=0, n_src=None, src_offsets=None, src_sizes=None,
              sel=None, boxes=None, uniform_box=None, flips=None, mean=IMAGENET_MEAN, std=IMAGENET_STD,
              normalize_01=True, channels_last=False, out_indices=None, labels_in=None, labels_out=None,
              max_crop_w=0, status=None, antialias=False, max_crop_h=0, jitter=None, launch_overlap=False):
    """Fill a ``tlb_transform_desc`` from CUDA tensors (all tables on the device).

    ``jitter``: optional float32 ``(n, 3)`` CUDA tensor of per-sample (brightness, contrast,
    saturation) factors.  ``launch_overlap``: set ``TLB_FLAG_LAUNCH_OVERLAP`` -- only for a stream
    in which the kernel directly before this launch neither writes its inputs nor touches its
    outputs (e.g. a prefetch stream carrying only this library's launches)."""
    import torch

    d = _capi.TransformDesc()
    d.src = _dev_ptr(src, torch.uint8, "src")
    d.src_bytes = src.numel()
    if n_src is None:
        n_src = src_sizes.shape[0] if src_sizes is not None else (src.shape[0] if src.dim() == 4 else n)
    d.n_src = int(n_src)
    d.src_offsets = _dev_ptr(src_offsets, torch.int64, "src_offsets")
    d.src_sizes = _dev_ptr(src_sizes, torch.int32, "src_sizes")
    if src.dim() == 4 and not (src_w and src_h):
        src_h, src_w = src.shape[1], src.shape[2]
    d.src_w, d.src_h = int(src_w), int(src_h)
    d.n = int(n)
    d.sel = _dev_ptr(sel, torch.int64, "sel")
    d.boxes = _dev_ptr(boxes, torch.int32, "boxes")
    if uniform_box is not None:
        d.uniform_box = (C.c_int32 * 4)(*[int(v) for v in uniform_box])
    d.flips = _dev_ptr(flips, torch.uint8, "flips")
    d.dst_h, d.dst_w = int(dst_h), int(dst_w)
    if out.dtype == torch.float32:
        d.out_dtype = _capi.TLB_F32
    elif out.dtype == torch.bfloat16:
        d.out_dtype = _capi.TLB_BF16
    else:
        raise TypeError("out must be float32 or bfloat16")
    if not out.is_cuda or not out.is_contiguous() or out.numel() != n * 3 * dst_h * dst_w:
        raise ValueError("out must be a contiguous CUDA tensor of n*3*dst_h*dst_w elements")
    d.out = out.data_ptr()
    d.out_layout = _capi.TLB_NHWC if channels_last else _capi.TLB_NCHW
    d.out_indices = _dev_ptr(out_indices, torch.int64, "out_indices")
    d.labels_in = _dev_ptr(labels_in, torch.int64, "labels_in")
    d.labels_out = _dev_ptr(labels_out, torch.int64, "labels_out")
    d.mean = _capi.f3(mean)
    d.std = _capi.f3(std)
    d.normalize_01 = int(bool(normalize_01))
    d.max_crop_w = int(max_crop_w)
    d.antialias = int(bool(antialias))  # the reference's opt-in triangle-filter resize
    d.max_crop_h = int(max_crop_h)
    d.status = _dev_ptr(status, torch.int32, "status")
    if jitter is not None:
        if tuple(jitter.shape) != (int(n), 3):
            raise ValueError("jitter must have shape (n, 3)")
        d.jitter = _dev_ptr(jitter, torch.float32, "jitter")
    d.flags = _capi.FLAG_LAUNCH_OVERLAP if launch_overlap else 0
    return d


def fused_transform(src, *, stream=None, **kw):
    """Enqueue one fused batch on ``stream`` (default: torch's current stream); returns
    immediately.  See ``make_desc`` for the keyword arguments."""
    import torch

    d = make_desc(src, **kw)
    st = stream if stream is not None else torch.cuda.current_stream(src.device)
    with torch.cuda.device(src.device):
        _capi.check(_capi.load().tlb_fused_transform(C.byref(d), C.c_void_p(st.cuda_stream)))
    return kw["out"]


def fused_plan(desc):
    vals = [C.c_int32() for _ in range(5)]
    _capi.check(_capi.load().tlb_fused_plan(C.byref(desc), *[C.byref(v) for v in vals]))
    keys = ("grid", "block", "smem_bytes", "tile_rows", "tile_cols")
    return {k: v.value for k, v in zip(keys, vals)}


def features() -> dict:
    """Capability dict in the spirit of ``turboloader.features()``
    (turboloader_bindings.cpp:1977-2055), honest about what this build contains."""
    ok = cuda_available()
    return {
        "version": _capi.load().tlb_version().decode(),
        "gpu_transforms": ok,
        "sm100_fused_transform": ok,
        "bf16_output": True,
        "channels_last_output": True,
        "cpu_fallback": False,
        "nvjpeg": False,
        "nvimgcodec": False,
    }
