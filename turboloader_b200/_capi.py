"""ctypes binding of the C ABI in ``include/turboloader_b200.h``.

The shared library is the only compute path of this package: if it is missing the import
fails loudly (``build.build()`` creates it with nvcc); there is no CPU or eager fallback.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

TLB_OK = 0
ERR_NAMES = {1: "INVALID_ARG", 2: "BAD_BOX", 3: "BAD_INDEX", 4: "TOO_WIDE", 5: "CUDA", 6: "NO_DEVICE",
             7: "TOO_LARGE"}
TLB_F32, TLB_BF16 = 0, 1
TLB_NCHW, TLB_NHWC = 0, 1
STATIC_SCRATCH_BYTES = 32 * 1024 * 1024  # TLB_STATIC_SCRATCH_BYTES
STATIC_MAX_SAMPLES = 4096                # TLB_STATIC_MAX_SAMPLES
DEV_BAD_INDEX, DEV_BAD_BOX, DEV_TOO_WIDE, DEV_COPY_TIMEOUT = 1, 2, 4, 8
FLAG_LAUNCH_OVERLAP = 1                  # TLB_FLAG_LAUNCH_OVERLAP


class TransformDesc(C.Structure):
    """``tlb_transform_desc`` (field order and types must match the header)."""
    _fields_ = [
        ("src", C.c_void_p),
        ("src_bytes", C.c_uint64),
        ("n_src", C.c_int64),
        ("src_offsets", C.c_void_p),
        ("src_sizes", C.c_void_p),
        ("src_w", C.c_int32),
        ("src_h", C.c_int32),
        ("n", C.c_int32),
        ("sel", C.c_void_p),
        ("boxes", C.c_void_p),
        ("uniform_box", C.c_int32 * 4),
        ("flips", C.c_void_p),
        ("dst_h", C.c_int32),
        ("dst_w", C.c_int32),
        ("out", C.c_void_p),
        ("out_dtype", C.c_int32),
        ("out_layout", C.c_int32),
        ("out_indices", C.c_void_p),
        ("labels_in", C.c_void_p),
        ("labels_out", C.c_void_p),
        ("mean", C.c_float * 3),
        ("std", C.c_float * 3),
        ("normalize_01", C.c_int32),
        ("max_crop_w", C.c_int32),
        ("status", C.c_void_p),
        ("antialias", C.c_int32),
        ("max_crop_h", C.c_int32),
        ("jitter", C.c_void_p),
        ("flags", C.c_uint32),
    ]


class VideoDesc(C.Structure):
    """``tlb_video_desc`` (field order and types must match the header)."""
    _fields_ = [
        ("y_ptrs", C.c_void_p),
        ("cb_ptrs", C.c_void_p),
        ("cr_ptrs", C.c_void_p),
        ("n", C.c_int32),
        ("y_stride", C.c_int32),
        ("c_stride", C.c_int32),
        ("c_px_stride", C.c_int32),
        ("src_w", C.c_int32),
        ("src_h", C.c_int32),
        ("dst_h", C.c_int32),
        ("dst_w", C.c_int32),
        ("crops", C.c_void_p),
        ("flips", C.c_void_p),
        ("clip_len", C.c_int32),
        ("bt709", C.c_int32),
        ("mean", C.c_float * 3),
        ("std", C.c_float * 3),
        ("out", C.c_void_p),
        ("out_dtype", C.c_int32),
        ("status", C.c_void_p),
        ("flags", C.c_uint32),
    ]


class ImageRef(C.Structure):
    _fields_ = [("data", C.c_void_p), ("w", C.c_int32), ("h", C.c_int32)]


class CropParams(C.Structure):
    _fields_ = [("x", C.c_float), ("y", C.c_float), ("w", C.c_float), ("h", C.c_float), ("flip", C.c_int32)]


class TurboLoaderB200Error(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"turboloader_b200: {ERR_NAMES.get(code, code)}: {message}")
        self.code = code


_F3 = C.c_float * 3
_lib = None


def lib_path() -> str:
    return _build.LIB


def load() -> C.CDLL:
    """Load (building first if the sources are newer) the C-ABI library."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB
    if not os.path.exists(path) or os.environ.get("TLB_REBUILD"):
        path = _build.build()
    lib = C.CDLL(path)
    lib.tlb_available.restype = C.c_int
    lib.tlb_device_name.restype = C.c_int
    lib.tlb_device_name.argtypes = [C.c_int, C.c_char_p, C.c_size_t]
    lib.tlb_version.restype = C.c_char_p
    lib.tlb_last_error.restype = C.c_char_p
    lib.tlb_fused_transform.restype = C.c_int
    lib.tlb_fused_transform.argtypes = [C.POINTER(TransformDesc), C.c_void_p]
    lib.tlb_fused_transform_host_params.restype = C.c_int
    lib.tlb_fused_transform_host_params.argtypes = [C.POINTER(TransformDesc), C.c_void_p]
    lib.tlb_resize_normalize_batch.restype = C.c_int
    lib.tlb_resize_normalize_batch.argtypes = [C.POINTER(ImageRef), C.c_int32, C.c_int32, C.c_int32, _F3, _F3,
                                               C.c_void_p]
    lib.tlb_crop_resize_normalize_batch.restype = C.c_int
    lib.tlb_crop_resize_normalize_batch.argtypes = [C.POINTER(ImageRef), C.POINTER(CropParams), C.c_int32,
                                                    C.c_int32, C.c_int32, _F3, _F3, C.c_void_p]
    lib.tlb_crop_resize_normalize_to_device.restype = C.c_int
    lib.tlb_crop_resize_normalize_to_device.argtypes = [C.POINTER(ImageRef), C.POINTER(CropParams), C.c_int32,
                                                        C.c_int32, C.c_int32, _F3, _F3, C.c_int32, C.c_void_p,
                                                        C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    lib.tlb_crop_resize_normalize_to_device_static.restype = C.c_int
    lib.tlb_crop_resize_normalize_to_device_static.argtypes = lib.tlb_crop_resize_normalize_to_device.argtypes
    lib.tlb_normalize_resident_batch.restype = C.c_size_t
    lib.tlb_normalize_resident_batch.argtypes = [C.c_size_t, C.c_int32, C.c_int32, C.c_int32, _F3, _F3]
    lib.tlb_normalize_resident_gather_batch.restype = C.c_size_t
    lib.tlb_normalize_resident_gather_batch.argtypes = [C.c_size_t, C.c_size_t, C.c_int32, C.c_int32, C.c_int32,
                                                        _F3, _F3]
    up = C.POINTER(C.c_size_t)
    lib.tlb_resize_normalize_device_batch.restype = C.c_size_t
    lib.tlb_resize_normalize_device_batch.argtypes = [up, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.c_int32,
                                                      C.c_int32, C.c_int32, _F3, _F3]
    lib.tlb_video_yuv420.restype = C.c_int
    lib.tlb_video_yuv420.argtypes = [C.POINTER(VideoDesc), C.c_void_p]
    lib.tlb_video_yuv420_batch.restype = C.c_size_t
    lib.tlb_video_yuv420_batch.argtypes = [up, up, up] + [C.c_int32] * 9 + [_F3, _F3]
    lib.tlb_video_clip_yuv420.restype = C.c_size_t
    lib.tlb_video_clip_yuv420.argtypes = [up, up, up] + [C.c_int32] * 8 + [C.c_float * 4, C.c_int32, C.c_int32, _F3, _F3]
    lib.tlb_stream_create.restype = C.c_void_p
    lib.tlb_stream_create.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, _F3, _F3, C.c_int32,
                                      C.c_int32, C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.c_int32, C.c_int32]
    lib.tlb_stream_destroy.restype = None
    lib.tlb_stream_destroy.argtypes = [C.c_void_p]
    lib.tlb_stream_num_batches.restype = C.c_int64
    lib.tlb_stream_num_batches.argtypes = [C.c_void_p]
    lib.tlb_stream_begin_epoch.restype = C.c_int
    lib.tlb_stream_begin_epoch.argtypes = [C.c_void_p, C.c_void_p]
    lib.tlb_stream_next.restype = C.c_int
    lib.tlb_stream_next.argtypes = [C.c_void_p, C.POINTER(C.c_size_t), C.POINTER(C.c_int32), C.c_void_p]
    lib.tlb_stream_status.restype = C.c_int
    lib.tlb_stream_status.argtypes = [C.c_void_p, C.POINTER(C.c_uint32)]
    lib.tlb_epoch_create.restype = C.c_void_p
    lib.tlb_epoch_create.argtypes = [C.POINTER(TransformDesc), C.c_int64, C.c_int32, C.c_int64, C.c_int32, C.c_int32,
                                     C.c_int64, C.c_int64, C.c_int64]
    lib.tlb_epoch_next.restype = C.c_int
    lib.tlb_epoch_next.argtypes = [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                   C.c_void_p]
    lib.tlb_epoch_destroy.restype = None
    lib.tlb_epoch_destroy.argtypes = [C.c_void_p]
    lib.tlb_fused_plan.restype = C.c_int
    lib.tlb_fused_plan.argtypes = [C.POINTER(TransformDesc)] + [C.POINTER(C.c_int32)] * 5
    lib.tlb_launch_count.restype = C.c_uint64
    i64p = C.POINTER(C.c_int64)
    lib.tlb_shard_indices.restype = C.c_int64
    lib.tlb_shard_indices.argtypes = [C.c_int32, C.c_int64, C.c_int64, C.c_int64, i64p, C.c_int64]
    lib.tlb_sampler_indices.restype = C.c_int64
    lib.tlb_sampler_indices.argtypes = [C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_uint64, C.c_uint64,
                                        C.c_int32, i64p, C.c_int64]
    lib.tlb_direct_order.restype = C.c_int64
    lib.tlb_direct_order.argtypes = [C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                     i64p, C.c_int64]
    lib.tlb_pick_crops.restype = C.c_int64
    lib.tlb_pick_crops.argtypes = [C.c_int32, C.c_int32, i64p, C.POINTER(C.c_int32), C.c_int64, C.c_float,
                                   C.POINTER(C.c_int32), C.POINTER(C.c_uint8)]
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != TLB_OK:
        raise TurboLoaderB200Error(rc, load().tlb_last_error().decode(errors="replace"))


def f3(v) -> "_F3":
    v = [float(x) for x in v]
    if len(v) != 3:
        raise ValueError("mean/std must have 3 elements")
    return _F3(*v)
