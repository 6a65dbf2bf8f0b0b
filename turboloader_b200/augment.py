"""Per-sample RandomResizedCrop + horizontal-flip parameters, drawn on the host for a whole
epoch up front (TurboLoader's ``train_aug=True``: DirectBatchCore::pick_crop,
src/pipeline/direct_batch_loader.hpp:141-178).  The rects are integers in source pixels and the
flags are what the fused kernel takes as ``boxes`` / ``flips``."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi

__all__ = ["pick_crops"]


def pick_crops(seed, epoch, sizes_wh, indices=None, hflip_prob=0.5):
    """``(boxes int32[n,4] (x,y,w,h), flips uint8[n])`` for images of ``sizes_wh`` = n x (w, h);
    sample i's generator is seeded with (seed, epoch, indices[i]) (indices default 0..n-1)."""
    sizes = np.ascontiguousarray(sizes_wh, dtype=np.int32).reshape(-1, 2)
    n = sizes.shape[0]
    idx = None if indices is None else np.ascontiguousarray(indices, dtype=np.int64)
    if idx is not None and idx.shape != (n,):
        raise ValueError("indices must have one entry per size")
    boxes = np.empty((n, 4), dtype=np.int32)
    flips = np.empty(n, dtype=np.uint8)
    rc = _capi.load().tlb_pick_crops(int(seed), int(epoch),
                                     None if idx is None else idx.ctypes.data_as(C.POINTER(C.c_int64)),
                                     sizes.ctypes.data_as(C.POINTER(C.c_int32)), n, float(hflip_prob),
                                     boxes.ctypes.data_as(C.POINTER(C.c_int32)), flips.ctypes.data_as(C.POINTER(C.c_uint8)))
    if rc != n:
        raise ValueError("pick_crops: every image size must be positive")
    return boxes, flips
