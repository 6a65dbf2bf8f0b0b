"""Streaming GPU loader for pre-processed uint8 datasets larger than device memory.

Keeps the constructor and iteration contract of TurboLoader's ``CudaStreamLoader``
(turboloader/cuda_loader.py:538-674): the dataset is decoded and resized once into pinned host
memory and streamed to the GPU every epoch; batches are ``(n, 3, H, W)`` float32.  The iteration
runs in the C-ABI streaming core (``tlb_stream_*``): per batch one asynchronous host-to-device copy
and one fused kernel on the slot's own stream, ``slots - 1`` batches ahead of the consumer.

Differences from the reference, on purpose: batches arrive in index order (it yields them "as
completed"); there are no worker threads; and by default nothing synchronises with the host --
the consumer's current stream is made to wait for each batch by an event
(``synchronize=True`` restores the blocking hand-over).  Optional ``crop_size`` / ``output_size``
(centre crop + bilinear resize, fused), ``dtype`` and ``channels_last`` default to the
reference's behaviour.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi, ops
from .cuda_loader import _CudaArray

__all__ = ["CudaStreamLoader"]


class CudaStreamLoader:
    def __init__(self, paths, image_size=160, batch_size=64, *, mean=ops.IMAGENET_MEAN, std=ops.IMAGENET_STD,
                 drop_last=True, num_workers=8, slots=3, **extra):
        from .tbl import decode_to_array

        arr = decode_to_array(paths, int(image_size), int(image_size), workers=num_workers)
        self._init_common(arr, batch_size, mean=mean, std=std, drop_last=drop_last, slots=slots, **extra)

    @classmethod
    def from_array(cls, array, batch_size=64, **kw):
        """Build from an in-memory or memory-mapped ``(N, H, W, 3)`` uint8 array (copied once into
        pinned memory), or from a pinned CPU uint8 torch tensor of that shape (used in place)."""
        self = cls.__new__(cls)
        self._init_common(array, batch_size, **kw)
        return self

    @classmethod
    def from_tbl(cls, path, batch_size=64, **kw):
        """Build from a pre-processed RAW_U8 ``.tbl`` file through a memory map."""
        from .tbl import open_raw_view

        view, _, _ = open_raw_view(path)
        return cls.from_array(view, batch_size, **kw)

    def _init_common(self, array, batch_size, *, mean=ops.IMAGENET_MEAN, std=ops.IMAGENET_STD, drop_last=True, slots=3,
                     crop_size=None, output_size=None, dtype=None, channels_last=False, synchronize=False, as_tensor=None):
        import torch

        if not ops.cuda_available():
            raise RuntimeError("CudaStreamLoader needs an sm_100 CUDA device and the built C-ABI library.")
        self._torch = torch
        if isinstance(array, torch.Tensor):
            if array.dtype != torch.uint8 or array.dim() != 4 or array.shape[3] != 3 or array.is_cuda:
                raise ValueError("expected a CPU uint8 tensor of shape (N, H, W, 3)")
            host = array.contiguous()
            if not host.is_pinned():
                host = host.pin_memory()
        else:
            a = np.asarray(array) if not isinstance(array, np.memmap) else array
            if a.dtype != np.uint8 or a.ndim != 4 or a.shape[3] != 3:
                raise ValueError("expected a uint8 array of shape (N, H, W, 3)")
            host = torch.empty(a.shape, dtype=torch.uint8).pin_memory()
            host.numpy()[...] = a  # one pass, straight into the pinned buffer
        self._host = host  # the core keeps a raw pointer into it
        self._n, self._H, self._W = int(host.shape[0]), int(host.shape[1]), int(host.shape[2])
        self.batch_size = int(batch_size)
        self.mean, self.std = list(mean), list(std)
        self.drop_last = bool(drop_last)
        self.dtype = dtype if dtype is not None else torch.float32
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError("dtype must be torch.float32 or torch.bfloat16")
        self.channels_last = bool(channels_last)
        self.synchronize = bool(synchronize)
        # float32 NCHW batches are yielded as __cuda_array_interface__ objects like the reference's;
        # bf16 / channels-last batches (no CAI typestr for bf16) as torch tensors.
        self._as_tensor = (self.dtype != torch.float32 or self.channels_last) if as_tensor is None else bool(as_tensor)
        box = None
        oh = ow = 0
        if crop_size is not None:
            ch, cw = (crop_size, crop_size) if np.isscalar(crop_size) else crop_size
            box = (C.c_int32 * 4)((self._W - int(cw)) // 2, (self._H - int(ch)) // 2, int(cw), int(ch))
        if output_size is not None:
            oh, ow = (output_size, output_size) if np.isscalar(output_size) else output_size
        lib = _capi.load()
        self._core = lib.tlb_stream_create(host.data_ptr(), self._n, self._H, self._W, self.batch_size, _capi.f3(mean),
                                           _capi.f3(std), int(slots), int(self.drop_last), box, int(oh), int(ow),
                                           _capi.TLB_F32 if self.dtype == torch.float32 else _capi.TLB_BF16,
                                           _capi.TLB_NHWC if self.channels_last else _capi.TLB_NCHW)
        if not self._core:
            raise RuntimeError("CudaStreamLoader: " + lib.tlb_last_error().decode(errors="replace"))
        self._out_h = int(oh) if oh else (int(box[3]) if box else self._H)
        self._out_w = int(ow) if ow else (int(box[2]) if box else self._W)

    def __len__(self):
        return self._n // self.batch_size if self.drop_last else -(-self._n // self.batch_size)

    def __del__(self):
        core, self._core = getattr(self, "_core", None), None
        if core:
            try:
                _capi.load().tlb_stream_destroy(core)
            except Exception:
                pass

    def device_status(self) -> int:
        """Drains the pipeline and returns the OR of the device status bits (0 = all samples valid)."""
        v = C.c_uint32(0)
        _capi.check(_capi.load().tlb_stream_status(self._core, C.byref(v)))
        return int(v.value)

    def __iter__(self):
        torch = self._torch
        lib = _capi.load()
        stream = None if self.synchronize else C.c_void_p(torch.cuda.current_stream().cuda_stream)
        _capi.check(lib.tlb_stream_begin_epoch(self._core, stream))
        ptr, n = C.c_size_t(0), C.c_int32(0)
        while True:
            stream = None if self.synchronize else C.c_void_p(torch.cuda.current_stream().cuda_stream)
            _capi.check(lib.tlb_stream_next(self._core, C.byref(ptr), C.byref(n), stream))
            if n.value == 0:
                return
            shape = ((n.value, self._out_h, self._out_w, 3) if self.channels_last
                     else (n.value, 3, self._out_h, self._out_w))
            if not self._as_tensor:
                yield _CudaArray(ptr.value, shape, owner=self)
                continue
            if self.dtype == torch.float32:
                yield torch.as_tensor(_CudaArray(ptr.value, shape, owner=self), device="cuda")
            else:
                # no bf16 typestr in the array interface: adopt the bytes as int16 and reinterpret
                raw = _CudaArray(ptr.value, shape, owner=self)
                raw.__cuda_array_interface__["typestr"] = "<i2"
                yield torch.as_tensor(raw, device="cuda").view(torch.bfloat16)
