"""Direct-batch image loader over the fused sm_100a transform.

The GPU form of TurboLoader's ``DirectBatchCore`` (src/pipeline/direct_batch_loader.hpp:32-327)
for PRE-DECODED images: a store of variable-size HWC uint8 images lives in device memory, and
every batch is one launch of the fused kernel (gather by the epoch order, RandomResizedCrop
rect, horizontal flip, bilinear or antialiased resize to ``(H, W)``, normalize, layout, cast).

Host-side rules are the reference's own and are checked against that class executed unmodified
(tests/test_direct_batch.py):

* epoch order: ``iota`` shuffled by ``mt19937_64(seed + epoch)``, then the rank's equal block of
  ``total // world_size`` samples (``build_order``, :116-135) -- ``direct_order``;
* ``train_aug=True``: per sample a rect and a flip flag from a generator seeded with
  ``(seed, epoch, sample index)`` (``pick_crop``, :141-178) -- ``pick_crops``;
* batches of ``batch_size`` in that order, the ragged last one kept unless ``drop_last``
  (``acquire_batch``, :98-108); ``begin_epoch(epoch, start_batch)`` resumes mid-epoch (:91-95).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi, ops
from .augment import pick_crops
from .sharding import direct_order

__all__ = ["DirectBatchLoader"]


class DirectBatchLoader:
    def __init__(self, images, batch_size, target_h, target_w, *, mean=None, std=None, shuffle=False, seed=0,
                 distributed=False, world_rank=0, world_size=1, drop_last=False, antialias=False, train_aug=False,
                 hflip_prob=0.5, dtype=None, channels_last=False, jitter=None, ring=8, device=None):
        """``images``: a sequence of HWC uint8 RGB arrays (any sizes), or a tuple
        ``(packed uint8 buffer, int64 offsets, int32 sizes[n,2] as (w,h))`` whose buffer is a host
        array or a uint8 tensor already on the device.  ``mean``/``std`` in
        [0,1] units (None: plain [0,1] floats, as the reference without a Normalize).  ``jitter``:
        optional callable ``(epoch, order) -> float32[len(order), 3]`` of per-sample (brightness,
        contrast, saturation) factors."""
        import torch

        if not ops.cuda_available():
            raise RuntimeError("DirectBatchLoader needs an sm_100 CUDA device and the built C-ABI library.")
        self._torch = torch
        self._device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        resident = None  # a store that is already a device tensor is used where it lies
        if isinstance(images, tuple) and len(images) == 3 and np.ndim(images[1]) == 1:
            packed, offsets, sizes = images
            if torch.is_tensor(packed) and packed.is_cuda:
                if packed.dtype != torch.uint8:
                    raise ValueError("a device-resident store must be a uint8 tensor")
                resident = packed.contiguous().view(-1)
                self._device = resident.device
            else:
                packed = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)
            offsets = np.ascontiguousarray(offsets, dtype=np.int64)
            sizes = np.ascontiguousarray(sizes, dtype=np.int32).reshape(-1, 2)
        else:
            images = list(images)
            for im in images:
                if im.ndim != 3 or im.shape[2] != 3 or im.dtype != np.uint8:
                    raise ValueError("every image must be HxWx3 uint8 (RGB)")
            sizes = np.array([(im.shape[1], im.shape[0]) for im in images], dtype=np.int32).reshape(-1, 2)
            nbytes = sizes[:, 0].astype(np.int64) * sizes[:, 1] * 3
            offsets = np.concatenate([[0], np.cumsum(nbytes)[:-1]]).astype(np.int64)
            packed = np.empty(int(nbytes.sum()), dtype=np.uint8)
            for im, o, b in zip(images, offsets, nbytes):
                packed[o:o + b] = np.ascontiguousarray(im).reshape(-1)
        if sizes.shape[0] == 0 or (sizes <= 0).any():
            raise ValueError("the store is empty or holds an image without pixels")
        self._n = int(sizes.shape[0])
        self._sizes = sizes
        self._src = resident if resident is not None else torch.from_numpy(packed).to(self._device)
        self._offsets = torch.from_numpy(offsets).to(self._device)
        self._d_sizes = torch.from_numpy(sizes).to(self._device)
        self.batch_size = int(batch_size)
        self._oh, self._ow = int(target_h), int(target_w)
        self.mean = list(mean) if mean is not None else [0.0, 0.0, 0.0]
        self.std = list(std) if std is not None else [1.0, 1.0, 1.0]
        self.shuffle, self.seed = bool(shuffle), int(seed)
        self.distributed, self.world_rank, self.world_size = bool(distributed), int(world_rank), int(world_size)
        self.drop_last, self.antialias, self.train_aug = bool(drop_last), bool(antialias), bool(train_aug)
        self.hflip_prob = float(hflip_prob)
        self.channels_last = bool(channels_last)
        self.dtype = torch.float32 if dtype is None else dtype
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("dtype must be torch.float32 or torch.bfloat16")
        self._jitter_fn = jitter
        self._ring_slots = max(3, int(ring))
        self._ahead = max(1, (self._ring_slots - 1) // 2)
        self._ring = None
        self._lookahead = None
        self._epoch = 0
        self._resume_batches = 0
        self._served = 0
        self._status = torch.zeros(1, dtype=torch.int32, device=self._device)

    # ---- the reference's surface -----------------------------------------------------------------
    def epoch_order(self, epoch=None) -> np.ndarray:
        e = self._epoch if epoch is None else int(epoch)
        return direct_order(self._n, self.shuffle, self.seed, e, self.distributed, self.world_rank, self.world_size)

    def num_samples(self) -> int:
        n = self.epoch_order().size
        return (n // self.batch_size) * self.batch_size if self.drop_last else n

    def __len__(self):
        n = self.epoch_order().size
        return n // self.batch_size if self.drop_last else -(-n // self.batch_size)

    def set_epoch(self, epoch):
        self._epoch = int(epoch)

    def begin_epoch(self, epoch, start_batch=0):
        self._epoch = int(epoch)
        self._resume_batches = int(start_batch)

    def state_dict(self):
        return {"version": 1, "epoch": int(self._epoch), "batches_served": int(self._served)}

    def load_state_dict(self, sd):
        self._epoch = int(sd["epoch"])
        self._resume_batches = int(sd["batches_served"])

    def device_status(self) -> int:
        """Status bits the kernels OR-ed so far (synchronises); 0 when every sample was valid."""
        return int(self._status.item())

    def epoch_crops(self, epoch=None):
        """``(boxes int32[n,4], flips uint8[n])`` per epoch position, or ``(None, None)`` without train_aug."""
        if not self.train_aug:
            return None, None
        e = self._epoch if epoch is None else int(epoch)
        order = self.epoch_order(e)
        return pick_crops(self.seed, e, self._sizes[order], indices=order, hflip_prob=self.hflip_prob)

    def _host_tables(self, epoch):
        """(order, boxes or None, flips or None) of an epoch: everything drawn on the host from
        (seed, epoch, rank) alone."""
        order = self.epoch_order(epoch)
        if not self.train_aug:
            return order, None, None
        boxes, flips = pick_crops(self.seed, epoch, self._sizes[order], indices=order, hflip_prob=self.hflip_prob)
        return order, boxes, flips

    def _epoch_tables(self, epoch):
        """This epoch's host tables, from the look-ahead if it drew them already; the NEXT epoch's are
        then drawn on a helper thread while this one is served (the shuffle of a large epoch and its
        crop rects take longer on the host than the epoch takes on the GPU)."""
        import threading

        key = lambda e: (e, self.seed, self.shuffle, self.train_aug, self.hflip_prob, self.distributed,
                         self.world_rank, self.world_size)
        pending, self._lookahead = self._lookahead, None
        tables = None
        if pending is not None:
            thread, box = pending
            thread.join()
            if box.get("key") == key(epoch):
                tables = box["tables"]
        if tables is None:
            tables = self._host_tables(epoch)
        box = {}

        def work(e=epoch + 1, k=key(epoch + 1)):
            box["tables"] = self._host_tables(e)
            box["key"] = k

        thread = threading.Thread(target=work, daemon=True)
        thread.start()
        self._lookahead = (thread, box)
        return tables

    # ---- iteration -----------------------------------------------------------------------------------
    def __iter__(self):
        torch = self._torch
        lib = _capi.load()
        bs = self.batch_size
        order, boxes, flips = self._epoch_tables(self._epoch)
        total = int(order.size)
        start = self._resume_batches
        self._resume_batches = 0
        self._served = start
        if total == 0:
            return
        with torch.cuda.device(self._device):
            d_order = torch.from_numpy(order).to(self._device)
            d_boxes = torch.from_numpy(boxes).to(self._device) if boxes is not None else None
            d_flips = torch.from_numpy(flips).to(self._device) if flips is not None else None
            d_jit = None
            if self._jitter_fn is not None:
                j = np.ascontiguousarray(self._jitter_fn(self._epoch, order), dtype=np.float32).reshape(-1, 3)
                if j.shape[0] != total:
                    raise ValueError("jitter callable must return one (brightness, contrast, saturation) per sample")
                d_jit = torch.from_numpy(j).to(self._device)
            R = self._ring_slots
            shape = (bs, self._oh, self._ow, 3) if self.channels_last else (bs, 3, self._oh, self._ow)
            if self._ring is None or tuple(self._ring.shape) != (R,) + shape:
                self._ring = torch.empty((R,) + shape, dtype=self.dtype, device=self._device)
            ring = self._ring
            d = _capi.TransformDesc()
            d.src = self._src.data_ptr()
            d.src_bytes = self._src.numel()
            d.n_src = self._n
            d.src_offsets = self._offsets.data_ptr()
            d.src_sizes = self._d_sizes.data_ptr()
            d.src_w, d.src_h = int(self._sizes[:, 0].max()), int(self._sizes[:, 1].max())
            d.n = bs
            d.sel = d_order.data_ptr()
            if d_boxes is not None:
                d.boxes = d_boxes.data_ptr()
                d.flips = d_flips.data_ptr()
                d.max_crop_w = int(boxes[:, 2].max())
                d.max_crop_h = int(boxes[:, 3].max())
            else:
                d.max_crop_w, d.max_crop_h = d.src_w, d.src_h
            if d_jit is not None:
                d.jitter = d_jit.data_ptr()
            d.dst_h, d.dst_w = self._oh, self._ow
            d.out = ring.data_ptr()
            d.out_dtype = _capi.TLB_F32 if self.dtype == torch.float32 else _capi.TLB_BF16
            d.out_layout = _capi.TLB_NHWC if self.channels_last else _capi.TLB_NCHW
            d.mean = _capi.f3(self.mean)
            d.std = _capi.f3(self.std)
            d.normalize_01 = 1
            d.antialias = int(self.antialias)
            d.status = self._status.data_ptr()
            plan = lib.tlb_epoch_create(C.byref(d), total, int(self.drop_last), start, R, self._ahead,
                                        ring[0].numel() * ring.element_size(), 0, 0)
            if not plan:
                raise _capi.TurboLoaderB200Error(1, lib.tlb_last_error().decode(errors="replace"))
            b_no, n_out, slot = C.c_int64(0), C.c_int32(0), C.c_int32(0)
            try:
                while True:
                    stream = torch.cuda.current_stream(self._device)
                    _capi.check(lib.tlb_epoch_next(plan, C.byref(b_no), C.byref(n_out), C.byref(slot),
                                                   C.c_void_p(stream.cuda_stream)))
                    n = n_out.value
                    if n == 0:
                        break
                    out = ring[slot.value, :n]
                    self._served += 1
                    b0 = b_no.value * bs
                    idx = order[b0:b0 + n].copy()
                    images = out.permute(0, 3, 1, 2) if self.channels_last else out
                    yield images, {"indices": idx, "batch_size": int(n)}
            finally:
                lib.tlb_epoch_destroy(plan)
            self._served = 0
