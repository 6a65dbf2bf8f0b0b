"""GPU-resident image loader over the fused sm_100a transform.

Keeps the constructor, iteration and ``return_indices`` contract of TurboLoader's
``CudaResidentLoader`` (turboloader/cuda_loader.py:385-535): the uint8 dataset is uploaded
once, every epoch is served from HBM with one kernel launch per batch, the shuffle is the
device-side index gather fused into that kernel, and the permutation is
``np.random.default_rng(seed + epoch).permutation(n)`` (cuda_loader.py:506-510).

Additions that default to the reference behaviour: ``crop_size`` / ``output_size`` /
``hflip_prob`` / explicit ``boxes`` (crop + flip + resize fused into the same launch),
``dtype`` (float32 | bfloat16), ``channels_last``, and ``state_dict`` /
``load_state_dict`` with the same dict the CPU loaders use
(turboloader/__init__.py:689-700).  Unlike the reference there is no per-batch
synchronisation: the library prefetches batches on its own stream (``tlb_epoch_*``) and the
consumer's current stream is made to wait for each batch as it is handed out.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi, ops

__all__ = ["CudaResidentLoader", "_CudaArray"]


class _CudaArray:
    """A CUDA device pointer as a ``__cuda_array_interface__`` v3 float32 array
    (turboloader/cuda_loader.py:37-55) so torch/cupy adopt it without a copy:
    ``torch.as_tensor(x, device='cuda')``.  ``owner`` keeps the backing allocation alive.
    It also speaks DLPack (``__dlpack__`` / ``__dlpack_device__``), so ``torch.from_dlpack(x)``,
    ``cupy.from_dlpack(x)`` or ``jax.dlpack.from_dlpack(x)`` adopt the same memory; bfloat16 and
    channels-last batches are handed out as torch tensors, whose own ``__dlpack__`` serves those."""

    def __init__(self, ptr, shape, owner=None, stream=None, device=None):
        self.__cuda_array_interface__ = {
            "data": (int(ptr), False),
            "shape": tuple(int(s) for s in shape),
            "typestr": "<f4",
            "version": 3,
        }
        if stream is not None:
            self.__cuda_array_interface__["stream"] = int(stream)
        self._owner = owner
        self._device = device

    @property
    def shape(self):
        return self.__cuda_array_interface__["shape"]

    def __len__(self):
        return self.shape[0]

    def _device_index(self):
        if self._device is None:
            import torch
            self._device = torch.cuda.current_device()
        return int(self._device)

    def __dlpack_device__(self):
        return (2, self._device_index())  # (kDLCUDA, ordinal)

    def __dlpack__(self, stream=None, **kwargs):
        """Zero-copy DLPack capsule of the same device memory (the capsule keeps this object, and
        with it the backing allocation, alive)."""
        import torch
        t = torch.as_tensor(self, device=torch.device("cuda", self._device_index()))
        return t.__dlpack__(stream=stream) if stream is not None else t.__dlpack__()


class CudaResidentLoader:
    def __init__(self, paths, image_size=160, batch_size=64, *, mean=ops.IMAGENET_MEAN, std=ops.IMAGENET_STD,
                 drop_last=True, num_workers=8, shuffle=False, seed=42, return_indices=False, **extra):
        from .tbl import decode_to_array

        arr = decode_to_array(paths, int(image_size), int(image_size), workers=num_workers)
        self._init_common(arr, batch_size, mean=mean, std=std, drop_last=drop_last, shuffle=shuffle, seed=seed,
                          return_indices=return_indices, **extra)

    @classmethod
    def from_array(cls, array, batch_size=64, **kw):
        """Build from an in-memory or memory-mapped ``(N, H, W, 3)`` uint8 array (or an
        already-resident CUDA uint8 tensor of that shape)."""
        self = cls.__new__(cls)
        self._init_common(array, batch_size, **kw)
        return self

    @classmethod
    def from_tbl(cls, path, batch_size=64, **kw):
        """Build from a pre-processed RAW_U8 ``.tbl`` file (turboloader/cuda_loader.py:453-492):
        the upload reads straight through a memory map."""
        from .tbl import open_raw_view

        view, H, W = open_raw_view(path)
        if H != W:
            raise ValueError(f"resident loader needs square samples, file is {W}x{H}")
        return cls.from_array(view, batch_size, **kw)

    # ------------------------------------------------------------------------------------
    def _init_common(self, array, batch_size, *, mean=ops.IMAGENET_MEAN, std=ops.IMAGENET_STD, drop_last=True,
                     shuffle=False, seed=42, return_indices=False, crop_size=None, output_size=None,
                     hflip_prob=0.0, boxes=None, dtype=None, channels_last=False, as_tensor=None, labels=None,
                     ring=8, device=None, flips=None, train_aug=False, antialias=False, jitter=None):
        import torch

        if not ops.cuda_available():
            raise RuntimeError("CudaResidentLoader needs an sm_100 CUDA device and the built C-ABI library.")
        self._torch = torch
        self._device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if isinstance(array, torch.Tensor):
            if array.dtype != torch.uint8 or array.dim() != 4 or array.shape[3] != 3:
                raise ValueError("dataset tensor must be (N, H, W, 3) uint8")
            self._gpu = array.to(self._device).contiguous()
        else:
            if array.ndim != 4 or array.shape[3] != 3 or array.dtype != np.uint8:
                raise ValueError("dataset must be (N, H, W, 3) uint8")
            n, H, W, _ = array.shape
            # Chunked upload (~64 MB): peak host memory is one chunk even for a memory map.
            self._gpu = torch.empty((n, H, W, 3), dtype=torch.uint8, device=self._device)
            step = max(1, (64 << 20) // max(1, H * W * 3))
            for s in range(0, n, step):
                chunk = np.array(array[s:s + step])  # a writable copy (memory maps are read-only)
                self._gpu[s:s + chunk.shape[0]] = torch.from_numpy(chunk)
        self._n, self._H, self._W = int(self._gpu.shape[0]), int(self._gpu.shape[1]), int(self._gpu.shape[2])
        self.batch_size = int(batch_size)
        self.mean, self.std = list(mean), list(std)
        self.drop_last, self.shuffle, self.seed = bool(drop_last), bool(shuffle), int(seed)
        self.return_indices = bool(return_indices)
        self.hflip_prob = float(hflip_prob)
        self.channels_last = bool(channels_last)
        self.antialias = bool(antialias)  # DirectBatchCore's antialias option: triangle filter on downscale
        self.dtype = torch.float32 if dtype is None else dtype
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("dtype must be torch.float32 or torch.bfloat16")
        if crop_size is None:
            self._box = (0, 0, self._W, self._H)
        else:
            cw, ch = (crop_size, crop_size) if np.isscalar(crop_size) else (crop_size[1], crop_size[0])
            if cw > self._W or ch > self._H or cw <= 0 or ch <= 0:
                raise ValueError("crop_size must fit inside the stored images")
            # Centre crop: offset (W - cw) / 2 (src/transforms/crop_transform.hpp:37-38).
            self._box = ((self._W - int(cw)) // 2, (self._H - int(ch)) // 2, int(cw), int(ch))
        if output_size is None:
            self._oh, self._ow = self._box[3], self._box[2]
        else:
            self._oh, self._ow = (output_size, output_size) if np.isscalar(output_size) else tuple(output_size)
        self._boxes_fn = boxes  # callable(epoch, order) -> int32[len(order), 4], or None
        self._flips_fn = flips  # callable(epoch, n, start_batch) -> uint8[n] per epoch position, or None
        # train_aug: RandomResizedCrop + flip per sample and epoch, seeded by (seed, epoch, sample index)
        # like the direct-batch loader's train_aug (src/pipeline/direct_batch_loader.hpp:141-178).
        self._train_aug = bool(train_aug)
        if self._train_aug and (boxes is not None or flips is not None):
            raise ValueError("train_aug draws its own boxes and flips")
        if self._train_aug and hflip_prob == 0.0:
            self.hflip_prob = 0.5
        # Plain float32 NCHW batches are handed out as __cuda_array_interface__ objects like the
        # reference's; bf16 has no CAI typestr and channels-last needs strides, so those are tensors.
        plain = self.dtype == torch.float32 and not self.channels_last
        self._as_tensor = (not plain) if as_tensor is None else bool(as_tensor) or not plain
        self._labels = None if labels is None else torch.as_tensor(np.asarray(labels), dtype=torch.int64).to(self._device)
        # Batches are prefetched on streams of the library: `ring` output slots, `ahead` batches in
        # flight beyond the one handed out.  A batch stays valid for ring - ahead - 1 further batches
        # (4 by default).
        self._ring_slots = max(3, int(ring))
        self._ahead = max(1, (self._ring_slots - 1) // 2)
        self._ring = None
        self._lookahead = None
        self._stage = {}        # (table name, parity) -> page-locked staging tensor
        self._stage_parity = 0
        self._jitter_fn = jitter  # callable(epoch, order) -> float32[len(order), 3] (brightness, contrast, saturation), or None
        self._epoch = 0
        self._resume_batches = 0
        self._batches_served = 0
        self._status = torch.zeros(1, dtype=torch.int32, device=self._device)

    # ---- reference surface ------------------------------------------------------------------
    def set_epoch(self, epoch):
        self._epoch = int(epoch)

    def __len__(self):
        return self._n // self.batch_size if self.drop_last else -(-self._n // self.batch_size)

    def state_dict(self):
        return {"version": 1, "epoch": int(self._epoch), "batches_served": int(self._batches_served)}

    def load_state_dict(self, state):
        if int(state.get("version", 0)) != 1:
            raise ValueError("unsupported state_dict version")
        self._epoch = int(state["epoch"])
        self._resume_batches = int(state["batches_served"])

    def device_status(self) -> int:
        """Status bits the kernels OR-ed so far (synchronises); 0 when every sample was valid."""
        return int(self._status.item())

    # ---- epoch plan ---------------------------------------------------------------------------
    def epoch_order(self, epoch=None) -> np.ndarray:
        e = self._epoch if epoch is None else int(epoch)
        if self.shuffle:
            return np.random.default_rng(self.seed + e).permutation(self._n).astype(np.int64)
        return np.arange(self._n, dtype=np.int64)

    def epoch_flips(self, epoch=None) -> np.ndarray:
        """Flip flag per epoch position: Bernoulli(hflip_prob) from ``default_rng([seed, epoch, 7])``."""
        e = self._epoch if epoch is None else int(epoch)
        if self.hflip_prob <= 0.0:
            return np.zeros(self._n, dtype=np.uint8)
        return (np.random.default_rng([self.seed, e, 7]).random(self._n) < self.hflip_prob).astype(np.uint8)

    def _host_tables(self, epoch):
        """(order, flips, RandomResizedCrop boxes or None) of an epoch -- everything that is drawn on
        the host from (seed, epoch) alone."""
        order = self.epoch_order(epoch)
        if self._train_aug:
            from .augment import pick_crops
            sizes = np.tile(np.array([[self._W, self._H]], dtype=np.int32), (self._n, 1))
            boxes, flips = pick_crops(self.seed, epoch, sizes, indices=order, hflip_prob=self.hflip_prob)
            return order, flips, boxes
        return order, self.epoch_flips(epoch), None

    def _epoch_tables(self, epoch):
        """The epoch's host tables, from the look-ahead if it already drew them; then the NEXT
        epoch's tables are drawn on a helper thread while this epoch is being served, so that the
        usual ``for e in range(E): set_epoch(e); for batch in loader`` loop pays the permutation of
        a large dataset (milliseconds) only once."""
        import threading

        pending = self._lookahead
        self._lookahead = None
        tables = None
        if pending is not None:
            thread, box = pending
            thread.join()
            if box.get("key") == (epoch, self.seed, self.hflip_prob, self.shuffle, self._train_aug):
                tables = box["tables"]
        if tables is None:
            tables = self._host_tables(epoch)
        box = {}

        def work(e=epoch + 1, key=(epoch + 1, self.seed, self.hflip_prob, self.shuffle, self._train_aug)):
            box["tables"] = self._host_tables(e)
            box["key"] = key

        thread = threading.Thread(target=work, daemon=True)
        thread.start()
        self._lookahead = (thread, box)
        return tables

    def __iter__(self):
        torch = self._torch
        bs = self.batch_size
        order, flips, aug_boxes = self._epoch_tables(self._epoch)
        if self._flips_fn is not None:
            flips = np.ascontiguousarray(self._flips_fn(self._epoch, self._n, self._resume_batches), dtype=np.uint8)
            if flips.shape != (self._n,):
                raise ValueError("flips callable must return one flag per epoch position")
        lib = _capi.load()
        with torch.cuda.device(self._device):
            # ---- whole-epoch tables on the device, once -----------------------------------------
            # Host table -> device through page-locked staging that the loader keeps (two sets, used by
            # alternate epochs): a copy into it and an asynchronous upload, ordered before the first
            # launch (which waits for the consumer stream's position), instead of a blocking copy from
            # pageable memory per table.
            self._stage_parity ^= 1

            def upload(name, host):
                host = np.ascontiguousarray(host)
                slot = (name, self._stage_parity)
                buf = self._stage.get(slot)
                if buf is None or buf.shape != host.shape or buf.dtype != torch.from_numpy(host).dtype:
                    buf = torch.empty(host.shape, dtype=torch.from_numpy(host).dtype, pin_memory=True)
                    self._stage[slot] = buf
                buf.numpy()[...] = host
                return buf.to(self._device, non_blocking=True)

            d_order = upload("order", order) if self.shuffle else None
            d_flips = upload("flips", flips) if (self.hflip_prob > 0.0 or self._flips_fn is not None) else None
            d_boxes = None
            if self._boxes_fn is not None or aug_boxes is not None:
                b = aug_boxes if aug_boxes is not None else \
                    np.ascontiguousarray(self._boxes_fn(self._epoch, order), dtype=np.int32).reshape(-1, 4)
                if b.shape[0] != self._n:
                    raise ValueError("boxes callable must return one box per epoch position")
                if (b[:, 2] <= 0).any() or (b[:, 3] <= 0).any() or (b[:, 0] < 0).any() or (b[:, 1] < 0).any() or \
                        (b[:, 0] + b[:, 2] > self._W).any() or (b[:, 1] + b[:, 3] > self._H).any():
                    raise ValueError("a crop box leaves the stored image")
                d_boxes = upload("boxes", b)
                max_cw = int(b[:, 2].max())
            else:
                max_cw = self._box[2]
            d_jit = None
            if self._jitter_fn is not None:
                j = np.ascontiguousarray(self._jitter_fn(self._epoch, order), dtype=np.float32).reshape(-1, 3)
                if j.shape[0] != self._n:
                    raise ValueError("jitter callable must return one (brightness, contrast, saturation) per epoch position")
                d_jit = upload("jitter", j)
            # ---- output ring: slot s of every buffer belongs to batch b with b % ring == s --------
            R = self._ring_slots
            shape = (bs, self._oh, self._ow, 3) if self.channels_last else (bs, 3, self._oh, self._ow)
            if self._ring is None or tuple(self._ring.shape) != (R,) + shape:
                self._ring = torch.empty((R,) + shape, dtype=self.dtype, device=self._device)
            ring = self._ring
            want_idx = self.return_indices and self.shuffle
            idx_ring = torch.empty((R, bs), dtype=torch.int64, device=self._device) if want_idx else None
            lab_ring = torch.empty((R, bs), dtype=torch.int64, device=self._device) if self._labels is not None else None
            # ---- batch 0 as the fused transform takes it; the library walks the epoch from there ----
            d = _capi.TransformDesc()
            d.src = self._gpu.data_ptr()
            d.src_bytes = self._gpu.numel()
            d.n_src = self._n
            d.src_w, d.src_h = self._W, self._H
            d.n = bs
            if d_order is not None:
                d.sel = d_order.data_ptr()
            if d_boxes is not None:
                d.boxes = d_boxes.data_ptr()
            else:
                d.uniform_box = (C.c_int32 * 4)(*self._box)
            if d_flips is not None:
                d.flips = d_flips.data_ptr()
            if d_jit is not None:
                d.jitter = d_jit.data_ptr()
            d.dst_h, d.dst_w = self._oh, self._ow
            d.out = ring.data_ptr()
            d.out_dtype = _capi.TLB_F32 if self.dtype == torch.float32 else _capi.TLB_BF16
            d.out_layout = _capi.TLB_NHWC if self.channels_last else _capi.TLB_NCHW
            if idx_ring is not None:
                d.out_indices = idx_ring.data_ptr()
            if lab_ring is not None:
                d.labels_in = self._labels.data_ptr()
                d.labels_out = lab_ring.data_ptr()
            d.mean = _capi.f3(self.mean)
            d.std = _capi.f3(self.std)
            d.normalize_01 = 1
            d.max_crop_w = max_cw
            d.antialias = int(self.antialias)
            d.status = self._status.data_ptr()
            start = self._resume_batches
            self._batches_served = start
            self._resume_batches = 0
            plan = lib.tlb_epoch_create(C.byref(d), self._n, int(self.drop_last), start, R, self._ahead,
                                        ring[0].numel() * ring.element_size(), 8 * bs, 8 * bs)
            if not plan:
                raise _capi.TurboLoaderB200Error(1, lib.tlb_last_error().decode(errors="replace"))
            b_no, n_out, slot = C.c_int64(0), C.c_int32(0), C.c_int32(0)
            try:
                while True:
                    stream = torch.cuda.current_stream(self._device)  # the consumer's stream, asked at every batch
                    _capi.check(lib.tlb_epoch_next(plan, C.byref(b_no), C.byref(n_out), C.byref(slot),
                                                   C.c_void_p(stream.cuda_stream)))
                    n = n_out.value
                    if n == 0:
                        break
                    out = ring[slot.value, :n]
                    self._batches_served += 1
                    if self._as_tensor:
                        batch = out.permute(0, 3, 1, 2) if self.channels_last else out
                    else:
                        batch = _CudaArray(out.data_ptr(), (n, 3, self._oh, self._ow), owner=ring,
                                           device=self._device.index)
                    items = [batch]
                    if lab_ring is not None:
                        items.append(lab_ring[slot.value, :n])
                    if self.return_indices:
                        b0 = b_no.value * bs
                        items.append(idx_ring[slot.value, :n] if idx_ring is not None else np.arange(b0, b0 + n))
                    yield items[0] if len(items) == 1 else tuple(items)
            finally:
                lib.tlb_epoch_destroy(plan)
            self._batches_served = 0
            self._epoch_done = True
