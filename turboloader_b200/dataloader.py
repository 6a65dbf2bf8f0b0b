"""``DataLoader(path.tbl, output_format='pytorch', ...)`` served from GPU memory.

Keeps the contract of TurboLoader's unified ``DataLoader`` for pre-processed RAW_U8 ``.tbl``
files (turboloader/__init__.py:839-889 routes them to ``TblRawImageLoader``,
turboloader/tbl.py:139-330): iteration yields ``(images, meta)`` with ``images`` a
``(B, 3, H, W)`` float32 batch and ``meta['indices']`` the sample indices; the order is
``np.random.default_rng(seed + epoch).permutation(n)`` under ``shuffle``; flips follow
``default_rng((seed, epoch, 1)).random(k) < hflip_prob`` drawn batch by batch;
``state_dict()`` / ``load_state_dict()`` resume mid-epoch with the same dict.  The difference is
where the work happens: the dataset is uploaded once and every batch is one launch of the fused
sm_100a kernel, so ``images`` is a CUDA tensor (ready for the model, no H2D per batch).

With ``image_size=`` different from the stored size, ``train_aug=True``, ``antialias=True``, a list
of variable-size pre-decoded images (``arrays=[HxWx3 uint8, ...]``) or ``enable_distributed`` with
``world_size > 1`` the loader follows the unified DataLoader's direct-batch route instead
(turboloader/__init__.py:288-320, 1001-1019 -> ``DirectBatchCore``): ``mt19937_64`` epoch order,
the rank's equal block, per-sample RandomResizedCrop + flip, resize to ``image_size`` -- all inside
the same fused kernel (``DirectBatchLoader``).

Only what these paths can serve is accepted: ``.tbl`` paths or in-memory pre-decoded arrays,
``transform=None`` or an ``ImageNetNormalize`` instance, ``output_format='pytorch'``.  Decoding
TAR/JPEG datasets is outside this package.
"""
from __future__ import annotations

import os

import numpy as np

from . import ops
from .cuda_loader import CudaResidentLoader

__all__ = ["DataLoader", "ImageNetNormalize"]


class ImageNetNormalize:
    """Marker for ImageNet mean/std normalization (the one transform the RAW serve path fuses;
    matched by class name exactly as turboloader/__init__.py:857 does)."""
    mean = ops.IMAGENET_MEAN
    std = ops.IMAGENET_STD


class DataLoader:
    def __init__(self, data_path=None, batch_size=32, num_workers=4, shuffle=False, transform=None, image_size=None,
                 output_format="pytorch", modality="image", arrays=None, seed=42, enable_distributed=False,
                 world_rank=0, world_size=1, drop_last=False, pin_memory=False, prefetch_batches=4, train_aug=False,
                 hflip_prob=None, antialias=False, dtype=None, channels_last=False, **unused):
        if modality != "image":
            raise ValueError("turboloader_b200.DataLoader serves images only")
        if output_format != "pytorch":
            raise ValueError("turboloader_b200.DataLoader yields (images, meta) batches: use output_format='pytorch'")
        mean, std = (0.0, 0.0, 0.0), (1.0, 1.0, 1.0)
        if transform is not None:
            if type(transform).__name__ != "ImageNetNormalize":
                raise ValueError("the fused path supports transform=None ([0,1] floats) or ImageNetNormalize(); other "
                                 "transforms are not expressible in the fused pass")
            mean, std = ops.IMAGENET_MEAN, ops.IMAGENET_STD
        ragged = isinstance(arrays, (list, tuple))
        if arrays is not None:
            array = arrays
        elif data_path is not None and os.fspath(data_path).lower().endswith(".tbl"):
            from .tbl import open_raw_view
            array, _, _ = open_raw_view(data_path)
        else:
            raise ValueError("turboloader_b200.DataLoader needs a RAW_U8 .tbl path, arrays=(N,H,W,3) uint8 or "
                             "arrays=[HxWx3 uint8, ...]; decoding TAR/JPEG datasets is not part of this package")
        self._bs = int(batch_size)
        want = None
        if image_size is not None:
            want = (image_size, image_size) if isinstance(image_size, int) else tuple(int(v) for v in image_size)
        stored = None if ragged else (int(array.shape[1]), int(array.shape[2]))
        sharded = bool(enable_distributed) and int(world_size) > 1
        # The direct-batch route (DirectBatchCore's rules: mt19937_64 order + rank block, per-sample
        # RandomResizedCrop, resize to image_size) serves everything the plain RAW route cannot:
        # variable-size stores, a target size other than the stored one, train_aug, antialias, ranks.
        self._direct = ragged or train_aug or antialias or sharded or (want is not None and want != stored)
        if self._direct:
            from .direct_loader import DirectBatchLoader
            if want is None:
                if ragged:
                    raise ValueError("image_size is required for a store of variable-size images")
                want = stored
            if not ragged:
                n, h, w, _ = array.shape
                flat = np.ascontiguousarray(array).reshape(-1)
                array = (flat, np.arange(n, dtype=np.int64) * (h * w * 3), np.tile(np.array([[w, h]], np.int32), (n, 1)))
            self._loader = DirectBatchLoader(
                array, batch_size, want[0], want[1], mean=mean, std=std, shuffle=shuffle, seed=seed,
                distributed=sharded, world_rank=world_rank, world_size=world_size, drop_last=drop_last,
                antialias=antialias, train_aug=train_aug, hflip_prob=0.5 if hflip_prob is None else hflip_prob,
                dtype=dtype, channels_last=channels_last)
            self.num_samples = self._loader.num_samples()
            self.batch_size = self._bs
            return
        self._seed, self._hflip = int(seed), float(hflip_prob or 0.0)

        def flips(epoch, n, start_batch):
            # Drawn batch by batch from the first served batch on, as the reference loader does.
            out = np.zeros(n, dtype=np.uint8)
            if self._hflip > 0:
                rng = np.random.default_rng((self._seed, epoch, 1))
                for b in range(start_batch * self._bs, n, self._bs):
                    k = min(self._bs, n - b)
                    out[b:b + k] = rng.random(k) < self._hflip
            return out

        self._loader = CudaResidentLoader.from_array(
            array, batch_size=batch_size, mean=mean, std=std, drop_last=drop_last, shuffle=shuffle, seed=seed,
            return_indices=True, flips=flips if self._hflip > 0 else None, dtype=dtype, channels_last=channels_last,
            as_tensor=True)
        self.num_samples = self._loader._n
        self.batch_size = self._bs

    def __len__(self):
        return len(self._loader)

    def set_epoch(self, epoch):
        self._loader.set_epoch(epoch)

    def state_dict(self):
        return self._loader.state_dict()

    def load_state_dict(self, sd):
        self._loader.load_state_dict(sd)

    def __iter__(self):
        if self._direct:
            yield from self._loader
            return
        order = self._loader.epoch_order()
        bs = self._bs
        b = self._loader._resume_batches
        for batch, _ in self._loader:
            idx = order[b * bs:(b + 1) * bs].copy()
            yield batch, {"indices": idx, "batch_size": int(idx.size)}
            b += 1

    def close(self):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False
