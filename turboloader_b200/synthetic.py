"""Seeded synthetic workloads with the shapes, sizes and value distributions of the five
benchmark configurations of the fused image-transform path.  They stand in for the
ImageNet-style datasets the reference measures on; no dataset item is reproduced.

Every generator takes the counts as arguments so that tests can run the same recipe at
a size a CPU oracle finishes in seconds.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)


@dataclass
class Workload:
    name: str
    src: np.ndarray            # uint8, flat, packed images (16-byte aligned starts)
    offsets: np.ndarray        # int64[n_src]
    sizes: np.ndarray          # int32[n_src, 2] as (w, h)
    n: int
    dst_h: int
    dst_w: int
    sel: np.ndarray | None = None     # int64[n]
    boxes: np.ndarray | None = None   # int32[n, 4] (x, y, w, h)
    flips: np.ndarray | None = None   # uint8[n]
    mean: tuple = IMAGENET_MEAN
    std: tuple = IMAGENET_STD
    normalize_01: bool = True
    dtype: str = "f32"                # "f32" | "bf16"
    channels_last: bool = False
    uniform_hw: tuple | None = None   # (h, w) when every dataset image has the same size
    notes: dict = field(default_factory=dict)

    @property
    def n_src(self) -> int:
        return int(self.sizes.shape[0])

    def crop_wh(self) -> np.ndarray:
        """int64[n, 2] crop (w, h) of every sample."""
        if self.boxes is not None:
            return self.boxes[:, 2:4].astype(np.int64)
        s = self.sel if self.sel is not None else np.arange(self.n)
        return self.sizes[s].astype(np.int64)

    def algorithmic_bytes(self) -> tuple[int, int]:
        """(read, write) bytes one pass over the batch must move: the crop footprint plus the
        per-sample tables in, the output tensor (plus returned indices) out."""
        wh = self.crop_wh()
        read = int((wh[:, 0] * wh[:, 1] * 3).sum())
        if self.sel is not None:
            read += 8 * self.n
        if self.boxes is not None:
            read += 16 * self.n
        if self.flips is not None:
            read += self.n
        if self.uniform_hw is None:
            read += 16 * self.n  # offset + size of the image each sample reads
        esz = 4 if self.dtype == "f32" else 2
        write = self.n * 3 * self.dst_h * self.dst_w * esz
        if self.sel is not None:
            write += 8 * self.n
        return read, write


def pack_images(images) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Pack HWC uint8 images into one buffer with 16-byte aligned starts."""
    sizes = np.array([(im.shape[1], im.shape[0]) for im in images], dtype=np.int32).reshape(-1, 2)
    nbytes = sizes[:, 0].astype(np.int64) * sizes[:, 1] * 3
    padded = (nbytes + 15) // 16 * 16
    offsets = np.concatenate([[0], np.cumsum(padded)[:-1]]).astype(np.int64)
    buf = np.zeros(int(padded.sum()), dtype=np.uint8)
    for im, o, b in zip(images, offsets, nbytes):
        buf[o:o + b] = np.ascontiguousarray(im, dtype=np.uint8).reshape(-1)
    return buf, offsets, sizes


def uniform_dataset(arr: np.ndarray):
    """(N, H, W, 3) uint8 -> (flat, offsets, sizes)."""
    n, h, w, _ = arr.shape
    offsets = np.arange(n, dtype=np.int64) * (h * w * 3)
    sizes = np.tile(np.array([[w, h]], dtype=np.int32), (n, 1))
    return arr.reshape(-1), offsets, sizes


def smooth_field(rng: np.random.Generator, h: int, w: int) -> np.ndarray:
    """Sum of 4 random 2-D sinusoids per channel scaled to [0,255], plus uniform +-8 noise."""
    yy, xx = np.meshgrid(np.arange(h, dtype=np.float32), np.arange(w, dtype=np.float32), indexing="ij")
    out = np.empty((h, w, 3), dtype=np.float32)
    for c in range(3):
        acc = np.zeros((h, w), dtype=np.float32)
        for _ in range(4):
            fx, fy = rng.uniform(-0.03, 0.03, size=2)
            ph = rng.uniform(0, 2 * math.pi)
            amp = rng.uniform(0.5, 1.0)
            acc += amp * np.sin(2 * math.pi * (fx * xx + fy * yy) + ph).astype(np.float32)
        lo, hi = float(acc.min()), float(acc.max())
        out[..., c] = (acc - lo) * (255.0 / max(hi - lo, 1e-6))
    out += rng.uniform(-8.0, 8.0, size=out.shape).astype(np.float32)
    return np.clip(out, 0, 255).astype(np.uint8)


def rrc_boxes(sizes_wh, scale, ratio=(3 / 4, 4 / 3), seed=0) -> np.ndarray:
    """Crop boxes drawn with torchvision's ``RandomResizedCrop.get_params`` under a fixed torch
    seed (10 tries, then the centre-crop fallback); returns int32[n, 4] as (x, y, w, h)."""
    import torch
    from torchvision.transforms import RandomResizedCrop

    state = torch.random.get_rng_state()
    torch.manual_seed(int(seed))
    try:
        dummies: dict = {}
        out = np.empty((len(sizes_wh), 4), dtype=np.int32)
        for i, (w, h) in enumerate(sizes_wh):
            key = (int(h), int(w))
            if key not in dummies:
                dummies[key] = torch.empty((3, key[0], key[1]), dtype=torch.uint8)
            top, left, ch, cw = RandomResizedCrop.get_params(dummies[key], list(scale), list(ratio))
            out[i] = (left, top, cw, ch)
    finally:
        torch.random.set_rng_state(state)
    return out


def _flips(rng, n):
    return (rng.random(n) < 0.5).astype(np.uint8)


def config1(seed=0, n=256, src=256, dst=224) -> Workload:
    """Fixed-size resize: uniform-noise images, full-image box, flips, mean/std in 0..255 units."""
    rng = np.random.default_rng(seed)
    arr = rng.integers(0, 256, size=(n, src, src, 3), dtype=np.uint8)
    flat, offsets, sizes = uniform_dataset(arr)
    return Workload("fixed_resize", flat, offsets, sizes, n, dst, dst, flips=_flips(rng, n),
                    mean=tuple(m * 255 for m in IMAGENET_MEAN), std=tuple(s * 255 for s in IMAGENET_STD),
                    normalize_01=False, uniform_hw=(src, src))


def config2(seed=0, n=512, lo=200, hi=500, dst=224) -> Workload:
    """Variable-size RandomResizedCrop: H, W ~ U[lo, hi], smooth-field pixels, RRC(0.08, 1)."""
    rng = np.random.default_rng(seed)
    hs = rng.integers(lo, hi + 1, size=n)
    ws = rng.integers(lo, hi + 1, size=n)
    images = [smooth_field(rng, int(h), int(w)) for h, w in zip(hs, ws)]
    flat, offsets, sizes = pack_images(images)
    boxes = rrc_boxes(sizes, (0.08, 1.0), seed=seed + 1)
    return Workload("variable_rrc", flat, offsets, sizes, n, dst, dst, boxes=boxes, flips=_flips(rng, n))


def config3(seed=0, n_dataset=100_000, batch=1024, src=160, crop=144, dst=128, epoch=0, batch_index=0,
            dataset=None) -> Workload:
    """Resident-loader epoch: uniform-noise dataset, ``default_rng(seed+epoch).permutation`` gather,
    centre crop, flips, bf16 NCHW + returned indices.  One batch of the epoch is described."""
    rng = np.random.default_rng(seed)
    if dataset is None:
        dataset = rng.integers(0, 256, size=(n_dataset, src, src, 3), dtype=np.uint8)
    flat, offsets, sizes = uniform_dataset(dataset)
    perm = np.random.default_rng(seed + epoch).permutation(n_dataset).astype(np.int64)
    sel = perm[batch_index * batch:(batch_index + 1) * batch]
    n = len(sel)
    off = (src - crop) // 2
    boxes = np.tile(np.array([[off, off, crop, crop]], dtype=np.int32), (n, 1))
    frng = np.random.default_rng([seed, epoch, 7])
    all_flips = _flips(frng, n_dataset)  # drawn per epoch position
    flips = all_flips[batch_index * batch:batch_index * batch + n]
    return Workload("resident_epoch", flat, offsets, sizes, n, dst, dst, sel=sel, boxes=boxes, flips=flips,
                    dtype="bf16", uniform_hw=(src, src), notes={"perm": perm})


def config4(seed=0, n=256, src=512, dst=384) -> Workload:
    """High-resolution crop: smooth-field 512x512 images, RRC(0.25, 1), bf16 NHWC."""
    rng = np.random.default_rng(seed)
    arr = np.stack([smooth_field(rng, src, src) for _ in range(n)])
    flat, offsets, sizes = uniform_dataset(arr)
    boxes = rrc_boxes(sizes, (0.25, 1.0), seed=seed + 1)
    return Workload("highres_nhwc", flat, offsets, sizes, n, dst, dst, boxes=boxes, flips=_flips(rng, n),
                    dtype="bf16", channels_last=True, uniform_hw=(src, src))


def config5_params(seed=0, total=32768, src=256):
    """Boxes and flips of the 8-GPU sharded scaling set, drawn for the GLOBAL index so that a
    sample's result does not depend on the world size."""
    sizes = np.tile(np.array([[src, src]], dtype=np.int32), (total, 1))
    boxes = rrc_boxes(sizes, (0.08, 1.0), seed=seed + 1)
    flips = _flips(np.random.default_rng([seed, 5]), total)
    return boxes, flips


def config5(seed=0, total=32768, world=1, rank=0, batch=1024, batch_index=0, src=256, dst=224,
            params=None, shard=None) -> Workload:
    """One batch of rank ``rank``'s contiguous shard of the global uniform-noise dataset.  The
    pixels of image g come from ``default_rng([seed, g])`` so that any rank can make its own."""
    boxes_all, flips_all = params if params is not None else config5_params(seed, total, src)
    if shard is None:
        per = total // world
        shard = np.arange(rank * per, (rank + 1) * per, dtype=np.int64)
    glob = shard[batch_index * batch:(batch_index + 1) * batch]
    n = len(glob)
    arr = np.stack([np.random.default_rng([seed, int(g)]).integers(0, 256, size=(src, src, 3), dtype=np.uint8)
                    for g in glob])
    flat, offsets, sizes = uniform_dataset(arr)
    return Workload("sharded_scaling", flat, offsets, sizes, n, dst, dst, boxes=boxes_all[glob].copy(),
                    flips=flips_all[glob].copy(), dtype="bf16", uniform_hw=(src, src),
                    notes={"global_indices": glob})
