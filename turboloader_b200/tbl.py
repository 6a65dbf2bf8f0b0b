"""RAW_U8 ``.tbl`` ingest for the GPU-resident loader.

Reads TurboLoader's TBL v2 container directly (src/formats/tbl_v2_format.hpp:14-46, 103-104:
a 64-byte header ``"TBL\\x02"``, then ``num_samples`` 24-byte index entries, then payloads)
and exposes an uncompressed, uniform-size RAW_U8 file as a zero-copy ``(N, H, W, 3)`` uint8
memory map -- the contract of ``turboloader.tbl.open_raw_view`` (turboloader/tbl.py:31-74).
``write_raw_tbl`` writes such a file from an array so that datasets can be prepared without
the reference's decode pipeline (JPEG decode is outside this package).
"""
from __future__ import annotations

import os

import numpy as np

MAGIC = b"TBL\x02"
VERSION = 2
RAW_U8 = 8
SAMPLE_FLAG_COMPRESSED = 1

HEADER_DTYPE = np.dtype([
    ("magic", "S4"), ("version", "<u4"), ("num_samples", "<u8"), ("header_size", "<u4"), ("padding1", "<u4"),
    ("metadata_offset", "<u8"), ("metadata_size", "<u8"), ("flags", "<u4"), ("checksum", "<u4"),
    ("reserved", "V16"),
])
INDEX_DTYPE = np.dtype([
    ("offset", "<u8"), ("size", "<u4"), ("uncompressed_size", "<u4"), ("width", "<u2"), ("height", "<u2"),
    ("format", "u1"), ("flags", "u1"), ("checksum", "<u2"),
])
assert HEADER_DTYPE.itemsize == 64 and INDEX_DTYPE.itemsize == 24

__all__ = ["open_raw_view", "write_raw_tbl", "read_index"]


def read_index(path):
    """(header record, index record array) of a TBL v2 file."""
    path = os.fspath(path)
    with open(path, "rb") as f:
        raw = f.read(64)
        if len(raw) < 64:
            raise ValueError(f"{path}: too short for a TBL v2 header")
        hdr = np.frombuffer(raw, dtype=HEADER_DTYPE)[0]
        if bytes(hdr["magic"]).ljust(4, b"\0") != MAGIC or int(hdr["version"]) != VERSION:
            raise ValueError(f"{path}: not a TBL v2 file")
        n = int(hdr["num_samples"])
        idx = np.frombuffer(f.read(24 * n), dtype=INDEX_DTYPE)
        if idx.shape[0] != n:
            raise ValueError(f"{path}: truncated index table")
    return hdr, idx


def open_raw_view(path):
    """Memory-map an uncompressed, uniform-size RAW_U8 ``.tbl`` as ``(N, H, W, 3)`` uint8.
    Returns ``(view, H, W)``; raises ValueError for anything the fast path cannot serve
    (other formats, mixed sizes, LZ4 samples, non-contiguous payloads), as the reference does."""
    path = os.fspath(path)
    _, idx = read_index(path)
    n = idx.shape[0]
    if n == 0:
        raise ValueError(f"{path} contains no samples")
    if set(np.unique(idx["format"]).tolist()) != {RAW_U8}:
        raise ValueError(f"{path} holds non-RAW_U8 samples; the resident loader serves pre-processed RAW_U8 files")
    dims = set(zip(idx["height"].tolist(), idx["width"].tolist()))
    if len(dims) != 1:
        raise ValueError(f"samples have mixed sizes {sorted(dims)}; batching needs uniform dims")
    H, W = dims.pop()
    sz = H * W * 3
    if (idx["flags"] & SAMPLE_FLAG_COMPRESSED).any():
        raise ValueError("this .tbl is LZ4-compressed; the mmap path needs uncompressed RAW samples")
    if (idx["size"] != sz).any():
        raise ValueError("corrupt RAW_U8 file: sample size != W*H*3")
    offs = idx["offset"].astype(np.int64)
    if not np.array_equal(offs, offs[0] + np.arange(n, dtype=np.int64) * sz):
        raise ValueError("non-contiguous payload layout; refusing mmap view")
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    if offs[0] + n * sz > mm.shape[0]:
        raise ValueError("corrupt RAW_U8 file: payload runs past the end of the file")
    return mm[offs[0]:offs[0] + n * sz].reshape(n, H, W, 3), H, W


def write_raw_tbl(path, array) -> int:
    """Write an ``(N, H, W, 3)`` uint8 array as an uncompressed RAW_U8 TBL v2 file."""
    a = np.ascontiguousarray(array, dtype=np.uint8)
    if a.ndim != 4 or a.shape[3] != 3:
        raise ValueError("array must be (N, H, W, 3) uint8")
    n, H, W, _ = a.shape
    if H >= 65536 or W >= 65536:
        raise ValueError("TBL v2 stores 16-bit dimensions")
    sz = H * W * 3
    hdr = np.zeros(1, dtype=HEADER_DTYPE)
    hdr["magic"], hdr["version"], hdr["num_samples"] = MAGIC, VERSION, n
    hdr["header_size"] = 64 + 24 * n
    idx = np.zeros(n, dtype=INDEX_DTYPE)
    idx["offset"] = 64 + 24 * n + np.arange(n, dtype=np.uint64) * np.uint64(sz)
    idx["size"], idx["width"], idx["height"], idx["format"] = sz, W, H, RAW_U8
    with open(os.fspath(path), "wb") as f:
        f.write(hdr.tobytes())
        f.write(idx.tobytes())
        f.write(a.tobytes())
    return n


def decode_to_array(paths, height, width, workers=8) -> np.ndarray:
    """One-time ingest of image FILES for the resident and streaming loaders: every file is opened
    with PIL, converted to RGB and resized to ``width`` x ``height``; returns ``(N, height, width, 3)``
    uint8.  (Decode is outside the GPU path; this mirrors what the reference's loaders do once at
    construction, turboloader/cuda_loader.py:417-436.)"""
    from concurrent.futures import ThreadPoolExecutor

    from PIL import Image

    files = [os.fspath(f) for f in paths]
    out = np.empty((len(files), int(height), int(width), 3), dtype=np.uint8)

    def fill(slot_and_file):
        slot, name = slot_and_file
        with Image.open(name) as picture:
            out[slot] = np.asarray(picture.convert("RGB").resize((int(width), int(height))))

    with ThreadPoolExecutor(max_workers=max(1, int(workers))) as pool:
        for _ in pool.map(fill, enumerate(files)):
            pass
    return out
