"""RAW_U8 .tbl ingest (TBL v2 container, src/formats/tbl_v2_format.hpp:14-46, 103-104): the
reader exposes the payload as a zero-copy (N, H, W, 3) view and refuses what the mmap path
cannot serve, like turboloader/tbl.py:31-74."""
import numpy as np
import pytest

from turboloader_b200 import tbl


def _data(n=7, h=6, w=5, seed=0):
    return np.random.RandomState(seed).randint(0, 256, size=(n, h, w, 3), dtype=np.uint8)


def test_round_trip_is_zero_copy_view(tmp_path):
    a = _data()
    path = tmp_path / "x.tbl"
    assert tbl.write_raw_tbl(path, a) == 7
    view, H, W = tbl.open_raw_view(path)
    assert (H, W) == (6, 5) and view.shape == a.shape and view.dtype == np.uint8
    assert np.array_equal(view, a)
    assert isinstance(view.base, np.memmap) or isinstance(view, np.memmap) or view.base is not None
    hdr, idx = tbl.read_index(path)
    assert bytes(hdr["magic"]) == b"TBL\x02" and int(hdr["version"]) == 2 and int(hdr["num_samples"]) == 7
    assert int(hdr["header_size"]) == 64 + 24 * 7
    assert (idx["format"] == tbl.RAW_U8).all() and (idx["size"] == 6 * 5 * 3).all()


def test_rejects_what_the_mmap_path_cannot_serve(tmp_path):
    a = _data()
    path = tmp_path / "x.tbl"
    tbl.write_raw_tbl(path, a)
    raw = bytearray(open(path, "rb").read())

    def variant(mutate):
        b = bytearray(raw)
        mutate(b)
        p = tmp_path / "v.tbl"
        open(p, "wb").write(b)
        return p

    ent = 64  # first index entry: offset u64, size u32, usize u32, w u16, h u16, format u8, flags u8, crc u16
    with pytest.raises(ValueError, match="not a TBL v2"):
        tbl.open_raw_view(variant(lambda b: b.__setitem__(slice(0, 4), b"XXXX")))
    with pytest.raises(ValueError, match="non-RAW_U8"):
        tbl.open_raw_view(variant(lambda b: b.__setitem__(ent + 20, 1)))       # JPEG
    with pytest.raises(ValueError, match="mixed sizes"):
        tbl.open_raw_view(variant(lambda b: b.__setitem__(ent + 16, 9)))       # width of sample 0
    with pytest.raises(ValueError, match="LZ4"):
        tbl.open_raw_view(variant(lambda b: b.__setitem__(ent + 21, 1)))       # compressed flag
    with pytest.raises(ValueError, match="non-contiguous"):
        tbl.open_raw_view(variant(lambda b: b.__setitem__(ent + 24, (b[ent + 24] + 1) % 256)))  # offset of sample 1
    empty = tmp_path / "e.tbl"
    tbl.write_raw_tbl(empty, np.zeros((0, 2, 2, 3), np.uint8))
    with pytest.raises(ValueError, match="no samples"):
        tbl.open_raw_view(empty)
    with pytest.raises(ValueError):
        tbl.write_raw_tbl(tmp_path / "bad.tbl", np.zeros((2, 2, 2), np.uint8))


def test_dataloader_argument_errors_do_not_need_a_gpu(tmp_path):
    import turboloader_b200 as t
    with pytest.raises(ValueError, match="output_format"):
        t.DataLoader("x.tbl", output_format="dict")
    with pytest.raises(ValueError, match="image_size is required"):
        t.DataLoader(arrays=[np.zeros((4, 5, 3), np.uint8), np.zeros((6, 3, 3), np.uint8)], train_aug=True)
    with pytest.raises(ValueError, match="ImageNetNormalize"):
        t.DataLoader("x.tbl", transform=object())
    with pytest.raises(ValueError, match="RAW_U8 .tbl"):
        t.DataLoader("x.tar")
