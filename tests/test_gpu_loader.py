"""GPU tests of the reference-facing surface: the pointer-returning resident operators, the
host-image operators, the host-to-device streaming entry point and CudaResidentLoader."""
import ctypes as C

import numpy as np
import pytest

import turboloader_b200 as t
from oracle import oracle as O
from turboloader_b200 import _capi
from turboloader_b200 import synthetic as S

from helpers import check_bf16, expected

pytestmark = pytest.mark.gpu
MEAN, STD = t.IMAGENET_MEAN, t.IMAGENET_STD


def _dataset(n=40, hw=24, seed=0):
    return np.random.RandomState(seed).randint(0, 256, size=(n, hw, hw, 3), dtype=np.uint8)


def _oracle_uniform(data, sel=None, box=None, flips=None, dst=None, mean=MEAN, std=STD):
    n, h, w, _ = data.shape
    flat, offsets, sizes = S.uniform_dataset(data)
    m = len(sel) if sel is not None else n
    boxes = None if box is None else np.tile(np.array([box], np.int32), (m, 1))
    dh, dw = dst if dst else ((box[3], box[2]) if box else (h, w))
    return O.fused_batch(flat, offsets, sizes, sel, boxes, flips, dh, dw, mean, std, True)


def test_normalize_resident_and_gather_pointer_forms():
    import torch
    data = _dataset()
    gpu = torch.from_numpy(data).cuda()
    ptr = t.cuda_normalize_resident(gpu.data_ptr(), 40, 24, 24, mean=MEAN, std=STD)
    got = torch.as_tensor(t._CudaArray(ptr, (40, 3, 24, 24)), device="cuda").cpu().numpy()
    assert np.array_equal(got, _oracle_uniform(data))
    # numpy formula within 1e-5 (reference tests/test_tbl_raw.py:228-240 compares GPU and CPU serve)
    want = ((data.astype(np.float32) / 255 - np.array(MEAN, np.float32)) / np.array(STD, np.float32)).transpose(0, 3, 1, 2)
    assert np.abs(got - want).max() < 1e-5
    sel = torch.from_numpy(np.array([5, 0, 39, 5, 17], dtype=np.int64)).cuda()
    ptr2 = t.cuda_normalize_resident_gather(gpu.data_ptr(), sel.data_ptr(), 5, 24, 24)
    got2 = torch.as_tensor(t._CudaArray(ptr2, (5, 3, 24, 24)), device="cuda").cpu().numpy()
    assert np.array_equal(got2, _oracle_uniform(data, sel=sel.cpu().numpy()))


def test_pointer_ring_is_four_deep():
    import torch
    gpu = torch.from_numpy(_dataset(8, 16)).cuda()
    ptrs = [t.cuda_normalize_resident(gpu.data_ptr(), 8, 16, 16) for _ in range(5)]
    assert len(set(ptrs[:4])) == 4 and ptrs[4] == ptrs[0]
    with pytest.raises(RuntimeError):
        t.cuda_normalize_resident(0, 8, 16, 16)


def test_host_image_operators():
    rs = np.random.RandomState(3)
    images = [rs.randint(0, 256, size=(h, w, 3), dtype=np.uint8) for h, w in [(50, 70), (33, 20), (64, 64), (9, 200)]]
    flat, offsets, sizes = S.pack_images(images)
    got = t.cuda_resize_normalize(images, 32, 48)
    want = O.fused_batch(flat, offsets, sizes, None, None, None, 32, 48, MEAN, STD, True)
    assert got.shape == (4, 3, 32, 48) and np.array_equal(got, want)
    crops = np.array([[3, 4, 40, 30], [0, 0, 20, 33], [10, 10, 54, 54], [100, 2, 90, 7]], dtype=np.float32)
    flips = np.array([1, 0, 1, 0], dtype=np.int32)
    got = t.cuda_crop_resize_normalize(images, crops, flips, 32, 48)
    want = O.fused_batch(flat, offsets, sizes, None, crops.astype(np.int32), flips.astype(np.uint8), 32, 48, MEAN, STD, True)
    assert np.array_equal(got, want)
    with pytest.raises(RuntimeError):
        t.cuda_resize_normalize([], 8, 8)
    with pytest.raises(RuntimeError):
        t.cuda_crop_resize_normalize(images, crops[:3], flips, 8, 8)
    bad = crops.copy()
    bad[1] = (5, 0, 20, 33)
    with pytest.raises(_capi.TurboLoaderB200Error) as e:
        t.cuda_crop_resize_normalize(images, bad, flips, 8, 8)
    assert e.value.code == 2
    frac = crops.copy()
    frac[0, 0] = 3.5
    with pytest.raises(_capi.TurboLoaderB200Error):
        t.cuda_crop_resize_normalize(images, frac, flips, 8, 8)


def test_host_to_device_streaming_entry():
    import torch
    wl = S.config2(seed=21, n=10, lo=50, hi=120, dst=64)
    wl.dtype = "bf16"
    lib = _capi.load()
    refs = (_capi.ImageRef * wl.n)()
    crops = (_capi.CropParams * wl.n)()
    for i in range(wl.n):
        refs[i].data = wl.src.ctypes.data + int(wl.offsets[i])
        refs[i].w, refs[i].h = int(wl.sizes[i, 0]), int(wl.sizes[i, 1])
        crops[i].x, crops[i].y, crops[i].w, crops[i].h = (float(v) for v in wl.boxes[i])
        crops[i].flip = int(wl.flips[i])
    out = torch.empty((wl.n, 3, 64, 64), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(3):  # exercises the two-deep staging ring
        rc = lib.tlb_crop_resize_normalize_to_device(refs, crops, wl.n, 64, 64, _capi.f3(wl.mean), _capi.f3(wl.std), 1,
                                                     out.data_ptr(), _capi.TLB_BF16, _capi.TLB_NCHW, status.data_ptr(),
                                                     C.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, lib.tlb_last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert check_bf16(out.view(torch.int16).cpu().numpy().view(np.uint16), expected(wl)) == 0


@pytest.mark.parametrize("direct", [True, False])
def test_pinned_host_images_need_no_host_packing(direct, monkeypatch):
    """Images in page-locked host memory are read by the GPU itself: by default the fused kernel
    pulls the crop rows straight out of the mapped host images (one launch per call); with
    TLB_HOST_DIRECT=0 a gather kernel packs them into device memory first (two launches).  Either
    way the result must equal the oracle exactly, for odd widths, any alignment, all output forms."""
    import torch
    lib = _capi.load()
    monkeypatch.setenv("TLB_HOST_DIRECT", "1" if direct else "0")
    for seed, dtype, layout, cl in [(41, _capi.TLB_F32, _capi.TLB_NCHW, False), (42, _capi.TLB_BF16, _capi.TLB_NHWC, True)]:
        wl = S.config2(seed=seed, n=14, lo=33, hi=131, dst=56)
        wl.dtype, wl.channels_last = ("f32" if dtype == _capi.TLB_F32 else "bf16"), cl
        pad = 5  # shift the packed images off the 16-byte grid
        pinned = torch.empty(wl.src.size + pad, dtype=torch.uint8).pin_memory()
        pinned[pad:] = torch.from_numpy(wl.src)
        refs = (_capi.ImageRef * wl.n)()
        crops = (_capi.CropParams * wl.n)()
        for i in range(wl.n):
            refs[i].data = pinned.data_ptr() + pad + int(wl.offsets[i])
            refs[i].w, refs[i].h = int(wl.sizes[i, 0]), int(wl.sizes[i, 1])
            crops[i].x, crops[i].y, crops[i].w, crops[i].h = (float(v) for v in wl.boxes[i])
            crops[i].flip = int(wl.flips[i])
        tdt = torch.float32 if dtype == _capi.TLB_F32 else torch.bfloat16
        shape = (wl.n, 56, 56, 3) if cl else (wl.n, 3, 56, 56)
        out = torch.empty(shape, dtype=tdt, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        before = t.launch_count()
        for _ in range(3):
            rc = lib.tlb_crop_resize_normalize_to_device(refs, crops, wl.n, 56, 56, _capi.f3(wl.mean), _capi.f3(wl.std), 1,
                                                         out.data_ptr(), dtype, layout, status.data_ptr(),
                                                         C.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert rc == 0, lib.tlb_last_error()
        torch.cuda.synchronize()
        assert t.launch_count() - before == (3 if direct else 6)
        assert int(status.item()) == 0
        want = expected(wl)
        if dtype == _capi.TLB_F32:
            assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
        else:
            assert check_bf16(out.view(torch.int16).cpu().numpy().view(np.uint16), want) == 0


def test_separately_pinned_host_images_whole_and_edge_crops():
    """Every image in its own page-locked allocation (as a decoder pool hands them out), with crops
    that touch the first and the last byte of their image: the direct path may not read a byte
    outside an image, and must still produce the oracle's bits."""
    import torch
    lib = _capi.load()
    wl = S.config2(seed=43, n=9, lo=17, hi=90, dst=40)
    for i in range(wl.n):  # whole image, top-left corner, bottom-right corner, ...
        w, h = int(wl.sizes[i, 0]), int(wl.sizes[i, 1])
        wl.boxes[i] = [(0, 0, w, h), (0, 0, max(1, w // 2), max(1, h // 3)), (w - max(1, w // 3), h - max(1, h // 2), max(1, w // 3), max(1, h // 2))][i % 3]
    pins, refs, crops = [], (_capi.ImageRef * wl.n)(), (_capi.CropParams * wl.n)()
    for i in range(wl.n):
        w, h = int(wl.sizes[i, 0]), int(wl.sizes[i, 1])
        o = int(wl.offsets[i])
        pimg = torch.from_numpy(wl.src[o:o + w * h * 3].copy()).pin_memory()
        pins.append(pimg)
        refs[i].data, refs[i].w, refs[i].h = pimg.data_ptr(), w, h
        crops[i].x, crops[i].y, crops[i].w, crops[i].h = (float(v) for v in wl.boxes[i])
        crops[i].flip = int(wl.flips[i])
    out = torch.empty((wl.n, 3, 40, 40), dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.tlb_crop_resize_normalize_to_device(refs, crops, wl.n, 40, 40, _capi.f3(wl.mean), _capi.f3(wl.std), 1,
                                                 out.data_ptr(), _capi.TLB_F32, _capi.TLB_NCHW, status.data_ptr(),
                                                 C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.tlb_last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert np.array_equal(out.cpu().numpy().view(np.uint32), expected(wl).view(np.uint32))


def test_resident_loader_reference_contract():
    import torch
    data = _dataset(50, 20, seed=4)
    ld = t.CudaResidentLoader.from_array(data, batch_size=16, shuffle=True, seed=42, return_indices=True)
    assert len(ld) == 3
    perm = np.random.default_rng(42).permutation(50)
    seen = []
    for b, (batch, idx) in enumerate(ld):
        x = torch.as_tensor(batch, device="cuda")
        assert x.shape == (16, 3, 20, 20) and x.dtype == torch.float32
        idx = idx.cpu().numpy()
        assert np.array_equal(idx, perm[b * 16:(b + 1) * 16])
        assert np.array_equal(x.cpu().numpy(), _oracle_uniform(data, sel=idx))
        seen.append(idx)
    assert len(seen) == 3
    ld.set_epoch(1)
    first = next(iter(ld))[1].cpu().numpy()
    assert np.array_equal(first, np.random.default_rng(43).permutation(50)[:16])
    # sequential, ragged tail kept, numpy arange indices (turboloader/cuda_loader.py:528-533)
    ld2 = t.CudaResidentLoader.from_array(data, batch_size=16, drop_last=False, return_indices=True)
    got = list(ld2)
    assert len(got) == 4 and len(got[-1][0]) == 2
    assert np.array_equal(got[-1][1], np.arange(48, 50))
    assert np.array_equal(torch.as_tensor(got[1][0], device="cuda").cpu().numpy(), _oracle_uniform(data[16:32]))
    assert ld.device_status() == 0 and ld2.device_status() == 0


def test_resident_loader_crop_flip_bf16_channels_last_labels_and_resume():
    import torch
    data = _dataset(64, 40, seed=5)
    labels = np.arange(64) * 3 + 1
    kw = dict(batch_size=8, shuffle=True, seed=7, return_indices=True, crop_size=36, output_size=32, hflip_prob=0.5,
              dtype=torch.bfloat16, channels_last=True, labels=labels)
    ld = t.CudaResidentLoader.from_array(data, **kw)
    order, flips = ld.epoch_order(), ld.epoch_flips()
    assert flips.sum() not in (0, 64)
    batches = []
    for b, (x, y, idx) in enumerate(ld):
        assert x.shape == (8, 3, 32, 32) and x.is_contiguous(memory_format=torch.channels_last)
        idx = idx.cpu().numpy()
        assert np.array_equal(idx, order[b * 8:(b + 1) * 8])
        assert np.array_equal(y.cpu().numpy(), labels[idx])
        ref = _oracle_uniform(data, sel=idx, box=(2, 2, 36, 36), flips=flips[b * 8:(b + 1) * 8], dst=(32, 32))
        got = x.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)  # logical NCHW order
        assert check_bf16(got, O.bf16_bits(ref)) == 0
        batches.append(got.copy())
        if b == 2:
            state = ld.state_dict()
    assert state == {"version": 1, "epoch": 0, "batches_served": 3}
    ld2 = t.CudaResidentLoader.from_array(data, **kw)
    ld2.load_state_dict(state)
    rest = [x.contiguous().view(torch.int16).cpu().numpy().view(np.uint16) for x, _, _ in ld2]
    assert len(rest) == 5
    for a, b in zip(rest, batches[3:]):
        assert np.array_equal(a, b)


def test_resident_loader_explicit_boxes():
    import torch
    data = _dataset(20, 48, seed=6)

    def boxes(epoch, order):
        rs = np.random.RandomState(epoch)
        w = rs.randint(8, 49, size=len(order))
        h = rs.randint(8, 49, size=len(order))
        return np.stack([rs.randint(0, 48 - w + 1), rs.randint(0, 48 - h + 1), w, h], axis=1)

    ld = t.CudaResidentLoader.from_array(data, batch_size=10, shuffle=True, boxes=boxes, output_size=24, hflip_prob=0.3,
                                         return_indices=True, as_tensor=True)
    bx = boxes(0, ld.epoch_order()).astype(np.int32)
    fl = ld.epoch_flips()
    flat, offsets, sizes = S.uniform_dataset(data)
    for b, (x, idx) in enumerate(ld):
        want = O.fused_batch(flat, offsets, sizes, idx.cpu().numpy(), bx[b * 10:(b + 1) * 10], fl[b * 10:(b + 1) * 10], 24, 24,
                             MEAN, STD, True)
        assert np.array_equal(x.cpu().numpy(), want)


def test_dataloader_tbl_contract(tmp_path):
    """DataLoader('x.tbl', output_format='pytorch'): (images, meta) batches, TblRawImageLoader's
    order and flip rules (turboloader/tbl.py:213-264), state_dict resume, ragged last batch."""
    import torch
    from turboloader_b200 import tbl
    data = _dataset(37, 16, seed=9)
    path = tmp_path / "d.tbl"
    tbl.write_raw_tbl(path, data)
    dl = t.DataLoader(path, batch_size=8, shuffle=True, seed=5, transform=t.ImageNetNormalize(), image_size=16,
                      hflip_prob=0.5)
    assert len(dl) == 5
    order = np.random.default_rng(5).permutation(37)
    frng = np.random.default_rng((5, 0, 1))
    got = []
    for b, (x, meta) in enumerate(dl):
        idx = order[b * 8:(b + 1) * 8]
        assert x.is_cuda and x.dtype == torch.float32 and x.shape == (len(idx), 3, 16, 16)
        assert np.array_equal(meta["indices"], idx) and meta["batch_size"] == len(idx)
        flips = (frng.random(len(idx)) < 0.5).astype(np.uint8)
        assert np.array_equal(x.cpu().numpy(), _oracle_uniform(data, sel=idx, flips=flips))
        got.append(x.cpu().numpy().copy())
        if b == 1:
            sd = dl.state_dict()
    assert sd == {"version": 1, "epoch": 0, "batches_served": 2}
    # plain [0,1] floats without a transform; sequential order
    dl2 = t.DataLoader(arrays=data, batch_size=16)
    x, meta = next(iter(dl2))
    assert np.array_equal(meta["indices"], np.arange(16))
    assert np.abs(x.cpu().numpy() - data[:16].transpose(0, 3, 1, 2).astype(np.float32) / 255.0).max() < 1e-6
    # resume: unflipped loader continues exactly where the state says
    dl3 = t.DataLoader(path, batch_size=8, shuffle=True, seed=5, transform=t.ImageNetNormalize())
    ref = [x.cpu().numpy().copy() for x, _ in dl3]
    dl4 = t.DataLoader(path, batch_size=8, shuffle=True, seed=5, transform=t.ImageNetNormalize())
    dl4.load_state_dict({"version": 1, "epoch": 0, "batches_served": 3})
    rest = [x.cpu().numpy().copy() for x, _ in dl4]
    assert len(rest) == 2 and all(np.array_equal(a, b) for a, b in zip(rest, ref[3:]))


def test_resident_loader_train_aug():
    """train_aug: per-sample RandomResizedCrop + flip drawn for (seed, epoch, sample index),
    fused with the resize; batches equal the oracle run on the same rects."""
    data = _dataset(30, 64, seed=12)
    ld = t.CudaResidentLoader.from_array(data, batch_size=10, shuffle=True, seed=3, train_aug=True, output_size=32,
                                         return_indices=True, as_tensor=True)
    flat, offsets, sizes = S.uniform_dataset(data)
    for epoch in (0, 1):
        ld.set_epoch(epoch)
        order = ld.epoch_order()
        boxes, flips = t.pick_crops(3, epoch, np.tile([[64, 64]], (30, 1)), indices=order)
        assert flips.sum() not in (0, 30)
        for b, (x, idx) in enumerate(ld):
            idx = idx.cpu().numpy()
            assert np.array_equal(idx, order[b * 10:(b + 1) * 10])
            want = O.fused_batch(flat, offsets, sizes, idx, boxes[b * 10:(b + 1) * 10], flips[b * 10:(b + 1) * 10], 32, 32,
                                 MEAN, STD, True)
            assert np.array_equal(x.cpu().numpy(), want)


@pytest.mark.skipif(O.ref_cuda() is None, reason="reference CUDA kernels were not compiled (oracle/_ref)")
def test_against_the_reference_gpu_kernels():
    """The reference's own CUDA kernels (compiled in place for this GPU) as a second statement of the
    math.  Normalize / gather: they divide by 255 where the CPU path multiplies by 1/255, so the
    agreement is to rounding, not to the bit (the reference reports 4e-07 against numpy).  Resize:
    they skip the 8-bit truncation of the CPU path, so they sit within one code step of it."""
    import torch
    lib = O.ref_cuda()
    assert lib.tlrefcuda_available() == 1
    data = _dataset(64, 32, seed=13)
    gpu = torch.from_numpy(data).cuda()
    mean = np.asarray(MEAN, np.float32)
    std = np.asarray(STD, np.float32)
    f32p = C.POINTER(C.c_float)
    sel = torch.from_numpy(np.random.RandomState(1).permutation(64)[:40].astype(np.int64)).cuda()
    rptr = lib.tlrefcuda_normalize_resident_gather(gpu.data_ptr(), sel.data_ptr(), 40, 32, 32,
                                                   mean.ctypes.data_as(f32p), std.ctypes.data_as(f32p))
    assert rptr
    ref = torch.as_tensor(t._CudaArray(rptr, (40, 3, 32, 32)), device="cuda").cpu().numpy()
    ours = torch.as_tensor(t._CudaArray(t.cuda_normalize_resident_gather(gpu.data_ptr(), sel.data_ptr(), 40, 32, 32),
                                        (40, 3, 32, 32)), device="cuda").cpu().numpy()
    assert np.abs(ours - ref).max() < 1e-6
    # full-image resize of host images: within one 8-bit code step of the reference GPU kernel
    rs = np.random.RandomState(2)
    images = [rs.randint(0, 256, size=(h, w, 3), dtype=np.uint8) for h, w in [(40, 60), (64, 64), (33, 21)]]
    ref = O.ref_cuda_crop_resize_normalize(images, None, None, 24, 24, MEAN, STD)
    ours = t.cuda_resize_normalize(images, 24, 24)
    step = 1.0 / (255.0 * np.asarray(STD, np.float64)).reshape(1, 3, 1, 1)
    d = np.abs(ours.astype(np.float64) - ref)
    # 1.001: the two coordinate formulas round differently, which moves a blend by ~2e-4 of a code
    assert (d <= step * 1.001).all() and d.mean() > 1e-4  # truncation really differs, by < 1 code


def test_device_images_in_separate_allocations():
    """cuda_resize_normalize_from_device (resize_normalize_device_batch, cuda_transforms.hpp:141-144):
    every image lives in its own device allocation, sizes are ragged and odd so that rows and image
    ends sit off the 16-byte grid; the result is the oracle's, the ring is shared with the other
    pointer-returning forms, and an image that does not fit its allocation is refused."""
    import torch
    rs = np.random.RandomState(21)
    shapes = [(50, 70), (33, 21), (64, 64), (9, 201), (17, 5), (1, 1), (120, 37)]
    images = [rs.randint(0, 256, size=(h, w, 3), dtype=np.uint8) for h, w in shapes]
    # One device buffer per image (small blocks of torch's allocator, spread apart by 2 MiB fillers),
    # passed in an order that is not the address order.
    devs = [torch.empty(im.size + 0, dtype=torch.uint8, device="cuda") for im in images]
    pad = [torch.empty(1 << 21, dtype=torch.uint8, device="cuda") for _ in images]  # spread the blocks apart
    for d, im in zip(devs, images):
        d.copy_(torch.from_numpy(im.reshape(-1)))
    order = [3, 0, 6, 1, 5, 2, 4]  # not in address order
    ptrs = [devs[i].data_ptr() for i in order]
    ws = [shapes[i][1] for i in order]
    hs = [shapes[i][0] for i in order]
    flat, offsets, sizes = S.pack_images([images[i] for i in order])
    want = O.fused_batch(flat, offsets, sizes, None, None, None, 40, 56, MEAN, STD, True)
    out = t.cuda_resize_normalize_from_device(ptrs, ws, hs, 40, 56)
    got = torch.as_tensor(t._CudaArray(out, (len(order), 3, 40, 56)), device="cuda").cpu().numpy()
    assert np.array_equal(got, want)
    out2 = t.cuda_resize_normalize_from_device(ptrs[:2], ws[:2], hs[:2], 40, 56)
    assert out2 != out
    with pytest.raises(RuntimeError):
        t.cuda_resize_normalize_from_device(ptrs, ws, hs[:-1], 40, 56)
    with pytest.raises(RuntimeError):
        t.cuda_resize_normalize_from_device([0], [4], [4], 8, 8)
    # an image claimed larger than the allocation that holds it
    whole = torch.empty(1 << 22, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError):
        t.cuda_resize_normalize_from_device([whole.data_ptr()], [4096], [4096], 8, 8)
    del pad


def test_resident_gather_is_bounded_by_the_allocation():
    """The legacy gather form does not say how many images the dataset holds; the bound is the end
    of the device allocation, so an index far beyond it is not read (the sample is zero-filled)."""
    import torch
    data = _dataset(16, 24)
    gpu = torch.empty(1 << 22, dtype=torch.uint8, device="cuda")  # a whole 4 MiB block of its own
    gpu[:data.size] = torch.from_numpy(data.reshape(-1)).cuda()
    sel = torch.from_numpy(np.array([3, 1 << 34, 7], dtype=np.int64)).cuda()
    ptr = t.cuda_normalize_resident_gather(gpu.data_ptr(), sel.data_ptr(), 3, 24, 24)
    got = torch.as_tensor(t._CudaArray(ptr, (3, 3, 24, 24)), device="cuda").cpu().numpy()
    want = _oracle_uniform(data, sel=np.array([3, 7], np.int64))
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[2], want[1]) and (got[1] == 0).all()


def test_cuda_array_speaks_dlpack():
    """The float32 hand-off object implements __dlpack__ / __dlpack_device__ beside
    __cuda_array_interface__: torch.from_dlpack adopts the same device memory without a copy."""
    import torch
    data = _dataset(12, 16)
    gpu = torch.from_numpy(data).cuda()
    ptr = t.cuda_normalize_resident(gpu.data_ptr(), 12, 16, 16)
    arr = t._CudaArray(ptr, (12, 3, 16, 16))
    assert arr.__dlpack_device__() == (2, torch.cuda.current_device())
    via_dlpack = torch.from_dlpack(arr)
    via_cai = torch.as_tensor(arr, device="cuda")
    assert via_dlpack.data_ptr() == ptr == via_cai.data_ptr()
    assert via_dlpack.dtype == torch.float32 and tuple(via_dlpack.shape) == (12, 3, 16, 16)
    assert np.array_equal(via_dlpack.cpu().numpy(), _oracle_uniform(data))
    # the loader's float32 batches are such objects; bf16 batches are torch tensors with their own __dlpack__
    ld = t.CudaResidentLoader.from_array(data, batch_size=4)
    first = next(iter(ld))
    assert hasattr(first, "__dlpack__") and hasattr(first, "__cuda_array_interface__")
    assert np.array_equal(torch.from_dlpack(first).cpu().numpy(), _oracle_uniform(data[:4]))
