"""The allocation-free host-image entry point (tlb_crop_resize_normalize_to_device_static).

Some users of this library cannot allocate memory when they ask for a batch: their process has
handed the whole GPU to a training memory pool, or runs under a rule that forbids allocation
after start-up.  For them the library offers one entry point that stages the crops in a fixed
device array inside the library instead of a growable ring.  This file checks, through the C
ABI, that it produces exactly what the regular entry point and the CPU oracle produce -- twice in
a row, because the fixed array keeps the bytes of the previous call --, that a call leaves the
amount of free device memory as it found it, and that it refuses batches beyond its stated
limits.  It is named to be collected last.
"""
import ctypes as C

import numpy as np
import pytest

from turboloader_b200 import _capi
from turboloader_b200 import synthetic as S

from helpers import expected

pytestmark = pytest.mark.gpu


def _refs(wl):
    refs = (_capi.ImageRef * wl.n)()
    crops = (_capi.CropParams * wl.n)()
    for i in range(wl.n):
        refs[i].data = wl.src.ctypes.data + int(wl.offsets[i])
        refs[i].w, refs[i].h = int(wl.sizes[i, 0]), int(wl.sizes[i, 1])
        crops[i].x, crops[i].y, crops[i].w, crops[i].h = (float(v) for v in wl.boxes[i])
        crops[i].flip = int(wl.flips[i])
    return refs, crops


def _run(fn, wl, refs, crops, dtype, layout):
    import torch
    tdt = torch.float32 if dtype == _capi.TLB_F32 else torch.bfloat16
    out = torch.full((wl.n * 3 * wl.dst_h * wl.dst_w,), -3.0, dtype=tdt, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = fn(refs, crops, wl.n, wl.dst_h, wl.dst_w, _capi.f3(wl.mean), _capi.f3(wl.std), 1, out.data_ptr(), dtype, layout,
            status.data_ptr(), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, _capi.load().tlb_last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out.view(torch.int16 if tdt == torch.bfloat16 else torch.int32).cpu().numpy()


def test_static_entry_matches_the_regular_entry_twice_in_a_row():
    lib = _capi.load()
    first = S.config2(seed=31, n=12, lo=40, hi=150, dst=64)
    second = S.config2(seed=32, n=7, lo=20, hi=90, dst=48)   # a smaller batch afterwards: stale bytes stay behind it
    for wl, dtype, layout in [(first, _capi.TLB_F32, _capi.TLB_NCHW), (second, _capi.TLB_BF16, _capi.TLB_NHWC),
                              (first, _capi.TLB_BF16, _capi.TLB_NCHW)]:
        refs, crops = _refs(wl)
        want = _run(lib.tlb_crop_resize_normalize_to_device, wl, refs, crops, dtype, layout)
        got = _run(lib.tlb_crop_resize_normalize_to_device_static, wl, refs, crops, dtype, layout)
        assert np.array_equal(got, want)  # bit-identical: same kernel, same inputs, different staging
        # ... and directly against the CPU oracle, in the same layout and dtype
        wl.dtype = "f32" if dtype == _capi.TLB_F32 else "bf16"
        wl.channels_last = layout == _capi.TLB_NHWC
        ref = expected(wl)
        ref = ref.view(np.int32) if dtype == _capi.TLB_F32 else ref.view(np.int16)
        assert np.array_equal(got, ref.reshape(-1))


def test_static_entry_allocates_no_device_memory():
    """After the first call on the device (which only looks the array's address up), a call must
    leave the free device memory exactly as it found it: the staging lives in the library image."""
    import torch
    lib = _capi.load()
    wl = S.config2(seed=33, n=9, lo=30, hi=120, dst=56)
    refs, crops = _refs(wl)
    _run(lib.tlb_crop_resize_normalize_to_device_static, wl, refs, crops, _capi.TLB_F32, _capi.TLB_NCHW)  # set-up call
    out = torch.empty(wl.n * 3 * wl.dst_h * wl.dst_w, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        rc = lib.tlb_crop_resize_normalize_to_device_static(refs, crops, wl.n, wl.dst_h, wl.dst_w, _capi.f3(wl.mean),
                                                            _capi.f3(wl.std), 1, out.data_ptr(), _capi.TLB_F32,
                                                            _capi.TLB_NCHW, status.data_ptr(), stream)
        assert rc == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before and int(status.item()) == 0


def test_static_entry_rejects_what_does_not_fit():
    import torch
    lib = _capi.load()
    out = torch.empty(16, dtype=torch.float32, device="cuda")
    m, s = _capi.f3((0, 0, 0)), _capi.f3((1, 1, 1))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # too many samples
    n = _capi.STATIC_MAX_SAMPLES + 1
    img = np.zeros((2, 2, 3), dtype=np.uint8)
    refs = (_capi.ImageRef * n)()
    for i in range(n):
        refs[i].data, refs[i].w, refs[i].h = img.ctypes.data, 2, 2
    rc = lib.tlb_crop_resize_normalize_to_device_static(refs, None, n, 1, 1, m, s, 1, out.data_ptr(), 0, 0, None, stream)
    assert rc == 7 and b"samples" in lib.tlb_last_error()
    # too many bytes: three 3400x3400 images are 104 MB of crops, the array holds 32 MiB
    big = np.zeros((3400, 3400, 3), dtype=np.uint8)
    refs = (_capi.ImageRef * 3)()
    for i in range(3):
        refs[i].data, refs[i].w, refs[i].h = big.ctypes.data, 3400, 3400
    rc = lib.tlb_crop_resize_normalize_to_device_static(refs, None, 3, 1, 1, m, s, 1, out.data_ptr(), 0, 0, None, stream)
    assert rc == 7 and b"bytes" in lib.tlb_last_error()
