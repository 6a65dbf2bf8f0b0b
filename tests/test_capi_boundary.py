"""The C-ABI library loads without a GPU, exports every symbol the header declares, and
rejects bad arguments on the host before any CUDA call."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from turboloader_b200 import _capi, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "turboloader_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"TLB_API\s+[\w\s\*]+?\b(tlb_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    lib = _capi.load()
    names = _declared_symbols()
    assert len(names) >= 16
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"


def test_struct_layout_matches_header_order():
    text = open(os.path.join(ROOT, "include", "turboloader_b200.h")).read()
    start = text.index("typedef struct tlb_transform_desc {") + len("typedef struct tlb_transform_desc {")
    body = text[start:text.index("} tlb_transform_desc;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        for part in decl.split(","):
            m = re.search(r"(\w+)\s*(\[\d+\])?\s*$", part.strip())
            fields.append(m.group(1))
    assert fields == [f[0] for f in _capi.TransformDesc._fields_]


def _desc(**kw):
    d = _capi.TransformDesc()
    d.src = 0x1000
    d.src_bytes = 1 << 20
    d.n_src = 4
    d.src_w, d.src_h = 32, 32
    d.n = 4
    d.dst_h, d.dst_w = 16, 16
    d.out = 0x2000
    d.mean = _capi.f3((0, 0, 0))
    d.std = _capi.f3((1, 1, 1))
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def test_plan_is_computed_without_a_gpu():
    plan = ops.fused_plan(_desc(dst_h=224, dst_w=224, src_w=256, src_h=256, n=256, n_src=256))
    # Two columns per lane (c and c + 32 of a 64-column strip), one planner warp on top.
    assert plan["tile_cols"] == 256 and plan["block"] == 32 * (4 + 1) and plan["smem_bytes"] <= 227 * 1024
    assert plan["grid"] == 256 * -(-224 // plan["tile_rows"])
    narrow = ops.fused_plan(_desc(dst_h=24, dst_w=24, src_w=256, src_h=256, n=256, n_src=256))
    assert narrow["tile_cols"] == 32 and narrow["block"] == 32 * (1 + 1)  # one column per lane
    wide = ops.fused_plan(_desc(dst_h=8, dst_w=1200, src_w=1400, src_h=60))
    assert wide["tile_cols"] <= 512 and wide["tile_cols"] % 32 == 0 and wide["block"] <= 288
    assert wide["grid"] == 4 * -(-1200 // wide["tile_cols"])


@pytest.mark.parametrize("kw,code", [
    (dict(dst_h=0), 1), (dict(out_dtype=7), 1), (dict(out_layout=3), 1), (dict(src=None), 1), (dict(n_src=0), 1),
    (dict(std=_capi.f3((1, 0, 1))), 1), (dict(n=9), 3), (dict(uniform_box=(C.c_int32 * 4)(30, 0, 8, 8)), 2),
    (dict(src_w=0, src_h=0), 1), (dict(flags=2), 1), (dict(jitter=0x3000, normalize_01=0), 1),
])
def test_invalid_descriptors_are_rejected_on_the_host(kw, code):
    lib = _capi.load()
    rc = lib.tlb_fused_transform(C.byref(_desc(**kw)), None)
    assert rc == code
    assert lib.tlb_last_error()


def test_host_params_validation_names_the_sample():
    lib = _capi.load()
    sel = np.array([0, 1, 4, 2], dtype=np.int64)
    d = _desc(sel=sel.ctypes.data)
    assert lib.tlb_fused_transform_host_params(C.byref(d), None) == 3
    assert b"sample 2" in lib.tlb_last_error()
    boxes = np.array([[0, 0, 32, 32], [1, 0, 32, 32], [0, 0, 1, 1], [0, 0, 1, 1]], dtype=np.int32)
    d = _desc(boxes=boxes.ctypes.data)
    assert lib.tlb_fused_transform_host_params(C.byref(d), None) == 2
    assert b"sample 1" in lib.tlb_last_error()


def test_empty_batch_is_a_no_op():
    assert _capi.load().tlb_fused_transform(C.byref(_desc(n=0)), None) == 0


def test_host_image_forms_validate_before_touching_cuda():
    lib = _capi.load()
    img = np.zeros((8, 8, 3), dtype=np.uint8)
    refs = (_capi.ImageRef * 1)()
    refs[0].data, refs[0].w, refs[0].h = img.ctypes.data, 8, 8
    out = np.zeros((1, 3, 4, 4), dtype=np.float32)
    crops = (_capi.CropParams * 1)()
    crops[0].x, crops[0].y, crops[0].w, crops[0].h = 0.5, 0, 4, 4
    m, s = _capi.f3((0, 0, 0)), _capi.f3((1, 1, 1))
    if not ops.cuda_available():
        pytest.skip("host-image forms look up the current device first")
    assert lib.tlb_crop_resize_normalize_batch(refs, crops, 1, 4, 4, m, s, out.ctypes.data) == 1


def test_no_gpu_means_unavailable_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    assert ops.cuda_available() is False
    assert ops.cuda_device_name() == ""
    assert ops.features()["cpu_fallback"] is False
    with pytest.raises(RuntimeError):
        ops.cuda_resize_normalize([np.zeros((4, 4, 3), np.uint8)], 2, 2)


def test_video_descriptor_is_validated_on_the_host():
    lib = _capi.load()
    ptrs = (C.c_size_t * 2)(4096, 8192)
    out = np.zeros(16, np.float32)

    def vd(**kw):
        d = _capi.VideoDesc()
        d.y_ptrs = d.cb_ptrs = d.cr_ptrs = C.cast(ptrs, C.c_void_p)
        d.n, d.y_stride, d.c_stride, d.c_px_stride = 2, 32, 16, 1
        d.src_w, d.src_h, d.dst_h, d.dst_w = 32, 32, 8, 8
        d.mean, d.std = _capi.f3((0, 0, 0)), _capi.f3((1, 1, 1))
        d.out = out.ctypes.data
        for k, v in kw.items():
            setattr(d, k, v)
        return d

    assert lib.tlb_video_yuv420(None, None) == 1
    assert lib.tlb_video_yuv420(C.byref(vd(n=0)), None) == 0  # empty batch: nothing to do
    for kw in (dict(y_stride=31), dict(c_px_stride=3), dict(c_stride=15), dict(dst_w=0), dict(out=None),
               dict(out_dtype=5), dict(clip_len=-1), dict(std=_capi.f3((1, 0, 1)))):
        assert lib.tlb_video_yuv420(C.byref(vd(**kw)), None) == 1, kw
        assert lib.tlb_last_error()
    assert lib.tlb_video_yuv420(C.byref(vd(n=70000)), None) == 7
    bad_crop = np.array([0, 0, np.inf, 4], np.float32)
    assert lib.tlb_video_yuv420(C.byref(vd(crops=bad_crop.ctypes.data)), None) == 2
    null_plane = (C.c_size_t * 2)(4096, 0)
    assert lib.tlb_video_yuv420(C.byref(vd(cb_ptrs=C.cast(null_plane, C.c_void_p))), None) == 1
    assert b"frame 1" in lib.tlb_last_error()
    m, s = _capi.f3((0, 0, 0)), _capi.f3((1, 1, 1))
    assert lib.tlb_video_yuv420_batch(ptrs, ptrs, ptrs, 0, 32, 16, 1, 32, 32, 8, 8, 0, m, s) == 0


def test_stream_core_arguments_are_validated_on_the_host():
    lib = _capi.load()
    img = np.zeros((4, 8, 8, 3), np.uint8)
    m, s = _capi.f3((0, 0, 0)), _capi.f3((1, 1, 1))
    assert not lib.tlb_stream_create(None, 4, 8, 8, 2, m, s, 3, 1, None, 0, 0, 0, 0)
    assert not lib.tlb_stream_create(img.ctypes.data, 0, 8, 8, 2, m, s, 3, 1, None, 0, 0, 0, 0)
    assert not lib.tlb_stream_create(img.ctypes.data, 4, 8, 8, 2, m, s, 3, 1, None, 0, 0, 9, 0)
    assert lib.tlb_last_error()
    assert lib.tlb_stream_num_batches(None) == -1
    assert lib.tlb_stream_begin_epoch(None, None) == 1
    lib.tlb_stream_destroy(None)  # a no-op


def test_video_descriptor_from_python_and_no_device_error():
    import torch
    out = torch.empty((2, 3, 8, 8), dtype=torch.float32)
    d = ops.make_video_desc([4096, 8192], [4096, 8192], [4100, 8200], y_stride=32, c_stride=16, c_px_stride=1, src_w=32,
                            src_h=32, out=out, crops=[[0, 0, 16, 16]], flips=[1], clip_len=0, bt709=True)
    assert (d.n, d.dst_h, d.dst_w, d.bt709, d.out_dtype) == (2, 8, 8, 1, _capi.TLB_F32)
    assert d.crops and d.flips and d.out == out.data_ptr()
    with pytest.raises(ValueError):
        ops.make_video_desc([1], [1, 2], [1], y_stride=8, c_stride=4, c_px_stride=1, src_w=8, src_h=8, out=out)
    with pytest.raises(TypeError):
        ops.make_video_desc([1, 2], [1, 2], [1, 2], y_stride=8, c_stride=4, c_px_stride=1, src_w=8, src_h=8,
                            out=out.to(torch.float16))
    if torch.cuda.is_available():
        pytest.skip("GPU present: the enqueue would run")
    with pytest.raises(_capi.TurboLoaderB200Error) as e:
        ops.enqueue_video(d, 0)
    assert e.value.code == 6  # TLB_ERR_NO_DEVICE: there is no CPU fallback


def test_epoch_pipeline_rejects_bad_arguments_on_the_host():
    """tlb_epoch_create validates its descriptor and pipeline geometry before any CUDA call."""
    lib = _capi.load()
    d = _desc(n=4, n_src=64)
    d.sel = 0x4000
    args = dict(total=64, drop_last=0, start=0, ring=8, ahead=3, out=4 * 3 * 16 * 16 * 4, idx=0, lab=0)

    def create(desc=d, **kw):
        a = dict(args, **kw)
        return lib.tlb_epoch_create(C.byref(desc), a["total"], a["drop_last"], a["start"], a["ring"], a["ahead"],
                                    a["out"], a["idx"], a["lab"])

    assert not create(ring=4, ahead=3) and b"ring" in lib.tlb_last_error()   # no slot left for a valid batch
    assert not create(ahead=0)
    assert not create(total=0)
    assert not create(out=0)
    assert not create(start=-1)
    seq = _desc(n=4, n_src=8)                                                  # in order, but total > n_src
    assert not create(desc=seq) and b"n_src" in lib.tlb_last_error()
    assert not create(desc=_desc(n=4, n_src=64, dst_h=0))
    assert lib.tlb_epoch_next(None, None, None, None, None) == 1
    lib.tlb_epoch_destroy(None)
