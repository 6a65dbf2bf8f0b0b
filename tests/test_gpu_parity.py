"""GPU parity: the sm_100a kernel, called through the C ABI, against the CPU oracle on the
same seeded inputs (reduced-size versions of the five benchmark configurations), plus the
edge cases the reference's own resize tests use."""
import numpy as np
import pytest

from turboloader_b200 import _capi
from turboloader_b200 import synthetic as S

from helpers import check_bf16, check_f32, expected, run_gpu

pytestmark = pytest.mark.gpu


def _compare(wl, **kw):
    res = run_gpu(wl, **kw)
    ref = expected(wl)
    assert res["status"] == 0
    if wl.dtype == "f32":
        nbad = check_f32(res["out"], ref, wl, channel_axis=3 if wl.channels_last else 1)
    else:
        nbad = check_bf16(res["out"], ref)
    assert nbad == 0, f"{nbad} elements are not bit-identical to the oracle"
    want_idx = wl.sel if wl.sel is not None else np.arange(wl.n)
    assert np.array_equal(res["indices"], want_idx)
    return res


def test_config1_fixed_resize():
    _compare(S.config1(seed=1, n=24))


def test_config2_variable_rrc():
    _compare(S.config2(seed=2, n=48))


def test_config2_host_params():
    _compare(S.config2(seed=3, n=16), host_params=True)


def test_config3_resident_gather_bf16():
    wl = S.config3(seed=4, n_dataset=300, batch=64, batch_index=2)
    labels = np.arange(300, dtype=np.int64) * 7 + 3
    res = _compare(wl, labels=labels)
    assert np.array_equal(res["labels"], labels[wl.sel])


def test_config4_highres_nhwc_bf16():
    _compare(S.config4(seed=5, n=6))


def test_config5_shard_bf16():
    _compare(S.config5(seed=6, total=64, world=2, rank=1, batch=16, batch_index=1))


@pytest.mark.parametrize("dtype,cl", [("f32", False), ("f32", True), ("bf16", False), ("bf16", True)])
def test_all_output_forms(dtype, cl):
    wl = S.config2(seed=7, n=12, lo=60, hi=140, dst=64)
    wl.dtype, wl.channels_last = dtype, cl
    _compare(wl)


# Size cases of the reference's tests/test_simd_bilinear.cpp:111-251 (sw, sh, dw, dh).
SIZE_CASES = [(224, 224, 112, 112), (112, 112, 224, 224), (320, 240, 224, 224), (100, 100, 127, 97), (8, 8, 16, 16),
              (64, 64, 64, 64), (100, 1, 224, 1), (1, 100, 1, 224), (1, 1, 5, 7), (2, 2, 17, 3), (3840, 2160, 224, 224),
              (201, 333, 50, 50), (499, 200, 300, 31), (37, 41, 640, 33)]


@pytest.mark.parametrize("case", SIZE_CASES)
@pytest.mark.parametrize("dtype,cl", [("f32", False), ("bf16", True)])
def test_size_cases(case, dtype, cl):
    sw, sh, dw, dh = case
    rng = np.random.default_rng(sw * 7 + dh)
    imgs = [rng.integers(0, 256, size=(sh, sw, 3), dtype=np.uint8) for _ in range(3)]
    flat, offsets, sizes = S.pack_images(imgs)
    wl = S.Workload("case", flat, offsets, sizes, 3, dh, dw, flips=np.array([0, 1, 1], dtype=np.uint8), dtype=dtype,
                    channels_last=cl)
    _compare(wl)


def test_crops_at_all_borders_and_odd_pitch():
    rng = np.random.default_rng(11)
    imgs = [rng.integers(0, 256, size=(97, 201, 3), dtype=np.uint8) for _ in range(8)]
    flat, offsets, sizes = S.pack_images(imgs)
    boxes = np.array([[0, 0, 201, 97], [0, 0, 1, 1], [200, 96, 1, 1], [0, 96, 201, 1], [200, 0, 1, 97],
                      [13, 7, 150, 60], [100, 50, 101, 47], [1, 1, 199, 95]], dtype=np.int32)
    flips = np.array([0, 1, 0, 1, 0, 1, 0, 1], dtype=np.uint8)
    for dst in [(33, 47), (1, 1), (16, 128)]:
        wl = S.Workload("borders", flat, offsets, sizes, 8, dst[0], dst[1], boxes=boxes, flips=flips)
        _compare(wl)


def test_source_off_the_16_byte_grid():
    wl = S.config2(seed=12, n=6, lo=30, hi=90, dst=40)
    for pad in (1, 7, 15):
        _compare(wl, src_pad_front=pad)


def test_steep_downscale_uses_row_pairs():
    rng = np.random.default_rng(13)
    imgs = [rng.integers(0, 256, size=(900, 300, 3), dtype=np.uint8) for _ in range(2)]
    flat, offsets, sizes = S.pack_images(imgs)
    wl = S.Workload("steep", flat, offsets, sizes, 2, 40, 64)
    _compare(wl)


def test_wide_output_uses_column_tiles():
    rng = np.random.default_rng(14)
    imgs = [rng.integers(0, 256, size=(60, 700, 3), dtype=np.uint8) for _ in range(2)]
    flat, offsets, sizes = S.pack_images(imgs)
    for dtype, cl in [("f32", False), ("bf16", True)]:
        wl = S.Workload("wide", flat, offsets, sizes, 2, 20, 600, flips=np.array([1, 0], dtype=np.uint8), dtype=dtype,
                        channels_last=cl)
        _compare(wl)


def test_invalid_samples_are_zero_filled_and_reported():
    from turboloader_b200 import _capi
    wl = S.config2(seed=15, n=6, lo=40, hi=80, dst=32)
    good = expected(wl)
    wl.sel = np.array([0, 1, 99, 3, -1, 5], dtype=np.int64)  # two invalid gather indices
    wl.boxes = wl.boxes.copy()
    wl.boxes[3] = (0, 0, 10_000, 5)                          # a box that leaves its image
    res = run_gpu(wl, max_crop_w=int(wl.sizes[:, 0].max()))
    assert res["status"] == (_capi.DEV_BAD_INDEX | _capi.DEV_BAD_BOX)
    for k in (2, 3, 4):
        assert (res["out"][k] == 0).all()
    for k in (0, 1, 5):
        assert np.array_equal(res["out"][k], good[k])
    assert np.array_equal(res["indices"], wl.sel)


def test_back_to_back_launches_may_overlap():
    """TLB_FLAG_LAUNCH_OVERLAP (per call): consecutive flagged launches into distinct outputs give
    the same bits as plain launches."""
    import torch

    import turboloader_b200 as t
    wl = S.config2(n=24, seed=5, lo=60, hi=140, dst=64)
    want = expected(wl)
    flat = torch.from_numpy(wl.src).cuda()
    offs = torch.from_numpy(wl.offsets).cuda()
    sizes = torch.from_numpy(np.ascontiguousarray(wl.sizes)).cuda()
    boxes = torch.from_numpy(np.ascontiguousarray(wl.boxes)).cuda()
    flips = torch.from_numpy(wl.flips).cuda()
    outs = [torch.full((wl.n, 3, 64, 64), -7.0, device="cuda") for _ in range(8)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for o in outs:
        t.fused_transform(flat, n=wl.n, dst_h=64, dst_w=64, out=o, src_offsets=offs, src_sizes=sizes, boxes=boxes,
                          flips=flips, mean=wl.mean, std=wl.std, max_crop_w=int(wl.boxes[:, 2].max()), status=status,
                          launch_overlap=True)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for o in outs:
        assert np.array_equal(o.cpu().numpy(), want)


def test_unflagged_launch_keeps_stream_order_behind_a_producer_kernel():
    """A launch WITHOUT the overlap flag must see what a kernel directly before it in the same
    stream wrote -- here the gather indices and the flip flags -- even when other launches in the
    process use the flag.  (The flag is per call; it must never change an unflagged launch.)"""
    import torch

    import turboloader_b200 as t
    wl = S.config3(seed=11, n_dataset=64, batch=32, batch_index=0)
    data = torch.from_numpy(wl.src).cuda()
    boxes = torch.from_numpy(np.ascontiguousarray(wl.boxes)).cuda()
    sel_final = torch.from_numpy(wl.sel).cuda()
    flips_final = torch.from_numpy(wl.flips).cuda()
    h, w = wl.uniform_hw
    want = expected(wl)
    for rep in range(6):
        sel = torch.zeros_like(sel_final)
        flips = torch.zeros_like(flips_final)
        out = torch.empty((wl.n, 3, wl.dst_h, wl.dst_w), dtype=torch.bfloat16, device="cuda")
        warm = torch.empty_like(out)
        # A flagged launch first, so that the stream's previous kernel is one that signals early.
        t.fused_transform(data, n=wl.n, n_src=wl.n_src, src_w=w, src_h=h, dst_h=wl.dst_h, dst_w=wl.dst_w, out=warm,
                          sel=sel_final, boxes=boxes, flips=flips_final, mean=wl.mean, std=wl.std,
                          max_crop_w=int(wl.boxes[:, 2].max()), launch_overlap=True)
        sel.copy_(sel_final + 0)        # producer kernels (elementwise add, then copy) on the same stream
        flips.copy_(flips_final | 0)
        t.fused_transform(data, n=wl.n, n_src=wl.n_src, src_w=w, src_h=h, dst_h=wl.dst_h, dst_w=wl.dst_w, out=out,
                          sel=sel, boxes=boxes, flips=flips, mean=wl.mean, std=wl.std,
                          max_crop_w=int(wl.boxes[:, 2].max()))
        torch.cuda.synchronize()
        assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), want), f"repetition {rep}"


def _jitter_run(wl, jit):
    import torch
    from oracle import oracle as O
    table = torch.from_numpy(np.ascontiguousarray(jit, np.float32)).cuda()
    res = run_gpu(wl, mutate=lambda d: setattr(d, "jitter", table.data_ptr()))
    assert res["status"] == 0
    ref = O.fused_batch(wl.src, wl.offsets, wl.sizes, wl.sel, wl.boxes, wl.flips, wl.dst_h, wl.dst_w, wl.mean, wl.std,
                        jitter=jit)
    if wl.channels_last:
        ref = O.nchw_to_nhwc(ref)
    return res["out"], (O.bf16_bits(ref) if wl.dtype == "bf16" else ref)


def test_colour_jitter_matches_the_restatement_bit_for_bit():
    """Per-sample (brightness, contrast, saturation) between the 8-bit code and the normalize, in the
    order of the reference's train_transform shader (src/metal/metal_transforms.mm:111-115).  The
    oracle is a CPU restatement of those lines (the shader itself cannot run here)."""
    rs = np.random.RandomState(4)
    wl = S.config2(n=40, seed=21, lo=60, hi=260, dst=96)
    jit = rs.uniform(0.6, 1.4, size=(wl.n, 3)).astype(np.float32)
    jit[0] = (1.0, 1.0, 1.0)
    jit[1] = (3.0, 2.0, 0.0)   # saturates, then grey
    jit[2] = (0.0, 1.0, 1.0)   # black before contrast
    got, want = _jitter_run(wl, jit)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # bf16 NHWC, gather + uniform crop (two columns per lane and the ragged last strip)
    wl3 = S.config3(seed=5, n_dataset=90, batch=33, batch_index=1, src=100, crop=90, dst=80)
    wl3.channels_last = True
    jit3 = rs.uniform(0.5, 1.5, size=(wl3.n, 3)).astype(np.float32)
    got, want = _jitter_run(wl3, jit3)
    assert check_bf16(got, want) == 0
    # narrow output: one column per lane
    wln = S.config2(n=9, seed=22, lo=30, hi=80, dst=24)
    got, want = _jitter_run(wln, rs.uniform(0.7, 1.3, size=(9, 3)).astype(np.float32))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_identity_jitter_and_brightness():
    """The reference's own two checks (tests/test_metal.py:205-228): identity factors reproduce the
    plain transform within 1e-4, a brightness factor changes the output."""
    wl = S.config2(n=6, seed=23, lo=100, hi=200, dst=64)
    plain = run_gpu(wl)["out"]
    ident, _ = _jitter_run(wl, np.ones((6, 3), np.float32))
    assert np.abs(ident - plain).max() < 1e-4
    bright, _ = _jitter_run(wl, np.tile(np.array([[1.5, 1.0, 1.0]], np.float32), (6, 1)))
    assert np.abs(bright - plain).mean() > 0.01


def test_jitter_needs_unit_range():
    import torch
    wl = S.config1(n=2, seed=1, src=32, dst=16)   # mean/std in 0..255 units
    table = torch.ones((2, 3), device="cuda")
    with pytest.raises(_capi.TurboLoaderB200Error):
        run_gpu(wl, mutate=lambda d: setattr(d, "jitter", table.data_ptr()))
