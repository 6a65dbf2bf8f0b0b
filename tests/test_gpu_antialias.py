"""GPU parity of the antialiased (triangle filter) variant of the fused transform against the
CPU oracle, which itself equals the reference's resize_triangle_antialias bit for bit
(tests/test_oracle.py).  Bit-exact for fp32; bf16 is the rounded fp32 result."""
import numpy as np
import pytest

from oracle import oracle as O
from turboloader_b200 import synthetic as S

from helpers import check_bf16, expected_antialias, run_gpu

pytestmark = pytest.mark.gpu


def _aa(d):
    d.antialias = 1
    d.max_crop_h = 0  # derived from src_h = the tallest image


def _check(wl, **kw):
    res = run_gpu(wl, mutate=_aa, **kw)
    want = expected_antialias(wl)
    assert res["status"] == 0
    if wl.channels_last:
        want = O.nchw_to_nhwc(want)
    if wl.dtype == "f32":
        bad = int((res["out"].view(np.uint32) != want.view(np.uint32)).sum())
    else:
        bad = check_bf16(res["out"], O.bf16_bits(want))
    assert bad == 0, f"{bad} elements differ from the oracle"
    return res


def test_variable_size_downscale_with_boxes_and_flips():
    _check(S.config2(seed=11, n=24, lo=80, hi=300, dst=64))


def test_strong_downscale_many_taps():
    wl = S.config2(seed=12, n=6, lo=300, hi=420, dst=24)  # scale up to ~17: 36 taps per axis
    _check(wl)


def test_upscale_and_identity_reduce_to_two_or_one_tap():
    wl = S.config1(seed=13, n=6, src=40, dst=56)  # upscale: support 1
    _check(wl)
    same = S.config1(seed=14, n=4, src=48, dst=48)  # identity: exact copy of the pixels
    res = _check(same)
    plain = run_gpu(same)
    assert np.array_equal(res["out"], plain["out"])


def test_bf16_nhwc_and_gather():
    wl = S.config4(seed=15, n=8, src=96, dst=72)
    _check(wl)
    wl = S.config3(seed=16, n_dataset=64, batch=16, src=40, crop=36, dst=32)
    res = _check(wl)
    assert np.array_equal(res["indices"], wl.sel)


def test_invalid_samples_are_zero_filled_and_reported():
    wl = S.config2(seed=17, n=8, lo=60, hi=100, dst=32)
    want = expected_antialias(wl)
    wl.boxes[3] = (5, 5, 400, 10)  # leaves the image
    res = run_gpu(wl, mutate=_aa, max_crop_w=100)
    assert res["status"] & 2
    assert (res["out"][3] == 0).all()
    keep = [i for i in range(8) if i != 3]
    assert np.array_equal(res["out"][keep], want[keep])


def test_tiny_crops_odd_widths_and_two_column_tiles():
    """Crops narrower than the filter (the tap window is the whole crop row), an output width that is
    no multiple of 32 (the second column of some threads does not exist), and an output wide enough
    for two column tiles of which the second is mostly empty."""
    wl = S.config2(seed=21, n=12, lo=20, hi=60, dst=40)
    wl.dst_w = 50
    for i, (w, h) in enumerate([(1, 1), (2, 3), (3, 2), (1, 7), (5, 1), (4, 4)]):
        wl.boxes[i] = (i % 3, (i + 1) % 4, w, h)
    _check(wl)
    wide = S.config2(seed=22, n=3, lo=200, hi=400, dst=20)
    wide.dst_w = 300
    _check(wide)
    wide.dtype, wide.channels_last = "bf16", True
    _check(wide)


@pytest.mark.parametrize("pad", [1, 2, 3])
def test_source_off_the_word_grid(pad):
    """The packed kernel fetches tap windows as aligned 32-bit words.  A source that starts 1..3 bytes
    off the word grid sends its first image (words would start before the buffer) and its last one
    (words would end after it) through byte loads, and every other image through realigned words."""
    wl = S.config2(seed=23 + pad, n=10, lo=50, hi=130, dst=48)
    _check(wl, src_pad_front=pad)


def test_one_column_kernel_still_matches():
    """The packed kernel and the one-column kernel it replaced are the same function."""
    import subprocess, sys, textwrap
    code = textwrap.dedent("""
        import numpy as np
        from turboloader_b200 import synthetic as S
        import sys; sys.path.insert(0, 'tests')
        from helpers import expected_antialias, run_gpu
        def aa(d):
            d.antialias = 1; d.max_crop_h = 0
        wl = S.config2(seed=29, n=8, lo=80, hi=300, dst=64)
        out = run_gpu(wl, mutate=aa)["out"]
        assert np.array_equal(out.view(np.uint32), expected_antialias(wl).view(np.uint32))
        print("ok")
    """)
    import os
    env = dict(os.environ, TLB_AA_ONE_COLUMN="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]


def test_colour_jitter_after_the_antialiased_resize():
    """Per-sample (brightness, contrast, saturation) applied to the antialiased 8-bit image before the
    normalize; oracle: the C restatement of both (the shader lines src/metal/metal_transforms.mm:111-115
    after resize_triangle_antialias)."""
    import torch
    rs = np.random.RandomState(9)
    for wl in (S.config2(seed=31, n=16, lo=60, hi=260, dst=72), S.config4(seed=32, n=5, src=96, dst=80)):
        jit = rs.uniform(0.6, 1.4, size=(wl.n, 3)).astype(np.float32)
        jit[0] = (1.0, 1.0, 1.0)
        jit[1] = (3.0, 2.0, 0.0)   # saturates, then grey
        table = torch.from_numpy(jit).cuda()

        def mutate(d):
            _aa(d)
            d.jitter = table.data_ptr()

        res = run_gpu(wl, mutate=mutate)
        assert res["status"] == 0
        want = O.fused_batch(wl.src, wl.offsets, wl.sizes, wl.sel, wl.boxes, wl.flips, wl.dst_h, wl.dst_w, wl.mean, wl.std,
                             antialias=True, jitter=jit)
        if wl.channels_last:
            want = O.nchw_to_nhwc(want)
        if wl.dtype == "f32":
            assert np.array_equal(res["out"].view(np.uint32), want.view(np.uint32))
        else:
            assert check_bf16(res["out"], O.bf16_bits(want)) == 0
