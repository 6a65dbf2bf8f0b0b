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
