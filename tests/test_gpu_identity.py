"""GPU tests of the identity-size fast path (crop size == output size on a uniform dataset: gather,
flip, normalize, layout, dtype -- the reference's resident-loader operation): bit-identical to the
CPU oracle and to the general kernel, which is forced with TLB_IDENTITY_FAST=0."""
import ctypes as C

import numpy as np
import pytest

import turboloader_b200 as t
from oracle import oracle as O
from turboloader_b200 import synthetic as S

from helpers import check_bf16, expected, run_gpu

pytestmark = pytest.mark.gpu


def _uniform_box(box):
    def mutate(d):
        d.boxes = None
        d.uniform_box = (C.c_int32 * 4)(*box)
    return mutate


@pytest.mark.parametrize("dtype,channels_last", [("f32", False), ("f32", True), ("bf16", False), ("bf16", True)])
@pytest.mark.parametrize("hw,crop", [(40, 32), (37, 37), (50, 29)])
def test_identity_path_matches_oracle_and_general_kernel(monkeypatch, dtype, channels_last, hw, crop):
    wl = S.config3(seed=21, n_dataset=48, batch=20, src=hw, crop=crop, dst=crop)
    wl.dtype, wl.channels_last = dtype, channels_last
    off = (hw - crop) // 2
    mutate = _uniform_box((off, off, crop, crop)) if crop != hw else _uniform_box((0, 0, 0, 0))
    before = t.launch_count()
    fast = run_gpu(wl, mutate=mutate)
    assert t.launch_count() == before + 1
    want = expected(wl)
    if dtype == "f32":
        assert np.array_equal(fast["out"].view(np.uint32), want.view(np.uint32))
    else:
        assert check_bf16(fast["out"], want) == 0
    assert fast["status"] == 0 and np.array_equal(fast["indices"], wl.sel)
    monkeypatch.setenv("TLB_IDENTITY_FAST", "0")
    general = run_gpu(wl, mutate=mutate)
    assert np.array_equal(fast["out"], general["out"])


def test_invalid_gather_index_is_zero_filled_and_reported():
    wl = S.config3(seed=22, n_dataset=32, batch=8, src=24, crop=24, dst=24)
    wl.dtype = "f32"
    want = expected(wl)
    wl.sel = wl.sel.copy()
    wl.sel[5] = 99  # outside the dataset
    res = run_gpu(wl, mutate=_uniform_box((0, 0, 0, 0)))
    assert res["status"] & 1
    assert (res["out"][5] == 0).all()
    keep = [i for i in range(8) if i != 5]
    assert np.array_equal(res["out"][keep], want[keep])
