"""CPU checks of the YUV 4:2:0 video oracle (oracle/video_ref.c): against an independent numpy
statement of the sampling + colour math (the one the reference's tests/test_cuda_video.py:74-111
uses, within its own tolerance and a much tighter one), I420 == NV12, flip and crop algebra, and
the golden vectors written on a B200 by the reference's own kernels."""
import os

import numpy as np
import pytest

from oracle import oracle as O

MEAN = (0.485, 0.456, 0.406)
STD = (0.229, 0.224, 0.225)
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def make_frame(seed, h, w, smooth=True):
    """Deterministic I420 planes (y (h,w), cb, cr ((h+1)//2,(w+1)//2))."""
    rs = np.random.RandomState(seed)
    ch, cw = (h + 1) // 2, (w + 1) // 2
    if smooth:
        yy, xx = np.mgrid[0:h, 0:w].astype(np.float32)
        y = np.clip(127 + 90 * np.sin(xx / 17 + seed) * np.cos(yy / 23) + rs.randint(-6, 7, (h, w)), 16, 235)
        cb = np.clip(128 + 60 * np.cos(xx[:ch, :cw] / 9 - seed) + rs.randint(-4, 5, (ch, cw)), 16, 240)
        cr = np.clip(128 + 60 * np.sin((xx + yy)[:ch, :cw] / 11 + seed) + rs.randint(-4, 5, (ch, cw)), 16, 240)
        return y.astype(np.uint8), cb.astype(np.uint8), cr.astype(np.uint8)
    return (rs.randint(0, 256, (h, w), dtype=np.uint8), rs.randint(0, 256, (ch, cw), dtype=np.uint8),
            rs.randint(0, 256, (ch, cw), dtype=np.uint8))


def to_nv12(cb, cr):
    uv = np.empty((cb.shape[0], cb.shape[1] * 2), dtype=np.uint8)
    uv[:, 0::2], uv[:, 1::2] = cb, cr
    return uv


def numpy_statement(y, cb, cr, dh, dw, bt709, crop=None, flip=False):
    """float64 statement of the transform -> rgb in [0,1], (3, dh, dw)."""
    H, W = y.shape
    if crop is None:
        sx = np.maximum(0.0, (np.arange(dw) + 0.5) * W / dw - 0.5)
        sy = np.maximum(0.0, (np.arange(dh) + 0.5) * H / dh - 0.5)
    else:
        x, yy, cw_, ch_ = crop
        ox = np.arange(dw)[::-1] if flip else np.arange(dw)
        sx = np.clip(x + (ox + 0.5) / dw * cw_ - 0.5, 0, W - 1)
        sy = np.clip(yy + (np.arange(dh) + 0.5) / dh * ch_ - 0.5, 0, H - 1)

    def gather(plane, yf, xf):
        y0 = np.floor(yf).astype(np.int64)
        x0 = np.floor(xf).astype(np.int64)
        y1 = np.minimum(y0 + 1, plane.shape[0] - 1)
        x1 = np.minimum(x0 + 1, plane.shape[1] - 1)
        dy = (yf - y0)[:, None]
        dx = (xf - x0)[None, :]
        p = plane.astype(np.float64)
        return (p[y0][:, x0] * (1 - dx) + p[y0][:, x1] * dx) * (1 - dy) + (p[y1][:, x0] * (1 - dx) + p[y1][:, x1] * dx) * dy

    cxf = np.clip(sx * 0.5, 0, cb.shape[1] - 1)
    cyf = np.clip(sy * 0.5 - 0.25, 0, cb.shape[0] - 1)
    Y = gather(y, sy, sx)
    Cb = gather(cb, cyf, cxf) - 128.0
    Cr = gather(cr, cyf, cxf) - 128.0
    yv = (Y - 16.0) * (255.0 / 219.0)
    if bt709:
        r, g, b = yv + 1.792741 * Cr, yv - 0.213249 * Cb - 0.532909 * Cr, yv + 2.112402 * Cb
    else:
        r, g, b = yv + 1.596027 * Cr, yv - 0.391762 * Cb - 0.812968 * Cr, yv + 2.017232 * Cb
    return np.clip(np.stack([r, g, b]) / 255.0, 0.0, 1.0)


def denorm(out):
    return out * np.asarray(STD, np.float32).reshape(3, 1, 1) + np.asarray(MEAN, np.float32).reshape(3, 1, 1)


@pytest.mark.parametrize("dst,bt709", [((48, 64), False), ((97, 111), False), ((31, 45), True), ((120, 200), True)])
def test_whole_frame_matches_numpy_statement(dst, bt709):
    y, cb, cr = make_frame(3, 96, 128)
    dh, dw = dst
    got = denorm(O.yuv420_frame(y, cb, cr, 1, 128, 96, dh, dw, MEAN, STD, bt709=bt709))
    ref = numpy_statement(y, cb, cr, dh, dw, bt709)
    d = np.abs(got - ref)
    assert d.max() < 0.03 and d.mean() < 0.004  # the reference's own bound (tests/test_cuda_video.py:141-142)
    assert d.max() < 2e-5                       # what separately rounded fp32 really achieves


@pytest.mark.parametrize("flip", [False, True])
def test_crop_window_and_flip(flip):
    y, cb, cr = make_frame(5, 90, 122, smooth=False)  # odd chroma width: (122+1)//2 = 61
    crop = (10.0, 7.0, 71.0, 53.0)
    got = denorm(O.yuv420_frame(y, cb, cr, 1, 122, 90, 40, 56, MEAN, STD, crop=crop, flip=flip))
    ref = numpy_statement(y, cb, cr, 40, 56, False, crop=crop, flip=flip)
    assert np.abs(got - ref).max() < 5e-5
    if flip:
        plain = O.yuv420_frame(y, cb, cr, 1, 122, 90, 40, 56, MEAN, STD, crop=crop, flip=False)
        flipped = O.yuv420_frame(y, cb, cr, 1, 122, 90, 40, 56, MEAN, STD, crop=crop, flip=True)
        assert np.array_equal(flipped, plain[:, :, ::-1])  # the flip mirrors the sampling positions exactly


def test_nv12_equals_i420():
    y, cb, cr = make_frame(7, 64, 80, smooth=False)
    uv = to_nv12(cb, cr)
    a = O.yuv420_frame(y, cb, cr, 1, 80, 64, 50, 70, MEAN, STD)
    b = O.yuv420_frame(y, uv, uv.reshape(-1)[1:], 2, 80, 64, 50, 70, MEAN, STD, c_stride=uv.strides[0])
    assert np.array_equal(a, b)


def test_full_frame_crop_reduces_to_whole_frame_rule_within_rounding():
    """tests/test_cuda_video.py:165-174: with the crop equal to the frame the clip rule matches the
    batch rule to 1e-6 (the two coordinate formulas round differently, so not to the bit)."""
    y, cb, cr = make_frame(9, 96, 128)
    a = O.yuv420_frame(y, cb, cr, 1, 128, 96, 48, 64, MEAN, STD)
    b = O.yuv420_frame(y, cb, cr, 1, 128, 96, 48, 64, MEAN, STD, crop=(0.0, 0.0, 128.0, 96.0))
    assert np.abs(a - b).max() < 5e-5


def test_golden_vectors_from_the_reference_kernels():
    """tests/golden/video_golden.npz holds outputs of the reference's own CUDA kernels (compiled
    without FMA contraction) on a B200 for seeded frames; the restatement must reproduce them
    bit for bit."""
    path = os.path.join(GOLD, "video_golden.npz")
    if not os.path.exists(path):
        pytest.skip("golden file not generated yet")
    g = np.load(path, allow_pickle=False)
    cases = int(g["n_cases"])
    assert cases >= 4
    for i in range(cases):
        seed, h, w, dh, dw, nv12, bt709, use_crop, flip, smooth = [int(v) for v in g[f"case{i}_params"]]
        crop = tuple(float(v) for v in g[f"case{i}_crop"]) if use_crop else None
        y, cb, cr = make_frame(seed, h, w, smooth=bool(smooth))
        if nv12:
            uv = to_nv12(cb, cr)
            got = O.yuv420_frame(y, uv, uv.reshape(-1)[1:], 2, w, h, dh, dw, MEAN, STD, crop=crop, flip=bool(flip),
                                 bt709=bool(bt709), c_stride=uv.strides[0])
        else:
            got = O.yuv420_frame(y, cb, cr, 1, w, h, dh, dw, MEAN, STD, crop=crop, flip=bool(flip), bt709=bool(bt709))
        want = g[f"case{i}_out"]
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"case {i}"
