"""GPU parity of the fused YUV 4:2:0 video kernel, called through the C ABI: bit-identical to the
CPU oracle; bit-identical to the reference's own CUDA kernels when those are compiled without FMA
contraction, and within rounding of them as the reference builds them."""
import numpy as np
import pytest

import turboloader_b200 as t
from oracle import oracle as O
from turboloader_b200 import _capi

from test_video_oracle import MEAN, STD, make_frame, to_nv12

pytestmark = pytest.mark.gpu


class Frames:
    """n seeded frames on the device, I420 or NV12, optionally with padded row strides."""

    def __init__(self, n, h, w, nv12=False, pad=0, smooth=True, seed=0):
        import torch
        self.n, self.h, self.w, self.nv12 = n, h, w, nv12
        self.host = []
        self.keep = []
        self.y_ptrs, self.cb_ptrs, self.cr_ptrs = [], [], []
        ch, cw = (h + 1) // 2, (w + 1) // 2
        self.y_stride = w + pad
        self.c_px = 2 if nv12 else 1
        self.c_stride = cw * self.c_px + pad
        for i in range(n):
            y, cb, cr = make_frame(seed + i, h, w, smooth=smooth)
            yb = np.zeros((h, self.y_stride), np.uint8)
            yb[:, :w] = y
            if nv12:
                cbuf = np.zeros((ch, self.c_stride), np.uint8)
                cbuf[:, :2 * cw] = to_nv12(cb, cr)
                dc = torch.from_numpy(cbuf).cuda()
                self.keep.append(dc)
                self.cb_ptrs.append(dc.data_ptr())
                self.cr_ptrs.append(dc.data_ptr() + 1)
                self.host.append((yb, cbuf, cbuf.reshape(-1)[1:]))
            else:
                b0 = np.zeros((ch, self.c_stride), np.uint8)
                b1 = np.zeros((ch, self.c_stride), np.uint8)
                b0[:, :cw], b1[:, :cw] = cb, cr
                d0, d1 = torch.from_numpy(b0).cuda(), torch.from_numpy(b1).cuda()
                self.keep += [d0, d1]
                self.cb_ptrs.append(d0.data_ptr())
                self.cr_ptrs.append(d1.data_ptr())
                self.host.append((yb, b0, b1))
            dy = torch.from_numpy(yb).cuda()
            self.keep.append(dy)
            self.y_ptrs.append(dy.data_ptr())

    def oracle(self, i, dh, dw, crop=None, flip=False, bt709=False):
        y, cb, cr = self.host[i]
        return O.yuv420_frame(y, cb, cr, self.c_px, self.w, self.h, dh, dw, MEAN, STD, crop=crop, flip=flip, bt709=bt709,
                              y_stride=self.y_stride, c_stride=self.c_stride)

    def run(self, dh, dw, dtype=None, **kw):
        import torch
        out = torch.full((self.n, 3, dh, dw), -9.0, dtype=dtype or torch.float32, device="cuda")
        t.video_yuv420(self.y_ptrs, self.cb_ptrs, self.cr_ptrs, y_stride=self.y_stride, c_stride=self.c_stride,
                       c_px_stride=self.c_px, src_w=self.w, src_h=self.h, out=out, mean=MEAN, std=STD, **kw)
        torch.cuda.synchronize()
        return out

    def args(self):
        return (self.y_ptrs, self.cb_ptrs, self.cr_ptrs, self.y_stride, self.c_stride, self.c_px, self.w, self.h)


@pytest.fixture(params=["direct", "direct-uploaded-tables", "staged"], autouse=True)
def kernel_choice(request, monkeypatch):
    """Every test runs against the direct-load kernel with its tables in the kernel parameters (the
    default for small batches), the same kernel with the tables uploaded to device memory (what
    larger batches get; TLB_VIDEO_INLINE_TABLES=0), and the shared-memory staged kernel
    (TLB_VIDEO_STAGED=1)."""
    monkeypatch.delenv("TLB_VIDEO_STAGED", raising=False)
    monkeypatch.delenv("TLB_VIDEO_INLINE_TABLES", raising=False)
    if request.param == "staged":
        monkeypatch.setenv("TLB_VIDEO_STAGED", "1")
    elif request.param == "direct-uploaded-tables":
        monkeypatch.setenv("TLB_VIDEO_INLINE_TABLES", "0")
    return request.param


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("nv12,bt709,dst,pad", [(False, False, (48, 64), 0), (True, False, (97, 111), 0),
                                                (False, True, (120, 300), 5), (True, True, (31, 45), 3)])
def test_whole_frame_resize_is_bit_identical_to_the_oracle(nv12, bt709, dst, pad):
    f = Frames(5, 96, 128, nv12=nv12, pad=pad, smooth=not nv12)
    got = f.run(*dst, bt709=bt709).cpu().numpy()
    for i in range(f.n):
        assert np.array_equal(_bits(got[i]), _bits(f.oracle(i, *dst, bt709=bt709))), f"frame {i}"


def test_clips_share_their_crop_and_flip():
    f = Frames(8, 90, 122, smooth=False, seed=20)  # odd chroma width
    crops = np.array([[10.0, 7.0, 71.0, 53.0], [0.5, 2.25, 100.0, 80.0]], np.float32)  # fractional windows too
    flips = np.array([1, 0], np.int32)
    got = f.run(40, 56, crops=crops, flips=flips, clip_len=4).cpu().numpy()
    for i in range(8):
        want = f.oracle(i, 40, 56, crop=tuple(crops[i // 4]), flip=bool(flips[i // 4]))
        assert np.array_equal(_bits(got[i]), _bits(want)), f"frame {i}"


def test_upscale_and_windows_touching_the_frame_edges():
    """Right/bottom edge taps (x1 == x0, y1 == y0), windows partly outside the frame (coordinates
    clamp), odd frame sizes, an output wider than one block of threads."""
    f = Frames(3, 37, 53, nv12=True, pad=1, smooth=False, seed=60)
    got = f.run(80, 300).cpu().numpy()
    for i in range(3):
        assert np.array_equal(_bits(got[i]), _bits(f.oracle(i, 80, 300)))
    crops = np.array([[30.0, 20.0, 40.0, 30.0]], np.float32)  # reaches past the right and bottom edges
    for flip in (0, 1):
        got = f.run(33, 47, crops=crops, flips=np.array([flip], np.int32)).cpu().numpy()
        for i in range(3):
            assert np.array_equal(_bits(got[i]), _bits(f.oracle(i, 33, 47, crop=tuple(crops[0]), flip=bool(flip))))


def test_back_to_back_launches_with_the_overlap_flag():
    """TLB_FLAG_LAUNCH_OVERLAP: consecutive launches into their own outputs may overlap head to tail;
    every one of them must still produce the oracle's bits."""
    import torch
    f = Frames(6, 72, 100, nv12=True, smooth=False, seed=33)
    crops = np.array([[4.0, 3.0, 80.0, 60.0], [10.0, 8.0, 50.0, 40.0]], np.float32)
    flips = np.array([0, 1], np.int32)
    outs = [torch.full((6, 3, 48, 64), -9.0, device="cuda") for _ in range(4)]
    for out in outs:
        t.video_yuv420(f.y_ptrs, f.cb_ptrs, f.cr_ptrs, y_stride=f.y_stride, c_stride=f.c_stride, c_px_stride=f.c_px,
                       src_w=f.w, src_h=f.h, out=out, mean=MEAN, std=STD, crops=crops, flips=flips, clip_len=3,
                       launch_overlap=True)
    torch.cuda.synchronize()
    want = [f.oracle(i, 48, 64, crop=tuple(crops[i // 3]), flip=bool(flips[i // 3])) for i in range(6)]
    for out in outs:
        got = out.cpu().numpy()
        for i in range(6):
            assert np.array_equal(_bits(got[i]), _bits(want[i])), f"frame {i}"


def test_bf16_output_is_the_rounded_fp32_result():
    import torch
    f = Frames(3, 64, 80, nv12=True)
    got = f.run(50, 70, dtype=torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16)
    for i in range(3):
        assert np.array_equal(got[i], O.bf16_bits(f.oracle(i, 50, 70)))


def test_pointer_forms_keep_the_reference_lifetime():
    """cuda_transforms.hpp:62-64: the returned buffer stays valid until the NEXT call (two buffers)."""
    import torch
    f = Frames(4, 72, 96)
    p1 = t.cuda_video_yuv420_batch(*f.args(), 36, 48, False, MEAN, STD)
    a1 = torch.as_tensor(t._CudaArray(p1, (4, 3, 36, 48)), device="cuda")
    first = a1.cpu().numpy()
    p2 = t.cuda_video_clip_yuv420(*f.args(), 36, 48, (4.0, 6.0, 60.0, 50.0), True, False, MEAN, STD)
    assert p2 != p1
    a2 = torch.as_tensor(t._CudaArray(p2, (4, 3, 36, 48)), device="cuda").cpu().numpy()
    assert np.array_equal(a1.cpu().numpy(), first)  # the previous result survived one more call
    for i in range(4):
        assert np.array_equal(_bits(first[i]), _bits(f.oracle(i, 36, 48)))
        assert np.array_equal(_bits(a2[i]), _bits(f.oracle(i, 36, 48, crop=(4.0, 6.0, 60.0, 50.0), flip=True)))


def test_invalid_arguments_are_rejected_on_the_host():
    f = Frames(2, 32, 32)
    with pytest.raises(RuntimeError):
        t.cuda_video_yuv420_batch(f.y_ptrs, f.cb_ptrs, f.cr_ptrs, 16, f.c_stride, 1, 32, 32, 8, 8)  # y_stride < w
    with pytest.raises(RuntimeError):
        t.cuda_video_yuv420_batch(f.y_ptrs, f.cb_ptrs, f.cr_ptrs, 32, f.c_stride, 3, 32, 32, 8, 8)  # bad px stride
    with pytest.raises(RuntimeError):
        t.cuda_video_yuv420_batch([0, 0], f.cb_ptrs, f.cr_ptrs, 32, f.c_stride, 1, 32, 32, 8, 8)  # NULL plane
    with pytest.raises(ValueError):
        t.cuda_video_yuv420_batch(f.y_ptrs, f.cb_ptrs[:1], f.cr_ptrs, 32, f.c_stride, 1, 32, 32, 8, 8)


@pytest.mark.skipif(O.ref_cuda(nofma=True) is None, reason="reference CUDA kernels were not compiled (oracle/_ref)")
@pytest.mark.parametrize("nv12,bt709", [(False, False), (True, True)])
def test_against_the_reference_video_kernels(nv12, bt709):
    """The reference's own kernels on the same device frames.  Compiled without FMA contraction they
    must equal this library (and hence the oracle) bit for bit; as the reference builds them
    (contraction on) they agree to rounding."""
    import torch
    f = Frames(4, 96, 128, nv12=nv12, smooth=not nv12, seed=40)
    shape = (4, 3, 60, 84)
    crop = (9.0, 5.5, 101.0, 77.25)
    for kw in (dict(), dict(crop=crop, flip=True)):
        ours = f.run(60, 84, bt709=bt709, **({} if not kw else dict(crops=np.array([crop], np.float32),
                                                                      flips=np.array([1], np.int32)))).cpu().numpy()
        p = O.ref_cuda_video(*f.args(), 60, 84, MEAN, STD, bt709=bt709, nofma=True, **kw)
        ref = torch.as_tensor(t._CudaArray(p, shape), device="cuda").cpu().numpy()
        assert np.array_equal(_bits(ours), _bits(ref))
        p = O.ref_cuda_video(*f.args(), 60, 84, MEAN, STD, bt709=bt709, nofma=False, **kw)
        ref = torch.as_tensor(t._CudaArray(p, shape), device="cuda").cpu().numpy()
        assert np.abs(ours - ref).max() < 2e-4  # contraction moves noise-frame results by a few 1e-5
