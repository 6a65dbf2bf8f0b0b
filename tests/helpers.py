"""Shared test helpers: run a synthetic workload through the C ABI on the GPU, and through
the CPU oracle, and compare under the stated tolerances."""
from __future__ import annotations

import ctypes as C

import numpy as np

from oracle import oracle as O
from turboloader_b200 import _capi
from turboloader_b200.synthetic import IMAGENET_STD, Workload


def oracle_f32(wl: Workload, impl="port") -> np.ndarray:
    """fp32 NCHW oracle result for the workload."""
    return O.fused_batch(wl.src, wl.offsets, wl.sizes, wl.sel, wl.boxes, wl.flips, wl.dst_h, wl.dst_w, wl.mean,
                         wl.std, wl.normalize_01, impl=impl)


def expected_antialias(wl):
    """Oracle result with the reference's opt-in antialiased resize (NCHW fp32)."""
    return O.fused_batch(wl.src, wl.offsets, wl.sizes, wl.sel, wl.boxes, wl.flips, wl.dst_h, wl.dst_w, wl.mean, wl.std,
                         wl.normalize_01, antialias=True)


def expected(wl: Workload, impl="port") -> np.ndarray:
    """Oracle result in the workload's layout; bf16 as uint16 bit patterns."""
    ref = oracle_f32(wl, impl)
    if wl.channels_last:
        ref = O.nchw_to_nhwc(ref)
    return O.bf16_bits(ref) if wl.dtype == "bf16" else ref


def run_gpu(wl: Workload, *, host_params=False, device_tables=True, status=True, src_pad_front=0, stream=None,
            want_indices=True, labels=None, max_crop_w=None, mutate=None):
    """Run the workload through tlb_fused_transform (device tables) or
    tlb_fused_transform_host_params (host tables).  Returns dict(out, indices, labels, status)."""
    import torch

    lib = _capi.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    # Optional front padding shifts the source off the 16-byte grid (alignment tests).
    raw = torch.empty(src_pad_front + wl.src.size, dtype=torch.uint8, device=dev)
    raw[src_pad_front:] = torch.from_numpy(np.ascontiguousarray(wl.src)).to(dev)
    src = raw[src_pad_front:]
    n = wl.n
    tdtype = torch.float32 if wl.dtype == "f32" else torch.bfloat16
    shape = (n, wl.dst_h, wl.dst_w, 3) if wl.channels_last else (n, 3, wl.dst_h, wl.dst_w)
    guard = 64
    flat = torch.full((int(np.prod(shape)) + 2 * guard,), -512.0, dtype=tdtype, device=dev)
    out = flat[guard:guard + int(np.prod(shape))].view(shape)
    keep = [raw, flat]
    d = _capi.TransformDesc()
    d.src = src.data_ptr()
    d.src_bytes = wl.src.size
    d.n_src = wl.n_src
    d.n = n

    def table(a, dtype):
        if a is None:
            return None
        a = np.ascontiguousarray(a, dtype=dtype)
        if host_params:
            keep.append(a)
            return a.ctypes.data
        t = torch.from_numpy(a).to(dev)
        keep.append(t)
        return t.data_ptr()

    if wl.uniform_hw is not None:
        d.src_h, d.src_w = wl.uniform_hw
    else:
        d.src_offsets = table(wl.offsets, np.int64)
        d.src_sizes = table(wl.sizes, np.int32)
        d.src_w = int(wl.sizes[:, 0].max())
        d.src_h = int(wl.sizes[:, 1].max())
    d.sel = table(wl.sel, np.int64)
    d.boxes = table(wl.boxes, np.int32)
    d.flips = table(wl.flips, np.uint8)
    d.dst_h, d.dst_w = wl.dst_h, wl.dst_w
    d.out = out.data_ptr()
    d.out_dtype = _capi.TLB_F32 if wl.dtype == "f32" else _capi.TLB_BF16
    d.out_layout = _capi.TLB_NHWC if wl.channels_last else _capi.TLB_NCHW
    idx = lab = None
    if want_indices:
        idx = torch.full((n,), -5, dtype=torch.int64, device=dev)
        d.out_indices = idx.data_ptr()
    if labels is not None:
        lab_in = torch.from_numpy(np.ascontiguousarray(labels, dtype=np.int64)).to(dev)
        lab = torch.full((n,), -5, dtype=torch.int64, device=dev)
        keep.append(lab_in)
        d.labels_in = lab_in.data_ptr()
        d.labels_out = lab.data_ptr()
    d.mean = _capi.f3(wl.mean)
    d.std = _capi.f3(wl.std)
    d.normalize_01 = int(wl.normalize_01)
    d.max_crop_w = int(wl.crop_wh()[:, 0].max()) if max_crop_w is None else int(max_crop_w)
    st = torch.zeros(1, dtype=torch.int32, device=dev) if status else None
    if st is not None:
        d.status = st.data_ptr()
    if mutate is not None:
        mutate(d)
    cs = torch.cuda.current_stream() if stream is None else stream
    fn = lib.tlb_fused_transform_host_params if host_params else lib.tlb_fused_transform
    rc = fn(C.byref(d), C.c_void_p(cs.cuda_stream))
    if rc != 0:
        raise _capi.TurboLoaderB200Error(rc, lib.tlb_last_error().decode())
    torch.cuda.synchronize()
    res = {"status": int(st.item()) if st is not None else None}
    g0 = flat[:guard].float().cpu().numpy()
    g1 = flat[guard + int(np.prod(shape)):].float().cpu().numpy()
    assert (g0 == -512.0).all() and (g1 == -512.0).all(), "guard band around the output was overwritten"
    if wl.dtype == "f32":
        res["out"] = out.cpu().numpy()
    else:
        res["out"] = out.view(torch.int16).cpu().numpy().view(np.uint16)
    res["indices"] = idx.cpu().numpy() if idx is not None else None
    res["labels"] = lab.cpu().numpy() if lab is not None else None
    return res


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def check_f32(got: np.ndarray, ref: np.ndarray, wl: Workload, channel_axis=1):
    """Tolerance stated by the parity contract: per element |d| <= 1/(255*std_c) (std in [0,1]
    units), mean |d| <= 1e-3.  Returns the number of elements that are not bit-identical."""
    std01 = np.asarray(wl.std, dtype=np.float64) / (1.0 if wl.normalize_01 else 255.0)
    bound = 1.0 / (255.0 * std01)
    shape = [1] * got.ndim
    shape[channel_axis] = 3
    d = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    assert (d <= bound.reshape(shape) * (1 + 1e-6)).all(), f"max |d| = {d.max()}"
    assert d.mean() <= 1e-3, f"mean |d| = {d.mean()}"
    return int((got.view(np.uint32) != ref.view(np.uint32)).sum())


def check_bf16(got_bits: np.ndarray, ref_bits: np.ndarray):
    """bf16 output must be the correctly rounded fp32 oracle value within one bf16 ulp.
    Returns the number of elements that differ at all."""
    g = got_bits.astype(np.int32)
    r = ref_bits.astype(np.int32)
    # Map the sign-magnitude bit patterns to a monotone integer line before differencing.
    g = np.where(g & 0x8000, 0x8000 - g, g)
    r = np.where(r & 0x8000, 0x8000 - r, r)
    ulp = np.abs(g - r)
    assert ulp.max() <= 1, f"bf16 differs by {ulp.max()} ulp"
    return int((ulp != 0).sum())
