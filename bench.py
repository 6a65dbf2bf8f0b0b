#!/usr/bin/env python
"""Benchmark of the fused image-transform path (crop + flip + bilinear resize + normalize
-> 224x224) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one pass of the fused transform over one batch of synthetic pre-decoded uint8
images.  The default workload is the variable-size RandomResizedCrop configuration
(512 images, H and W uniform in [200, 500], explicit torchvision-style RRC boxes, flips,
fp32 NCHW 224x224).  Under torchrun every rank transforms batches of its own disjoint
shard with no collective ("weak" scaling: per-rank work is fixed).

Prints ONE JSON line (rank 0).  ``value`` is images/s over all ranks with inputs resident
in HBM (median of several repeats of the K-step loop); ``e2e`` is the same metric through the
host-image C-ABI entry point (pinned host pixels -> crop rows pulled across PCIe -> kernel ->
device batch, status word read back every step); ``roofline`` compares the kernel's algorithmic
bytes per second with the measured HBM copy bandwidth; ``cpu_baseline`` times the reference's own
CPU fused path on this box's host cores; ``sharded_scaling`` (at every N) runs the 8-GPU scaling
configuration -- 32,768 images split over the ranks by the package's own sharding functions.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "img/s (crop+flip+resize+normalize->224)"
UNIT = "img/s"
WORKLOADS = ("variable_rrc", "fixed_resize", "resident_epoch", "highres_nhwc", "sharded_scaling")


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s)"


def ncu_traffic(workload):
    """DRAM bytes per launch from the committed ncu capture summary, or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            return json.load(f).get(workload)
    except Exception:
        return None


# ---- workloads -----------------------------------------------------------------------------

def make_host_workload(name, seed, sets):
    """``sets`` distinct host workloads of the named configuration (full size)."""
    from turboloader_b200 import synthetic as S

    if name == "variable_rrc":
        return [S.config2(seed=seed + 17 * i, n=512) for i in range(sets)]
    if name == "fixed_resize":
        return [S.config1(seed=seed + 17 * i, n=256) for i in range(sets)]
    if name == "highres_nhwc":
        return [S.config4(seed=seed + 17 * i, n=256) for i in range(sets)]
    raise ValueError(name)


class DeviceBatch:
    """One batch with every table resident on the device, ready to launch repeatedly."""

    def __init__(self, wl, device, src=None, keep=None):
        import torch

        from turboloader_b200 import _capi

        self.wl = wl
        self.keep = [] if keep is None else list(keep)
        dev = device
        if src is None:
            src = torch.from_numpy(np.ascontiguousarray(wl.src)).to(dev)
        self.src = src
        d = _capi.TransformDesc()
        d.src = src.data_ptr()
        d.src_bytes = src.numel()
        d.n_src = wl.n_src
        d.n = wl.n

        def up(a, dt):
            if a is None:
                return None
            t = torch.from_numpy(np.ascontiguousarray(a, dtype=dt)).to(dev)
            self.keep.append(t)
            return t.data_ptr()

        if wl.uniform_hw is not None:
            d.src_h, d.src_w = wl.uniform_hw
        else:
            d.src_offsets = up(wl.offsets, np.int64)
            d.src_sizes = up(wl.sizes, np.int32)
            d.src_w = int(wl.sizes[:, 0].max())
            d.src_h = int(wl.sizes[:, 1].max())
        d.sel = up(wl.sel, np.int64)
        d.boxes = up(wl.boxes, np.int32)
        d.flips = up(wl.flips, np.uint8)
        d.dst_h, d.dst_w = wl.dst_h, wl.dst_w
        tdt = torch.float32 if wl.dtype == "f32" else torch.bfloat16
        shape = (wl.n, wl.dst_h, wl.dst_w, 3) if wl.channels_last else (wl.n, 3, wl.dst_h, wl.dst_w)
        self.out = torch.empty(shape, dtype=tdt, device=dev)
        d.out = self.out.data_ptr()
        d.out_dtype = _capi.TLB_F32 if wl.dtype == "f32" else _capi.TLB_BF16
        d.out_layout = _capi.TLB_NHWC if wl.channels_last else _capi.TLB_NCHW
        if wl.sel is not None:
            self.idx = torch.empty(wl.n, dtype=torch.int64, device=dev)
            d.out_indices = self.idx.data_ptr()
        d.mean = _capi.f3(wl.mean)
        d.std = _capi.f3(wl.std)
        d.normalize_01 = int(wl.normalize_01)
        d.max_crop_w = int(wl.crop_wh()[:, 0].max())
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        d.status = self.status.data_ptr()
        self.desc = d

    def set_overlap(self, on):
        """Per-call launch flag: back-to-back launches of a stream that carries only this library's
        kernels may overlap head to tail (TLB_FLAG_LAUNCH_OVERLAP)."""
        self.desc.flags = 1 if on else 0

    def launch(self, lib, stream_ptr):
        rc = lib.tlb_fused_transform(C.byref(self.desc), stream_ptr)
        if rc != 0:
            raise RuntimeError(lib.tlb_last_error().decode())


def make_device_batches(name, seed, device, sets, resident_images=100_000):
    """Device-resident batches of the named workload (distinct data per set)."""
    import torch

    from turboloader_b200 import synthetic as S

    if name in ("variable_rrc", "fixed_resize", "highres_nhwc"):
        return [DeviceBatch(w, device) for w in make_host_workload(name, seed, sets)]
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    if name == "resident_epoch":
        # 100,000 x 160x160x3 uniform-noise images resident in HBM (7.68 GB); batches of 1024
        # gathered through default_rng(seed).permutation; centre crop 144 -> 128, bf16 NCHW + indices.
        n_ds, src, batch = int(resident_images), 160, 1024
        data = torch.randint(0, 256, (n_ds, src, src, 3), dtype=torch.uint8, device=device, generator=g)
        perm = np.random.default_rng(seed).permutation(n_ds).astype(np.int64)
        flips = (np.random.default_rng([seed, 0, 7]).random(n_ds) < 0.5).astype(np.uint8)
        out = []
        for b in range(sets):
            sel = perm[b * batch:(b + 1) * batch]
            off = (src - 144) // 2
            wl = S.Workload("resident_epoch", np.empty(0, np.uint8), np.empty(0, np.int64),
                            np.tile(np.array([[src, src]], np.int32), (n_ds, 1)), batch, 128, 128, sel=sel,
                            boxes=np.tile(np.array([[off, off, 144, 144]], np.int32), (batch, 1)),
                            flips=flips[b * batch:(b + 1) * batch], dtype="bf16", uniform_hw=(src, src))
            out.append(DeviceBatch(wl, device, src=data.view(-1)))
        return out
    if name == "sharded_scaling":
        # Per-rank batches of 1024 uniform-noise 256x256x3 images, RRC(0.08, 1) boxes, bf16 NCHW.
        src, batch = 256, 1024
        out = []
        for b in range(sets):
            data = torch.randint(0, 256, (batch, src, src, 3), dtype=torch.uint8, device=device, generator=g)
            sizes = np.tile(np.array([[src, src]], np.int32), (batch, 1))
            wl = S.Workload("sharded_scaling", np.empty(0, np.uint8), np.empty(0, np.int64), sizes, batch, 224, 224,
                            boxes=S.rrc_boxes(sizes, (0.08, 1.0), seed=seed + b),
                            flips=(np.random.default_rng([seed, b]).random(batch) < 0.5).astype(np.uint8), dtype="bf16",
                            uniform_hw=(src, src))
            out.append(DeviceBatch(wl, device, src=data.view(-1)))
        return out
    raise ValueError(name)


# ---- clocks --------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the bench runs."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz, self._stop, self._h = [], set(), None, threading.Event(), None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if vis:
                ids = [v for v in vis.split(",") if v.strip()]
                if index < len(ids) and ids[index].strip().isdigit():
                    phys = int(ids[index])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None
        self._t = threading.Thread(target=self._run, daemon=True)

    def sample(self):
        if self._h is None:
            return
        try:
            self.samples.append(int(self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM)))
            mask = int(self._nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self.sample()
            self._stop.wait(0.02)

    def start(self):
        self._t.start()

    def stop(self):
        self._stop.set()
        self._t.join(timeout=1)

    def summary(self):
        return {"sm_mhz": int(statistics.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---- CPU legs ------------------------------------------------------------------------------

def cpu_reference_pass(wl, flavour, threads):
    """One pass of the reference's CPU fused path over the batch; returns seconds."""
    from oracle import oracle as O

    out = np.empty((wl.n, 3, wl.dst_h, wl.dst_w), dtype=np.float32)
    impl = f"ref-{flavour}" if flavour != "port" else "port"
    t0 = time.perf_counter()
    O.fused_batch(wl.src, wl.offsets, wl.sizes, wl.sel, wl.boxes, wl.flips, wl.dst_h, wl.dst_w, wl.mean, wl.std,
                  wl.normalize_01, impl=impl, threads=threads, out=out)
    return time.perf_counter() - t0


def pick_cpu_flavour():
    from oracle import oracle as O

    for fl in ("avx2fma", "parity"):
        if O.ref_available(fl):
            return fl, "reference"
    O.build_port()
    return "port", "port"


def cpu_baseline(wl, budget_s=4.0, min_passes=3):
    from oracle import oracle as O

    flavour, kind = pick_cpu_flavour()
    threads = O.ref_threads(flavour) if kind == "reference" else 1
    cpu_reference_pass(wl, flavour, threads)  # warm-up (thread pool start, page faults)
    times, t_end = [], time.perf_counter() + budget_s
    while len(times) < min_passes or (time.perf_counter() < t_end and len(times) < 50):
        times.append(cpu_reference_pass(wl, flavour, threads))
    med = statistics.median(times)
    build = {"avx2fma": "-O3 -mavx2 -mfma -funroll-loops (hand-written AVX2 branch)",
             "parity": "-O2 -mavx2 -ffp-contract=off", "port": "C restatement, -O2, scalar"}[flavour]
    res = {"value": wl.n / med, "unit": UNIT, "cores": threads, "kind": kind,
           "sample": f"{len(times)} passes over the {wl.n}-image batch of '{wl.name}' (median), build {build}, "
                     f"host has {os.cpu_count()} logical cores"}
    # The reference's own build flags (-march=native, setup.py:678) on an AVX-512 host select the
    # header's scalar resize branch: reported beside the hand-written AVX2 branch above.
    if kind == "reference" and flavour != "avx512" and O.ref_available("avx512"):
        try:
            cpu_reference_pass(wl, "avx512", threads)
            ts = [cpu_reference_pass(wl, "avx512", threads) for _ in range(max(3, min(len(times), 10)))]
            res["march_native"] = {"value": wl.n / statistics.median(ts), "unit": UNIT,
                                   "build": "-O3 -mavx2 -mfma -mavx512f/bw/vl/dq -funroll-loops",
                                   "branch": O.ref_branch("avx512")}
        except Exception as e:  # the extra figure must never take the baseline down
            res["march_native"] = {"error": repr(e)}
    return res


def reference_gpu_leg(wl, lib, torch, device, sample=512):
    """The reference's own CUDA kernels, compiled for this GPU from its tree (oracle/_ref), timed
    beside the same contract of this library.  (a) host images -> host float32: its
    crop_resize_normalize_batch against tlb_crop_resize_normalize_batch on the first `sample` images
    of the batch; (b) resident gather + normalize of 1024 x 160x160 from a 20 000-image device
    array: its normalize_resident_gather_batch against tlb_normalize_resident_gather_batch (both
    synchronise before returning).  Returns None when the library was not compiled."""
    from oracle import oracle as O
    from turboloader_b200 import _capi

    rlib = O.ref_cuda()
    if rlib is None or not rlib.tlrefcuda_available():
        return None
    n = min(sample, wl.n)
    images, crops, flips = [], np.zeros((n, 4), np.float32), np.zeros(n, np.int32)
    refs, cps = (_capi.ImageRef * n)(), (_capi.CropParams * n)()
    for i in range(n):
        s_ = int(wl.sel[i]) if wl.sel is not None else i
        w, h = int(wl.sizes[s_, 0]), int(wl.sizes[s_, 1])
        off = int(wl.offsets[s_])
        images.append(wl.src[off:off + w * h * 3].reshape(h, w, 3))
        crops[i] = wl.boxes[i] if wl.boxes is not None else (0, 0, w, h)
        flips[i] = int(wl.flips[i]) if wl.flips is not None else 0
        refs[i].data, refs[i].w, refs[i].h = images[-1].ctypes.data, w, h
        cps[i].x, cps[i].y, cps[i].w, cps[i].h = [float(v) for v in crops[i]]
        cps[i].flip = int(flips[i])
    out = np.empty((n, 3, wl.dst_h, wl.dst_w), np.float32)

    def best(fn, reps=5):
        fn()
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return min(ts)

    t_ref = best(lambda: O.ref_cuda_crop_resize_normalize(images, crops, flips, wl.dst_h, wl.dst_w, wl.mean, wl.std))

    def ours_host():
        rc = lib.tlb_crop_resize_normalize_batch(refs, cps, n, wl.dst_h, wl.dst_w, _capi.f3(wl.mean), _capi.f3(wl.std),
                                                 out.ctypes.data)
        if rc != 0:
            raise RuntimeError(lib.tlb_last_error().decode())

    t_ours = best(ours_host)
    res = {"host_to_host": {"sample": f"first {n} images of '{wl.name}', pageable host memory, float32 NCHW to host",
                            "reference_img_per_s": n / t_ref, "ours_img_per_s": n / t_ours}}

    nsrc, hw, bs = 20000, 160, 1024
    g = torch.Generator(device=device)
    g.manual_seed(7)
    data = torch.randint(0, 256, (nsrc, hw, hw, 3), dtype=torch.uint8, device=device, generator=g)
    sels = [torch.randperm(nsrc, device=device, generator=g)[:bs].contiguous() for _ in range(8)]
    mean = np.asarray(wl.mean, np.float32)
    std = np.asarray(wl.std, np.float32)
    f32p = C.POINTER(C.c_float)

    def loop(fn, reps=40):
        for i in range(4):
            fn(sels[i % 8])
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(reps):
            if not fn(sels[i % 8]):
                raise RuntimeError("resident gather call failed")
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / reps

    t_ref = loop(lambda s_: rlib.tlrefcuda_normalize_resident_gather(data.data_ptr(), s_.data_ptr(), bs, hw, hw,
                                                                     mean.ctypes.data_as(f32p), std.ctypes.data_as(f32p)))
    t_ours = loop(lambda s_: lib.tlb_normalize_resident_gather_batch(data.data_ptr(), s_.data_ptr(), bs, hw, hw,
                                                                     _capi.f3(mean), _capi.f3(std)))
    nbytes = bs * hw * hw * 3 * 5
    res["resident_gather"] = {"sample": f"{bs} x {hw}x{hw} gathered from {nsrc} resident images, float32 NCHW, "
                                        "call + stream synchronise, 40 calls",
                              "reference_img_per_s": bs / t_ref, "ours_img_per_s": bs / t_ours,
                              "reference_GB_per_s": nbytes / t_ref / 1e9, "ours_GB_per_s": nbytes / t_ours / 1e9}
    del data

    # (c) streaming from pinned host memory (dataset larger than device memory): one epoch of 20 000
    # 160x160 images in batches of 1024, 3 slots: its CudaStreamCore (3 worker threads, blocking
    # hand-over) against tlb_stream_* (no threads, blocking hand-over here too for a like-for-like loop).
    ns, bs_s = 20000, 1024
    host = torch.empty((ns, hw, hw, 3), dtype=torch.uint8).pin_memory()
    host.numpy()[...] = np.random.RandomState(3).randint(0, 256, size=(64, hw, hw, 3), dtype=np.uint8)[np.arange(ns) % 64]
    core = rlib.tlrefcuda_stream_create(host.data_ptr(), ns, hw, hw, bs_s, mean.ctypes.data_as(f32p),
                                        std.ctypes.data_as(f32p), 3, 1)
    nn = C.c_int(0)

    def ref_epoch():
        rlib.tlrefcuda_stream_begin_epoch(core)
        got = 0
        while rlib.tlrefcuda_stream_next(core, C.byref(nn)):
            got += nn.value
        return got

    ref_epoch()
    t0 = time.perf_counter()
    got = ref_epoch()
    t_ref = time.perf_counter() - t0
    rlib.tlrefcuda_stream_destroy(core)
    ours = lib.tlb_stream_create(host.data_ptr(), ns, hw, hw, bs_s, _capi.f3(mean), _capi.f3(std), 3, 1, None, 0, 0, 0, 0)
    ptr = C.c_size_t(0)
    n32 = C.c_int32(0)

    def our_epoch():
        lib.tlb_stream_begin_epoch(ours, None)
        tot = 0
        while True:
            lib.tlb_stream_next(ours, C.byref(ptr), C.byref(n32), None)
            if n32.value == 0:
                return tot
            tot += n32.value

    our_epoch()
    t0 = time.perf_counter()
    got2 = our_epoch()
    t_ours = time.perf_counter() - t0
    lib.tlb_stream_destroy(ours)
    res["streaming"] = {"sample": f"one epoch of {ns} x {hw}x{hw} uint8 images from pinned host memory, batch {bs_s}, 3 slots, "
                                  "float32 NCHW on the device, host waits for every batch",
                        "reference_img_per_s": got / t_ref, "ours_img_per_s": got2 / t_ours,
                        "ours_h2d_GB_per_s": got2 * hw * hw * 3 / t_ours / 1e9}
    return res


def video_leg(torch, device, stream, peak, steps=30):
    """Fused YUV 4:2:0 clip assembly: 8 clips x 16 NV12 frames of 1280x720 (seeded noise), one crop
    window + flip per clip (area 35-100 % of the frame), -> (128, 3, 224, 224) float32, one launch
    per step.  Algorithmic bytes per frame: 1.5 x crop_w x crop_h read + 3 x 224 x 224 x 4 written.
    Beside it the reference's own clip kernel (one call per clip, as its loader does) on the same
    frames, when it was compiled."""
    from oracle import oracle as O
    from turboloader_b200 import ops

    n_clips, T, W, H, D = 8, 16, 1280, 720, 224
    n = n_clips * T
    g = torch.Generator(device=device)
    g.manual_seed(11)
    sets = []
    for _ in range(3):
        yb = torch.randint(0, 256, (n, H, W), dtype=torch.uint8, device=device, generator=g)
        uv = torch.randint(0, 256, (n, H // 2, W), dtype=torch.uint8, device=device, generator=g)
        out = torch.empty((n, 3, D, D), dtype=torch.float32, device=device)
        sets.append((yb, uv, out))
    rs = np.random.RandomState(5)
    crops = np.zeros((n_clips, 4), np.float32)
    for c in range(n_clips):
        area = rs.uniform(0.35, 1.0)
        cw = int(min(W, round(W * np.sqrt(area))))
        ch = int(min(H, round(H * np.sqrt(area))))
        crops[c] = (rs.randint(0, W - cw + 1), rs.randint(0, H - ch + 1), cw, ch)
    flips = rs.randint(0, 2, n_clips).astype(np.int32)
    rd = float((1.5 * crops[:, 2] * crops[:, 3]).sum() * T)
    wr = float(n * 3 * D * D * 4)

    def ptrs(yb, uv):
        yp = [yb.data_ptr() + i * H * W for i in range(n)]
        cb = [uv.data_ptr() + i * (H // 2) * W for i in range(n)]
        return yp, cb, [p + 1 for p in cb]

    plist = [ptrs(yb, uv) for yb, uv, _ in sets]

    def timed(overlap):
        descs = [ops.make_video_desc(*plist[i], y_stride=W, c_stride=W, c_px_stride=2, src_w=W, src_h=H, out=sets[i][2],
                                     crops=crops, flips=flips, clip_len=T, launch_overlap=overlap) for i in range(3)]
        for i in range(3):
            ops.enqueue_video(descs[i % 3], stream.cuda_stream)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for i in range(steps):
            ops.enqueue_video(descs[i % 3], stream.cuda_stream)
        stop.record(stream)
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / 1e3 / steps

    sec = statistics.median(timed(True) for _ in range(3))       # back-to-back launches overlap head to tail
    sec_ser = statistics.median(timed(False) for _ in range(3))  # every launch behind the previous one
    res = {"workload": f"{n_clips} clips x {T} NV12 frames {W}x{H} -> {D}x{D} f32, per-clip crop window + flip",
           "frames_per_s": n / sec, "GB_per_s": (rd + wr) / sec / 1e9, "frac_of_peak": (rd + wr) / sec / 1e9 / peak,
           "serialized": {"frames_per_s": n / sec_ser, "frac_of_peak": (rd + wr) / sec_ser / 1e9 / peak},
           "launch_overlap": "on (TLB_FLAG_LAUNCH_OVERLAP per call; tables in the kernel parameters)",
           "algorithmic_bytes_per_launch": rd + wr, "kernel": "yuv420_kernel", "launches_per_step": 1}
    if O.ref_cuda() is not None:
        yp, cb, cr = plist[0]

        def ref_step():
            for c in range(n_clips):
                sl = slice(c * T, (c + 1) * T)
                O.ref_cuda_video(yp[sl], cb[sl], cr[sl], W, W, 2, W, H, D, D, (0.485, 0.456, 0.406), (0.229, 0.224, 0.225),
                                 crop=crops[c], flip=bool(flips[c]))

        ref_step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(5):
            ref_step()
        torch.cuda.synchronize()
        res["reference_gpu_frames_per_s"] = n * 5 / (time.perf_counter() - t0)
    return res


# ---- main ----------------------------------------------------------------------------------

def bench_config(wl, seed):
    """The ``config`` object: identical for both arms, so that their lines describe one workload."""
    return {"workload": wl.name, "batch_per_gpu": wl.n, "dst": [wl.dst_h, wl.dst_w],
            "out": f"{wl.dtype} {'NHWC' if wl.channels_last else 'NCHW'}", "seed": int(seed),
            "sharding": "disjoint shard per rank, no collective"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = make_host_workload(args.workload if args.workload in ("variable_rrc", "fixed_resize", "highres_nhwc")
                            else "variable_rrc", args.seed, 1)[0]
    from oracle import oracle as O

    flavour, kind = pick_cpu_flavour()
    threads = O.ref_threads(flavour) if kind == "reference" else 1
    for _ in range(max(1, min(args.warmup, 3))):
        cpu_reference_pass(wl, flavour, threads)
    steps = max(1, min(args.steps, 200))
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_reference_pass(wl, flavour, threads)
    dt = time.perf_counter() - t0
    val = steps * wl.n / dt
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * dt / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": bench_config(wl, args.seed),
            "note": "reference CPU fused path (resize_bilinear_simd + deinterleave_hwc_to_chw_f32 on its own "
                    "parallel_for), one host, rank 0 only",
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": kind,
                             "sample": f"each step = one pass over the {wl.n}-image batch, flavour {flavour}"},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def time_steps(batches, lib, stream, steps, warmup, torch, barrier):
    sp = C.c_void_p(stream.cuda_stream)
    for i in range(warmup):
        batches[i % len(batches)].launch(lib, sp)
    torch.cuda.synchronize()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for i in range(steps):
        batches[i % len(batches)].launch(lib, sp)
    stop.record(stream)
    torch.cuda.synchronize()
    barrier()
    return start.elapsed_time(stop) / 1e3


def time_steps_repeated(batches, lib, stream, steps, warmup, torch, barrier, repeats=5):
    """The K-step loop `repeats` times (a step stays one batch); returns the list of seconds."""
    out = [time_steps(batches, lib, stream, steps, warmup, torch, barrier)]
    for _ in range(repeats - 1):
        out.append(time_steps(batches, lib, stream, steps, 0, torch, barrier))
    return out


def _cpulist(text):
    out = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        out.update(range(int(lo), int(hi or lo) + 1))
    return out


def gpu_numa_node(torch, index):
    """NUMA node the GPU's PCIe slot hangs off (sysfs), or None when the host does not say."""
    try:
        pr = torch.cuda.get_device_properties(index)
        addr = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{addr}/numa_node") as f:
            node = int(f.read().strip())
        return node if node >= 0 else None
    except Exception:
        return None


def rank_cores(rank, world, torch=None):
    """A disjoint set of host cores for this rank.  When the host tells which NUMA node each GPU
    is attached to, a rank gets cores of ITS GPU's node (split among the ranks that share the
    node), so that the pinned buffers it allocates and fills afterwards are local to the PCIe root
    its GPU reads them through; otherwise the allowed cores are split into `world` equal blocks.
    Returns (cores, numa node or None)."""
    allowed = sorted(os.sched_getaffinity(0))
    per = max(1, len(allowed) // world)
    fallback = allowed[rank * per:(rank + 1) * per] or allowed
    if torch is None:
        return fallback, None
    try:
        nodes = [gpu_numa_node(torch, r) for r in range(world)]
        if any(n is None for n in nodes):
            return fallback, None
        chosen = {}
        for node in sorted(set(nodes)):
            with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
                local = sorted(_cpulist(f.read()) & set(allowed))
            sharers = [r for r in range(world) if nodes[r] == node]
            share = len(local) // len(sharers)
            if share < 1:
                return fallback, None
            for i, r in enumerate(sharers):
                chosen[r] = local[i * share:(i + 1) * share]
        return chosen[rank], nodes[rank]
    except Exception:
        return fallback, None


def sharded_scaling_leg(args, lib, torch, device, stream, rank, world, dist, barrier, peak, epochs=7):
    """The 8-GPU sharded scaling configuration at this world size: a global set of 32,768 uint8
    256x256x3 images (uniform noise) split into contiguous per-rank shards by the package's own
    sharding functions, batches of 1024, RandomResizedCrop boxes (scale (0.08, 1)) and flips keyed by
    the GLOBAL index, -> 224x224 bf16 NCHW.  Each rank keeps only its shard in HBM and transforms
    it batch by batch with no collective; the epoch is timed on the device, max over ranks.  Pixels
    of global image g come from a generator seeded with (seed, g // 1024), so a sample's bytes do
    not depend on the world size.  After the timed region one rank-local batch is compared with the
    CPU oracle, bit for bit."""
    import turboloader_b200 as t
    from turboloader_b200 import synthetic as S

    total, batch, src, dst = 32768, 1024, 256, 224
    shard = t.shard_indices("contiguous", total, world, rank)
    order = t.direct_order(total, False, args.seed, 0, world > 1, rank, world)
    if not np.array_equal(shard, order):
        raise SystemExit("bench.py: shard_indices and direct_order disagree")
    boxes_all, flips_all = S.config5_params(args.seed, total, src)
    blocks = shard.reshape(-1, batch)
    sizes = np.tile(np.array([[src, src]], np.int32), (batch, 1))
    outs = [torch.empty((batch, 3, dst, dst), dtype=torch.bfloat16, device=device) for _ in range(3)]
    batches = []
    for i, glob in enumerate(blocks):
        g = torch.Generator(device=device)
        g.manual_seed(int(args.seed) * 1_000_003 + int(glob[0]) // batch)
        data = torch.randint(0, 256, (batch, src, src, 3), dtype=torch.uint8, device=device, generator=g)
        wl = S.Workload("sharded_scaling", np.empty(0, np.uint8), np.empty(0, np.int64), sizes, batch, dst, dst,
                        boxes=boxes_all[glob].copy(), flips=flips_all[glob].copy(), dtype="bf16", uniform_hw=(src, src),
                        notes={"global_indices": glob})
        b = DeviceBatch(wl, device, src=data.view(-1))
        b.out = outs[i % 3]
        b.desc.out = b.out.data_ptr()
        b.set_overlap(True)
        batches.append(b)
    sp = C.c_void_p(stream.cuda_stream)
    secs = []
    for e in range(epochs + 1):  # the first epoch is the warm-up
        torch.cuda.synchronize()
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for b in batches:
            b.launch(lib, sp)
        stop.record(stream)
        torch.cuda.synchronize()
        tt = torch.tensor([start.elapsed_time(stop) / 1e3], dtype=torch.float64, device=device)
        if dist is not None:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        if e > 0:
            secs.append(float(tt.item()))
    for b in batches:
        if int(b.status.item()) != 0:
            raise SystemExit("bench.py: device status word is non-zero (sharded_scaling)")
    # parity, outside the timing: this rank's batch `pick` against the CPU oracle
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import expected
    pick = rank % len(batches)
    b = batches[pick]
    b.set_overlap(False)
    b.launch(lib, sp)
    torch.cuda.synchronize()
    wl = b.wl
    wl.src = b.src.cpu().numpy()
    wl.offsets = np.arange(batch, dtype=np.int64) * (src * src * 3)
    got = b.out.view(torch.int16).cpu().numpy().view(np.uint16)
    exact = bool(np.array_equal(got, expected(wl)))
    flag = torch.tensor([1 if exact else 0], dtype=torch.int32, device=device)
    if dist is not None:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag.item()) != 1:
        raise SystemExit("bench.py: sharded_scaling output differs from the CPU oracle")
    med = statistics.median(secs)
    r, w = wl.algorithmic_bytes()
    per_rank_gbs = (r + w) * len(batches) / med / 1e9
    return {"workload": "32,768 x 256x256x3 uint8 split by tlb_shard_indices(contiguous) == tlb_direct_order, batch 1024, "
                        "RRC(0.08,1) boxes + flips keyed by the global index, -> 224x224 bf16 NCHW",
            "img_per_s": total / med, "epoch_ms_median": 1e3 * med, "epoch_ms_min": 1e3 * min(secs),
            "epoch_ms_max": 1e3 * max(secs), "epochs_timed": len(secs), "batches_per_rank": len(batches),
            "per_rank_GB_per_s": per_rank_gbs, "per_rank_frac_of_peak": per_rank_gbs / peak,
            "timing": "CUDA events around each rank's epoch, max over ranks, median over epochs",
            "parity": f"bit-exact against the CPU oracle on every rank (rank r checked its batch r % {len(batches)})"}


def loader_epoch_leg(args, torch, device, peak, n_images):
    """The product API on the resident-epoch configuration: CudaResidentLoader iterated over one
    whole epoch (batches of 1024 gathered through the shuffled order, centre crop 144 -> 128, flips,
    bf16 NCHW + indices), CUDA events around the epoch on the consumer's stream."""
    import turboloader_b200 as t

    g = torch.Generator(device=device)
    g.manual_seed(args.seed + 3)
    data = torch.randint(0, 256, (n_images, 160, 160, 3), dtype=torch.uint8, device=device, generator=g)
    ld = t.CudaResidentLoader.from_array(data, batch_size=1024, shuffle=True, seed=args.seed, return_indices=True,
                                         crop_size=144, output_size=128, hflip_prob=0.5, dtype=torch.bfloat16,
                                         drop_last=True)
    stream = torch.cuda.current_stream()
    times = []
    for ep in range(8):  # the first epoch warms up; median of the other seven
        ld.set_epoch(ep)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record(stream)
        nb = 0
        for x, idx in ld:
            nb += 1
        stop.record(stream)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        if ep > 0:
            times.append(max(start.elapsed_time(stop) / 1e3, wall))
    if ld.device_status() != 0:
        raise SystemExit("bench.py: device status word is non-zero (loader_epoch)")
    med = statistics.median(times)
    per_img = 144 * 144 * 3 + 8 + 1 + 3 * 128 * 128 * 2 + 8
    n = nb * 1024
    del data
    return {"api": "for x, idx in CudaResidentLoader(...)", "images": n_images, "batches": nb, "img_per_s": n / med,
            "GB_per_s": n * per_img / med / 1e9, "frac_of_peak": n * per_img / med / 1e9 / peak,
            "epochs_timed": len(times), "timing": "max(CUDA events on the consumer stream, host wall clock) per epoch, median"}


def direct_loader_leg(args, torch, device, peak, n_images=32768):
    """The product API of the variable-size route (what DataLoader(image_size=224, train_aug=True)
    runs): DirectBatchLoader over a device-resident store of 256x256 images, epoch order from
    tlb_direct_order, RandomResizedCrop rects and flips from tlb_pick_crops, -> 224x224 bf16 NCHW,
    batches of 1024; CUDA events around the epoch on the consumer's stream."""
    import turboloader_b200 as t

    g = torch.Generator(device=device)
    g.manual_seed(args.seed + 5)
    store = torch.randint(0, 256, (n_images * 256 * 256 * 3,), dtype=torch.uint8, device=device, generator=g)
    offsets = np.arange(n_images, dtype=np.int64) * (256 * 256 * 3)
    sizes = np.tile(np.array([[256, 256]], np.int32), (n_images, 1))
    ld = t.DirectBatchLoader((store, offsets, sizes), 1024, 224, 224, mean=(0.485, 0.456, 0.406), std=(0.229, 0.224, 0.225),
                             shuffle=True, seed=args.seed, train_aug=True, dtype=torch.bfloat16)
    stream = torch.cuda.current_stream()
    times, read = [], 0
    for ep in range(5):
        ld.set_epoch(ep)
        boxes, _ = ld.epoch_crops(ep)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record(stream)
        nb = 0
        for x, meta in ld:
            nb += 1
        stop.record(stream)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        if ep > 0:
            times.append(max(start.elapsed_time(stop) / 1e3, wall))
            read = int((boxes[:, 2].astype(np.int64) * boxes[:, 3] * 3).sum())
    if ld.device_status() != 0:
        raise SystemExit("bench.py: device status word is non-zero (direct_loader_epoch)")
    med = statistics.median(times)
    total = read + n_images * (8 + 16 + 1 + 16 + 3 * 224 * 224 * 2)
    del store
    return {"api": "for x, meta in DirectBatchLoader(..., train_aug=True)", "images": n_images, "batches": nb,
            "img_per_s": n_images / med, "GB_per_s": total / med / 1e9, "frac_of_peak": total / med / 1e9 / peak,
            "epochs_timed": len(times), "timing": "max(CUDA events on the consumer stream, host wall clock) per epoch, median"}


def identity_leg(lib, torch, device, stream, peak, barrier, seed, dtypes=("f32", "bf16")):
    """The identity-size case of the resident loader (gather -> flip -> normalize -> layout/dtype, the
    reference's normalize_gather_kernel operation): 1024 x 160x160 gathered from 20,000 resident
    images, fp32 and bf16 NCHW."""
    from turboloader_b200 import synthetic as S

    n_ds, hw, bs = 20000, 160, 1024
    g = torch.Generator(device=device)
    g.manual_seed(seed + 5)
    data = torch.randint(0, 256, (n_ds, hw, hw, 3), dtype=torch.uint8, device=device, generator=g)
    res = {}
    for dt in dtypes:
        batches = []
        for b in range(3):
            sel = np.random.default_rng([seed, b]).permutation(n_ds)[:bs].astype(np.int64)
            wl = S.Workload("identity_gather", np.empty(0, np.uint8), np.empty(0, np.int64),
                            np.tile(np.array([[hw, hw]], np.int32), (n_ds, 1)), bs, hw, hw, sel=sel,
                            flips=(np.random.default_rng([seed, b, 1]).random(bs) < 0.5).astype(np.uint8), dtype=dt,
                            uniform_hw=(hw, hw))
            batches.append(DeviceBatch(wl, device, src=data.view(-1)))
        esz = 4 if dt == "f32" else 2
        nbytes = bs * (hw * hw * 3 * (1 + esz) + 8 + 1 + 8)
        for on in (True, False):  # back-to-back launches overlapping head to tail, then every launch serialized
            for b in batches:
                b.set_overlap(on)
            s = statistics.median(time_steps_repeated(batches, lib, stream, 50, 5, torch, barrier, repeats=3))
            fig = {"img_per_s": 50 * bs / s, "GB_per_s": nbytes / (s / 50) / 1e9, "frac_of_peak": nbytes / (s / 50) / 1e9 / peak}
            if on:
                res[dt] = fig
            else:
                res[dt]["serialized"] = fig
    res["kernel"] = "normalize_copy_kernel"
    res["workload"] = f"{bs} x {hw}x{hw} gathered from {n_ds} resident images, flips, NCHW"
    del data
    return res


def e2e_steps(wl_sets, lib, stream, steps, warmup, torch, device):
    """Host images (pinned) -> device batch through tlb_crop_resize_normalize_to_device."""
    from turboloader_b200 import _capi

    prepared = []
    for wl in wl_sets:
        pinned = torch.from_numpy(np.ascontiguousarray(wl.src)).pin_memory()
        base = pinned.data_ptr()
        n = wl.n
        refs = (_capi.ImageRef * n)()
        crops = (_capi.CropParams * n)()
        for i in range(n):
            s = int(wl.sel[i]) if wl.sel is not None else i
            refs[i].data = base + int(wl.offsets[s])
            refs[i].w, refs[i].h = int(wl.sizes[s, 0]), int(wl.sizes[s, 1])
            x, y, w, h = (wl.boxes[i] if wl.boxes is not None else (0, 0, refs[i].w, refs[i].h))
            crops[i].x, crops[i].y, crops[i].w, crops[i].h = float(x), float(y), float(w), float(h)
            crops[i].flip = int(wl.flips[i]) if wl.flips is not None else 0
        tdt = torch.float32 if wl.dtype == "f32" else torch.bfloat16
        out = torch.empty((n, 3, wl.dst_h, wl.dst_w), dtype=tdt, device=device)
        prepared.append((wl, pinned, refs, crops, out))
    status = torch.zeros(1, dtype=torch.int32, device=device)
    status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
    sp = C.c_void_p(stream.cuda_stream)

    def step(i):
        wl, _, refs, crops, out = prepared[i % len(prepared)]
        rc = lib.tlb_crop_resize_normalize_to_device(
            refs, crops, wl.n, wl.dst_h, wl.dst_w, _capi.f3(wl.mean), _capi.f3(wl.std), int(wl.normalize_01),
            out.data_ptr(), _capi.TLB_F32 if wl.dtype == "f32" else _capi.TLB_BF16,
            _capi.TLB_NHWC if wl.channels_last else _capi.TLB_NCHW, status.data_ptr(), sp)
        if rc != 0:
            raise RuntimeError(lib.tlb_last_error().decode())
        status_host.copy_(status, non_blocking=True)  # the step's result word comes back to the host
        stream.synchronize()
        if int(status_host.item()) != 0:
            raise RuntimeError("device status word is non-zero")

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record(stream)
    for i in range(steps):
        step(i)
    stop.record(stream)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    dev_s = start.elapsed_time(stop) / 1e3
    wl = prepared[0][0]
    wh = wl.crop_wh()
    h2d = int((((wh[:, 0] * wh[:, 1] * 3) + 15) // 16 * 16).sum()) + wl.n * 33
    return max(wall, dev_s), h2d, 4


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="variable_rrc", choices=WORKLOADS)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--sets", type=int, default=3, help="distinct input/output sets cycled through")
    ap.add_argument("--repeats", type=int, default=5, help="times the K-step loop is timed (median reported)")
    ap.add_argument("--no-extras", action="store_true", help="skip e2e, CPU baseline and the other workloads")
    ap.add_argument("--resident-images", type=int, default=100_000,
                    help="dataset size of the resident_epoch workload (smaller for profiler captures)")
    ap.add_argument("--video-only", action="store_true",
                    help="run only the YUV 4:2:0 clip leg and print its JSON (used for profiling that kernel)")
    ap.add_argument("--identity-only", nargs="?", const="both", default=None, choices=["both", "f32", "bf16"],
                    help="run only the identity-size gather leg and print its JSON (used for profiling that kernel)")
    ap.add_argument("--e2e-only", action="store_true",
                    help="run only the host-image end-to-end leg and print its JSON (used for profiling the gather kernel)")
    ap.add_argument("--antialias", action="store_true", help="set the descriptor's antialias flag on the workload")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch

    from turboloader_b200 import _capi, ops

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cores = None
    numa_node = None
    all_cores = os.sched_getaffinity(0)
    if world > 1:
        # Every rank feeds its GPU from its own block of host cores.
        try:
            cores, numa_node = rank_cores(local_rank, world, torch)
            os.sched_setaffinity(0, cores)
        except OSError:
            cores = None
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if dist is not None:
            dist.barrier()

    if not ops.cuda_available():
        raise SystemExit("bench.py: the C-ABI library did not find an sm_100 device (no fallback exists)")
    lib = _capi.load()
    stream = torch.cuda.current_stream()
    peak, peak_src = measured_peak_gbs()
    if args.video_only:
        print(json.dumps(video_leg(torch, device, stream, peak, steps=max(3, min(args.steps, 30)))))
        return
    if args.identity_only:
        dts = ("f32", "bf16") if args.identity_only == "both" else (args.identity_only,)
        print(json.dumps(identity_leg(lib, torch, device, stream, peak, barrier, args.seed, dtypes=dts)))
        return
    if args.e2e_only:
        hs = make_host_workload(args.workload, args.seed, 2)
        es, h2d, d2h = e2e_steps(hs, lib, stream, max(3, min(args.steps, 20)), 3, torch, device)
        print(json.dumps({"img_per_s": max(3, min(args.steps, 20)) * hs[0].n / es, "h2d_bytes_per_step": h2d}))
        return
    sampler = ClockSampler(local_rank)
    sampler.start()

    # Every rank owns a disjoint shard: its data are generated from a rank-specific seed.
    seed = args.seed + 100_003 * rank
    batches = make_device_batches(args.workload, seed, device, args.sets, args.resident_images)
    # The timed stream carries nothing but this library's launches, one batch after another, each
    # into its own output set: the condition under which consecutive launches may overlap.
    for b in batches:
        b.set_overlap(True)
        if args.antialias:
            b.desc.antialias = 1
    wl = batches[0].wl
    launches0 = ops.launch_count()
    sampler.sample()
    secs_all = time_steps_repeated(batches, lib, stream, args.steps, args.warmup, torch, barrier, repeats=args.repeats)
    sampler.sample()
    launches = (ops.launch_count() - launches0 - args.warmup) // max(1, args.repeats)
    for b in batches:
        if int(b.status.item()) != 0:
            raise SystemExit("bench.py: device status word is non-zero")
    t = torch.tensor(secs_all, dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    secs_max_all = [float(v) for v in t.tolist()]
    secs_max = statistics.median(secs_max_all)
    secs = statistics.median(secs_all)
    value = world * args.steps * wl.n / secs_max

    rd, wr = wl.algorithmic_bytes()
    achieved = (rd + wr) / (secs / args.steps) / 1e9
    cfg = bench_config(wl, args.seed)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * secs_max / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 arithmetic, %s output" % wl.dtype, "data": "synthetic",
        "config": cfg,
        "timing": {"repeats": args.repeats, "value_is": "median over repeats of the K-step loop (max over ranks each)",
                   "img_per_s_min": world * args.steps * wl.n / max(secs_max_all),
                   "img_per_s_max": world * args.steps * wl.n / min(secs_max_all),
                   "launch_overlap": "on (TLB_FLAG_LAUNCH_OVERLAP per call): back-to-back batches overlap head to "
                                     "tail; the figure with every launch serialized is under 'serialized'",
                   "l2": f"per-step traffic {(rd + wr) / 1e6:.0f} MB exceeds the 126 MB L2; {args.sets} distinct "
                         "input/output sets are cycled"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": ncu_traffic(("antialias_" if args.antialias else "") + wl.name), "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": rd + wr,
                     "kernel": "antialias_pair_kernel" if args.antialias else "fused_transform_kernel"},
        "gpu_launches": int(launches),
    }
    if cores is not None:
        line["host_cores_per_rank"] = len(cores)

    host_sets = None
    e_steps = max(3, min(args.steps, 20))
    if not args.no_extras:
        for b in batches:
            b.set_overlap(False)
        s_ser = statistics.median(time_steps_repeated(batches, lib, stream, args.steps, args.warmup, torch, barrier,
                                                      repeats=max(1, min(args.repeats, 3))))
        for b in batches:
            b.set_overlap(True)
        line["serialized"] = {"value": args.steps * wl.n / s_ser, "unit": UNIT,
                              "GB_per_s": (rd + wr) / (s_ser / args.steps) / 1e9,
                              "frac_of_peak": (rd + wr) / (s_ser / args.steps) / 1e9 / peak, "per": "rank"}
    if not args.no_extras and args.workload in ("variable_rrc", "fixed_resize", "highres_nhwc"):
        host_sets = [b.wl for b in batches]
        path = ("tlb_crop_resize_normalize_to_device: pinned host pixels -> the fused kernel pulls the crop rows "
                "over PCIe itself (no staging copy); status word read back")
        if world == 1:
            es, h2d, d2h = e2e_steps(host_sets, lib, stream, e_steps, 3, torch, device)
            line["e2e"] = {"value": e_steps * wl.n / es, "unit": UNIT, "h2d_bytes_per_step": h2d,
                           "d2h_bytes_per_step": d2h, "steps": e_steps, "h2d_GB_per_s": e_steps * h2d / es / 1e9,
                           "path": path}
        else:
            # Every rank feeds its own GPU from its own pinned host shard: first one rank at a time
            # (what one host-to-device path can do alone), then all together (what the host can feed).
            alone = torch.zeros(world, dtype=torch.float64, device=device)
            for r in range(world):
                barrier()
                if r == rank:
                    es1, h2d, d2h = e2e_steps(host_sets, lib, stream, e_steps, 3, torch, device)
                    alone[r] = e_steps * h2d / es1 / 1e9
            dist.all_reduce(alone, op=dist.ReduceOp.SUM)
            barrier()
            es, h2d, d2h = e2e_steps(host_sets, lib, stream, e_steps, 3, torch, device)
            te = torch.tensor([es], dtype=torch.float64, device=device)
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
            tog = torch.zeros(world, dtype=torch.float64, device=device)
            tog[rank] = e_steps * h2d / es / 1e9
            dist.all_reduce(tog, op=dist.ReduceOp.SUM)
            line["e2e"] = {"value": world * e_steps * wl.n / float(te.item()), "unit": UNIT, "h2d_bytes_per_step": h2d,
                           "d2h_bytes_per_step": d2h, "steps": e_steps, "path": path,
                           "h2d_GB_per_s_per_rank_alone": [round(float(v), 2) for v in alone.tolist()],
                           "h2d_GB_per_s_per_rank_together": [round(float(v), 2) for v in tog.tolist()],
                           "host_cores_per_rank": len(cores) if cores else None,
                           "numa_node_of_rank0": numa_node,
                           "note": "no collective is involved: the ranks share the host's memory system and PCIe "
                                   "root ports; compare each rank's rate alone with its rate when all ranks run"}
        if rank == 0:
            # The CPU baseline uses every host core (its worker threads are created here, after the
            # rank's own core block has been lifted), while the other ranks wait.
            try:
                os.sched_setaffinity(0, all_cores)
                line["cpu_baseline"] = cpu_baseline(host_sets[0])
            finally:
                if cores is not None:
                    os.sched_setaffinity(0, cores)
    # The sharded scaling configuration runs at EVERY world size, 1 included.
    if not args.no_extras:
        del batches
        torch.cuda.empty_cache()
        line["sharded_scaling"] = sharded_scaling_leg(args, lib, torch, device, stream, rank, world, dist, barrier, peak)
        torch.cuda.empty_cache()

    if rank == 0 and world == 1 and not args.no_extras:
        if host_sets is not None:
            try:
                rg = reference_gpu_leg(host_sets[0], lib, torch, device)
            except Exception as e:  # the comparison leg must never take the bench line down
                rg = {"error": repr(e)}
            if rg is not None:
                line["reference_gpu"] = rg
            try:
                line["video_clip"] = video_leg(torch, device, stream, peak)
            except Exception as e:
                line["video_clip"] = {"error": repr(e)}
        others = {}
        for name in WORKLOADS:
            if name in (args.workload, "sharded_scaling"):
                continue
            torch.cuda.empty_cache()
            bb = make_device_batches(name, seed, device, 3)
            for b in bb:
                b.set_overlap(True)
            s = statistics.median(time_steps_repeated(bb, lib, stream, 50, 5, torch, barrier, repeats=3))
            r, w = bb[0].wl.algorithmic_bytes()
            for b in bb:
                b.set_overlap(False)
            s1 = statistics.median(time_steps_repeated(bb, lib, stream, 50, 5, torch, barrier, repeats=3))
            others[name] = {"img_per_s": 50 * bb[0].wl.n / s, "GB_per_s": (r + w) / (s / 50) / 1e9,
                            "frac_of_peak": (r + w) / (s / 50) / 1e9 / peak, "batch": bb[0].wl.n,
                            "frac_of_peak_serialized": (r + w) / (s1 / 50) / 1e9 / peak}
            del bb
        line["other_workloads"] = others
        try:
            torch.cuda.empty_cache()
            line["identity_gather"] = identity_leg(lib, torch, device, stream, peak, barrier, args.seed)
        except Exception as e:
            line["identity_gather"] = {"error": repr(e)}
        try:
            torch.cuda.empty_cache()
            line["loader_epoch"] = loader_epoch_leg(args, torch, device, peak, args.resident_images)
            if "resident_epoch" in others:
                line["loader_epoch"]["vs_raw_launch_loop"] = line["loader_epoch"]["img_per_s"] / others["resident_epoch"]["img_per_s"]
        except Exception as e:
            line["loader_epoch"] = {"error": repr(e)}
        try:
            torch.cuda.empty_cache()
            line["direct_loader_epoch"] = direct_loader_leg(args, torch, device, peak)
            ss = line.get("sharded_scaling") or {}
            if ss.get("img_per_s"):
                line["direct_loader_epoch"]["vs_raw_launch_loop"] = line["direct_loader_epoch"]["img_per_s"] / ss["img_per_s"]
        except Exception as e:
            line["direct_loader_epoch"] = {"error": repr(e)}
        # The opt-in antialiased (triangle filter) resize on the default workload: same inputs, the
        # descriptor's antialias flag set.  Quality path: about twice the arithmetic of the bilinear kernel.
        try:
            torch.cuda.empty_cache()
            bb = make_device_batches(args.workload, seed, device, 2)
            r, w = bb[0].wl.algorithmic_bytes()
            aa = {"workload": args.workload, "kernel": "antialias_pair_kernel",
                  "traffic": ncu_traffic("antialias_" + args.workload)}
            for on in (True, False):  # as `value` (launches overlap head to tail), then every launch serialized
                for b in bb:
                    b.desc.antialias = 1
                    b.set_overlap(on)
                s = time_steps(bb, lib, stream, 20, 3, torch, barrier)
                fig = {"img_per_s": 20 * bb[0].wl.n / s, "GB_per_s": (r + w) / (s / 20) / 1e9,
                       "frac_of_peak": (r + w) / (s / 20) / 1e9 / peak}
                if on:
                    aa.update(fig)
                else:
                    aa["serialized"] = fig
            line["antialias"] = aa
            del bb
        except Exception as e:
            line["antialias"] = {"error": repr(e)}
    sampler.stop()
    line["clocks"] = sampler.summary()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
