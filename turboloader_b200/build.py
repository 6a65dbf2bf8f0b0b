"""In-tree build of the C-ABI shared library (``turboloader_b200/libturboloader_b200.so``).

The library is compiled for sm_100a only.  nvcc cross-compiles without a GPU, so this
runs on a CPU-only machine; the built file sits next to the package sources.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.environ.get("TLB_LIB") or os.path.join(HERE, "libturboloader_b200.so")
SOURCES = ["fused_transform.cu", "host_gather.cu", "video_yuv420.cu", "antialias.cu", "normalize_copy.cu", "capi.cu", "sharding.cpp"]
HEADERS = ["fused_params.h", "host_gather.h", "video_params.h", "antialias_params.h", os.path.join("..", "..", "include", "turboloader_b200.h")]

NVCC_FLAGS = [
    "-std=c++20", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-O2",
    "--fmad=false", *[f"-D{m}" for m in os.environ.get("TLB_DEFINES", "").split() if m],  # belt and braces: every fp32 op in the kernels is an explicit _rn intrinsic anyway
    "-shared", "-cudart", "static",
]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libturboloader_b200.so")
    cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []),
           *[os.path.join(CSRC, s) for s in SOURCES], "-o", LIB + ".tmp"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libturboloader_b200.so")
    if verbose:
        sys.stderr.write(res.stderr)
    os.replace(LIB + ".tmp", LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
