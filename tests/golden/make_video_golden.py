"""Writes tests/golden/video_golden.npz: outputs of the reference's OWN CUDA video kernels
(TurboLoader src/cuda/cuda_transforms.cu:143-268, compiled in place by `make -C oracle refcuda`
into oracle/_ref/libtl_ref_cuda_nofma.so, i.e. without FMA contraction) for seeded frames.

Needs a CUDA device and the compiled reference library, so it runs on a GPU machine:

    python tests/golden/make_video_golden.py [output.npz]

Frames come from tests/test_video_oracle.py:make_frame (numpy RandomState, version-stable); only the
parameters and the outputs are stored."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import oracle as O  # noqa: E402
from test_video_oracle import MEAN, STD, make_frame, to_nv12  # noqa: E402
from turboloader_b200.cuda_loader import _CudaArray  # noqa: E402

# seed, h, w, dh, dw, nv12, bt709, use_crop, flip, smooth ; crop
CASES = [
    ((1, 96, 128, 48, 64, 0, 0, 0, 0, 1), None),
    ((2, 96, 128, 67, 81, 1, 0, 0, 0, 0), None),
    ((3, 90, 122, 40, 56, 0, 1, 1, 1, 0), (10.0, 7.0, 71.0, 53.0)),
    ((4, 64, 80, 50, 70, 1, 1, 1, 0, 1), (0.5, 2.25, 70.0, 55.5)),
    ((5, 48, 64, 90, 120, 0, 0, 0, 0, 1), None),
    ((6, 50, 66, 20, 30, 1, 0, 1, 1, 0), (0.0, 0.0, 66.0, 50.0)),
]


def main(path):
    out = {"n_cases": np.int64(len(CASES))}
    for i, (params, crop) in enumerate(CASES):
        seed, h, w, dh, dw, nv12, bt709, use_crop, flip, smooth = params
        y, cb, cr = make_frame(seed, h, w, smooth=bool(smooth))
        dy = torch.from_numpy(y).cuda()
        if nv12:
            uv = torch.from_numpy(to_nv12(cb, cr)).cuda()
            cbp, crp, cs, cpx = uv.data_ptr(), uv.data_ptr() + 1, uv.shape[1], 2
        else:
            dcb, dcr = torch.from_numpy(cb).cuda(), torch.from_numpy(cr).cuda()
            cbp, crp, cs, cpx = dcb.data_ptr(), dcr.data_ptr(), cb.shape[1], 1
        p = O.ref_cuda_video([dy.data_ptr()], [cbp], [crp], w, cs, cpx, w, h, dh, dw, MEAN, STD,
                             crop=crop if use_crop else None, flip=bool(flip), bt709=bool(bt709), nofma=True)
        res = torch.as_tensor(_CudaArray(p, (1, 3, dh, dw)), device="cuda").cpu().numpy()[0]
        out[f"case{i}_params"] = np.array(params, dtype=np.int64)
        out[f"case{i}_crop"] = np.array(crop if crop else (0, 0, 0, 0), dtype=np.float32)
        out[f"case{i}_out"] = res.astype(np.float32)
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "video_golden.npz"))
