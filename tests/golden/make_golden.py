"""Regenerates the golden vectors in this directory from the REFERENCE ITSELF: the TurboLoader
headers compiled in place by ``make -C oracle ref`` (flavour ``parity``: -O2 -mavx2
-ffp-contract=off).  Needs the reference tree; the committed outputs do not.

    python tests/golden/make_golden.py

Inputs come from ``np.random.RandomState`` (a frozen, version-stable stream), so the tests
can rebuild them without storing megabytes of pixels.

Files written:
  resize_cases.json   sha256 of the uint8 result of resize_bilinear_simd for the size cases of
                      the reference's tests/test_simd_bilinear.cpp:111-251 and a few more
  fused_small.npz     full fp32 outputs of the fused crop/flip/resize/normalize replay
                      (direct_batch_loader.hpp:219-243) on small ragged inputs
  fused_hashes.json   sha256 of fused outputs at config-like shapes
  antialias_hashes.json  the same pipeline with DirectBatchCore's antialias option
                      (resize_triangle_antialias) on
  sharding.json       index lists of the reference sharding rules, sampler and epoch order
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle as O  # noqa: E402

RESIZE_CASES = [(224, 224, 112, 112), (112, 112, 224, 224), (320, 240, 224, 224), (100, 100, 127, 97), (8, 8, 16, 16),
                (3840, 2160, 224, 224), (64, 64, 64, 64), (100, 1, 224, 1), (1, 100, 1, 224), (256, 256, 224, 224),
                (144, 144, 128, 128), (499, 200, 300, 31), (1, 1, 5, 7)]
MEAN = (0.485, 0.456, 0.406)
STD = (0.229, 0.224, 0.225)


def rs_image(seed, h, w):
    return np.random.RandomState(seed).randint(0, 256, size=(h, w, 3), dtype=np.uint8)


def fused_case(seed, n, lo, hi, dst_h, dst_w, with_sel):
    """Ragged images, boxes touching borders, mixed flips; all drawn from RandomState(seed)."""
    rs = np.random.RandomState(seed)
    hs = rs.randint(lo, hi + 1, size=n)
    ws = rs.randint(lo, hi + 1, size=n)
    imgs = [rs.randint(0, 256, size=(int(h), int(w), 3), dtype=np.uint8) for h, w in zip(hs, ws)]
    sizes = np.array([(w, h) for h, w in zip(hs, ws)], dtype=np.int32)
    nbytes = sizes[:, 0].astype(np.int64) * sizes[:, 1] * 3
    padded = (nbytes + 15) // 16 * 16
    offsets = np.concatenate([[0], np.cumsum(padded)[:-1]]).astype(np.int64)
    src = np.zeros(int(padded.sum()), dtype=np.uint8)
    for im, o, b in zip(imgs, offsets, nbytes):
        src[o:o + b] = im.reshape(-1)
    m = 2 * n if with_sel else n
    sel = rs.randint(0, n, size=m).astype(np.int64) if with_sel else None
    pick = sel if with_sel else np.arange(n)
    boxes = np.empty((m, 4), dtype=np.int32)
    for k, s in enumerate(pick):
        w, h = sizes[s]
        cw = rs.randint(1, w + 1)
        ch = rs.randint(1, h + 1)
        boxes[k] = (rs.randint(0, w - cw + 1), rs.randint(0, h - ch + 1), cw, ch)
    boxes[0] = (0, 0, sizes[pick[0]][0], sizes[pick[0]][1])  # one full-image box
    flips = rs.randint(0, 2, size=m).astype(np.uint8)
    return dict(src=src, offsets=offsets, sizes=sizes, sel=sel, boxes=boxes, flips=flips, dst_h=dst_h, dst_w=dst_w)


def run_ref(c, mean=MEAN, std=STD, n01=True, antialias=False):
    return O.fused_batch(c["src"], c["offsets"], c["sizes"], c["sel"], c["boxes"], c["flips"], c["dst_h"], c["dst_w"],
                         mean, std, n01, impl="ref-parity", antialias=antialias)


FUSED_SMALL = [dict(seed=101, n=5, lo=9, hi=40, dst_h=12, dst_w=20, with_sel=False),
               dict(seed=102, n=4, lo=1, hi=6, dst_h=7, dst_w=5, with_sel=True),
               dict(seed=103, n=3, lo=30, hi=64, dst_h=33, dst_w=17, with_sel=True)]
FUSED_HASHED = [dict(seed=201, n=6, lo=200, hi=500, dst_h=224, dst_w=224, with_sel=False),
                dict(seed=202, n=8, lo=160, hi=160, dst_h=128, dst_w=128, with_sel=True),
                dict(seed=203, n=2, lo=512, hi=512, dst_h=384, dst_w=384, with_sel=False)]


ANTIALIAS_HASHED = [dict(seed=301, n=5, lo=60, hi=260, dst_h=48, dst_w=64, with_sel=False),
                    dict(seed=302, n=4, lo=300, hi=420, dst_h=24, dst_w=24, with_sel=True),
                    dict(seed=303, n=4, lo=20, hi=40, dst_h=56, dst_w=40, with_sel=False)]


def main():
    if not O.build_ref():
        raise SystemExit("reference tree not found: golden vectors can only be regenerated next to it")
    out = {}
    for i, (sw, sh, dw, dh) in enumerate(RESIZE_CASES):
        img = rs_image(1000 + i, sh, sw)
        res = O.resize_bilinear_u8(img, dh, dw, impl="ref-parity")
        out[f"{sw}x{sh}->{dw}x{dh}"] = {"seed": 1000 + i, "sha256": hashlib.sha256(res.tobytes()).hexdigest()}
    with open(os.path.join(HERE, "resize_cases.json"), "w") as f:
        json.dump(out, f, indent=1)

    small = {}
    for j, spec in enumerate(FUSED_SMALL):
        c = fused_case(**spec)
        small[f"case{j}_out01"] = run_ref(c)
        small[f"case{j}_out255"] = run_ref(c, tuple(m * 255 for m in MEAN), tuple(s * 255 for s in STD), False)
        small[f"case{j}_spec"] = np.array(json.dumps(spec))
    np.savez_compressed(os.path.join(HERE, "fused_small.npz"), **small)

    hashes = {}
    for spec in FUSED_HASHED:
        c = fused_case(**spec)
        hashes[json.dumps(spec, sort_keys=True)] = hashlib.sha256(run_ref(c).tobytes()).hexdigest()
    with open(os.path.join(HERE, "fused_hashes.json"), "w") as f:
        json.dump(hashes, f, indent=1)

    hashes = {}
    for spec in ANTIALIAS_HASHED:
        c = fused_case(**spec)
        hashes[json.dumps(spec, sort_keys=True)] = hashlib.sha256(run_ref(c, antialias=True).tobytes()).hexdigest()
    with open(os.path.join(HERE, "antialias_hashes.json"), "w") as f:
        json.dump(hashes, f, indent=1)

    sh = {"shard": [], "sampler": [], "order": []}
    for kind in (0, 1, 2):
        for total, world in [(100, 4), (103, 4), (7, 3), (5, 8), (32768, 8)]:
            for r in range(world):
                idx = O.ref_shard_indices(kind, total, world, r)
                rec = {"kind": kind, "total": total, "world": world, "rank": r, "size": int(idx.size)}
                if total <= 103:
                    rec["indices"] = idx.tolist()
                else:
                    rec["sha256"] = hashlib.sha256(idx.tobytes()).hexdigest()
                sh["shard"].append(rec)
    for total, world, shuffle, drop in [(100, 4, 1, 1), (103, 4, 1, 0), (103, 4, 0, 0), (10, 3, 1, 1), (1, 1, 1, 1)]:
        for r in range(world):
            for ep in (0, 3):
                idx = O.ref_sampler_indices(total, world, r, shuffle, 42, ep, drop)
                sh["sampler"].append({"total": total, "world": world, "rank": r, "shuffle": shuffle, "seed": 42,
                                      "epoch": ep, "drop_last": drop, "indices": idx.tolist()})
    for total, world, shuffle in [(100, 4, 1), (103, 4, 1), (10, 1, 1), (10, 2, 0)]:
        for r in range(world):
            idx = O.ref_direct_order(total, shuffle, 42, 2, int(world > 1), r, world)
            sh["order"].append({"total": total, "world": world, "rank": r, "shuffle": shuffle, "seed": 42, "epoch": 2,
                                "indices": idx.tolist()})
    with open(os.path.join(HERE, "sharding.json"), "w") as f:
        json.dump(sh, f)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
