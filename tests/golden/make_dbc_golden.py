"""Generates tests/golden/direct_batch.json from the reference's own DirectBatchCore
(src/pipeline/direct_batch_loader.hpp), compiled in place and unmodified by `make -C oracle refdbc`
(its libjpeg wrapper replaced by a stand-in that reads pre-decoded pixels).  Run where the
reference tree is present:

    python tests/golden/make_dbc_golden.py

Contents:
  sampler   rects and flips drawn by DirectBatchCore::pick_crop (:141-178) for seeded sizes/indices
  order     epoch orders built by DirectBatchCore::build_order (:116-135)
  epochs    whole epochs through begin_epoch / acquire_batch / fill_batch / process_one (:85-113,
            :189-290): per batch the sample indices and the sha256 of the float32 output
Inputs come from the version-stable np.random.RandomState, so the tests can rebuild them.
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import oracle as O  # noqa: E402

MEAN = (0.485, 0.456, 0.406)
STD = (0.229, 0.224, 0.225)

SAMPLER_CASES = [dict(seed=0, epoch=0, hflip_prob=0.5, n=48), dict(seed=42, epoch=3, hflip_prob=0.5, n=48),
                 dict(seed=7, epoch=11, hflip_prob=0.0, n=24), dict(seed=123456, epoch=1, hflip_prob=1.0, n=24),
                 dict(seed=2147483647, epoch=2, hflip_prob=0.3, n=24)]
ORDER_CASES = [dict(total=100, world=4, shuffle=1, seed=42, epoch=2), dict(total=103, world=4, shuffle=1, seed=42, epoch=2),
               dict(total=10, world=1, shuffle=1, seed=42, epoch=2), dict(total=10, world=2, shuffle=0, seed=42, epoch=2),
               dict(total=37, world=3, shuffle=1, seed=3, epoch=1)]
EPOCH_CASES = [
    dict(name="train_aug_shuffle", n=37, lo=40, hi=120, dst=32, batch=8, shuffle=1, seed=5, epoch=2, world=1,
         train_aug=1, antialias=0, drop_last=0, chw=1),
    dict(name="train_aug_two_ranks", n=41, lo=30, hi=90, dst=48, batch=6, shuffle=1, seed=9, epoch=1, world=2,
         train_aug=1, antialias=0, drop_last=1, chw=1),
    dict(name="resize_only_hwc", n=19, lo=50, hi=100, dst=40, batch=5, shuffle=0, seed=1, epoch=0, world=1,
         train_aug=0, antialias=0, drop_last=0, chw=0),
    dict(name="train_aug_antialias", n=16, lo=60, hi=160, dst=32, batch=8, shuffle=1, seed=3, epoch=4, world=1,
         train_aug=1, antialias=1, drop_last=0, chw=1),
]


def sampler_inputs(case):
    rs = np.random.RandomState(case["seed"] % 65536 + 17 * case["epoch"])
    n = case["n"]
    sizes = np.stack([rs.randint(1, 700, n), rs.randint(1, 700, n)], 1).astype(np.int32)
    q = n // 4
    sizes[:q, 0] = rs.randint(1, 20, q)          # tall and narrow: reaches the central-crop fallback
    sizes[:q, 1] = rs.randint(200, 2000, q)
    sizes[q:2 * q, 1] = rs.randint(1, 20, q)     # wide and flat
    sizes[q:2 * q, 0] = rs.randint(200, 2000, q)
    idx = rs.randint(0, 2 ** 31 - 1, n).astype(np.int64) * 977
    return sizes, idx


def epoch_images(case):
    rs = np.random.RandomState(1000 + case["seed"])
    return [rs.randint(0, 256, size=(rs.randint(case["lo"], case["hi"] + 1), rs.randint(case["lo"], case["hi"] + 1), 3),
                       dtype=np.uint8) for _ in range(case["n"])]


def main():
    if not O.build_ref_dbc():
        raise SystemExit("reference tree not found: cannot build oracle/_ref/libtl_ref_dbc.so")
    tiny = [np.zeros((2, 2, 3), np.uint8)] * 4
    gold = {"sampler": [], "order": [], "epochs": []}
    for case in SAMPLER_CASES:
        core = O.RefDirectBatchCore(tiny, 2, 2, 2, seed=case["seed"], train_aug=True, hflip_prob=case["hflip_prob"])
        core.begin_epoch(case["epoch"])
        sizes, idx = sampler_inputs(case)
        gold["sampler"].append(dict(case, rects=core.pick_crops(sizes, idx).tolist()))
    for case in ORDER_CASES:
        imgs = [np.zeros((1, 1, 3), np.uint8)] * case["total"]
        for r in range(case["world"]):
            core = O.RefDirectBatchCore(imgs, 4, 1, 1, shuffle=bool(case["shuffle"]), seed=case["seed"],
                                        distributed=case["world"] > 1, world_rank=r, world_size=case["world"])
            core.begin_epoch(case["epoch"])
            gold["order"].append(dict(case, rank=r, indices=core.order().tolist()))
    for case in EPOCH_CASES:
        imgs = epoch_images(case)
        for r in range(case["world"]):
            core = O.RefDirectBatchCore(imgs, case["batch"], case["dst"], case["dst"], chw=bool(case["chw"]), mean=MEAN,
                                        std=STD, shuffle=bool(case["shuffle"]), seed=case["seed"],
                                        distributed=case["world"] > 1, world_rank=r, world_size=case["world"],
                                        drop_last=bool(case["drop_last"]), antialias=bool(case["antialias"]),
                                        train_aug=bool(case["train_aug"]))
            core.begin_epoch(case["epoch"])
            batches = []
            while True:
                b = core.next()
                if b is None:
                    break
                batches.append({"indices": b[0].tolist(), "sha256": hashlib.sha256(b[1].tobytes()).hexdigest()})
            assert core.decode_failures() == 0
            gold["epochs"].append(dict(case, rank=r, batches=batches))
    with open(os.path.join(HERE, "direct_batch.json"), "w") as f:
        json.dump(gold, f)
    print("written", os.path.join(HERE, "direct_batch.json"))


if __name__ == "__main__":
    main()
