"""The host logic around the fused kernel -- epoch order, batch cursor, RandomResizedCrop + flip
sampler -- and the CPU oracle, checked against the reference's own DirectBatchCore
(src/pipeline/direct_batch_loader.hpp) executed unmodified: frozen outputs in
tests/golden/direct_batch.json (made by tests/golden/make_dbc_golden.py), and the compiled class
itself when oracle/_ref/libtl_ref_dbc.so is present."""
import hashlib
import json
import os
import sys

import numpy as np
import pytest

import turboloader_b200 as t
from oracle import oracle as O
from turboloader_b200 import synthetic as S

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_dbc_golden as G  # noqa: E402

GOLD = json.load(open(os.path.join(HERE, "golden", "direct_batch.json")))


def test_sampler_matches_pick_crop_of_the_reference():
    assert len(GOLD["sampler"]) == len(G.SAMPLER_CASES)
    for rec in GOLD["sampler"]:
        sizes, idx = G.sampler_inputs(rec)
        boxes, flips = t.pick_crops(rec["seed"], rec["epoch"], sizes, idx, rec["hflip_prob"])
        want = np.array(rec["rects"], np.int32)
        assert np.array_equal(boxes, want[:, :4]) and np.array_equal(flips, want[:, 4])
    # the fallback branch (central crop at the clamped ratio) is part of the frozen cases
    fell_back = sum(1 for rec in GOLD["sampler"] for (x, y, w, h, f), (sw, sh) in
                    zip(rec["rects"], G.sampler_inputs(rec)[0]) if (w == sw and x == 0 and 3 * h <= 4 * w + 3 and sh > 2 * h))
    assert fell_back > 0


def test_epoch_order_matches_build_order_of_the_reference():
    for rec in GOLD["order"]:
        got = t.direct_order(rec["total"], bool(rec["shuffle"]), rec["seed"], rec["epoch"], rec["world"] > 1,
                             rec["rank"], rec["world"])
        assert got.tolist() == rec["indices"]


def replay_epoch(case, rank):
    """The package's host logic + the CPU oracle standing in for the kernel: yields
    (indices, float32 batch) like DirectBatchCore's acquire_batch / fill_batch."""
    imgs = G.epoch_images(case)
    src, offsets, sizes = S.pack_images(imgs)
    order = t.direct_order(len(imgs), bool(case["shuffle"]), case["seed"], case["epoch"], case["world"] > 1, rank,
                           case["world"])
    bs = case["batch"]
    for b0 in range(0, len(order), bs):
        idx = order[b0:b0 + bs]
        if case["drop_last"] and len(idx) < bs:
            break
        boxes = flips = None
        if case["train_aug"]:
            boxes, flips = t.pick_crops(case["seed"], case["epoch"], sizes[idx], idx)
        out = O.fused_batch(src, offsets, sizes, idx, boxes, flips, case["dst"], case["dst"], G.MEAN, G.STD,
                            antialias=bool(case["antialias"]))
        yield idx, (out if case["chw"] else O.nchw_to_nhwc(out))


def test_whole_epochs_match_the_reference_loader():
    for rec in GOLD["epochs"]:
        got = list(replay_epoch(rec, rec["rank"]))
        assert len(got) == len(rec["batches"]), rec["name"]
        for (idx, out), want in zip(got, rec["batches"]):
            assert idx.tolist() == want["indices"], rec["name"]
            assert hashlib.sha256(out.tobytes()).hexdigest() == want["sha256"], rec["name"]


@pytest.mark.skipif(O.ref_dbc() is None, reason="compiled DirectBatchCore harness not present")
def test_against_the_live_reference_loader():
    rng = np.random.default_rng(0)
    tiny = [np.zeros((2, 2, 3), np.uint8)] * 4
    for seed, epoch, hp in [(0, 0, 0.5), (42, 3, 0.5), (7, 11, 0.0), (99, 1, 1.0)]:
        core = O.RefDirectBatchCore(tiny, 2, 2, 2, seed=seed, train_aug=True, hflip_prob=hp)
        core.begin_epoch(epoch)
        n = 5000
        sizes = np.stack([rng.integers(1, 700, n), rng.integers(1, 700, n)], 1).astype(np.int32)
        sizes[:300, 0] = rng.integers(1, 20, 300)
        sizes[:300, 1] = rng.integers(200, 2000, 300)
        idx = rng.integers(0, 1 << 40, n)
        ref = core.pick_crops(sizes, idx)
        boxes, flips = t.pick_crops(seed, epoch, sizes, idx, hp)
        assert np.array_equal(boxes, ref[:, :4]) and np.array_equal(flips, ref[:, 4])
    # a fresh epoch case that is not frozen: live class against the replay, including mid-epoch resume
    case = dict(n=23, lo=30, hi=70, dst=24, batch=4, shuffle=1, seed=77, epoch=6, world=1, train_aug=1, antialias=0,
                drop_last=0, chw=1)
    core = O.RefDirectBatchCore(G.epoch_images(case), case["batch"], case["dst"], case["dst"], mean=G.MEAN, std=G.STD,
                                shuffle=True, seed=case["seed"], train_aug=True)
    core.begin_epoch(case["epoch"], start_batch=2)
    got = list(replay_epoch(case, 0))[2:]
    for idx, out in got:
        ridx, rout = core.next()
        assert np.array_equal(idx, ridx) and np.array_equal(out.view(np.uint32), rout.view(np.uint32))
    assert core.next() is None
