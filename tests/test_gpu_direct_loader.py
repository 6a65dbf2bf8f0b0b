"""DataLoader / DirectBatchLoader on the GPU against the reference's own DirectBatchCore: whole
epochs frozen from that class (tests/golden/direct_batch.json, made by executing it unmodified),
the reference's acceptance tests for train_aug (tests/test_train_aug.py:45-110) and for exact
mid-epoch resume (tests/test_state_dict_resume.py:45-63), and sharding across ranks."""
import hashlib
import json
import os
import sys

import numpy as np
import pytest

import turboloader_b200 as t

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_dbc_golden as G  # noqa: E402

pytestmark = pytest.mark.gpu
GOLD = json.load(open(os.path.join(HERE, "golden", "direct_batch.json")))


def _loader(case, rank, **kw):
    return t.DataLoader(arrays=G.epoch_images(case), batch_size=case["batch"], image_size=case["dst"],
                        shuffle=bool(case["shuffle"]), seed=case["seed"], transform=t.ImageNetNormalize(),
                        enable_distributed=case["world"] > 1, world_rank=rank, world_size=case["world"],
                        drop_last=bool(case["drop_last"]), train_aug=bool(case["train_aug"]),
                        antialias=bool(case["antialias"]), channels_last=not case["chw"], **kw)


def _host(x, chw):
    """float32 bytes in the reference's output order (CHW planes, or HWC when chw is off)."""
    x = x if chw else x.permute(0, 2, 3, 1)
    return x.contiguous().cpu().numpy()


def test_whole_epochs_match_the_reference_loader_bit_for_bit():
    for rec in GOLD["epochs"]:
        dl = _loader(rec, rec["rank"])
        dl.set_epoch(rec["epoch"])
        assert len(dl) == len(rec["batches"]), rec["name"]
        n = 0
        for (x, meta), want in zip(dl, rec["batches"]):
            assert x.is_cuda and x.shape[1:] == (3, rec["dst"], rec["dst"])
            assert meta["indices"].tolist() == want["indices"] and meta["batch_size"] == len(want["indices"])
            assert hashlib.sha256(_host(x, rec["chw"]).tobytes()).hexdigest() == want["sha256"], (rec["name"], n)
            n += 1
        assert n == len(rec["batches"])
        assert dl._loader.device_status() == 0


def test_exact_midepoch_resume_with_train_aug():
    case = dict(n=48, lo=40, hi=90, dst=32, batch=8, shuffle=1, seed=11, epoch=2, world=1, train_aug=1, antialias=0,
                drop_last=0, chw=1)
    ref_loader = _loader(case, 0)
    ref_loader.set_epoch(2)
    ref = [(x.cpu().numpy().copy(), m["indices"].tolist()) for x, m in ref_loader]
    src = _loader(case, 0)
    src.set_epoch(2)
    it = iter(src)
    got = [next(it), next(it)]
    sd = src.state_dict()
    assert sd["epoch"] == 2 and sd["batches_served"] == 2
    del it
    dst = _loader(case, 0)
    dst.load_state_dict(sd)
    tail = [(x.cpu().numpy().copy(), m["indices"].tolist()) for x, m in dst]
    assert len(got) + len(tail) == len(ref) == 6
    for (xr, ir), (xt, it_) in zip(ref[2:], tail):
        assert ir == it_ and np.array_equal(xr, xt)


def _gradient_images(n=64, src=128):
    y, x = np.mgrid[0:src, 0:src]
    img = np.stack([x * 255 // (src - 1), y * 255 // (src - 1), np.full_like(x, 128)], axis=-1).astype(np.uint8)
    return [img] * n


def _crop_stats(batch):
    out = []
    for im in batch:  # CHW in [0,1]
        r, g = im[0], im[1]
        flipped = bool(r[:, 0].mean() > r[:, -1].mean())
        rr = r[:, ::-1] if flipped else r
        x0, x1 = float(rr[:, 0].mean()), float(rr[:, -1].mean())
        y0, y1 = float(g[0, :].mean()), float(g[-1, :].mean())
        cw, ch = max(x1 - x0, 1e-3), max(y1 - y0, 1e-3)
        out.append((cw * ch, cw / ch, flipped))
    return out


def _aug_loader(seed=0, hflip=0.5):
    return t.DataLoader(arrays=_gradient_images(), batch_size=64, image_size=64, shuffle=False, seed=seed,
                        train_aug=True, hflip_prob=hflip)


def test_crop_distribution_recovered_from_a_gradient_image():
    scales, ratios, flips = [], [], []
    loader = _aug_loader()
    for epoch in range(6):  # 384 samples
        loader.set_epoch(epoch)
        for im, _m in loader:
            for s, r, f in _crop_stats(im.cpu().numpy()):
                scales.append(s)
                ratios.append(r)
                flips.append(f)
    scales, ratios = np.array(scales), np.array(ratios)
    assert scales.min() > 0.05 and scales.max() <= 1.02, (scales.min(), scales.max())
    assert 0.45 < scales.mean() < 0.65, scales.mean()
    assert ratios.min() > 0.70 and ratios.max() < 1.40, (ratios.min(), ratios.max())
    assert abs(np.log(ratios).mean()) < 0.06
    assert 0.40 < np.mean(flips) < 0.60


def test_train_aug_determinism_and_flip_direction():
    a = _aug_loader(seed=7)
    a.set_epoch(3)
    b1 = next(iter(a))[0].cpu().numpy().copy()
    a.set_epoch(3)
    b2 = next(iter(a))[0].cpu().numpy().copy()
    a.set_epoch(4)
    b3 = next(iter(a))[0].cpu().numpy().copy()
    assert np.array_equal(b1, b2) and not np.array_equal(b1, b3)
    none = _crop_stats(next(iter(_aug_loader(hflip=0.0)))[0].cpu().numpy())
    all_ = _crop_stats(next(iter(_aug_loader(hflip=1.0)))[0].cpu().numpy())
    assert not any(f for _s, _r, f in none) and all(f for _s, _r, f in all_)


def test_ranks_partition_the_epoch():
    """enable_distributed: the ranks' epochs are disjoint equal blocks of the single-rank epoch order,
    and a sample gets the same pixels whichever rank serves it (its crop depends on seed, epoch and
    the sample index only)."""
    case = dict(n=45, lo=30, hi=70, dst=24, batch=5, shuffle=1, seed=21, epoch=1, world=1, train_aug=1, antialias=0,
                drop_last=0, chw=1)
    one = _loader(case, 0)
    one.set_epoch(1)
    whole = {}
    order = []
    for x, m in one:
        xs = x.cpu().numpy()
        for i, s in enumerate(m["indices"].tolist()):
            whole[s] = xs[i].copy()
            order.append(s)
    seen = []
    for r in range(4):
        dl = _loader(dict(case, world=4), r)
        dl.set_epoch(1)
        mine = []
        for x, m in dl:
            xs = x.cpu().numpy()
            for i, s in enumerate(m["indices"].tolist()):
                assert np.array_equal(xs[i], whole[s])
                mine.append(s)
        assert mine == order[r * 11:(r + 1) * 11]  # 45 // 4 = 11 per rank, the tail is dropped
        seen += mine
    assert len(set(seen)) == 44


def test_store_already_on_the_device_gives_the_same_batches():
    """The packed store may be a uint8 tensor that already lives on the GPU (no upload); two epochs
    with train_aug must equal the ones served from the same store given as a host array."""
    import torch
    rs = np.random.RandomState(5)
    sizes = rs.randint(30, 90, size=(37, 2)).astype(np.int32)
    nbytes = sizes[:, 0].astype(np.int64) * sizes[:, 1] * 3
    offsets = np.concatenate([[0], np.cumsum(nbytes)[:-1]]).astype(np.int64)
    packed = rs.randint(0, 256, size=int(nbytes.sum()), dtype=np.uint8)
    kw = dict(mean=(0.485, 0.456, 0.406), std=(0.229, 0.224, 0.225), shuffle=True, seed=11, train_aug=True)
    host = t.DirectBatchLoader((packed, offsets, sizes), 8, 32, 40, **kw)
    dev = t.DirectBatchLoader((torch.from_numpy(packed).cuda(), offsets, sizes), 8, 32, 40, **kw)
    for ep in range(2):
        host.set_epoch(ep)
        dev.set_epoch(ep)
        a = [(x.clone(), m["indices"]) for x, m in host]
        b = [(x.clone(), m["indices"]) for x, m in dev]
        assert len(a) == len(b) == 5
        for (xa, ia), (xb, ib) in zip(a, b):
            assert np.array_equal(ia, ib) and torch.equal(xa, xb)
    assert host.device_status() == 0 and dev.device_status() == 0
