"""RandomResizedCrop + flip sampler (host).  Statistical and structural checks in the spirit of
the reference's tests/test_train_aug.py:45-110: scale and ratio ranges, per-epoch determinism,
flip probability, and the clamped-ratio central-crop fallback."""
import numpy as np
import pytest

import turboloader_b200 as t


def test_ranges_and_statistics():
    sizes = np.tile([[320, 240]], (20000, 1))
    boxes, flips = t.pick_crops(42, 0, sizes)
    x, y, w, h = boxes.T
    assert (w > 0).all() and (h > 0).all() and (x >= 0).all() and (y >= 0).all()
    assert (x + w <= 320).all() and (y + h <= 240).all()
    area = w * h / (320 * 240)
    assert area.min() >= 0.075 and area.max() <= 1.0
    assert 0.40 < area.mean() < 0.47          # E[U(0.08,1)] = 0.54, lowered by rejected large crops
    ratio = w / h
    assert ratio.min() > 0.73 and ratio.max() < 1.37
    assert 0.48 < flips.mean() < 0.52
    assert len({tuple(b) for b in boxes}) > 19000  # per-sample seeds give distinct rects


def test_determinism_per_seed_epoch_index():
    sizes = np.tile([[200, 300]], (64, 1))
    a = t.pick_crops(7, 3, sizes)
    b = t.pick_crops(7, 3, sizes)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    assert not np.array_equal(a[0], t.pick_crops(7, 4, sizes)[0])
    assert not np.array_equal(a[0], t.pick_crops(8, 3, sizes)[0])
    # The rect depends on the sample index, not on its position in the call.
    idx = np.array([5, 9, 2], dtype=np.int64)
    sub = t.pick_crops(7, 3, sizes[:3], indices=idx)[0]
    assert np.array_equal(sub, a[0][idx])


def test_fallback_is_the_clamped_central_crop():
    # Extreme aspect ratios exhaust the 10 attempts: central crop at ratio 3/4 or 4/3.
    assert t.pick_crops(1, 0, [[10, 1000]])[0].tolist() == [[0, 493, 10, 13]]
    assert t.pick_crops(1, 0, [[1000, 10]])[0].tolist() == [[493, 0, 13, 10]]
    flips = t.pick_crops(1, 0, np.tile([[10, 1000]], (2000, 1)), hflip_prob=0.25)[1]
    assert 0.2 < flips.mean() < 0.3
    with pytest.raises(ValueError):
        t.pick_crops(1, 0, [[0, 10]])


def test_a_whole_epoch_drawn_on_all_cores_equals_the_serial_draw():
    """Large tables are drawn on several host threads (each sample has its own generator); the result
    must not depend on how the samples were split."""
    import numpy as np
    from turboloader_b200.augment import pick_crops
    rs = np.random.RandomState(3)
    n = 40_000
    sizes = rs.randint(20, 600, size=(n, 2)).astype(np.int32)
    order = rs.permutation(n).astype(np.int64)
    boxes, flips = pick_crops(7, 2, sizes, indices=order, hflip_prob=0.5)
    for i0 in range(0, n, 3000):  # below the threshold at which threads are used
        b, f = pick_crops(7, 2, sizes[i0:i0 + 3000], indices=order[i0:i0 + 3000], hflip_prob=0.5)
        assert np.array_equal(b, boxes[i0:i0 + 3000]) and np.array_equal(f, flips[i0:i0 + 3000])
