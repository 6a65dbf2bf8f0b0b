"""Shard index math of the C-ABI library against the reference's rules: golden index lists
generated from the compiled reference headers, the values its own tests state
(tests/test_sharding_strategies.cpp:19-104, 107-163, 287-336), and the live reference when present."""
import hashlib
import json
import os

import numpy as np
import pytest

import turboloader_b200 as t
from oracle import oracle as O

GOLD = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sharding.json")))


def test_shard_rules_match_golden():
    for rec in GOLD["shard"]:
        idx = t.shard_indices(rec["kind"], rec["total"], rec["world"], rec["rank"])
        assert idx.size == rec["size"]
        if "indices" in rec:
            assert idx.tolist() == rec["indices"]
        else:
            assert hashlib.sha256(idx.tobytes()).hexdigest() == rec["sha256"]


def test_sampler_and_epoch_order_match_golden():
    for rec in GOLD["sampler"]:
        s = t.DistributedSampler(rec["total"], rec["world"], rec["rank"], drop_last=bool(rec["drop_last"]),
                                 seed=rec["seed"], shuffle=bool(rec["shuffle"]))
        assert s.get_indices(rec["epoch"]).tolist() == rec["indices"]
    for rec in GOLD["order"]:
        got = t.direct_order(rec["total"], bool(rec["shuffle"]), rec["seed"], rec["epoch"], rec["world"] > 1, rec["rank"],
                             rec["world"])
        assert got.tolist() == rec["indices"]


def test_contiguous_values_stated_by_the_reference_tests():
    assert [t.ShardingStrategy("contiguous", 100, 4, r).size() for r in range(4)] == [25, 25, 25, 25]
    assert [t.ShardingStrategy("contiguous", 103, 4, r).size() for r in range(4)] == [26, 26, 26, 25]
    s = t.ShardingStrategy("contiguous", 100, 4, 1)
    assert s.get_indices()[0] == 25 and s.get_indices()[-1] == 49 and s.global_index(3) == 28
    assert s.owns_index(25) and not s.owns_index(50)
    with pytest.raises(IndexError):
        s.global_index(25)


def test_interleaved_and_hash_cover_everything_once():
    for kind in ("interleaved", "hash_based", "contiguous"):
        for total, world in [(100, 4), (103, 4), (1000, 7)]:
            c = t.ShardingCoordinator(total, world, kind)
            assert c.verify_coverage()
            assert sum(c.get_shard_sizes()) == total
            assert c.owner_rank(total - 1) in range(world)
    assert t.ShardingStrategy("interleaved", 100, 4, 1).get_indices()[:4].tolist() == [1, 5, 9, 13]
    assert t.ShardingCoordinator(10000, 4, "hash_based").imbalance_ratio() < 1.2


def test_constructor_errors():
    with pytest.raises(ValueError):
        t.ShardingStrategy("contiguous", 10, 0, 0)
    with pytest.raises(ValueError):
        t.ShardingStrategy("contiguous", 10, 2, 2)
    with pytest.raises(ValueError):
        t.ShardingStrategy("zigzag", 10, 2, 0)
    with pytest.raises(ValueError):
        t.DistributedSampler(10, 0, 0)


def test_sampler_determinism_and_epochs():
    a = t.DistributedSampler(100, 4, 2, seed=7).get_indices(1)
    assert np.array_equal(a, t.DistributedSampler(100, 4, 2, seed=7).get_indices(1))
    assert not np.array_equal(a, t.DistributedSampler(100, 4, 2, seed=7).get_indices(2))
    allr = np.concatenate([t.DistributedSampler(100, 4, r, seed=7).get_indices(1) for r in range(4)])
    assert sorted(allr.tolist()) == list(range(100))
    padded = [t.DistributedSampler(103, 4, r, drop_last=False).get_indices(0) for r in range(4)]
    assert all(p.size == 26 for p in padded)


def test_config5_shards_are_equal_blocks():
    for ws in (1, 2, 4, 8):
        for r in range(ws):
            idx = t.shard_indices("contiguous", 32768, ws, r)
            assert idx.size == 32768 // ws and idx[0] == r * (32768 // ws)
            assert np.array_equal(idx, t.direct_order(32768, False, 0, 0, True, r, ws))


@pytest.mark.skipif(not O.ref_available("parity") or O.ref_dbc() is None, reason="compiled reference harness not present")
def test_against_live_reference():
    for kind in (0, 1, 2):
        for total, world in [(0, 2), (1, 1), (17, 5), (4096, 8)]:
            for r in range(world):
                assert np.array_equal(t.shard_indices(kind, total, world, r), O.ref_shard_indices(kind, total, world, r))
    for total, world in [(37, 3), (64, 8)]:
        for r in range(world):
            assert np.array_equal(t.DistributedSampler(total, world, r, drop_last=False, seed=9).get_indices(5),
                                  O.ref_sampler_indices(total, world, r, 1, 9, 5, 0))
            assert np.array_equal(t.direct_order(total, True, 3, 1, True, r, world),
                                  O.ref_direct_order(total, 1, 3, 1, 1, r, world))
