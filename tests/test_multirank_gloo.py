"""Multi-rank behaviour on CPU (gloo, world size 2): every rank derives its own disjoint shard
from the library's index rules with no data-path collective, per-sample results do not depend
on the world size, and a rank that dies does not block the others (there is nothing to wait on)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, batch, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import turboloader_b200 as t
    from turboloader_b200 import synthetic as S
    from helpers import oracle_f32

    shard = t.shard_indices("contiguous", total, world, rank)
    assert np.array_equal(shard, t.direct_order(total, False, 0, 0, world > 1, rank, world))
    params = S.config5_params(seed=3, total=total, src=32)
    sums = {}
    for b in range(len(shard) // batch):
        wl = S.config5(seed=3, total=total, world=world, rank=rank, batch=batch, batch_index=b, src=32, dst=16,
                       params=params)
        out = oracle_f32(wl)  # stands in for the GPU kernel: same per-sample function of (pixels, box, flip)
        for g, o in zip(wl.notes["global_indices"], out):
            sums[int(g)] = float(np.abs(o).sum())
    # The ONLY communication is this test's own bookkeeping; the data path has none.
    gathered = [None] * world
    dist.all_gather_object(gathered, sorted(sums.items()))
    if rank == 0:
        q.put(gathered)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_shards_disjoint_complete_and_world_size_independent(world):
    total, batch = 24, 4
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, total, batch, q)) for r in range(world)]
    for p in procs:
        p.start()
    gathered = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    keys = [k for part in gathered for k, _ in part]
    assert sorted(keys) == list(range(total)) and len(set(keys)) == total
    # Same per-sample result at world size 1.
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from turboloader_b200 import synthetic as S
    from helpers import oracle_f32
    params = S.config5_params(seed=3, total=total, src=32)
    single = {}
    for b in range(total // batch):
        wl = S.config5(seed=3, total=total, world=1, rank=0, batch=batch, batch_index=b, src=32, dst=16, params=params)
        for g, o in zip(wl.notes["global_indices"], oracle_f32(wl)):
            single[int(g)] = float(np.abs(o).sum())
    multi = {k: v for part in gathered for k, v in part}
    assert multi == single


def _lonely_worker(rank, q):
    sys.path.insert(0, ROOT)
    import turboloader_b200 as t
    if rank == 1:
        os._exit(3)  # this rank dies before doing any work
    shard = t.shard_indices("contiguous", 10, 2, rank)
    q.put(shard.tolist())


def test_a_dead_rank_does_not_block_the_others():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_lonely_worker, args=(r, q)) for r in range(2)]
    for p in procs:
        p.start()
    assert q.get(timeout=60) == [0, 1, 2, 3, 4]
    for p in procs:
        p.join(timeout=30)
    assert procs[0].exitcode == 0 and procs[1].exitcode == 3


def _direct_worker(rank, world, port, total, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import turboloader_b200 as t

    # The host side of DataLoader(enable_distributed=True, shuffle=True, train_aug=True): this rank's
    # block of the shuffled epoch and the crops of its samples.
    sizes = np.stack([40 + np.arange(total) % 17, 50 + np.arange(total) % 23], 1).astype(np.int32)
    order = t.direct_order(total, True, 9, 4, True, rank, world)
    boxes, flips = t.pick_crops(9, 4, sizes[order], indices=order)
    mine = [(int(i), boxes[k].tolist(), int(flips[k])) for k, i in enumerate(order)]
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    if rank == 0:
        q.put(gathered)
    dist.barrier()
    dist.destroy_process_group()


def test_direct_batch_route_union_of_ranks_is_the_single_rank_epoch():
    import turboloader_b200 as t
    world, total = 2, 31
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_direct_worker, args=(r, world, port, total, q)) for r in range(world)]
    for p in procs:
        p.start()
    gathered = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    sizes = np.stack([40 + np.arange(total) % 17, 50 + np.arange(total) % 23], 1).astype(np.int32)
    whole = t.direct_order(total, True, 9, 4, False, 0, 1)
    boxes, flips = t.pick_crops(9, 4, sizes[whole], indices=whole)
    single = {int(i): (boxes[k].tolist(), int(flips[k])) for k, i in enumerate(whole)}
    per = total // world
    seen = []
    for r, part in enumerate(gathered):
        assert [i for i, _, _ in part] == whole[r * per:(r + 1) * per].tolist()  # equal blocks of the same shuffle
        for i, b, f in part:
            assert single[i] == (b, f)  # a sample's crop does not depend on the rank that serves it
        seen += [i for i, _, _ in part]
    assert len(set(seen)) == world * per
