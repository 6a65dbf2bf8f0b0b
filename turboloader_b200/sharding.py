"""Rank -> sample-index rules of TurboLoader's distributed layer, computed by the host
half of the C-ABI library (no GPU involved).

* ``ContiguousSharding`` / ``InterleavedSharding`` / ``HashBasedSharding``:
  src/distributed/sharding_strategies.hpp:150-316
* ``DistributedSampler``: src/distributed/distributed_dataloader.hpp:65-164
* ``direct_order``: DirectBatchCore::build_order, src/pipeline/direct_batch_loader.hpp:116-135

The fused transform path is embarrassingly parallel: every rank transforms the indices
these rules give it from its own GPU's memory, and no collective is involved.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi

CONTIGUOUS, INTERLEAVED, HASH_BASED = 0, 1, 2
_KINDS = {"contiguous": 0, "CONTIGUOUS": 0, "interleaved": 1, "INTERLEAVED": 1, "hash_based": 2, "HASH_BASED": 2}
_i64p = C.POINTER(C.c_int64)


def _kind(kind) -> int:
    if isinstance(kind, str):
        if kind not in _KINDS:
            raise ValueError(f"Unknown sharding type: {kind}")
        return _KINDS[kind]
    return int(kind)


def shard_indices(kind, total_samples: int, world_size: int, rank: int) -> np.ndarray:
    """Indices owned by ``rank`` (int64, ascending)."""
    if world_size <= 0:
        raise ValueError("world_size must be > 0")
    if rank < 0 or rank >= world_size:
        raise ValueError("rank must be < world_size")
    lib = _capi.load()
    out = np.empty(max(int(total_samples), 1), dtype=np.int64)
    k = lib.tlb_shard_indices(_kind(kind), int(total_samples), int(world_size), int(rank),
                              out.ctypes.data_as(_i64p), out.size)
    if k < 0:
        raise ValueError("invalid sharding arguments")
    return out[:k].copy()


class ShardingStrategy:
    """One rank's view of a sharding rule (``size``, ``get_indices``, ``global_index``,
    ``owns_index`` as in sharding_strategies.hpp:33-63)."""

    def __init__(self, kind, total_samples, world_size, rank):
        self.kind = _kind(kind)
        self.total_samples, self.world_size, self.rank = int(total_samples), int(world_size), int(rank)
        self._idx = shard_indices(self.kind, total_samples, world_size, rank)
        self._set = None

    def size(self) -> int:
        return int(self._idx.size)

    def __len__(self) -> int:
        return self.size()

    def get_indices(self) -> np.ndarray:
        return self._idx.copy()

    def global_index(self, local_idx: int) -> int:
        if local_idx < 0 or local_idx >= self._idx.size:
            raise IndexError("local index out of range")
        return int(self._idx[local_idx])

    def owns_index(self, global_idx: int) -> bool:
        if self._set is None:
            self._set = set(self._idx.tolist())
        return int(global_idx) in self._set

    def __iter__(self):
        return iter(self._idx.tolist())


class ShardingCoordinator:
    """All ranks' strategies at once (sharding_strategies.hpp:365-448)."""

    def __init__(self, total_samples, world_size, kind=CONTIGUOUS):
        self.total_samples, self.world_size, self.kind = int(total_samples), int(world_size), _kind(kind)
        self.strategies = [ShardingStrategy(self.kind, total_samples, world_size, r) for r in range(world_size)]

    def get_strategy(self, rank):
        if rank < 0 or rank >= self.world_size:
            raise IndexError("rank out of range")
        return self.strategies[rank]

    def owner_rank(self, global_idx):
        for r, s in enumerate(self.strategies):
            if s.owns_index(global_idx):
                return r
        raise IndexError("global index not owned by any rank")

    def verify_coverage(self) -> bool:
        seen = np.zeros(self.total_samples, dtype=bool)
        for s in self.strategies:
            idx = s.get_indices()
            if idx.size and (idx.max() >= self.total_samples or seen[idx].any()):
                return False
            seen[idx] = True
        return bool(seen.all())

    def get_shard_sizes(self):
        return [s.size() for s in self.strategies]

    def imbalance_ratio(self) -> float:
        sizes = self.get_shard_sizes()
        return float("inf") if min(sizes) == 0 else max(sizes) / min(sizes)


class DistributedSampler:
    """Shuffled, rank-strided sampler with pad-or-drop (distributed_dataloader.hpp:65-164)."""

    def __init__(self, total_samples, world_size=1, rank=0, drop_last=True, seed=42, shuffle=True):
        if world_size < 1:
            raise ValueError("world_size must be >= 1")
        if rank < 0 or rank >= world_size:
            raise ValueError("rank must be in [0, world_size)")
        self.total_samples, self.world_size, self.rank = int(total_samples), int(world_size), int(rank)
        self.drop_last, self.seed, self.shuffle = bool(drop_last), int(seed), bool(shuffle)
        per = total_samples // world_size if drop_last else -(-total_samples // world_size)
        self._per, self._total = per, per * world_size

    def num_samples(self) -> int:
        return self._per

    def total_size(self) -> int:
        return self._total

    def get_indices(self, epoch: int = 0) -> np.ndarray:
        lib = _capi.load()
        out = np.empty(self._per + 1, dtype=np.int64)
        k = lib.tlb_sampler_indices(self.total_samples, self.world_size, self.rank, int(self.shuffle), self.seed,
                                    int(epoch), int(self.drop_last), out.ctypes.data_as(_i64p), out.size)
        if k < 0:
            raise ValueError("invalid sampler arguments")
        return out[:k].copy()


def direct_order(total, shuffle=False, seed=0, epoch=0, distributed=False, rank=0, world_size=1) -> np.ndarray:
    """Epoch order of the direct-batch loader: optional seeded shuffle, then this rank's
    equal-size block (direct_batch_loader.hpp:116-135)."""
    lib = _capi.load()
    out = np.empty(max(int(total), 1), dtype=np.int64)
    k = lib.tlb_direct_order(int(total), int(shuffle), int(seed), int(epoch), int(distributed), int(rank),
                             int(world_size), out.ctypes.data_as(_i64p), out.size)
    if k < 0:
        raise ValueError("invalid order arguments")
    return out[:k].copy()
