"""Row-shard geometry of a multi-GPU run.

Same contract as the reference's ``compute_shard_layout`` / ``ShardLayout``
(src/coresets/cuda/multi/layout.py:8-50): ``N_global // world_size`` rows per rank, the
remainder on the LAST rank, contiguous ranges, empty shards legal.
"""
from __future__ import annotations

from bisect import bisect_right
from dataclasses import dataclass
from itertools import accumulate
from typing import List, Tuple


def compute_shard_layout(N_global: int, world_size: int) -> Tuple[List[int], List[int]]:
    """Return ``(sizes, offsets)`` per rank."""
    if world_size <= 0:
        raise ValueError(f"world_size must be positive, got {world_size}")
    base, rem = divmod(N_global, world_size)
    sizes = [base] * (world_size - 1) + [base + rem]
    offsets = [0, *accumulate(sizes[:-1])]
    return sizes, offsets


@dataclass(frozen=True)
class ShardLayout:
    rank: int
    world_size: int
    sizes: List[int]
    offsets: List[int]

    @property
    def shard_offset(self) -> int:
        return self.offsets[self.rank]

    @property
    def N_shard(self) -> int:
        return self.sizes[self.rank]

    @property
    def N_global(self) -> int:
        return sum(self.sizes)

    def owner_of(self, global_idx: int) -> int:
        """Rank whose range holds ``global_idx``; indices past the end map to the last rank
        (as the reference's linear scan does, layout.py:41-46).  Empty shards never own a row:
        among ranks that start at the same offset the last one wins, which is the one whose
        range is non-empty (or the last rank)."""
        r = bisect_right(self.offsets, global_idx) - 1
        return min(max(r, 0), self.world_size - 1)

    def to_local(self, global_idx: int) -> int:
        """No bounds check: the caller must own ``global_idx``."""
        return global_idx - self.shard_offset
