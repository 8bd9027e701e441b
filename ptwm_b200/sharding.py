"""Splitting one container across the GPUs of a box.

Tensors are independent, so a rank decodes a contiguous run of records (in
file order) and needs only that byte range of the file on its GPU.  There is
no exchange step; an optional all-gather of the decoded arena serves callers
that want a full replica on every rank.
"""
from __future__ import annotations

from typing import Sequence


def contiguous_shards(costs: Sequence[int], world: int) -> list[range]:
    """Partition items 0..n-1 into `world` contiguous ranges whose summed
    cost is as even as a greedy left-to-right cut makes it: rank r ends at
    the first item where the running cost reaches (r+1)/world of the total."""
    n = len(costs)
    total = sum(costs)
    bounds = [0]
    run = 0
    i = 0
    for r in range(1, world):
        target = total * r / world
        while i < n and run + costs[i] / 2 <= target:
            run += costs[i]
            i += 1
        bounds.append(i)
    bounds.append(n)
    return [range(bounds[r], bounds[r + 1]) for r in range(world)]


def shard_for_rank(infos: Sequence[dict], rank: int, world: int) -> list[int]:
    """Indices of the tensors rank `rank` of `world` decodes.  Cost of a
    tensor = compressed bytes read + decoded bytes written."""
    costs = [int(t["compressed"]) + int(t["orig_size"]) for t in infos]
    return list(contiguous_shards(costs, world)[rank])
