"""Host dispatcher for multi-GPU serving: independent engine replicas, no tensor crosses GPUs.

The ragged attention path shards only as whole requests, so scaling out means one engine process
per GPU and a host-side split of the request list.  ``partition_by_tokens`` balances the replicas by
token count (prompt + output budget); every rank can compute the same partition from the same list,
so no communication is needed to agree on it.  ``merge_outputs`` puts per-replica results back in
submission order.
"""
from __future__ import annotations

from typing import Sequence


def partition_by_tokens(costs: Sequence[int], n_parts: int) -> list[list[int]]:
    """Longest-first greedy: each request goes to the replica with the fewest tokens so far.

    Returns, per replica, the indices of its requests in ascending (submission) order.  Deterministic:
    ties go to the lower replica index and equal costs keep submission order.
    """
    if n_parts <= 0:
        raise ValueError("n_parts must be positive")
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    loads, parts = [0] * n_parts, [[] for _ in range(n_parts)]
    for i in order:
        j = min(range(n_parts), key=lambda r: (loads[r], r))
        parts[j].append(i)
        loads[j] += costs[i]
    return [sorted(p) for p in parts]


def merge_outputs(parts: list[list[int]], outputs_per_part: list[list], total: int) -> list:
    """Inverse of the partition: ``outputs_per_part[r][k]`` belongs to request ``parts[r][k]``."""
    merged = [None] * total
    for idx, outs in zip(parts, outputs_per_part):
        if len(idx) != len(outs):
            raise ValueError("a replica returned a different number of results than it was given requests")
        for i, o in zip(idx, outs):
            merged[i] = o
    if any(m is None for m in merged):
        raise ValueError("some requests have no result")
    return merged
