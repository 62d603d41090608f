"""Sharding of sequences over the GPUs of one node.

Sequences are independent on this path (no term of the append or of the attention couples two
sequences), so a GPU owns whole sequences and its cache never crosses NVLink; only the per-sequence
outputs are gathered.  Equal-length batches are split into contiguous blocks; ragged batches are balanced
by total tokens with the longest-processing-time greedy rule.
"""
from __future__ import annotations

import heapq
from typing import List, Sequence


def contiguous_partition(n_seq: int, world: int) -> List[List[int]]:
    """Sequence ids per rank, contiguous blocks whose sizes differ by at most one."""
    base, extra = divmod(n_seq, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append(list(range(start, start + n)))
        start += n
    return out


def lpt_partition(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Greedy LPT: longest sequence first, each to the rank with the fewest tokens so far.

    Deterministic (ties go to the lower rank, equal lengths keep their order); every rank's list is
    sorted by sequence id so that gathered outputs can be put back with one index_copy.
    """
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    heap = [(0, r) for r in range(world)]
    heapq.heapify(heap)
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        load, r = heapq.heappop(heap)
        out[r].append(i)
        heapq.heappush(heap, (load + int(lengths[i]), r))
    for lst in out:
        lst.sort()
    return out


def partition_loads(lengths: Sequence[int], parts: List[List[int]]) -> List[int]:
    return [sum(int(lengths[i]) for i in p) for p in parts]
