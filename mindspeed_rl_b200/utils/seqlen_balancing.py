"""Sequence-length aware partitioning: balanced k-way splits and token-budget micro-batches.

Provides the algorithms the data plane and the training engine rely on (reference:
``mindspeed_rl/utils/seqlen_balancing.py:12-388``):

* ``karmarkar_karp``       -- largest-differencing k-way number partitioning,
* ``heapq_partition``      -- greedy longest-first onto the lightest bin,
* ``get_seqlen_balanced_partitions`` -- validated wrapper returning sorted index lists,
* ``heapq_partition_with_max``       -- greedy bins that open a new bin on overflow,
* ``balanced_bin_packing`` -- best-fit-decreasing under a capacity, then pairwise rebalancing,
* ``rearrange_micro_batches`` -- token-budget micro-batches with the bin count agreed on
  (MAX) across the data-parallel group so every rank runs the same number of micro-steps,
* ``get_reverse_idx``.
"""
from __future__ import annotations

import heapq
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


# ----------------------------------------------------------------------------------------------
# k-way balanced partitioning
# ----------------------------------------------------------------------------------------------
class _Bucket:
    """A multiset of (index, length) with its running sum."""

    __slots__ = ("total", "members")

    def __init__(self, members=None):
        self.members = list(members or [])
        self.total = sum(v for _, v in self.members)

    def absorb(self, other: "_Bucket") -> None:
        self.members.extend(other.members)
        self.total += other.total

    def key(self):
        return (self.total, len(self.members))


class _PartialSolution:
    """k buckets kept sorted by descending sum; ordered in the heap by their spread."""

    def __init__(self, k: int, first=None):
        self.buckets = [_Bucket() for _ in range(k)]
        if first is not None:
            self.buckets[0] = _Bucket([first])
        self._sort()

    def _sort(self):
        self.buckets.sort(key=_Bucket.key, reverse=True)

    @property
    def spread(self) -> int:
        return self.buckets[0].total - self.buckets[-1].total

    def merge(self, other: "_PartialSolution") -> None:
        # largest of one with smallest of the other: cancels the differences
        k = len(self.buckets)
        for i in range(k):
            self.buckets[i].absorb(other.buckets[k - 1 - i])
        self._sort()

    def __lt__(self, other: "_PartialSolution") -> bool:
        # heapq is a min-heap; we want the largest spread first
        if self.spread != other.spread:
            return self.spread > other.spread
        return self.buckets[0].key() > other.buckets[0].key()


def karmarkar_karp(seqlen_list: Sequence[int], k_partitions: int, equal_size: bool) -> List[List[int]]:
    items = sorted(((int(v), i) for i, v in enumerate(seqlen_list)))
    heap: List[_PartialSolution] = []
    if equal_size:
        if len(items) % k_partitions != 0:
            raise ValueError(f"{len(items)} items cannot be split into {k_partitions} equal parts")
        # seed each solution with k items so that every bucket receives exactly one per round
        for off in range(0, len(items), k_partitions):
            sol = _PartialSolution(k_partitions)
            for slot, (v, i) in enumerate(items[off:off + k_partitions]):
                sol.buckets[slot] = _Bucket([(i, v)])
            sol._sort()
            heapq.heappush(heap, sol)
    else:
        for v, i in items:
            heapq.heappush(heap, _PartialSolution(k_partitions, first=(i, v)))
    if not heap:
        return [[] for _ in range(k_partitions)]
    while len(heap) > 1:
        a = heapq.heappop(heap)
        b = heapq.heappop(heap)
        a.merge(b)
        heapq.heappush(heap, a)
    final = heap[0]
    parts = [[i for i, _ in b.members] for b in final.buckets]
    if equal_size:
        size = len(items) // k_partitions
        if any(len(p) != size for p in parts):
            raise RuntimeError("equal-size partitioning failed")
    return parts


def heapq_partition(seqlen_list: Sequence[int], k_partitions: int, equal_size: bool) -> List[List[int]]:
    order = sorted(range(len(seqlen_list)), key=lambda i: (-int(seqlen_list[i]), i))
    cap = len(seqlen_list) // k_partitions if equal_size else None
    if equal_size and len(seqlen_list) % k_partitions != 0:
        raise ValueError("equal_size needs len(seqlen_list) % k_partitions == 0")
    heap = [(0, 0, b) for b in range(k_partitions)]  # (sum, count, bin)
    parts: List[List[int]] = [[] for _ in range(k_partitions)]
    for i in order:
        total, count, b = heapq.heappop(heap)
        parts[b].append(i)
        count += 1
        total += int(seqlen_list[i])
        if cap is None or count < cap:
            heapq.heappush(heap, (total, count, b))
    return parts


def get_seqlen_balanced_partitions(seqlen_list: Sequence[int], k_partitions: int,
                                   equal_size: bool) -> List[List[int]]:
    if len(seqlen_list) < k_partitions:
        raise ValueError(f"{len(seqlen_list)} items < {k_partitions} partitions")
    parts = karmarkar_karp(seqlen_list, k_partitions, equal_size)
    seen = set()
    out = []
    for p in parts:
        if len(p) == 0:
            raise RuntimeError("empty partition")
        seen.update(p)
        out.append(sorted(p))
    if seen != set(range(len(seqlen_list))):
        raise RuntimeError("partitions do not cover every item exactly once")
    return out


# ----------------------------------------------------------------------------------------------
# capacity-bounded packing
# ----------------------------------------------------------------------------------------------
def heapq_partition_with_max(seqlen_list: Sequence[int], k_partitions: int,
                             max_token_len: int) -> List[List[int]]:
    order = sorted(range(len(seqlen_list)), key=lambda i: (-int(seqlen_list[i]), -i))
    heap = [[0, 0, b, []] for b in range(max(k_partitions, 1))]
    next_id = len(heap)
    closed: List[List[int]] = []
    for i in order:
        v = int(seqlen_list[i])
        cur = heapq.heappop(heap)
        if cur[0] + v > max_token_len:
            closed.append(cur[3])
            cur = [0, 0, next_id, []]
            next_id += 1
        cur[0] += v
        cur[1] += 1
        cur[3].append(i)
        heapq.heappush(heap, cur)
    closed.extend(b[3] for b in heap)
    return closed


def balanced_bin_packing(seqlen_list: Sequence[int], max_capacity: int) -> List[List[int]]:
    """Best-fit decreasing into bins of ``max_capacity`` followed by move/swap rebalancing."""
    order = sorted(range(len(seqlen_list)), key=lambda i: -int(seqlen_list[i]))
    bins: List[dict] = []
    for i in order:
        v = int(seqlen_list[i])
        best, slack = None, None
        for b in bins:
            room = max_capacity - b["sum"] - v
            if room >= 0 and (slack is None or room < slack):
                best, slack = b, room
        if best is None:
            best = {"sum": 0, "items": []}
            bins.append(best)
        best["items"].append((i, v))
        best["sum"] += v
    _rebalance(bins, max_capacity)
    return [[i for i, _ in b["items"]] for b in bins]


def _rebalance(bins: List[dict], cap: int, max_rounds: int = 64) -> None:
    for _ in range(max_rounds):
        bins.sort(key=lambda b: b["sum"], reverse=True)
        heavy, light = bins[0], bins[-1]
        gap = heavy["sum"] - light["sum"]
        if gap <= 1:
            return
        moved = False
        for pos, (i, v) in enumerate(sorted(heavy["items"], key=lambda t: t[1])):
            if v < gap and light["sum"] + v <= cap:
                heavy["items"].remove((i, v))
                heavy["sum"] -= v
                light["items"].append((i, v))
                light["sum"] += v
                moved = True
                break
        if moved:
            continue
        for (ih, vh) in heavy["items"]:
            hit = None
            for (il, vl) in light["items"]:
                d = vh - vl
                if 0 < d < gap and light["sum"] + d <= cap:
                    hit = (il, vl)
                    break
            if hit:
                heavy["items"].remove((ih, vh)); light["items"].remove(hit)
                heavy["items"].append(hit); light["items"].append((ih, vh))
                heavy["sum"] -= vh - hit[1]; light["sum"] += vh - hit[1]
                moved = True
                break
        if not moved:
            return


def rearrange_micro_batches(seqlen_list: Sequence[int], max_token_len,
                            dynamic_max_batch_size: Optional[int] = None, dp_group=None,
                            multimodal: bool = False) -> List[List[int]]:
    """Split samples into the fewest micro-batches whose token sum stays under the budget."""
    if multimodal:
        return balanced_bin_packing(seqlen_list, max_token_len)
    total = int(sum(int(v) for v in seqlen_list))
    k = max(1, -(-total // int(max_token_len)))
    k = len(heapq_partition_with_max(seqlen_list, k, int(max_token_len)))
    if dynamic_max_batch_size is not None:
        k = max(k, -(-len(seqlen_list) // int(dynamic_max_batch_size)))
    if dist.is_available() and dist.is_initialized():
        dev = "cuda" if dist.get_backend(dp_group) == "nccl" else "cpu"
        t = torch.tensor([k], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=dp_group)
        k = int(t.item())
    k = min(k, len(seqlen_list)) if len(seqlen_list) else k
    return karmarkar_karp(seqlen_list, k, equal_size=False)


def get_reverse_idx(idx_map: Sequence[int]) -> List[int]:
    rev = [0] * len(idx_map)
    for pos, idx in enumerate(idx_map):
        rev[idx] = pos
    return rev
