"""How the path is partitioned across the GPUs of one box (one process per GPU).

Two partitionings, neither present in the single-GPU reference:
  * independent sequences / decode branches: data parallel, no collective; a fork family (pages
    shared by reference count) stays on one rank;
  * one long sequence: contiguous KV page ranges per rank; every rank attends its own range and
    the per-rank partial (m, l, o) are all-gathered and merged (log-sum-exp combine).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def page_range_for_rank(n_pages: int, rank: int, world: int) -> Tuple[int, int]:
    """Pages [lo, hi) of a sequence of n_pages that `rank` owns: contiguous, sizes differ by at most one,
    earlier ranks take the larger shares."""
    if world <= 0 or not (0 <= rank < world) or n_pages < 0:
        raise ValueError("bad rank / world / page count")
    base, extra = divmod(n_pages, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def key_range_for_rank(seq_len: int, page_size: int, rank: int, world: int) -> Tuple[int, int]:
    """Keys [begin, end) of a sequence of seq_len tokens that `rank` attends (page-aligned split)."""
    n_pages = (seq_len + page_size - 1) // page_size
    lo, hi = page_range_for_rank(n_pages, rank, world)
    return min(lo * page_size, seq_len), min(hi * page_size, seq_len)


def owner_of_position(pos: int, seq_len_after: int, page_size: int, world: int) -> int:
    """Rank whose page range holds token `pos` once the sequence has seq_len_after tokens: the rank
    that appends it."""
    n_pages = (seq_len_after + page_size - 1) // page_size
    page = pos // page_size
    for r in range(world):
        lo, hi = page_range_for_rank(n_pages, r, world)
        if lo <= page < hi:
            return r
    raise ValueError("position outside the sequence")


def shard_sequences(costs: Sequence[int], world: int, families: Sequence[int] | None = None) -> List[List[int]]:
    """Assigns sequences to ranks, balancing the summed cost (context length) greedily, largest first.
    families[i] groups sequences that share pages (forks): a family is placed as one unit."""
    if families is None:
        families = list(range(len(costs)))
    groups = {}
    for i, f in enumerate(families):
        groups.setdefault(f, []).append(i)
    units = sorted(groups.values(), key=lambda idx: (-sum(costs[i] for i in idx), idx[0]))
    loads = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for idx in units:
        r = min(range(world), key=lambda k: (loads[k], k))
        out[r].extend(idx)
        loads[r] += sum(costs[i] for i in idx)
    return [sorted(x) for x in out]
