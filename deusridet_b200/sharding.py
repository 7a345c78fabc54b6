"""How the path is partitioned across the GPUs of one box (one process per GPU): thin wrappers over the
drkv_shard_* entry points of libdrkv.so, so that a Python driver and a C++ host take the same decisions.

Two partitionings, neither present in the single-GPU reference:
  * independent sequences / decode branches: data parallel, no collective; a fork family (pages
    shared by reference count) stays on one rank;
  * one long sequence: contiguous KV page ranges per rank; every rank attends its own range and
    the per-rank partial (m, l, o) are all-gathered and merged (log-sum-exp combine).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence, Tuple

from . import capi


def _pair(fn, *args) -> Tuple[int, int]:
    a, b = C.c_int(), C.c_int()
    if fn(*args, C.byref(a), C.byref(b)) != 0:
        raise ValueError("bad rank / world / size")
    return a.value, b.value


def page_range_for_rank(n_pages: int, rank: int, world: int) -> Tuple[int, int]:
    """Pages [lo, hi) of a sequence of n_pages that `rank` owns: contiguous, sizes differ by at most one,
    earlier ranks take the larger shares."""
    return _pair(capi.load_library().drkv_shard_page_range, n_pages, rank, world)


def key_range_for_rank(seq_len: int, page_size: int, rank: int, world: int) -> Tuple[int, int]:
    """Keys [begin, end) of a sequence of seq_len tokens that `rank` attends (page-aligned split)."""
    return _pair(capi.load_library().drkv_shard_key_range, seq_len, page_size, rank, world)


def owner_of_position(pos: int, seq_len_after: int, page_size: int, world: int) -> int:
    """Rank whose page range holds token `pos` once the sequence has seq_len_after tokens: the rank
    that appends it."""
    r = capi.load_library().drkv_shard_owner_of_position(pos, seq_len_after, page_size, world)
    if r < 0:
        raise ValueError("position outside the sequence")
    return r


def shard_sequences(costs: Sequence[int], world: int, families: Sequence[int] | None = None) -> List[List[int]]:
    """Assigns sequences to ranks, balancing the summed cost (context length) greedily, largest first.
    families[i] groups sequences that share pages (forks): a family is placed as one unit."""
    n = len(costs)
    c = (C.c_int64 * max(n, 1))(*[int(x) for x in costs])
    fam = None if families is None else (C.c_int32 * max(n, 1))(*[int(x) for x in families])
    out = (C.c_int32 * max(n, 1))()
    if capi.load_library().drkv_shard_sequences(n, c, fam, world, out) != 0:
        raise ValueError("bad world / costs")
    parts: List[List[int]] = [[] for _ in range(world)]
    for i in range(n):
        parts[out[i]].append(i)
    return parts
