"""CPU model of the paged KV-cache bookkeeping: free stack, tables, reference counts, fork,
copy-on-write, eviction.  TEST INFRASTRUCTURE ONLY (the checker for libdrkv.so's host side).

Follows the reference where it has code, by file:line of the reference tree:
  free stack  src/memoria/block_pool.cpp:52-74    LIFO; first pops 0,1,2,...; free pushes back
  allocate    src/memoria/cache_manager.cpp:73-106, 306-326
  evict       src/memoria/cache_manager.cpp:118-164, 185-205 (no scorer: oldest allocated first)
and, for what the reference only describes (docs/en/architecture/02-memoria.md:25-26), the rules
this build fixed: fork shares pages (+1 reference each); a write into a page with more than one
reference first moves the sequence onto a fresh copy; release turns pages that reach zero
references into cached pages at the LRU tail (or frees them when discarded); an allocation takes
the free stack first, then the LRU head, then (stream mode) the sequence's own oldest unshared
page.  Pinned against the reference's compiled objects for the single-sequence subset
(tests/test_bookkeeping_vs_reference.py); the fork / copy-on-write / cached-LRU part is
"parity unpinned": nothing in the reference executes it.
"""
from __future__ import annotations

from collections import deque
from typing import List, Optional, Tuple

OK, ERR_INVALID, ERR_EXHAUSTED, ERR_STATE, ERR_CAPACITY = 0, -1, -2, -5, -6
FREE, ACTIVE, CACHED = 0, 1, 2


class Seq:
    def __init__(self, width: int):
        self.len = 0
        self.table = [-1] * width
        self.order = deque()  # logical indices, oldest allocation first (lru_order_)
        self.stored = set()   # logical pages held by the storage tier (BlockLocation::SSD)


class BookModel:
    def __init__(self, max_pages: int, page_size: int, max_seqs: int, row_width: int = 0,
                 stream_evict: bool = False):
        assert max_pages >= 4                                   # block_pool.cpp:31-36
        self.n, self.P = max_pages, page_size
        self.width = row_width or 2 * max_pages                 # cache_manager.cpp:39
        self.stream_evict = stream_evict
        self.free = list(range(max_pages - 1, -1, -1))          # block_pool.cpp:52-55
        self.ref = [0] * max_pages
        self.caller_owned = set()                               # pages handed out by pool_alloc(): only those go back by pool_free()
        self.state = [FREE] * max_pages
        self.lru = deque()                                      # cached pages, oldest release first
        self.seqs: List[Optional[Seq]] = [None] * max_seqs
        self.log: List[Tuple[int, int, int, int]] = []          # (kind, seq, logical, page)
        self.cow: List[Tuple[int, int, int]] = []               # (src, dst, valid slots) device copies
        self.n_cow = 0                                          # pages replaced, with or without a copy
        self.scores = None                                      # {seq: [float per logical page]} once a scorer is attached
        self.tier = False                                       # storage tier attached: own victims are stored, not discarded
        self.swap_ins = []                                      # (seq, logical, page) in order
        self.files = set()                                      # (seq, logical) files the tier holds

    # ---- pool ---------------------------------------------------------------------------
    def _alloc_raw(self) -> int:
        if not self.free:
            return -1                                           # block_pool.cpp:63-69
        p = self.free.pop()
        self.state[p], self.ref[p] = ACTIVE, 1
        return p

    def pool_alloc(self) -> int:
        p = self._alloc_raw()
        if p >= 0:
            self.caller_owned.add(p)
        return p

    def pool_free(self, p: int) -> int:
        if p < 0 or p >= self.n:
            return ERR_INVALID
        if self.state[p] != ACTIVE or p not in self.caller_owned or self.ref[p] != 1:
            return ERR_STATE                                    # not allocated, a sequence's page, or still shared
        self.caller_owned.discard(p)
        self.state[p], self.ref[p] = FREE, 0
        self.free.append(p)                                     # block_pool.cpp:71-74
        return OK

    def _unref(self, p: int, discard: bool):
        self.ref[p] -= 1
        if self.ref[p] > 0:
            return
        if discard:
            self.state[p] = FREE
            self.free.append(p)
        else:
            self.state[p] = CACHED
            self.lru.append(p)

    # ---- eviction -------------------------------------------------------------------------
    def evict_cached(self, n: int) -> int:
        done = 0
        while done < n and self.lru:
            p = self.lru.popleft()
            self.state[p] = FREE
            self.free.append(p)
            self.log.append((0, -1, -1, p))
            done += 1
        return done

    def _retire(self, s: int, pos_in_order: int, may_store: bool) -> None:
        """The victim leaves the allocation order, then is stored (kind 2, cache_manager.cpp:132-141,
        215-241) or discarded (kind 1, cache_manager.cpp:144-147)."""
        seq = self.seqs[s]
        idx = seq.order[pos_in_order]
        p = seq.table[idx]
        del seq.order[pos_in_order]
        stored = self.tier and may_store
        self.ref[p], self.state[p] = 0, FREE
        self.free.append(p)
        seq.table[idx] = -1
        if stored:
            seq.stored.add(idx)
            self.files.add((s, idx))
        else:
            if idx in seq.stored:
                seq.stored.discard(idx)
                self.files.discard((s, idx))
        self.log.append((2 if stored else 1, s, idx, p))

    def _evict_one_of(self, s: int, may_store: bool = True) -> bool:
        seq = self.seqs[s]
        if self.scores is not None:
            # cache_manager.cpp:185-205 + importance_scorer.cu:75-87: lowest score among the resident
            # (and here: unshared) entries, first minimum in allocation order
            best = -1
            for i, idx in enumerate(seq.order):
                p = seq.table[idx]
                if p < 0 or self.ref[p] > 1:
                    continue
                if best < 0 or self.scores[s][idx] < self.scores[s][seq.order[best]]:
                    best = i
            if best >= 0:
                self._retire(s, best, may_store)
                return True
        i = 0
        while i < len(seq.order):
            idx = seq.order[i]
            p = seq.table[idx]
            if p < 0:                                           # hole: dropped, not counted (cache_manager.cpp:129-130)
                del seq.order[i]
                continue
            if self.ref[p] > 1:                                 # shared with a fork: never a victim
                i += 1
                continue
            self._retire(s, i, may_store)
            return True
        return False

    def _live(self, s: int) -> bool:
        return 0 <= s < len(self.seqs) and self.seqs[s] is not None

    def _take(self, s: int, may_store: bool = True) -> int:
        p = self._alloc_raw()
        if p >= 0:
            return p
        if self.lru:
            self.evict_cached(1)
            return self._alloc_raw()
        if self.stream_evict and self._live(s) and self._evict_one_of(s, may_store):   # cache_manager.cpp:310-319
            return self._alloc_raw()
        return -1

    def seq_evict(self, s: int, n: int) -> int:
        if not self._live(s):
            return ERR_STATE
        done = 0
        while done < n and self._evict_one_of(s):
            done += 1
        return done

    def ensure_free(self, s: int, n_free: int) -> int:
        while len(self.free) < n_free:                          # cache_manager.cpp:158-164
            if self.evict_cached(1) == 1:
                continue
            if self._live(s) and self._evict_one_of(s):
                continue
            return 0
        return 1

    # ---- sequences ------------------------------------------------------------------------
    def seq_create(self) -> int:
        for i, s in enumerate(self.seqs):
            if s is None:
                self.seqs[i] = Seq(self.width)
                return i
        return ERR_CAPACITY

    def seq_release(self, s: int, discard: bool = False) -> int:
        if not self._live(s):
            return ERR_STATE
        for p in self.seqs[s].table:
            if p >= 0:
                self._unref(p, discard)
        for idx in self.seqs[s].stored:                         # stored copies go with the sequence
            self.files.discard((s, idx))
        self.seqs[s] = None
        return OK

    def seq_fork(self, parent: int) -> int:
        if not self._live(parent):
            return ERR_STATE
        c = self.seq_create()
        if c < 0:
            return c
        ps, cs = self.seqs[parent], self.seqs[c]
        cs.len = ps.len
        cs.order = deque(ps.order)
        for i, p in enumerate(ps.table):
            if p >= 0:
                cs.table[i] = p
                self.ref[p] += 1
        return c

    def seq_ensure_pos(self, s: int, pos: int) -> int:
        if not self._live(s):
            return ERR_STATE
        if pos < 0:
            return ERR_INVALID
        seq = self.seqs[s]
        idx = pos // self.P
        if idx >= self.width:                                   # cache_manager.cpp:77-81
            return ERR_CAPACITY
        p = seq.table[idx]
        if p >= 0:
            if self.ref[p] == 1:
                return OK                                       # cache_manager.cpp:84-86
            fresh = self._take(s)
            if fresh < 0:
                return ERR_EXHAUSTED
            valid = max(0, min(seq.len - idx * self.P, self.P))
            if valid > 0:
                self.cow.append((p, fresh, valid))
            self.ref[p] -= 1
            seq.table[idx] = fresh
            self.n_cow += 1
            return OK
        if self.tier and idx in seq.stored:
            # swap_block_from_ssd (cache_manager.cpp:243-292): the page for it may cost a victim, which is
            # discarded, never stored
            back = self._take(s, may_store=False)
            if back < 0:
                return ERR_EXHAUSTED
            seq.table[idx] = back
            seq.stored.discard(idx)
            self.files.discard((s, idx))                        # the pool holds the only copy again
            seq.order.append(idx)
            self.swap_ins.append((s, idx, back))
            return OK
        fresh = self._take(s)                                   # cache_manager.cpp:306-326
        if fresh < 0:
            return ERR_EXHAUSTED
        seq.table[idx] = fresh
        seq.order.append(idx)
        return OK

    def seq_ensure_range(self, s: int, pos_start: int, m: int) -> int:
        if not self._live(s):
            return ERR_STATE
        if pos_start < 0:
            return ERR_INVALID
        if m <= 0:
            return OK
        for b in range(pos_start // self.P, (pos_start + m - 1) // self.P + 1):   # cache_manager.cpp:97-106
            rc = self.seq_ensure_pos(s, b * self.P)
            if rc != OK:
                return rc
        return OK

    def seq_reserve(self, s: int, n: int) -> int:
        if not self._live(s):
            return ERR_STATE
        return self.seq_ensure_range(s, self.seqs[s].len, n)

    def seq_set_len(self, s: int, n: int) -> int:
        if not self._live(s):
            return ERR_STATE
        if n < 0 or n > self.width * self.P:
            return ERR_INVALID
        self.seqs[s].len = n
        return OK

    def seq_adopt(self, s: int, pages, n_tokens: int) -> int:
        if not self._live(s):
            return ERR_STATE
        seq = self.seqs[s]
        if seq.len != 0 or seq.order:
            return ERR_STATE
        if len(pages) > self.width or n_tokens < 0 or n_tokens > len(pages) * self.P:
            return ERR_INVALID
        for i, p in enumerate(pages):
            if p < 0 or p >= self.n or p in pages[:i]:
                return ERR_INVALID
            if self.state[p] == FREE:
                return ERR_STATE
        for i, p in enumerate(pages):
            if self.state[p] == CACHED:
                self.lru.remove(p)
                self.state[p] = ACTIVE
            self.ref[p] += 1
            seq.table[i] = p
            seq.order.append(i)
        seq.len = n_tokens
        return OK

    # ---- views ------------------------------------------------------------------------------
    def table(self, s: int):
        return list(self.seqs[s].table)

    def snapshot(self):
        return {"free": list(self.free), "ref": list(self.ref), "lru": list(self.lru),
                "tables": [None if s is None else list(s.table) for s in self.seqs],
                "lens": [None if s is None else s.len for s in self.seqs]}
