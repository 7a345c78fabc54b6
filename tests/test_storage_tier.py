"""Storage tier bookkeeping on an engine without a device (files are empty markers): which page is
stored or discarded, what comes back on access, what a swap-in may cost, which files exist — against
the Python model of the same rules (oracle/bookkeeping.py) on seeded operation mixes, plus the edge
cases by hand.  The reference's own tier is not run: KVSwapper::drain returns once the queue is empty,
which is before the popped request has been processed, and the completion callback then writes through
a reference to a dead stack variable (kv_swapper.cpp:84-87,155-176, cache_manager.cpp:226-229)."""
import os

import numpy as np
import pytest

from oracle.bookkeeping import BookModel


def _engine(tmp, pages=8, page=16, max_seqs=4, width=24):
    from deusridet_b200 import PagedKVEngine
    e = PagedKVEngine(num_layers=2, num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=page, dtype="bf16",
                      rope_theta=1e6, max_pages=pages, max_seqs=max_seqs, max_pages_per_seq=width, device=-1,
                      stream_evict=True)
    e.tier_enable(str(tmp))
    return e


def _files(tmp):
    return sorted(os.listdir(tmp))


def test_evicted_pages_are_stored_and_come_back(drkv_lib, tmp_path):
    e = _engine(tmp_path)
    try:
        s = e.seq_create()
        assert s == 0
        assert e.ensure_blocks_for_range(s, 0, 6 * 16)
        before = e.table(s).tolist()
        assert e.evict_blocks(s, 2) == 2                          # oldest two: logical 0 and 1
        assert e.table(s)[:2].tolist() == [-1, -1]
        assert e.locations(s)[:7].tolist() == [2, 2, 1, 1, 1, 1, 0]
        assert _files(tmp_path) == ["block_0.kv", "block_1.kv"]   # the reference's naming for row 0
        log = e.evict_log()
        assert log == [(2, 0, 0, before[0]), (2, 0, 1, before[1])]
        st = e.tier_stats()
        assert st["pages_stored"] == 2 and st["swap_outs"] == 2 and st["swap_ins"] == 0
        assert e.free_count() == 4
        # access brings logical 0 back into the page freed last (LIFO) and re-queues it as youngest
        assert e.ensure_blocks_for(s, 5)
        assert e.table(s)[0] == before[1]
        assert e.locations(s)[0] == 1 and e.tier_stats()["swap_ins"] == 1
        assert _files(tmp_path) == ["block_1.kv"]
        assert e.evict_blocks(s, 5) == 5                          # 2,3,4,5 then 0 (youngest)
        assert e.locations(s)[:6].tolist() == [2, 2, 2, 2, 2, 2]
        assert e.tier_stats()["pages_stored"] == 6
    finally:
        e.close()


def test_swap_in_with_an_empty_pool_discards_a_victim(drkv_lib, tmp_path):
    e = _engine(tmp_path, pages=4)
    try:
        s = e.seq_create()
        assert e.ensure_blocks_for_range(s, 0, 4 * 16)
        assert e.evict_blocks(s, 1) == 1                          # logical 0 stored
        assert e.ensure_blocks_for(s, 4 * 16)                     # logical 4 takes the freed page; pool empty again
        e.evict_log(clear=True)
        assert e.ensure_blocks_for(s, 0)                          # swap-in: oldest resident (logical 1) is DISCARDED
        log = e.evict_log()
        assert [(kind, logical) for kind, _, logical, _ in log] == [(1, 1)]
        assert e.locations(s)[:5].tolist() == [1, 0, 1, 1, 1]
        assert _files(tmp_path) == []
    finally:
        e.close()


def test_release_drops_stored_pages_and_forks_see_holes(drkv_lib, tmp_path):
    e = _engine(tmp_path, pages=12)
    try:
        a = e.seq_create()
        b = e.seq_create()
        assert e.ensure_blocks_for_range(a, 0, 3 * 16) and e.ensure_blocks_for_range(b, 0, 3 * 16)
        assert e.evict_blocks(a, 1) == 1 and e.evict_blocks(b, 2) == 2
        assert _files(tmp_path) == ["block_0.kv", "seq1_block_0.kv", "seq1_block_1.kv"]
        c = e.seq_fork(b)                                         # the child shares resident pages only
        assert e.locations(c)[:3].tolist() == [0, 0, 1]
        assert e.refcounts()[e.table(b)[2]] == 2
        assert e.evict_blocks(b, 1) == 0                          # its only resident page is shared: no victim
        e.seq_release(b, discard=True)
        assert _files(tmp_path) == ["block_0.kv"]
        with pytest.raises(RuntimeError, match="still stored"):
            e.tier_disable()
        e.seq_release(a, discard=True)
        assert _files(tmp_path) == []
        e.tier_disable()
        assert e.tier_stats()["pages_stored"] == 0
    finally:
        e.close()


@pytest.mark.parametrize("seed", range(8))
def test_random_mix_matches_model(drkv_lib, tmp_path, seed):
    rng = np.random.default_rng(seed)
    pages, page, max_seqs, width = int(rng.integers(4, 20)), 16, 4, 24
    e = _engine(tmp_path, pages=pages, page=page, max_seqs=max_seqs, width=width)
    m = BookModel(pages, page, max_seqs, width, True)
    m.tier = True
    if seed % 2:
        e.scorer_enable(0.5)
        m.scores = {i: np.zeros(width, dtype=np.float32) for i in range(max_seqs)}
    live = []
    try:
        for step in range(400):
            r = rng.random()
            if (r < 0.08 and len(live) < max_seqs) or not live:
                a, b = e.seq_create(), m.seq_create()
                assert a == b
                live.append(a)
                if m.scores is not None:
                    m.scores[a][:] = 0
            elif r < 0.13 and len(live) < max_seqs:
                parent = int(rng.choice(live))
                a, b = e.seq_fork(parent), m.seq_fork(parent)
                assert a == b
                live.append(a)
                if m.scores is not None:
                    m.scores[a][:] = m.scores[parent]
            elif r < 0.18:
                s = live.pop(int(rng.integers(len(live))))
                discard = bool(rng.random() < 0.5)
                e.seq_release(s, discard=discard)
                assert m.seq_release(s, discard) == 0
            elif r < 0.55:
                s = int(rng.choice(live))
                pos = int(rng.integers(0, width * page))
                got = e.ensure_blocks_for(s, pos)
                want = m.seq_ensure_pos(s, pos) == 0
                assert got == want, f"step {step}"
            elif r < 0.75:
                s = int(rng.choice(live))
                n = int(rng.integers(0, 4))
                assert e.evict_blocks(s, n) == m.seq_evict(s, n), f"step {step}"
            elif r < 0.85 and m.scores is not None:
                s = int(rng.choice(live))
                vals = (rng.integers(0, 4, size=width) * 0.25).astype(np.float32)
                e.scorer_update(s, vals)
                m.scores[s] = (m.scores[s] * np.float32(0.5) + vals).astype(np.float32)   # exact in fp32 for these values
            else:
                s = int(rng.choice(live))
                n = int(rng.integers(0, pages))
                assert int(e.ensure_free_blocks(s, n)) == m.ensure_free(s, n), f"step {step}"
            for s in live:
                assert e.table(s).tolist() == m.table(s), f"step {step} seq {s}"
                loc = e.locations(s).tolist()
                assert [i for i, v in enumerate(loc) if v == 2] == sorted(m.seqs[s].stored), f"step {step} seq {s}"
            assert e.free_stack().tolist() == m.free
            want_files = sorted(("block_%d.kv" % i) if s == 0 else ("seq%d_block_%d.kv" % (s, i)) for s, i in m.files)
            assert _files(tmp_path) == want_files, f"step {step}"
    finally:
        e.close()
