"""Multi-sequence bookkeeping of libdrkv.so (fork, reference counts, copy-on-write, cached-page
LRU, adoption) against the Python model in oracle/bookkeeping.py, operation by operation:
tables, reference counts, free stack, LRU list and the eviction log are integers and must agree
exactly.  The reference has no code for this part (parity unpinned); the single-sequence subset
of the same model is pinned in test_bookkeeping_vs_reference.py."""
import numpy as np
import pytest

from oracle.bookkeeping import BookModel


def _engine(pages, psize, max_seqs, width, stream_evict):
    from deusridet_b200 import PagedKVEngine
    return PagedKVEngine(num_layers=2, num_q_heads=8, num_kv_heads=2, head_dim=64, page_size=psize, dtype="bf16",
                         max_pages=pages, max_seqs=max_seqs, max_pages_per_seq=width, device=-1,
                         stream_evict=stream_evict)


def _same_state(eng, mod, live):
    assert eng.free_stack().tolist() == mod.free
    assert eng.refcounts().tolist() == mod.ref
    assert eng.cached_lru().tolist() == list(mod.lru)
    for s in live:
        assert eng.table(s).tolist() == mod.table(s), f"table of sequence {s}"
        assert eng.seq_len(s) == mod.seqs[s].len


@pytest.mark.parametrize("seed,stream_evict", [(s, bool(s % 2)) for s in range(10)])
def test_fuzz_against_model(drkv_lib, seed, stream_evict):
    from deusridet_b200 import DrkvError
    rng = np.random.default_rng(seed)
    pages, psize, max_seqs, width = int(rng.integers(6, 40)), 16, 6, 24
    eng, mod = _engine(pages, psize, max_seqs, width, stream_evict), BookModel(pages, psize, max_seqs, width, stream_evict)
    live = []
    for step in range(600):
        r = rng.random()
        if (r < 0.08 and len(live) < max_seqs) or not live:
            a, b = eng.lib.drkv_seq_create(eng.h), mod.seq_create()
            assert a == b
            if a >= 0:
                live.append(a)
        elif r < 0.16 and len(live) < max_seqs:
            parent = int(rng.choice(live))
            a, b = eng.lib.drkv_seq_fork(eng.h, parent), mod.seq_fork(parent)
            assert a == b
            if a >= 0:
                live.append(a)
        elif r < 0.24:
            s = live.pop(int(rng.integers(len(live))))
            discard = bool(rng.integers(2))
            assert eng.lib.drkv_seq_release(eng.h, s, int(discard)) == mod.seq_release(s, discard)
        elif r < 0.70:
            s = int(rng.choice(live))
            n = int(rng.integers(1, 3 * psize))
            a, b = eng.lib.drkv_seq_reserve(eng.h, s, n, None), mod.seq_reserve(s, n)
            assert a == b, f"step {step}: reserve({s},{n}) -> {a} vs {b}"
            if a == 0:
                new_len = mod.seqs[s].len + n
                assert eng.lib.drkv_seq_set_len(eng.h, s, new_len) == mod.seq_set_len(s, new_len)
        elif r < 0.78:
            s = int(rng.choice(live))
            pos = int(rng.integers(0, (width + 1) * psize))
            assert eng.lib.drkv_seq_ensure_pos(eng.h, s, pos, None) == mod.seq_ensure_pos(s, pos)
        elif r < 0.84:
            n = int(rng.integers(0, 4))
            assert eng.evict_cached(n) == mod.evict_cached(n)
        elif r < 0.90:
            s = int(rng.choice(live))
            n = int(rng.integers(0, 3))
            assert eng.evict_blocks(s, n) == mod.seq_evict(s, n)
        elif r < 0.95:
            s = int(rng.choice(live + [-1]))
            n = int(rng.integers(0, pages))
            assert int(eng.ensure_free_blocks(s, n)) == mod.ensure_free(s, n)
        else:
            # adopt the pages of a released sequence into a fresh one (prefix reuse)
            if len(live) < max_seqs and mod.lru:
                k = int(rng.integers(1, min(4, len(mod.lru)) + 1))
                pgs = [int(p) for p in list(mod.lru)[:k]]
                a, b = eng.lib.drkv_seq_create(eng.h), mod.seq_create()
                assert a == b and a >= 0
                live.append(a)
                ntok = k * psize - int(rng.integers(0, psize))
                eng.adopt(a, pgs, ntok)
                assert mod.seq_adopt(a, pgs, ntok) == 0
        _same_state(eng, mod, live)
        assert eng.evict_log(clear=False) == mod.log
        assert eng.stats()["cow_copies"] == mod.n_cow
    st = eng.stats()
    assert st["pages_free"] + st["pages_cached"] + st["pages_active"] == pages
    eng.close()


def test_fork_shares_pages_and_cow_splits_the_tail(drkv_lib):
    eng = _engine(32, 16, 10, 16, False)
    parent = eng.seq_create()
    eng.reserve(parent, 37)
    eng.set_seq_len(parent, 37)                 # 3 pages, the last holds 5 tokens
    kids = [eng.seq_fork(parent) for _ in range(7)]
    assert (eng.refcounts()[:3] == 8).all()
    before = eng.table(parent)[:3].tolist()
    # first writer: copy-on-write of the partial tail page only
    eng.reserve(kids[0], 1)
    t = eng.table(kids[0])[:3].tolist()
    assert t[:2] == before[:2] and t[2] != before[2]
    assert eng.refcounts()[before[2]] == 7 and eng.refcounts()[t[2]] == 1
    assert eng.stats()["cow_copies"] == 1
    # a second reserve by the same branch is private already
    eng.set_seq_len(kids[0], 38)
    eng.reserve(kids[0], 1)
    assert eng.stats()["cow_copies"] == 1
    # a fork at a page boundary shares nothing that is written to: no copy
    eng2 = _engine(32, 16, 4, 16, False)
    p2 = eng2.seq_create()
    eng2.reserve(p2, 32)
    eng2.set_seq_len(p2, 32)
    c2 = eng2.seq_fork(p2)
    eng2.reserve(c2, 1)
    assert eng2.stats()["cow_copies"] == 0
    assert eng2.table(c2)[2] >= 0 and eng2.table(p2)[2] == -1
    # releasing every holder turns the shared pages into cached pages, in release order
    for k in kids:
        eng.seq_release(k)
    assert eng.refcounts()[before[0]] == 1
    eng.seq_release(parent)
    assert eng.cached_lru().tolist()[-3:] == before
    eng.close()
    eng2.close()


def test_shared_pages_are_never_victims(drkv_lib):
    from deusridet_b200 import DrkvError
    eng = _engine(4, 16, 3, 8, True)
    a = eng.seq_create()
    eng.reserve(a, 64)
    eng.set_seq_len(a, 64)                      # all 4 pages
    b = eng.seq_fork(a)
    # stream-mode eviction may only take unshared pages: there are none
    assert eng.evict_blocks(a, 2) == 0
    with pytest.raises(DrkvError) as ei:
        eng.reserve(b, 1)
    assert ei.value.code == -2                  # DRKV_ERR_EXHAUSTED
    eng.seq_release(b)
    assert eng.evict_blocks(a, 2) == 2          # now private again
    eng.close()


def test_error_paths_do_not_corrupt_state(drkv_lib):
    from deusridet_b200 import DrkvError, capi
    eng = _engine(8, 16, 2, 8, False)
    p = eng.alloc_block()
    eng.free_block(p)
    with pytest.raises(DrkvError) as ei:
        eng.free_block(p)                       # double free: refused (the reference would corrupt its stack)
    assert ei.value.code == capi.ERR_STATE
    with pytest.raises(DrkvError):
        eng.free_block(99)
    assert eng.free_count() == 8
    with pytest.raises(DrkvError):
        eng.seq_fork(1)                         # unknown sequence
    s = eng.seq_create()
    assert not eng.ensure_blocks_for(s, 8 * 16)  # beyond the table (cache_manager.cpp:77-81)
    assert "beyond" in capi.last_error()
    s2 = eng.seq_create()
    with pytest.raises(DrkvError) as ei:
        eng.seq_create()                        # all rows in use
    assert ei.value.code == capi.ERR_CAPACITY
    # compute entry points refuse a bookkeeping-only engine: there is no CPU path
    with pytest.raises(DrkvError) as ei:
        eng.sync_block_table()
    assert ei.value.code == capi.ERR_NO_DEVICE
    with pytest.raises(DrkvError) as ei:
        eng.attend_decode(0, 1, 0, 0, 1, 0, 0, 1.0)
    assert ei.value.code in (capi.ERR_NO_DEVICE, capi.ERR_INVALID)
    eng.close()


def test_prefix_sharing_scenario_scaled(drkv_lib):
    """Scaled-down form of the multi-branch configuration: a common prefix forked into 8 decode
    branches (one at a page boundary, one 5 tokens past it), private growth per branch, a pool
    capped so that released filler pages get reclaimed in LRU order, 64 round-robin decode steps.
    Engine and model must agree on every table, count and log entry after every step."""
    rng = np.random.default_rng(77)
    P, prefix = 16, 16 * 24
    pages = 24 + 8 * 10 + 6
    eng, mod = _engine(pages, P, 16, 48, False), BookModel(pages, P, 16, 48, False)

    def both(fn_e, fn_m):
        a, b = fn_e(), fn_m()
        assert a == b
        return a

    # filler sequences, released: their pages become the unreferenced, evictable ones
    fillers = []
    for _ in range(4):
        s = both(lambda: eng.lib.drkv_seq_create(eng.h), mod.seq_create)
        n = int(rng.integers(20, 90))
        both(lambda: eng.lib.drkv_seq_reserve(eng.h, s, n, None), lambda: mod.seq_reserve(s, n))
        both(lambda: eng.lib.drkv_seq_set_len(eng.h, s, n), lambda: mod.seq_set_len(s, n))
        fillers.append(s)
    for s in fillers:
        both(lambda: eng.lib.drkv_seq_release(eng.h, s, 0), lambda: mod.seq_release(s, False))
    for plen in (prefix, prefix + 5):
        root = both(lambda: eng.lib.drkv_seq_create(eng.h), mod.seq_create)
        both(lambda: eng.lib.drkv_seq_reserve(eng.h, root, plen, None), lambda: mod.seq_reserve(root, plen))
        both(lambda: eng.lib.drkv_seq_set_len(eng.h, root, plen), lambda: mod.seq_set_len(root, plen))
        branches = [both(lambda: eng.lib.drkv_seq_fork(eng.h, root), lambda: mod.seq_fork(root)) for _ in range(3)]
        branches.append(root)
        lens = {b: plen for b in branches}
        for b in branches:
            grow = int(rng.integers(0, 40))
            rc = both(lambda: eng.lib.drkv_seq_reserve(eng.h, b, grow, None), lambda: mod.seq_reserve(b, grow))
            if rc == 0:
                lens[b] += grow
                both(lambda: eng.lib.drkv_seq_set_len(eng.h, b, lens[b]), lambda: mod.seq_set_len(b, lens[b]))
        for step in range(64):
            for b in branches:
                rc = both(lambda: eng.lib.drkv_seq_reserve(eng.h, b, 1, None), lambda: mod.seq_reserve(b, 1))
                if rc == 0:
                    lens[b] += 1
                    both(lambda: eng.lib.drkv_seq_set_len(eng.h, b, lens[b]), lambda: mod.seq_set_len(b, lens[b]))
            _same_state(eng, mod, branches)
            assert eng.evict_log(clear=False) == mod.log
        for b in branches:
            both(lambda: eng.lib.drkv_seq_release(eng.h, b, 0), lambda: mod.seq_release(b, False))
    assert len(mod.log) > 0, "the pool cap must force evictions of unreferenced pages"
    assert all(k == 0 for k, _, _, _ in mod.log)
    assert eng.stats()["cow_copies"] == mod.n_cow and len(mod.cow) >= 3
    eng.close()


def test_batch_reserve_and_advance(drkv_lib):
    eng = _engine(40, 16, 6, 12, False)
    mod = BookModel(40, 16, 6, 12, False)
    seqs = [eng.seq_create() for _ in range(5)]
    for _ in seqs:
        mod.seq_create()
    for step in range(40):
        eng.reserve_batch(seqs, 3)
        eng.advance_batch(seqs, 3)
        for s in seqs:
            assert mod.seq_reserve(s, 3) == 0
            assert mod.seq_set_len(s, mod.seqs[s].len + 3) == 0
    _same_state(eng, mod, seqs)
    assert eng.seq_len(seqs[2]) == 120
    eng.close()


def _c3_scenario(eng, mod, seed=2026, prefix=16384, branches=8, steps=256, P=16, check_every=1):
    """Multi-branch prefix sharing at full size: filler sequences are prefilled and released (their pages
    become unreferenced cached pages), a 16384-token prefix is forked into 8 branches (prefix pages at
    reference count 8), each branch appends U[0,2048] private tokens, then 256 decode steps round-robin.
    A second family forked at 16384 + 5 exercises copy-on-write of a shared partial tail page.  The pool
    is sized so that the active pages end at 90 % of it, which forces LRU eviction of the cached pages."""
    rng = np.random.default_rng(seed)          # filler sizes (depend on the pool size)
    rng_len = np.random.default_rng(seed + 1)  # private branch lengths (do not)

    def both(fe, fm):
        a, b = fe(), fm()
        assert a == b, (a, b)
        return a

    def grow(s, n):
        rc = both(lambda: eng.lib.drkv_seq_reserve(eng.h, s, n, None), lambda: mod.seq_reserve(s, n))
        if rc == 0:
            both(lambda: eng.lib.drkv_seq_advance_batch(eng.h, 1, (__import__("ctypes").c_int32 * 1)(s), n),
                 lambda: mod.seq_set_len(s, mod.seqs[s].len + n))
        return rc

    fillers = []
    while len(mod.free) > 64:
        s = both(lambda: eng.lib.drkv_seq_create(eng.h), mod.seq_create)
        assert grow(s, int(min(len(mod.free) - 32, rng.integers(40, 400))) * P) == 0
        fillers.append(s)
    for s in fillers:
        both(lambda: eng.lib.drkv_seq_release(eng.h, s, 0), lambda: mod.seq_release(s, False))
    live = []
    for plen, nb in ((prefix, branches), (prefix // 8 + 5, 3)):
        root = both(lambda: eng.lib.drkv_seq_create(eng.h), mod.seq_create)
        assert grow(root, plen) == 0
        fam = [root] + [both(lambda: eng.lib.drkv_seq_fork(eng.h, root), lambda: mod.seq_fork(root)) for _ in range(nb - 1)]
        for b in fam:
            assert grow(b, int(rng_len.integers(0, 2049 if plen == prefix else 200))) == 0
        live += fam
    _same_state(eng, mod, live)
    for step in range(steps):
        for b in live:
            assert grow(b, 1) == 0
        if step % check_every == 0 or step == steps - 1:
            _same_state(eng, mod, live)
            assert eng.evict_log(clear=False) == mod.log
    return live


def test_prefix_sharing_full_size(drkv_lib):
    # active pages at the end: 1024 shared + 8 private tails + 256 decode tokens each + the second family,
    # 1680 with this seed; the cap puts that at 90 % of the pool
    pages = 1867
    eng, mod = _engine(pages, 16, 64, 1300, False), BookModel(pages, 16, 64, 1300, False)
    live = _c3_scenario(eng, mod, check_every=16)
    st = eng.stats()
    assert 0.88 <= st["pages_active"] / pages <= 0.92 and st["evictions_cached"] > 100
    assert (eng.refcounts()[eng.table(live[0])[:1024]] == 8).all()        # the shared prefix
    assert st["cow_copies"] == mod.n_cow and st["cow_copies"] >= 2          # the 16384/8 + 5 family split its tail page
    assert all(k == 0 for k, _, _, _ in mod.log)                           # only unreferenced pages were victims
    # eviction order is release order of the fillers' pages
    assert [p for _, _, _, p in mod.log] == [p for _, _, _, p in eng.evict_log(clear=False)]
    eng.close()


def test_host_bookkeeping_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    """tests/cpp/page_book_fuzz.cpp drives csrc/page_book.cpp (no CUDA in it) with seeded operation mixes (valid calls,
    unknown sequences, double frees, frees of pages a block table still owns) and checks reference counts, free
    stack, cached list and stored-page counts after every operation, built with -fsanitize=address,undefined."""
    import os
    import subprocess
    ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "page_book_fuzz")
    subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined",
                    f"-I{ROOT}/deusridet_b200/csrc", f"-I{ROOT}/include", f"{ROOT}/tests/cpp/page_book_fuzz.cpp",
                    f"{ROOT}/deusridet_b200/csrc/page_book.cpp", "-o", exe], check=True)
    for seed in (11, 12, 13, 14):
        res = subprocess.run([exe, str(seed), "15000"], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0 and "PAGE_BOOK_FUZZ OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
