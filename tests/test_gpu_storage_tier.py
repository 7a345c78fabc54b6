"""Storage tier with a device: page files hold, for every layer, the K plane then the V plane of the page
(kv_swapper.cpp:183-200), byte for byte; a page read back — from the file or from a prefetched host copy —
restores the pool bytes at its new page id, and attention over the sequence returns the same bits as
before the round trip."""
import os

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("hkv,d,page,layers", [(8, 128, 16, 3), (2, 64, 64, 2)])
def test_page_files_and_round_trip(drkv_lib, oracle, tmp_path, hkv, d, page, layers):
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    hq, dtype = hkv * 4, ob.BF16
    max_pages, n_pages = 24, 14
    rng = np.random.default_rng(hkv + page)
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=max_pages, max_seqs=2, max_pages_per_seq=32, device=0,
                        stream_evict=True)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        eng.tier_enable(str(tmp_path))
        H.shuffled_free_stack(eng, rng)
        other = eng.seq_create()                                   # row 0, so that the sequence under test is row 1
        s = eng.seq_create()
        n_tok = n_pages * page - 3
        eng.reserve(s, n_tok)
        eng.set_seq_len(s, n_tok)
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        pool_dev = eng.pool_tensor()
        pool_dev.copy_(torch.from_numpy(pool_host.view(np.int16)))
        eng.sync_block_table()
        before = eng.table(s).copy()
        q = H.to_dev(H.randn_bits(rng, (1, hq, d), dtype), dtype)
        rows = torch.tensor([s], dtype=torch.int32, device="cuda")
        d_len = torch.tensor([n_tok], dtype=torch.int32, device="cuda")
        outs0 = []
        for layer in range(layers):
            o = torch.zeros(1, hq, d, dtype=torch.bfloat16, device="cuda")
            eng.attend_decode(layer, 1, rows, d_len, n_tok, q, o, 0.1)
            outs0.append(o)
        torch.cuda.synchronize()

        k = 6
        assert eng.evict_blocks(s, k) == k                          # oldest six logical pages
        per_layer = 2 * hkv * page * d                               # elements of one (layer, page): K plane, V plane
        by_layer = pool_host.reshape(layers, max_pages, per_layer)
        st = eng.tier_stats()
        assert st["page_file_bytes"] == layers * per_layer * 2 and st["bytes_out"] == k * st["page_file_bytes"]
        for j in range(k):
            with open(os.path.join(tmp_path, f"seq{s}_block_{j}.kv"), "rb") as f:
                got = np.frombuffer(f.read(), dtype=np.uint16)
            assert np.array_equal(got, by_layer[:, before[j], :].reshape(-1)), f"file of logical page {j}"
        # the freed pages are scribbled over: what comes back must come from the tier
        for j in range(k):
            pool_dev.view(layers, max_pages, per_layer)[:, int(before[j]), :] = 0x7F7F
        assert eng.locations(s)[:k + 1].tolist() == [2] * k + [1]
        for j in (1, 3, 5):
            assert eng.prefetch_block(s, j) == 1
        assert eng.prefetch_block(s, k) == 0                        # resident: nothing to prefetch
        eng.tier_drain()
        assert eng.ensure_blocks_for_range(s, 0, k * page)
        st = eng.tier_stats()
        assert st["swap_ins"] == k and st["prefetch_hits"] == 3 and st["pages_stored"] == 0
        assert sorted(os.listdir(tmp_path)) == []
        eng.sync_block_table()
        after = eng.table(s)
        assert (after[:n_pages] >= 0).all() and not np.array_equal(after[:k], before[:k])   # LIFO: ids come back reversed
        now = pool_dev.cpu().numpy().view(np.uint16).reshape(layers, max_pages, per_layer)
        for j in range(n_pages):
            assert np.array_equal(now[:, after[j], :], by_layer[:, before[j], :]), f"logical page {j}"
        for layer in range(layers):
            o = torch.zeros(1, hq, d, dtype=torch.bfloat16, device="cuda")
            eng.attend_decode(layer, 1, rows, d_len, n_tok, q, o, 0.1)
            torch.cuda.synchronize()
            assert torch.equal(o, outs0[layer]), f"layer {layer}"
        eng.check_kernels()
        eng.seq_release(other, discard=True)
    finally:
        eng.close()


def test_swap_out_waits_for_kernels_in_flight(drkv_lib, oracle, tmp_path):
    """An append enqueued on the engine's stream just before the eviction must be in the file."""
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, d, page, dtype = 2, 8, 2, 128, 16, ob.BF16
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=8, max_seqs=1, max_pages_per_seq=8, device=0, stream_evict=True)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    rng = np.random.default_rng(3)
    try:
        eng.tier_enable(str(tmp_path))
        s = eng.seq_create()
        eng.reserve(s, 5)
        eng.sync_block_table()
        pool_host = np.zeros(ob.pool_elems(g, 8), dtype=np.uint16)
        table = np.full((1, eng.table_stride()), -1, dtype=np.int32)
        table[0, :1] = eng.table(s)[:1]
        stream = torch.cuda.Stream()
        rows = torch.tensor([s], dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            for pos in range(5):
                for layer in range(layers):
                    k = H.randn_bits(rng, (1, hkv, d), dtype)
                    v = H.randn_bits(rng, (1, hkv, d), dtype)
                    eng.append_rope(layer, 1, rows, torch.tensor([pos], dtype=torch.int32, device="cuda"),
                                    H.to_dev(k, dtype), H.to_dev(v, dtype), stream)
                    ob.append(g, pool_host, 8, table[0], layer, pos, 1, k[0], v[0], rope=True)
        eng.set_seq_len(s, 5)
        page0 = int(table[0, 0])
        assert eng.evict_blocks(s, 1) == 1                          # no synchronisation in between
        per_layer = 2 * hkv * page * d
        with open(os.path.join(tmp_path, "block_0.kv"), "rb") as f:
            got = np.frombuffer(f.read(), dtype=np.uint16)
        assert np.array_equal(got, pool_host.reshape(layers, 8, per_layer)[:, page0, :].reshape(-1))
        torch.cuda.synchronize()
        eng.check_kernels()
    finally:
        eng.close()


def test_write_behind_round_trip_and_swapper_requests(drkv_lib, oracle, tmp_path):
    """With deferred file writes on: pages evicted in a burst (more than the four pinned buffers) come back with
    their bytes whether their file has been written yet or not, the freed pool pages may be overwritten at once,
    the files are complete after a drain, and nothing is left behind after the swap-ins.  Then the two moves a
    KVSwapper::submit request asks for (kv_swapper.h:36-44): one pool page to a file of the caller's choosing and
    back into another page."""
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, d, page, dtype = 3, 16, 4, 128, 16, ob.BF16
    max_pages, n_pages = 24, 16
    rng = np.random.default_rng(61)
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=max_pages, max_seqs=1, max_pages_per_seq=32, device=0,
                        stream_evict=True)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        eng.tier_enable(str(tmp_path))
        eng.tier_set_write_behind(True)
        H.shuffled_free_stack(eng, rng)
        s = eng.seq_create()
        n_tok = n_pages * page
        eng.reserve(s, n_tok)
        eng.set_seq_len(s, n_tok)
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        pool_dev = eng.pool_tensor()
        pool_dev.copy_(torch.from_numpy(pool_host.view(np.int16)))
        eng.sync_block_table()
        before = eng.table(s).copy()
        per_layer = 2 * hkv * page * d
        by_layer = pool_host.reshape(layers, max_pages, per_layer)
        k = 10
        assert eng.evict_blocks(s, k) == k                          # a burst: ten pages through four buffers
        for j in range(k):                                          # the pool pages are free: scribble over them at once
            pool_dev.view(layers, max_pages, per_layer)[:, int(before[j]), :] = 0x7F7F
        assert eng.prefetch_block(s, 2) == 1                        # queued behind the page's own file write
        assert eng.ensure_blocks_for_range(s, 0, 4 * page)          # four come back straight away
        eng.tier_drain()
        st = eng.tier_stats()
        assert st["writes_deferred"] == k and st["write_failures"] == 0 and st["swap_ins"] == 4
        for j in range(4, k):                                       # the others' files are complete
            with open(os.path.join(tmp_path, f"block_{j}.kv"), "rb") as f:
                got = np.frombuffer(f.read(), dtype=np.uint16)
            assert np.array_equal(got, by_layer[:, before[j], :].reshape(-1)), f"file of logical page {j}"
        assert eng.ensure_blocks_for_range(s, 0, k * page)
        assert sorted(os.listdir(tmp_path)) == []
        eng.sync_block_table()
        after = eng.table(s)
        now = pool_dev.cpu().numpy().view(np.uint16).reshape(layers, max_pages, per_layer)
        for j in range(n_pages):
            assert np.array_equal(now[:, after[j], :], by_layer[:, before[j], :]), f"logical page {j}"

        # one SwapRequest each way: pool page -> file -> another pool page
        src, dst = int(after[0]), eng.alloc_block()
        assert dst >= 0
        path = str(tmp_path / "request.kv")
        eng.page_to_file(src, path)
        eng.file_to_page(path, dst)
        torch.cuda.synchronize()
        now = pool_dev.cpu().numpy().view(np.uint16).reshape(layers, max_pages, per_layer)
        assert np.array_equal(now[:, dst, :], now[:, src, :]) and os.path.getsize(path) == layers * per_layer * 2
    finally:
        eng.close()
