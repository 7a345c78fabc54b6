"""Flat <-> paged K/V copies on the device against the CPU checker (bit-exact), with holes, and a
round trip at a size the checker is not asked to redo: extract, wipe the pages, inject, compare."""
import ctypes as C

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def test_extract_inject_match_checker_with_holes(drkv_lib, oracle):
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, d, page, dtype = 3, 24, 4, 256, 16, ob.F16
    rng = np.random.default_rng(41)
    total = 16 * 11 + 7
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="f16",
                        rotary_dim=64, max_pages=20, max_seqs=2, max_pages_per_seq=16, device=0, stream_evict=True)
    g = ob.geom(layers, hq, hkv, d, page, dtype, 64, 1e7)
    try:
        H.shuffled_free_stack(eng, rng)
        eng.seq_create()
        s = eng.seq_create()
        assert eng.ensure_blocks_for_range(s, 0, total)
        eng.set_seq_len(s, total)
        assert eng.evict_blocks(s, 2) == 2                  # logical pages 0 and 1 become holes
        eng.sync_block_table()
        table = eng.table(s)
        pool_host = H.randn_bits(rng, ob.pool_elems(g, 20), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        start, n = 5, total - 5
        want = ob.extract(g, pool_host, 20, table, start, n)
        flat = torch.full(want.shape, 0x1111, dtype=torch.int16, device="cuda")
        eng.extract(s, start, n, flat)
        torch.cuda.synchronize()
        assert np.array_equal(flat.cpu().numpy().view(np.uint16), want)
        assert not want[:, :, :16 * 2 - start].any()        # the holes read as zeros (cache_kernels.cu:66-69)
        # inject different data: holes are skipped, everything else lands where the checker puts it
        src = H.randn_bits(rng, want.shape, dtype)
        ob.inject(g, pool_host, src, 20, table, start, n)
        eng.inject(s, start, n, torch.from_numpy(src.view(np.int16)).cuda())
        torch.cuda.synchronize()
        assert np.array_equal(eng.pool_tensor().cpu().numpy().view(np.uint16), pool_host)
        # the raw-pointer entry points do the same
        from deusridet_b200 import capi
        cg = capi.Geometry(layers, hq, hkv, d, page, dtype, 64, 1e7)
        d_table = torch.from_numpy(table).cuda()
        flat2 = torch.zeros_like(flat)
        rc = drkv_lib.drkv_k_extract_kv(C.byref(cg), flat2.data_ptr(), eng.pool_ptr(), d_table.data_ptr(), start, n, 20, None)
        assert rc == 0
        torch.cuda.synchronize()
        assert np.array_equal(flat2.cpu().numpy().view(np.uint16), ob.extract(g, pool_host, 20, table, start, n))
    finally:
        eng.close()


def test_round_trip_large(drkv_lib):
    """8 layers x 20 000 tokens x 8 heads x 128 dims = 655 MB flat: extract -> clear pool -> inject -> extract."""
    import torch
    from deusridet_b200 import PagedKVEngine

    layers, hkv, d, page, n = 8, 8, 128, 16, 20000
    pages = (n + page - 1) // page
    eng = PagedKVEngine(num_layers=layers, num_q_heads=32, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        max_pages=pages + 3, max_seqs=1, max_pages_per_seq=pages + 1, device=0)
    try:
        H.shuffled_free_stack(eng, np.random.default_rng(3))
        s = eng.seq_create()
        assert eng.ensure_blocks_for_range(s, 0, n)
        eng.sync_block_table()
        torch.manual_seed(0)
        pool = eng.pool_tensor()
        pool.view(torch.bfloat16).normal_()
        flat = torch.empty(layers * 2 * n * hkv * d, dtype=torch.int16, device="cuda")
        eng.extract(s, 0, n, flat)
        checksum = int(flat.view(torch.int64).sum().item())
        pool.zero_()
        eng.inject(s, 0, n, flat)
        again = torch.empty_like(flat)
        eng.extract(s, 0, n, again)
        torch.cuda.synchronize()
        assert torch.equal(flat, again)
        assert int(again.view(torch.int64).sum().item()) == checksum and checksum != 0
    finally:
        eng.close()
