"""Decode items much longer than 32 pages: the kernel holds 32 page ids per lane window and switches windows
inside an item; items start in the middle of a table row (chunks 2, 3, ... of a sequence) and end ragged.
Also a key range that starts inside a page (attend_partial), and head_dim 256 (six warps per CTA).
Against the CPU checker."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d,page,chunk", [(128, 16, 2048), (128, 16, 1040), (256, 16, 1536), (128, 64, 4096), (64, 16, 2048)])
def test_items_across_page_id_windows(drkv_lib, oracle, d, page, chunk):
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, dtype = 2, 8, 2, ob.BF16
    rng = np.random.default_rng(d + page + chunk)
    lens = [3 * chunk + 517, chunk + 1, 33 * page + 5, 2 * chunk, 7]
    pages = sum((n + page - 1) // page for n in lens)
    max_pages, width = pages + 40, max((n + page - 1) // page for n in lens) + 3
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=max_pages, max_seqs=8, max_pages_per_seq=width, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        H.shuffled_free_stack(eng, rng)
        seqs = []
        for n in lens:
            s = eng.seq_create()
            eng.reserve(s, n)
            eng.set_seq_len(s, n)
            seqs.append(s)
        n = len(seqs)
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        eng.sync_block_table()
        tables = np.full((n, eng.table_stride()), -1, dtype=np.int32)
        for i, s in enumerate(seqs):
            t = eng.table(s)
            tables[i, :len(t)] = t
        eng.set_chunk_tokens(chunk)
        q = H.randn_bits(rng, (n, hq, d), dtype)
        scale = 1.0 / np.sqrt(d)
        for layer in range(layers):
            out = torch.zeros(n, hq, d, dtype=torch.bfloat16, device="cuda")
            eng.attend_decode(layer, n, torch.tensor(seqs, dtype=torch.int32, device="cuda"),
                              torch.tensor(lens, dtype=torch.int32, device="cuda"), max(lens), H.to_dev(q, dtype), out, scale)
            want = np.zeros((n, hq, d), dtype=np.uint16)
            ob.attend_decode(g, pool_host, max_pages, tables, np.arange(n), np.array(lens, dtype=np.int32), layer, q, want, scale)
            torch.cuda.synchronize()
            eng.check_kernels()
            got_f, want_f = ob.to_float(H.torch_bits(out), dtype), ob.to_float(want, dtype)
            tol = np.maximum(2e-3, H.ulp(want_f, dtype))
            bad = np.argwhere(np.abs(got_f - want_f) > tol)
            assert bad.size == 0, f"layer {layer}: {len(bad)} elements off, first {bad[:3].tolist()}, worst {np.abs(got_f - want_f).max()}"
    finally:
        eng.close()
