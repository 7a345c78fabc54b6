"""One long sequence split by contiguous KV page range across ranks, on one device: each rank's
share goes through drkv_attend_partial (un-normalised (m, l, o) per query head), the partials are
laid side by side as an all-gather would deliver them, and drkv_combine_partials merges them.
Ranks are emulated by consecutive calls; the partition is the one the multi-GPU path uses."""
import numpy as np
import pytest

from deusridet_b200 import sharding
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,seq_len,page", [(8, 8192 + 37, 64), (4, 3000, 64), (2, 100, 16), (8, 200, 64)])
def test_partials_of_page_ranges_merge_to_full_attention(drkv_lib, oracle, world, seq_len, page):
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, d, dtype = 2, 64, 8, 128, ob.BF16
    rng = np.random.default_rng(seq_len)
    n_pages = (seq_len + page - 1) // page
    max_pages = n_pages + 4
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=max_pages, max_seqs=1, max_pages_per_seq=n_pages + 1, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        H.shuffled_free_stack(eng, rng)
        s = eng.seq_create()
        assert eng.ensure_blocks_for_range(s, 0, seq_len)
        eng.set_seq_len(s, seq_len)
        eng.sync_block_table()
        table = eng.table(s)
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        q = H.randn_bits(rng, (hq, d), dtype)
        d_q = H.to_dev(q, dtype)
        scale = 1.0 / np.sqrt(d)
        nf = eng.partial_floats()
        assert nf == hq * (d + 2)
        layer = 1
        gathered = torch.zeros(world, nf, dtype=torch.float32, device="cuda")
        for r in range(world):
            begin, end = sharding.key_range_for_rank(seq_len, page, r, world)
            eng.attend_partial(layer, s, begin, end, d_q, gathered[r], scale)
            want = ob.attend_partial(g, pool_host, max_pages, table, layer, begin, end, q, scale)
            torch.cuda.synchronize()
            got = gathered[r].cpu().numpy()
            m_w, l_w = want[hq * d:hq * d + hq], want[hq * (d + 1):]
            m_g, l_g = got[hq * d:hq * d + hq], got[hq * (d + 1):]
            if end <= begin:
                assert (m_g == np.float32(-1e20)).all() and not l_g.any() and not got[:hq * d].any()
                continue
            # (m, l, o) may differ by a common factor exp(m_w - m_g); compare the normalised partial
            o_w = want[:hq * d].reshape(hq, d) / l_w[:, None]
            o_g = got[:hq * d].reshape(hq, d) / l_g[:, None]
            assert np.abs(o_w - o_g).max() <= 2e-3
            lse_w, lse_g = m_w + np.log(l_w), m_g + np.log(l_g)
            assert np.abs(lse_w - lse_g).max() <= 1e-3
        out = torch.zeros(hq, d, dtype=torch.bfloat16, device="cuda")
        eng.combine_partials(world, gathered, out)
        torch.cuda.synchronize()
        eng.check_kernels()
        whole = np.zeros((1, hq, d), dtype=np.uint16)
        ob.attend_decode(g, pool_host, max_pages, table[None, :], [0], [seq_len], layer, q[None], whole, scale)
        err = np.abs(ob.to_float(H.torch_bits(out), dtype) - ob.to_float(whole[0], dtype)).max()
        assert err <= 2e-3, err
    finally:
        eng.close()
