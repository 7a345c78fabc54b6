"""Decode branches on the device: fork, copy-on-write of the shared partial tail page (device
copy of the valid slots, every layer and head), private appends, attention per branch.  Pool bytes
bit-exact against the CPU checker applied to a host copy; attention within 2e-3."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def test_branches_share_prefix_and_split_on_write(drkv_lib, oracle):
    import torch
    from deusridet_b200 import PagedKVEngine
    from oracle.bookkeeping import BookModel

    ob = oracle
    layers, hq, hkv, d, page, dtype = 3, 32, 8, 128, 16, ob.BF16
    n_branch, prefix = 4, 16 * 20 + 5                     # the tail page holds 5 tokens: forces copy-on-write
    max_pages, width = 64, 40
    rng = np.random.default_rng(31)
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=max_pages, max_seqs=8, max_pages_per_seq=width, device=0)
    mod = BookModel(max_pages, page, 8, width, False)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        H.shuffled_free_stack(eng, rng)
        mod.free = eng.free_stack().tolist()              # same seeded pool order in the model
        root = eng.seq_create()
        assert mod.seq_create() == root
        eng.reserve(root, prefix)
        eng.set_seq_len(root, prefix)
        mod.seq_reserve(root, prefix)
        mod.seq_set_len(root, prefix)
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        branches = [root] + [eng.seq_fork(root) for _ in range(n_branch - 1)]
        for b in branches[1:]:
            assert mod.seq_fork(root) == b
        lens = {b: prefix for b in branches}
        scale = 1.0 / np.sqrt(d)
        for step in range(3):
            # allocate (+ copy-on-write on the first step) for every branch, then one decode step
            for b in branches:
                eng.reserve(b, 1)
                n_before = len(mod.cow)
                assert mod.seq_reserve(b, 1) == 0
                for src, dst, valid in mod.cow[n_before:]:
                    ob.cow_copy(g, pool_host, max_pages, src, dst, valid)
            eng.sync_block_table()
            tables = np.stack([eng.table(b) for b in branches])
            assert [t.tolist() for t in tables] == [mod.table(b) for b in branches]
            rows = torch.tensor(branches, dtype=torch.int32, device="cuda")
            pos = np.array([lens[b] for b in branches], dtype=np.int32)
            d_pos = torch.from_numpy(pos).cuda()
            for layer in range(layers):
                k = H.randn_bits(rng, (n_branch, hkv, d), dtype)
                v = H.randn_bits(rng, (n_branch, hkv, d), dtype)
                q = H.randn_bits(rng, (n_branch, hq, d), dtype)
                out = torch.zeros(n_branch, hq, d, dtype=torch.bfloat16, device="cuda")
                eng.append_rope(layer, n_branch, rows, d_pos, H.to_dev(k, dtype), H.to_dev(v, dtype))
                eng.attend_decode(layer, n_branch, rows, d_pos + 1, int(pos.max()) + 1, H.to_dev(q, dtype), out, scale)
                for i in range(n_branch):
                    ob.append(g, pool_host, max_pages, tables[i], layer, int(pos[i]), 1, k[i], v[i], rope=True)
                want = np.zeros((n_branch, hq, d), dtype=np.uint16)
                ob.attend_decode(g, pool_host, max_pages, tables, np.arange(n_branch), pos + 1, layer, q, want, scale)
                torch.cuda.synchronize()
                err = np.abs(ob.to_float(H.torch_bits(out), dtype) - ob.to_float(want, dtype)).max()
                assert err <= 2e-3, f"step {step} layer {layer}: {err}"
            eng.check_kernels()
            got_pool = eng.pool_tensor().cpu().numpy().view(np.uint16)
            assert np.array_equal(got_pool, pool_host), f"step {step}: pool bytes differ"
            for b in branches:
                lens[b] += 1
                eng.set_seq_len(b, lens[b])
                mod.seq_set_len(b, lens[b])
        st = eng.stats()
        assert st["cow_copies"] == n_branch - 1            # the last writer found the page private again
        assert eng.refcounts().tolist() == mod.ref
        assert (eng.refcounts()[tables[0][:20]] == n_branch).all()
    finally:
        eng.close()
