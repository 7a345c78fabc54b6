"""Tail split of the decode pass: the last chunks of every sequence are processed in pieces queued at the end.
Forced on small batches (the automatic rule only switches it on for passes several chunks deep per warp):
ragged lengths around every boundary, with and without a shared-prefix plan, against the CPU checker."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chunk,tail", [(64, 1), (64, 3), (128, 2), (256, 4), (32, 2)])
@pytest.mark.parametrize("planned", [False, True])
def test_tail_split_matches_checker(drkv_lib, oracle, chunk, tail, planned):
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, d, page, dtype = 1, 32, 8, 128, 16, ob.BF16
    rng = np.random.default_rng(chunk * 10 + tail)
    max_pages, width = 700, 80
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=max_pages, max_seqs=32, max_pages_per_seq=width, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        H.shuffled_free_stack(eng, rng)
        # lengths around the boundaries of chunks and pieces: 1, piece - 1, piece, piece + 1, chunk, k * chunk +- 1 ...
        piece = chunk // max(chunk // 64, 2)
        lens = [1, piece - 1, piece, piece + 1, chunk - 1, chunk, chunk + 1, 2 * chunk, 3 * chunk + piece, 4 * chunk + 5,
                tail * chunk, tail * chunk + 1, 700, 1023]
        seqs = []
        root = eng.seq_create()                                  # one family of three for the planned variant
        eng.reserve(root, 16 * 30 + 7)
        eng.set_seq_len(root, 16 * 30 + 7)
        fam = [root, eng.seq_fork(root), eng.seq_fork(root)]
        fam_lens = []
        for i, s in enumerate(fam):
            eng.reserve(s, 5 + 90 * i)
            eng.set_seq_len(s, 16 * 30 + 7 + 5 + 90 * i)
            fam_lens.append(16 * 30 + 7 + 5 + 90 * i)
        for n in lens:
            s = eng.seq_create()
            eng.reserve(s, n)
            eng.set_seq_len(s, n)
            seqs.append(s)
        seqs = fam + seqs
        lens = fam_lens + lens
        n = len(seqs)
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        eng.sync_block_table()
        tables = np.full((n, eng.table_stride()), -1, dtype=np.int32)
        for i, s in enumerate(seqs):
            t = eng.table(s)
            tables[i, :len(t)] = t
        eng.set_chunk_tokens(chunk)
        eng.set_tail_split(tail)
        q = H.randn_bits(rng, (n, hq, d), dtype)
        out = torch.zeros(n, hq, d, dtype=torch.bfloat16, device="cuda")
        scale = 1.0 / np.sqrt(d)
        if planned:
            info = eng.plan_decode(seqs, lens)
            assert info["n_families"] == 1
            eng.attend_decode_planned(0, H.to_dev(q, dtype), out, scale)
        else:
            eng.attend_decode(0, n, torch.tensor(seqs, dtype=torch.int32, device="cuda"),
                              torch.tensor(lens, dtype=torch.int32, device="cuda"), max(lens), H.to_dev(q, dtype), out, scale)
        want = np.zeros((n, hq, d), dtype=np.uint16)
        ob.attend_decode(g, pool_host, max_pages, tables, np.arange(n), np.array(lens, dtype=np.int32), 0, q, want, scale)
        torch.cuda.synchronize()
        eng.check_kernels()
        got_f, want_f = ob.to_float(H.torch_bits(out), dtype), ob.to_float(want, dtype)
        tol = np.maximum(2e-3, H.ulp(want_f, dtype))
        bad = np.argwhere(np.abs(got_f - want_f) > tol)
        assert bad.size == 0, f"{len(bad)} elements off, first {bad[:3].tolist()}, worst {np.abs(got_f - want_f).max()}"
        # and the pass without the split gives the same answer within the same bound
        eng.set_tail_split(0)
        plain = torch.zeros_like(out)
        if planned:
            eng.plan_decode(seqs, lens)
            eng.attend_decode_planned(0, H.to_dev(q, dtype), plain, scale)
        else:
            eng.attend_decode(0, n, torch.tensor(seqs, dtype=torch.int32, device="cuda"),
                              torch.tensor(lens, dtype=torch.int32, device="cuda"), max(lens), H.to_dev(q, dtype), plain, scale)
        torch.cuda.synchronize()
        assert np.abs(ob.to_float(H.torch_bits(plain), dtype) - got_f).max() <= 4e-3
    finally:
        eng.close()


def test_deep_batch_with_default_settings(drkv_lib, oracle):
    """A batch several 512-key items deep per warp, nothing forced: the engine picks 512-key items and splits
    every sequence's last chunk by itself.  Lengths sit on and around the chunk and piece boundaries."""
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, d, page, dtype = 1, 32, 8, 128, 16, ob.BF16
    rng = np.random.default_rng(77)
    lens = [1, 63, 64, 65, 511, 512, 513, 575, 576, 577, 1024, 1025, 4608, 5000] + \
        [int(x) for x in rng.integers(300, 5001, size=42)]
    n = len(lens)
    assert n * hkv * ((max(lens) + 511) // 512) >= 3 * 148 * 8          # deep enough for the automatic rule
    pages = sum((x + page - 1) // page for x in lens)
    max_pages, width = pages + 64, (max(lens) + page - 1) // page + 2
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=max_pages, max_seqs=n, max_pages_per_seq=width, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        H.shuffled_free_stack(eng, rng)
        seqs = []
        for x in lens:
            s = eng.seq_create()
            eng.reserve(s, x)
            eng.set_seq_len(s, x)
            seqs.append(s)
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        eng.sync_block_table()
        tables = np.full((n, eng.table_stride()), -1, dtype=np.int32)
        for i, s in enumerate(seqs):
            t = eng.table(s)
            tables[i, :len(t)] = t
        q = H.randn_bits(rng, (n, hq, d), dtype)
        scale = 1.0 / np.sqrt(d)
        d_rows = torch.tensor(seqs, dtype=torch.int32, device="cuda")
        d_len = torch.tensor(lens, dtype=torch.int32, device="cuda")
        out = torch.zeros(n, hq, d, dtype=torch.bfloat16, device="cuda")
        eng.attend_decode(0, n, d_rows, d_len, max(lens), H.to_dev(q, dtype), out, scale)
        want = np.zeros((n, hq, d), dtype=np.uint16)
        ob.attend_decode(g, pool_host, max_pages, tables, np.arange(n), np.array(lens, dtype=np.int32), 0, q, want, scale)
        torch.cuda.synchronize()
        eng.check_kernels()
        got_f, want_f = ob.to_float(H.torch_bits(out), dtype), ob.to_float(want, dtype)
        tol = np.maximum(2e-3, H.ulp(want_f, dtype))
        bad = np.argwhere(np.abs(got_f - want_f) > tol)
        assert bad.size == 0, f"{len(bad)} elements off, first {bad[:3].tolist()}, worst {np.abs(got_f - want_f).max()}"
        # the same batch with the split switched off: same answer within the same bound, and a second launch
        # with the defaults repeats the first bit for bit (the queue rewinds itself)
        eng.set_tail_split(0)
        plain = torch.zeros_like(out)
        eng.attend_decode(0, n, d_rows, d_len, max(lens), H.to_dev(q, dtype), plain, scale)
        eng.set_tail_split(-1)
        again = torch.zeros_like(out)
        eng.attend_decode(0, n, d_rows, d_len, max(lens), H.to_dev(q, dtype), again, scale)
        torch.cuda.synchronize()
        eng.check_kernels()
        assert np.abs(ob.to_float(H.torch_bits(plain), dtype) - got_f).max() <= 4e-3
        assert torch.equal(again, out)
    finally:
        eng.close()
