"""Importance-guided eviction on the device: the decode pass's per-page attention mass against the
CPU checker, the score update against what the reference's own ImportanceScorer kernel returned on a
B200 (tests/golden/importance_reference.npz), and eviction that follows the mirrored scores."""
import os

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _tables(eng, seqs):
    t = np.full((len(seqs), eng.table_stride()), -1, dtype=np.int32)
    for i, s in enumerate(seqs):
        row = eng.table(s)
        t[i, :len(row)] = row
    return t


@pytest.mark.parametrize("hq,hkv,d,page,dt", [(32, 8, 128, 16, "bf16"), (16, 2, 128, 64, "f16"), (8, 8, 64, 16, "f16"),
                                              (4, 1, 256, 32, "bf16")])
def test_page_mass_matches_checker(drkv_lib, oracle, hq, hkv, d, page, dt):
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    dtype = ob.BF16 if dt == "bf16" else ob.F16
    tdt = torch.bfloat16 if dt == "bf16" else torch.float16
    layers, max_pages, width = 3, 300, 48
    rng = np.random.default_rng(hq + d + page)
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype=dt,
                        rope_theta=1e6, max_pages=max_pages, max_seqs=8, max_pages_per_seq=width, device=0,
                        stream_evict=True)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        H.shuffled_free_stack(eng, rng)
        lens = [page * 20 + 3, 1, page * 7, page * 33 + page // 2, 17]
        seqs = []
        for n in lens:
            s = eng.seq_create()
            eng.reserve(s, n)
            eng.set_seq_len(s, n)
            seqs.append(s)
        assert eng.evict_blocks(seqs[3], 5) == 5                    # holes: the five oldest pages of one sequence
        eng.scorer_enable(0.9)
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        eng.sync_block_table()
        tables = _tables(eng, seqs)
        n = len(seqs)
        rows = torch.tensor(seqs, dtype=torch.int32, device="cuda")
        d_len = torch.tensor(lens, dtype=torch.int32, device="cuda")
        scale = 1.0 / np.sqrt(d)
        qs = [H.randn_bits(rng, (n, hq, d), dtype) for _ in range(layers)]
        want = np.zeros((n, eng.table_stride()), dtype=np.float64)
        out = torch.zeros(n, hq, d, dtype=tdt, device="cuda")
        for layer in range(layers):
            eng.attend_decode(layer, n, rows, d_len, max(lens), H.to_dev(qs[layer], dtype), out, scale)
            ob.page_mass(g, pool_host, max_pages, tables, np.arange(n), np.array(lens, dtype=np.int32), layer,
                         qs[layer], want, scale)
        eng.scorer_step()
        eng.scorer_sync()
        eng.check_kernels()
        first = np.stack([eng.scorer_scores(s) for s in seqs])
        # every head's probabilities sum to one: layers * heads in total (sequence 3 still has resident keys)
        assert np.allclose(first.sum(axis=1), layers * hq, rtol=2e-5)
        assert np.abs(first - want).max() <= 1e-4 * hq
        assert np.allclose(first, want, rtol=2e-3, atol=1e-5 * hq)
        assert (first[3, :5] == 0).all()                            # evicted pages received nothing
        # second token, same queries: the same masses fold in as score * decay + new, one fused multiply-add
        for layer in range(layers):
            eng.attend_decode(layer, n, rows, d_len, max(lens), H.to_dev(qs[layer], dtype), out, scale)
        eng.scorer_step()
        eng.scorer_sync()
        second = np.stack([eng.scorer_scores(s) for s in seqs])
        expect = first.copy()
        ob.importance_update(expect, first, 0.9)
        assert np.array_equal(second, expect)
        # eviction now takes the lowest-scored resident pages of a sequence, ties by allocation order
        resident = [j for j in range(eng.table_stride()) if tables[0][j] >= 0]
        order = sorted(resident, key=lambda j: (second[0][j], j))
        assert eng.evict_blocks(seqs[0], 4) == 4
        gone = [j for j in resident if eng.table(seqs[0])[j] < 0]
        assert sorted(gone) == sorted(order[:4])
    finally:
        eng.close()


def test_planned_pass_scores_like_the_per_sequence_pass(drkv_lib, oracle):
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    hq, hkv, d, page, dtype = 32, 8, 128, 16, ob.BF16
    rng = np.random.default_rng(77)
    scores = []
    for planned in (False, True):
        eng = PagedKVEngine(num_layers=1, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                            rope_theta=1e6, max_pages=200, max_seqs=8, max_pages_per_seq=64, device=0)
        try:
            eng.scorer_enable(0.5)
            root = eng.seq_create()
            eng.reserve(root, 16 * 30 + 5)
            eng.set_seq_len(root, 16 * 30 + 5)
            seqs = [root] + [eng.seq_fork(root) for _ in range(5)]
            lens = []
            for i, s in enumerate(seqs):
                eng.reserve(s, 3 + 11 * i)
                eng.set_seq_len(s, 16 * 30 + 5 + 3 + 11 * i)
                lens.append(16 * 30 + 5 + 3 + 11 * i)
            prng = np.random.default_rng(5)
            pool_host = H.randn_bits(prng, eng.pool_tensor().numel(), dtype)
            eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
            eng.sync_block_table()
            eng.set_chunk_tokens(64)
            q = H.to_dev(H.randn_bits(prng, (len(seqs), hq, d), dtype), dtype)
            out = torch.zeros(len(seqs), hq, d, dtype=torch.bfloat16, device="cuda")
            if planned:
                info = eng.plan_decode(seqs, lens)
                assert info["n_blocks"] == 2
                eng.attend_decode_planned(0, q, out, 0.088)
            else:
                eng.attend_decode(0, len(seqs), torch.tensor(seqs, dtype=torch.int32, device="cuda"),
                                  torch.tensor(lens, dtype=torch.int32, device="cuda"), max(lens), q, out, 0.088)
            eng.scorer_step()
            eng.scorer_sync()
            eng.check_kernels()
            scores.append(np.stack([eng.scorer_scores(s) for s in seqs]))
        finally:
            eng.close()
    assert np.array_equal(scores[0], scores[1])
    assert np.allclose(scores[0].sum(axis=1), hq, rtol=2e-5)


def test_update_matches_reference_kernel_record(drkv_lib):
    import torch
    from deusridet_b200 import PagedKVEngine
    from tests.golden.make_importance_golden import importance_cases

    gold = np.load(os.path.join(GOLD, "importance_reference.npz"))
    for name, (decay, new) in importance_cases().items():
        steps, n = new.shape
        eng = PagedKVEngine(num_layers=1, num_q_heads=4, num_kv_heads=4, head_dim=128, page_size=16, dtype="bf16",
                            rope_theta=1e6, max_pages=8, max_seqs=2, max_pages_per_seq=n, device=0)
        try:
            eng.scorer_enable(decay)
            eng.seq_create()
            s = eng.seq_create()
            for k in range(steps):
                eng.scorer_update(s, torch.from_numpy(new[k]).cuda())
                eng.scorer_sync()
                assert np.array_equal(eng.scorer_scores(s)[:n], gold[name][k]), f"{name} step {k}"
        finally:
            eng.close()
