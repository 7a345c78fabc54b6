"""Planned decode over forked branches: the pages a family of branches has in common are attended once
per 16 query rows of the family instead of once per branch.  The output must match the CPU checker
within 2e-3 and, with the chunk size pinned, the per-sequence pass bit for bit (every query row sees
the same keys in the same chunks; only the grouping of rows into tensor-core tiles differs)."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _build_batch(eng, rng, page, families, singles):
    """families: list of (prefix_tokens, [private tokens per branch]); singles: list of lengths.
    Returns batch order (sequence ids) and lengths; siblings of a family are consecutive."""
    seqs, lens = [], []
    for prefix, privates in families:
        root = eng.seq_create()
        eng.reserve(root, prefix)
        eng.set_seq_len(root, prefix)
        members = [root] + [eng.seq_fork(root) for _ in privates[1:]]
        for s, extra in zip(members, privates):
            if extra:
                eng.reserve(s, extra)
                eng.set_seq_len(s, prefix + extra)
            seqs.append(s)
            lens.append(prefix + extra)
    for n in singles:
        s = eng.seq_create()
        eng.reserve(s, n)
        eng.set_seq_len(s, n)
        seqs.append(s)
        lens.append(n)
    return seqs, lens


CASES = [
    # hq, hkv, d, page, dtype, families, singles, forced chunk
    (32, 8, 128, 16, "bf16", [(16 * 40 + 5, [3, 0, 17, 60, 1, 9]), (16 * 9, [1, 2])], [70, 1], 64),
    (32, 8, 128, 64, "bf16", [(64 * 11 + 63, [1, 130, 7, 64, 2, 300, 5, 9, 11])], [], 128),
    (16, 2, 128, 16, "f16", [(16 * 30, [4, 5, 6]), (16 * 13 + 1, [0, 0])], [200], 64),
    (8, 4, 64, 32, "f16", [(32 * 20 + 7, [1] * 11)], [33], 64),
    (8, 8, 256, 16, "bf16", [(16 * 12, [2] * 17)], [], 64),
    (32, 8, 128, 16, "bf16", [(16 * 40 + 5, [3, 0, 17, 60])], [50], 0),          # automatic chunk
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"hq{c[0]}kv{c[1]}d{c[2]}p{c[3]}{c[4]}c{c[7]}")
def test_planned_pass_matches_checker_and_per_sequence_pass(drkv_lib, oracle, case):
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    hq, hkv, d, page, dt, families, singles, chunk = case
    dtype = ob.BF16 if dt == "bf16" else ob.F16
    tdt = torch.bfloat16 if dt == "bf16" else torch.float16
    layers, max_pages, width = 2, 400, 64
    rng = np.random.default_rng(hq * 1000 + d + page)
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype=dt,
                        rope_theta=1e6, max_pages=max_pages, max_seqs=64, max_pages_per_seq=width, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        H.shuffled_free_stack(eng, rng)
        seqs, lens = _build_batch(eng, rng, page, families, singles)
        n = len(seqs)
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        eng.sync_block_table()
        tables = np.full((n, eng.table_stride()), -1, dtype=np.int32)
        for i, sq in enumerate(seqs):
            t = eng.table(sq)
            tables[i, :len(t)] = t
        if chunk:
            eng.set_chunk_tokens(chunk)
        info = eng.plan_decode(seqs, lens)
        assert info["n_seq"] == n
        assert info["n_families"] == len(families)
        assert info["keys_per_sequence_pass"] == sum(lens)
        assert info["keys_planned_pass"] < info["keys_per_sequence_pass"]
        if chunk:
            per_block = 16 // (hq // hkv)
            want_blocks, want_keys, at = 0, 0, 0
            for prefix, privates in families:
                # shared keys of a family, from the tables read back: leading pages equal to the first
                # member's (a branch that wrote nothing after the fork still shares the partial tail page)
                fam = range(at, at + len(privates))
                at += len(privates)
                shared = lens[fam[0]]
                for i in fam[1:]:
                    same = 0
                    while same < tables.shape[1] and tables[i][same] >= 0 and tables[i][same] == tables[fam[0]][same]:
                        same += 1
                    shared = min(shared, same * page, lens[i])
                assert shared >= prefix // page * page
                sc = shared // chunk
                nb = -(-len(privates) // per_block)
                want_blocks += nb
                want_keys += nb * sc * chunk + sum(prefix + e - sc * chunk for e in privates)
            want_keys += sum(singles)
            assert info["n_blocks"] == want_blocks
            assert info["keys_planned_pass"] == want_keys
        rows = torch.tensor(seqs, dtype=torch.int32, device="cuda")
        d_len = torch.tensor(lens, dtype=torch.int32, device="cuda")
        scale = 1.0 / np.sqrt(d)
        for layer in range(layers):
            q = H.randn_bits(rng, (n, hq, d), dtype)
            dq = H.to_dev(q, dtype)
            planned = torch.zeros(n, hq, d, dtype=tdt, device="cuda")
            plain = torch.zeros(n, hq, d, dtype=tdt, device="cuda")
            eng.attend_decode_planned(layer, dq, planned, scale)
            eng.attend_decode(layer, n, rows, d_len, max(lens), dq, plain, scale)
            want = np.zeros((n, hq, d), dtype=np.uint16)
            ob.attend_decode(g, pool_host, max_pages, tables, np.arange(n), np.array(lens, dtype=np.int32), layer, q,
                             want, scale)
            torch.cuda.synchronize()
            eng.check_kernels()
            err = np.abs(ob.to_float(H.torch_bits(planned), dtype) - ob.to_float(want, dtype)).max()
            assert err <= 2e-3, f"layer {layer}: {err}"
            if chunk:
                assert np.array_equal(H.torch_bits(planned), H.torch_bits(plain)), f"layer {layer}"
    finally:
        eng.close()


@pytest.mark.parametrize("case", [CASES[0], CASES[1], CASES[3], CASES[4], CASES[5]],
                         ids=lambda c: f"hq{c[0]}kv{c[1]}d{c[2]}p{c[3]}{c[4]}c{c[7]}")
def test_planned_pass_with_the_append_in_the_same_call(drkv_lib, oracle, case):
    """Every branch decodes one token: room is reserved (copy-on-write of a shared partial tail page), the plan
    counts the token, and one call per layer appends it and attends.  Pool bytes must equal the checker's append
    bit for bit and the outputs its attention within 2e-3."""
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    hq, hkv, d, page, dt, families, singles, chunk = case
    dtype = ob.BF16 if dt == "bf16" else ob.F16
    tdt = torch.bfloat16 if dt == "bf16" else torch.float16
    layers, max_pages, width = 2, 400, 64
    rng = np.random.default_rng(hq * 1000 + d + page + 1)
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype=dt,
                        rope_theta=1e6, max_pages=max_pages, max_seqs=64, max_pages_per_seq=width, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        H.shuffled_free_stack(eng, rng)
        seqs, lens = _build_batch(eng, rng, page, families, singles)
        n = len(seqs)
        for sq in seqs:
            eng.reserve(sq, 1)                                   # a page of its own where the token lands
        torch.cuda.synchronize()
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        eng.sync_block_table()
        tables = np.full((n, eng.table_stride()), -1, dtype=np.int32)
        for i, sq in enumerate(seqs):
            t = eng.table(sq)
            tables[i, :len(t)] = t
        if chunk:
            eng.set_chunk_tokens(chunk)
        new_lens = [x + 1 for x in lens]
        info = eng.plan_decode(seqs, new_lens)
        assert info["n_families"] == len(families)
        scale = 1.0 / np.sqrt(d)
        for layer in range(layers):
            q = H.randn_bits(rng, (n, hq, d), dtype)
            k_new = H.randn_bits(rng, (n, hkv, d), dtype)
            v_new = H.randn_bits(rng, (n, hkv, d), dtype)
            got = torch.zeros(n, hq, d, dtype=tdt, device="cuda")
            eng.append_attend_decode_planned(layer, H.to_dev(k_new, dtype), H.to_dev(v_new, dtype), H.to_dev(q, dtype),
                                             got, scale)
            torch.cuda.synchronize()
            eng.check_kernels()
            for i in range(n):
                ob.append(g, pool_host, max_pages, tables[i], layer, lens[i], 1, k_new[i], v_new[i], rope=True)
            want = np.zeros((n, hq, d), dtype=np.uint16)
            ob.attend_decode(g, pool_host, max_pages, tables, np.arange(n), np.array(new_lens, dtype=np.int32), layer,
                             q, want, scale)
            got_pool = eng.pool_tensor().cpu().numpy().view(np.uint16)
            assert np.array_equal(got_pool, pool_host), f"layer {layer}: pool bytes differ after the append"
            ref = ob.to_float(want, dtype)
            err = np.abs(ob.to_float(H.torch_bits(got), dtype) - ref)
            assert (err <= np.maximum(2e-3, H.ulp(ref, dtype))).all(), f"layer {layer}: {err.max()}"
    finally:
        eng.close()


def test_plan_without_families_is_the_per_sequence_pass(drkv_lib, oracle):
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    hq, hkv, d, page, dtype = 32, 8, 128, 16, ob.BF16
    rng = np.random.default_rng(5)
    eng = PagedKVEngine(num_layers=1, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=200, max_seqs=16, max_pages_per_seq=32, device=0)
    try:
        seqs, lens = _build_batch(eng, rng, page, [], [100, 37, 480, 1, 16])
        pool_host = H.randn_bits(rng, eng.pool_tensor().numel(), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        eng.sync_block_table()
        info = eng.plan_decode(seqs, lens)
        assert info["n_families"] == 0 and info["n_blocks"] == 0
        assert info["keys_planned_pass"] == info["keys_per_sequence_pass"] == sum(lens)
        eng.set_chunk_tokens(info["chunk_tokens"])
        n = len(seqs)
        q = H.to_dev(H.randn_bits(rng, (n, hq, d), dtype), dtype)
        a = torch.zeros(n, hq, d, dtype=torch.bfloat16, device="cuda")
        b = torch.zeros_like(a)
        eng.attend_decode_planned(0, q, a, 0.088)
        eng.attend_decode(0, n, torch.tensor(seqs, dtype=torch.int32, device="cuda"),
                          torch.tensor(lens, dtype=torch.int32, device="cuda"), max(lens), q, b, 0.088)
        torch.cuda.synchronize()
        eng.check_kernels()
        assert torch.equal(a, b)
    finally:
        eng.close()


def test_plan_rejects_bad_input(drkv_lib):
    from deusridet_b200 import PagedKVEngine

    eng = PagedKVEngine(num_layers=1, num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, dtype="bf16",
                        rope_theta=1e6, max_pages=32, max_seqs=4, max_pages_per_seq=8, device=0)
    try:
        import torch
        x = torch.zeros(8, 128, dtype=torch.bfloat16, device="cuda")
        with pytest.raises(RuntimeError, match="no decode plan"):
            eng.attend_decode_planned(0, x, x, 1.0)
        with pytest.raises(RuntimeError, match="not a live sequence"):
            eng.plan_decode([3], [5])
        s = eng.seq_create()
        with pytest.raises(RuntimeError, match="longer than a block table"):
            eng.plan_decode([s], [16 * 8 + 1])
    finally:
        eng.close()
