"""The benchmark configurations at their full batch, context and head shapes (two layers where a configuration has
dozens of identical ones), checked through properties that do not need the CPU checker to walk every key, plus the
checker on a sample:

* the split of a sequence into work items must not matter: automatic chunking with its tail split against 64-key
  items without one, and K/V ranges of 2, 4 and 8 ranks merged against the whole range (the log-sum-exp merge is
  exact up to rounding);
* the order of a batch must not matter: every sequence's rows are bit-identical when the batch is reversed;
* an append is idempotent: appending the same token again leaves a checksum of the whole pool unchanged;
* a chunk token of the prefill path sees exactly what a decode call with that many keys sees;
* the CPU checker agrees on the shortest, the longest and two other sequences (or on the whole single sequence)."""
import numpy as np
import pytest

from deusridet_b200 import sharding
from tests import helpers as H

pytestmark = pytest.mark.gpu

TOL = 2e-3


def _pool_checksum(eng):
    import torch
    t = eng.pool_tensor().view(torch.int16)
    # sum of the 16-bit words and of word x position weight: a swapped pair of rows changes the second
    s1 = int(t.to(torch.int64).sum().item())
    w = (torch.arange(t.numel(), device=t.device, dtype=torch.int64) % 65521) + 1
    s2 = int((t.to(torch.int64).flatten() * w).sum().item())
    return s1, s2


def test_batched_decode_at_full_size(drkv_lib, oracle):
    """64 sequences of U[1024, 8192] cached tokens, 32/8 heads, head_dim 128, bf16, page 16, pool of 1.1 x the pages
    handed out in a seeded shuffle (the Qwen3-8B-shaped decode configuration); 2 of its 36 identical layers."""
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, d, page, dtype = 2, 32, 8, 128, 16, ob.BF16
    rng = np.random.default_rng(1234)
    lens = rng.integers(1024, 8193, size=64).astype(np.int32)
    n = len(lens)
    pages_needed = int(sum((int(x) + 1 + page - 1) // page for x in lens))
    max_pages = int(np.ceil(1.1 * pages_needed))
    width = int(max((int(x) + 1 + page - 1) // page for x in lens)) + 1
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=max_pages, max_seqs=n, max_pages_per_seq=width, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        H.shuffled_free_stack(eng, rng)
        seqs = [eng.seq_create() for _ in range(n)]
        for s, x in zip(seqs, lens):
            assert eng.ensure_blocks_for_range(s, 0, int(x) + 1)
            eng.set_seq_len(s, int(x))
        eng.sync_block_table()
        torch.manual_seed(5)
        eng.pool_tensor().view(torch.bfloat16).normal_()
        rows = torch.tensor(seqs, dtype=torch.int32, device="cuda")
        d_len = torch.from_numpy(lens + 1).cuda()
        d_pos = torch.from_numpy(lens.copy()).cuda()
        max_kv = int(lens.max()) + 1
        scale = 1.0 / np.sqrt(d)
        layer = 1
        q = torch.randn(n, hq, d, dtype=torch.bfloat16, device="cuda")
        k_new = torch.randn(n, hkv, d, dtype=torch.bfloat16, device="cuda")
        v_new = torch.randn(n, hkv, d, dtype=torch.bfloat16, device="cuda")

        # the step as the benchmark runs it: append inside the attention launch, automatic chunking
        out = torch.zeros(n, hq, d, dtype=torch.bfloat16, device="cuda")
        eng.append_attend_decode(layer, n, rows, d_len, max_kv, k_new, v_new, q, out, scale)
        torch.cuda.synchronize()
        eng.check_kernels()
        sum_after_append = _pool_checksum(eng)

        # idempotence: the same token again, through the append kernel this time, changes no byte of the pool
        eng.append_rope(layer, n, rows, d_pos, k_new, v_new)
        torch.cuda.synchronize()
        assert _pool_checksum(eng) == sum_after_append

        # the split into items must not matter: 64-key items, no tail split
        eng.set_chunk_tokens(64)
        eng.set_tail_split(0)
        out64 = torch.zeros_like(out)
        eng.attend_decode(layer, n, rows, d_len, max_kv, q, out64, scale)
        eng.set_chunk_tokens(0)
        eng.set_tail_split(-1)
        torch.cuda.synchronize()
        assert (out.float() - out64.float()).abs().max().item() <= TOL

        # the order of the batch must not matter: same kernel configuration, reversed batch, identical bits per row
        rev = torch.arange(n - 1, -1, -1, device="cuda")
        out_rev = torch.zeros_like(out)
        eng.attend_decode(layer, n, rows[rev].contiguous(), d_len[rev].contiguous(), max_kv, q[rev].contiguous(), out_rev, scale)
        out_fwd = torch.zeros_like(out)
        eng.attend_decode(layer, n, rows, d_len, max_kv, q, out_fwd, scale)
        torch.cuda.synchronize()
        eng.check_kernels()
        assert torch.equal(out_rev[rev].view(torch.int16), out_fwd.view(torch.int16))
        assert (out_fwd.float() - out.float()).abs().max().item() <= TOL     # fused append against separate launches

        # the CPU checker on four of the sequences
        pool_host = H.torch_bits(eng.pool_tensor())
        sample = sorted({int(np.argmin(lens)), int(np.argmax(lens)), 7, 40})
        tables = np.stack([eng.table(seqs[i]) for i in sample])
        want = np.zeros((len(sample), hq, d), dtype=np.uint16)
        ob.attend_decode(g, pool_host, max_pages, tables, np.arange(len(sample)), (lens[sample] + 1).astype(np.int32), layer,
                         H.torch_bits(q[sample]), want, scale)
        err = np.abs(ob.to_float(H.torch_bits(out[sample]), dtype) - ob.to_float(want, dtype)).max()
        assert err <= TOL, err
    finally:
        eng.close()


def test_long_sequence_split_at_full_size(drkv_lib, oracle):
    """One 524 288-token sequence, 64/8 heads, head_dim 128, bf16, page 64 (the long-context configuration), one of
    its 8 identical layers: the partials of 2, 4 and 8 contiguous page ranges merge to the attention over the whole
    sequence, which the CPU checker confirms."""
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, d, page, dtype, S = 1, 64, 8, 128, 64, ob.BF16, 524288
    n_pages = S // page
    max_pages = n_pages + 8
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=max_pages, max_seqs=1, max_pages_per_seq=n_pages + 1, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        rng = np.random.default_rng(77)
        H.shuffled_free_stack(eng, rng)
        s = eng.seq_create()
        assert eng.ensure_blocks_for_range(s, 0, S)
        eng.set_seq_len(s, S)
        eng.sync_block_table()
        torch.manual_seed(6)
        eng.pool_tensor().view(torch.bfloat16).normal_()
        q = torch.randn(hq, d, dtype=torch.bfloat16, device="cuda")
        scale = 1.0 / np.sqrt(d)
        rows = torch.tensor([s], dtype=torch.int32, device="cuda")
        d_len = torch.tensor([S], dtype=torch.int32, device="cuda")
        whole = torch.zeros(1, hq, d, dtype=torch.bfloat16, device="cuda")
        eng.attend_decode(0, 1, rows, d_len, S, q.view(1, hq, d), whole, scale)
        nf = eng.partial_floats()
        for world in (2, 4, 8):
            gathered = torch.zeros(world, nf, dtype=torch.float32, device="cuda")
            covered = 0
            for r in range(world):
                begin, end = sharding.key_range_for_rank(S, page, r, world)
                assert begin == covered
                covered = end
                eng.attend_partial(0, s, begin, end, q, gathered[r], scale)
            assert covered == S
            merged = torch.zeros(hq, d, dtype=torch.bfloat16, device="cuda")
            eng.combine_partials(world, gathered, merged, None)
            torch.cuda.synchronize()
            eng.check_kernels()
            assert (merged.float() - whole[0].float()).abs().max().item() <= TOL, world
        pool_host = H.torch_bits(eng.pool_tensor())
        want = np.zeros((1, hq, d), dtype=np.uint16)
        ob.attend_decode(g, pool_host, max_pages, eng.table(s)[None, :], np.arange(1), np.array([S], dtype=np.int32), 0,
                         H.torch_bits(q.view(1, hq, d)), want, scale)
        err = np.abs(ob.to_float(H.torch_bits(whole), dtype) - ob.to_float(want, dtype)).max()
        assert err <= TOL, err
    finally:
        eng.close()


@pytest.mark.parametrize("hq,hkv,d,page", [(28, 4, 128, 16), (24, 4, 256, 256)], ids=["c4_shape", "reference_model_shape"])
def test_chunked_prefill_at_full_size(drkv_lib, oracle, hq, hkv, d, page):
    """A 32 768-token sequence prefilled in 2 048-token chunks, 28/4 heads, head_dim 128, bf16, page 16 (the chunked
    prefill configuration) and 24/4 heads, head_dim 256, 256-key pages (the reference model's own attention shape), one
    of the identical layers: every chunk is appended and attended; tokens of the first, a middle and the last chunk
    must see exactly what a decode call with that many keys sees."""
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, S, C = 1, 32768, 2048
    n_pages = S // page
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=n_pages + 8, max_seqs=1, max_pages_per_seq=n_pages + 1, device=0)
    try:
        rng = np.random.default_rng(78)
        H.shuffled_free_stack(eng, rng)
        s = eng.seq_create()
        torch.manual_seed(7)
        scale = 1.0 / np.sqrt(d)
        kept = {}
        for pos in range(0, S, C):
            assert eng.ensure_blocks_for_range(s, pos, C)
            eng.sync_block_table()
            k = torch.randn(C, hkv, d, dtype=torch.bfloat16, device="cuda")
            v = torch.randn(C, hkv, d, dtype=torch.bfloat16, device="cuda")
            q = torch.randn(C, hq, d, dtype=torch.bfloat16, device="cuda")
            out = torch.zeros(C, hq, d, dtype=torch.bfloat16, device="cuda")
            eng.append_rope_chunk(0, s, pos, C, k, v)
            eng.attend_prefill_chunk(0, s, pos, C, q, out, scale)
            eng.set_seq_len(s, pos + C)
            if pos in (0, 8 * C, S - C):
                kept[pos] = (q, out)
        torch.cuda.synchronize()
        eng.check_kernels()
        rows = torch.tensor([s], dtype=torch.int32, device="cuda")
        for pos, (q, out) in kept.items():
            for t in (0, 1, 63, 64, 1000, C - 1):
                n_keys = pos + t + 1
                d_len = torch.tensor([n_keys], dtype=torch.int32, device="cuda")
                dec = torch.zeros(1, hq, d, dtype=torch.bfloat16, device="cuda")
                eng.attend_decode(0, 1, rows, d_len, n_keys, q[t:t + 1].contiguous(), dec, scale)
                torch.cuda.synchronize()
                ref = dec[0].float()
                err = (out[t].float() - ref).abs()
                tol = torch.clamp(torch.from_numpy(H.ulp(ref.cpu().numpy(), ob.BF16)).cuda().float(), min=TOL)
                assert bool((err <= tol).all()), (pos, t, err.max().item())
                if n_keys >= 256:
                    assert err.max().item() <= TOL, (pos, t, err.max().item())
        eng.check_kernels()
    finally:
        eng.close()


def test_forked_branches_at_full_size(drkv_lib, oracle):
    """Eight decode branches forked from one 16 384-token prompt (minus five tokens, so that the shared tail page is
    partial and every branch copies it on its first write), private tails of U[0, 2048] tokens, 32/8 heads, head_dim
    128, bf16, page 16 (the prefix-sharing configuration), 2 of its 32 identical layers: the planned pass, which reads
    the shared pages once per 16 query rows, with the append inside it, must give what the per-sequence pass gives,
    and the CPU checker agrees on the shortest and the longest branch."""
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, d, page, dtype, prefix, n = 2, 32, 8, 128, 16, ob.BF16, 16384 - 5, 8
    rng = np.random.default_rng(79)
    private = rng.integers(0, 2049, size=n)
    max_pages = (prefix + page - 1) // page + int(sum((int(x) + 2 * page + 16) // page for x in private)) + 16
    width = (prefix + int(private.max())) // page + 4
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=max_pages, max_seqs=n, max_pages_per_seq=width, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        H.shuffled_free_stack(eng, rng)
        root = eng.seq_create()
        eng.reserve(root, prefix)
        eng.set_seq_len(root, prefix)
        seqs = [root] + [eng.seq_fork(root) for _ in range(n - 1)]
        assert int(eng.refcounts().max()) == n                         # the prompt's pages are shared by all eight
        lens = []
        for s, x in zip(seqs, private):
            eng.reserve(s, int(x) + 1)                                  # private tail + room for the token being decoded
            eng.set_seq_len(s, prefix + int(x))
            lens.append(prefix + int(x))
        assert eng.stats()["cow_copies"] >= n - 1                       # every branch but the last holder copied the tail page
        torch.cuda.synchronize()
        eng.sync_block_table()
        torch.manual_seed(8)
        eng.pool_tensor().view(torch.bfloat16).normal_()
        lens = np.asarray(lens, dtype=np.int32)
        info = eng.plan_decode(seqs, (lens + 1).tolist())
        assert info["n_families"] == 1 and info["keys_planned_pass"] < info["keys_per_sequence_pass"] // 3
        rows = torch.tensor(seqs, dtype=torch.int32, device="cuda")
        d_len = torch.from_numpy(lens + 1).cuda()
        scale = 1.0 / np.sqrt(d)
        layer = 1
        q = torch.randn(n, hq, d, dtype=torch.bfloat16, device="cuda")
        k_new = torch.randn(n, hkv, d, dtype=torch.bfloat16, device="cuda")
        v_new = torch.randn(n, hkv, d, dtype=torch.bfloat16, device="cuda")
        planned = torch.zeros(n, hq, d, dtype=torch.bfloat16, device="cuda")
        eng.append_attend_decode_planned(layer, k_new, v_new, q, planned, scale)
        plain = torch.zeros_like(planned)
        eng.attend_decode(layer, n, rows, d_len, int(lens.max()) + 1, q, plain, scale)   # the token is in the pool by now
        torch.cuda.synchronize()
        eng.check_kernels()
        assert (planned.float() - plain.float()).abs().max().item() <= TOL
        pool_host = H.torch_bits(eng.pool_tensor())
        sample = sorted({int(np.argmin(lens)), int(np.argmax(lens))})
        tables = np.stack([eng.table(seqs[i]) for i in sample])
        want = np.zeros((len(sample), hq, d), dtype=np.uint16)
        ob.attend_decode(g, pool_host, max_pages, tables, np.arange(len(sample)), (lens[sample] + 1).astype(np.int32), layer,
                         H.torch_bits(q[sample]), want, scale)
        err = np.abs(ob.to_float(H.torch_bits(planned[sample]), dtype) - ob.to_float(want, dtype)).max()
        assert err <= TOL, err
    finally:
        eng.close()
