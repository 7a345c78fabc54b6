"""Parity of the CUDA path (through the C ABI) with the CPU checker on one decode step:
block tables, appended K/V bytes and attention output."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu

TOL = 2e-3  # max-abs on attention outputs: fp16/bf16 out, fp32 accumulate


def _decode_case(oracle, *, layers, hq, hkv, d, page, dtype, theta, lens, seed, pool_slack=1.1, rot=None,
                 chunk=0, holes=0, fused=False, holes_first_only=False):
    """fused: the step goes through drkv_append_attend_decode (the new token is appended by the attention kernel's
    own work item) instead of the two separate calls."""
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    rng = np.random.default_rng(seed)
    rot = d if rot is None else rot
    lens = np.asarray(lens, dtype=np.int32)
    n_seq = len(lens)
    pages_needed = int(sum((int(n) + 1 + page - 1) // page for n in lens))
    max_pages = max(4, int(np.ceil(pool_slack * pages_needed)))
    width = int(max((int(n) + 1 + page - 1) // page for n in lens)) + 1
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page,
                        dtype="f16" if dtype == ob.F16 else "bf16", rotary_dim=rot, rope_theta=theta,
                        max_pages=max_pages, max_seqs=n_seq, max_pages_per_seq=width, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, rot, theta)
    try:
        if chunk:
            eng.set_chunk_tokens(chunk)
        H.shuffled_free_stack(eng, rng)
        seqs = [eng.seq_create() for _ in range(n_seq)]
        # cached context, then room for the token being decoded
        for s, n in zip(seqs, lens):
            assert eng.ensure_blocks_for_range(s, 0, int(n))
            eng.set_seq_len(s, int(n))
        for s in seqs:
            eng.reserve(s, 1)
        tables = np.stack([eng.table(s) for s in seqs])
        if holes:
            # evicted pages: the table entry becomes -1 and attention must skip it
            for s in (seqs[:1] if holes_first_only else seqs):
                eng.evict_blocks(s, holes)
            tables = np.stack([eng.table(s) for s in seqs])
            assert (tables[:1 if holes_first_only else None, :holes] == -1).all()
        eng.sync_block_table()

        # pool contents: N(0,1) everywhere (also in slots no sequence owns)
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))

        rows = np.asarray(seqs, dtype=np.int32)
        pos = lens.copy()
        d_rows = torch.from_numpy(rows).cuda()
        d_pos = torch.from_numpy(pos).cuda()
        d_len = torch.from_numpy(pos + 1).cuda()
        scale = 1.0 / np.sqrt(d)
        for layer in range(layers):
            k_new = H.randn_bits(rng, (n_seq, hkv, d), dtype)
            v_new = H.randn_bits(rng, (n_seq, hkv, d), dtype)
            q = H.randn_bits(rng, (n_seq, hq, d), dtype)
            out_dev = torch.full((n_seq, hq, d), 7.0, device="cuda",
                                 dtype=torch.float16 if dtype == ob.F16 else torch.bfloat16)
            if fused:
                eng.append_attend_decode(layer, n_seq, d_rows, d_len, int(pos.max()) + 1, H.to_dev(k_new, dtype),
                                         H.to_dev(v_new, dtype), H.to_dev(q, dtype), out_dev, scale)
            else:
                eng.append_rope(layer, n_seq, d_rows, d_pos, H.to_dev(k_new, dtype), H.to_dev(v_new, dtype))
                eng.attend_decode(layer, n_seq, d_rows, d_len, int(pos.max()) + 1, H.to_dev(q, dtype), out_dev, scale)
            torch.cuda.synchronize()
            eng.check_kernels()

            # checker on the host copy
            for i in range(n_seq):
                ob.append(g, pool_host, max_pages, tables[i], layer, int(pos[i]), 1, k_new[i], v_new[i], rope=True)
            want = H.torch_bits(torch.full((n_seq, hq, d), 7.0,
                                           dtype=torch.float16 if dtype == ob.F16 else torch.bfloat16))
            want = want.copy()
            ob.attend_decode(g, pool_host, max_pages, tables, np.arange(n_seq), pos + 1, layer, q, want, scale)

            got_pool = eng.pool_tensor().cpu().numpy().view(np.uint16)
            assert np.array_equal(got_pool, pool_host), f"layer {layer}: pool bytes differ after append"
            got = ob.to_float(H.torch_bits(out_dev), dtype)
            ref = ob.to_float(want, dtype)
            # 2e-3 max-abs; where one unit in the last place of the storage type is itself larger
            # than that (|out| >= 0.25 in bf16, >= 2 in fp16: only the very short sequences here),
            # a one-unit rounding flip is the most two correct fp32 results can differ by.
            tol = np.maximum(TOL, H.ulp(ref, dtype))
            err = np.abs(got - ref)
            exact = ob.attend_decode_f64(g, pool_host, max_pages, tables, np.arange(n_seq), pos + 1, layer, q, scale)
            err64 = np.abs(got - exact).max()
            assert (err <= tol).all(), f"layer {layer}: max-abs {err.max()} vs checker (vs fp64 {err64})"
            long_ctx = pos + 1 >= 512
            if long_ctx.any():
                assert err[long_ctx].max() <= TOL
        return eng.stats()
    finally:
        eng.close()


def test_toy_decode_step_fp16(drkv_lib, oracle):
    """1 layer, 16/4 heads, head_dim 128, fp16, page 16, 512 cached tokens on a seeded page
    permutation of a 64-page pool; append one token (RoPE base 1e4), attend over 513."""
    _decode_case(oracle, layers=1, hq=16, hkv=4, d=128, page=16, dtype=oracle.F16, theta=1e4, lens=[512], seed=1,
                 pool_slack=64 / 33)


def test_batched_decode_bf16_ragged(drkv_lib, oracle):
    """Qwen3-8B-shaped heads (32/8, bf16, page 16, RoPE base 1e6), 2 layers, ragged lengths."""
    _decode_case(oracle, layers=2, hq=32, hkv=8, d=128, page=16, dtype=oracle.BF16, theta=1e6,
                 lens=[1024, 1531, 4097, 2048, 777, 3000, 1, 15, 16, 17], seed=2)


@pytest.mark.parametrize("chunk", [16, 64, 256, 2048])
def test_decode_chunk_sizes(drkv_lib, oracle, chunk):
    _decode_case(oracle, layers=2, hq=32, hkv=8, d=128, page=16, dtype=oracle.BF16, theta=1e6,
                 lens=[1200, 63, 64, 65, 2500], seed=3, chunk=chunk)


def test_decode_group8_page64(drkv_lib, oracle):
    """64/8 heads (GQA 8), page 64: the long-context configuration's head shape."""
    _decode_case(oracle, layers=1, hq=64, hkv=8, d=128, page=64, dtype=oracle.BF16, theta=1e6, lens=[3000, 64, 129],
                 seed=4)


def test_decode_group16(drkv_lib, oracle):
    _decode_case(oracle, layers=1, hq=32, hkv=2, d=128, page=16, dtype=oracle.F16, theta=1e4, lens=[700, 33], seed=5)


def test_decode_reference_model_shape(drkv_lib, oracle):
    """The reference's own geometry: 24/4 heads, head_dim 256, page 256, partial rotary 64, fp16
    (src/memoria/block_pool.h:34-40, src/machina/model.h)."""
    _decode_case(oracle, layers=1, hq=24, hkv=4, d=256, page=256, dtype=oracle.F16, theta=1e7, lens=[1000, 300],
                 seed=6, rot=64)


def test_decode_head_dim_64(drkv_lib, oracle):
    _decode_case(oracle, layers=1, hq=8, hkv=2, d=64, page=32, dtype=oracle.BF16, theta=1e4, lens=[500, 100], seed=7)


def test_decode_with_evicted_pages(drkv_lib, oracle):
    """Holes in the table (evicted pages) contribute nothing."""
    _decode_case(oracle, layers=1, hq=16, hkv=4, d=128, page=16, dtype=oracle.BF16, theta=1e4, lens=[600, 900],
                 seed=8, holes=3)


# ---- the same step through the fused entry point: pool bytes and outputs must not change ----
def test_fused_append_toy_fp16(drkv_lib, oracle):
    _decode_case(oracle, layers=1, hq=16, hkv=4, d=128, page=16, dtype=oracle.F16, theta=1e4, lens=[512], seed=1,
                 pool_slack=64 / 33, fused=True)


def test_fused_append_batched_bf16_ragged(drkv_lib, oracle):
    """Lengths around page and chunk boundaries: the new token is the first slot of a fresh page (16, 1024, 2048),
    the last slot of one (15, 4095), the only key of its sequence (0)."""
    _decode_case(oracle, layers=2, hq=32, hkv=8, d=128, page=16, dtype=oracle.BF16, theta=1e6,
                 lens=[1024, 1531, 4095, 2048, 777, 3000, 0, 1, 15, 16, 17], seed=2, fused=True)


@pytest.mark.parametrize("chunk", [16, 64, 2048])
def test_fused_append_chunk_sizes(drkv_lib, oracle, chunk):
    _decode_case(oracle, layers=2, hq=32, hkv=8, d=128, page=16, dtype=oracle.BF16, theta=1e6,
                 lens=[1200, 63, 64, 65, 2500], seed=3, chunk=chunk, fused=True)


def test_fused_append_deep_batch_with_tail_pieces(drkv_lib, oracle):
    """A batch deep enough for 512-key items with the last chunk of every sequence in 64-key pieces: the piece
    that ends the sequence does the append."""
    lens = np.random.default_rng(9).integers(3600, 4400, size=64)
    _decode_case(oracle, layers=1, hq=32, hkv=8, d=128, page=16, dtype=oracle.BF16, theta=1e6, lens=lens, seed=9,
                 fused=True)


def test_fused_append_group8_page64_partial_rotary(drkv_lib, oracle):
    _decode_case(oracle, layers=1, hq=64, hkv=8, d=128, page=64, dtype=oracle.BF16, theta=1e6, lens=[3000, 64, 129],
                 seed=4, rot=64, fused=True)


def test_fused_append_head_dim_64(drkv_lib, oracle):
    _decode_case(oracle, layers=1, hq=8, hkv=2, d=64, page=32, dtype=oracle.BF16, theta=1e4, lens=[500, 100], seed=7,
                 fused=True)


def test_fused_append_head_dim_256(drkv_lib, oracle):
    _decode_case(oracle, layers=1, hq=24, hkv=4, d=256, page=256, dtype=oracle.F16, theta=1e7, lens=[1000, 300],
                 seed=6, rot=64, fused=True)


def test_fused_append_into_a_hole_writes_nothing(drkv_lib, oracle):
    """The first sequence's only page is evicted: its token has no page to go to, nothing is written and its output
    rows stay as they were; the other sequence is unaffected."""
    _decode_case(oracle, layers=1, hq=16, hkv=4, d=128, page=16, dtype=oracle.BF16, theta=1e4, lens=[5, 900], seed=10,
                 holes=1, holes_first_only=True, fused=True)


@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_head_dim_256_with_lengths_known_on_the_host(drkv_lib, oracle, dt):
    """A plan gives the lengths on the host; when every sequence has more than 1 024 keys the head_dim 256 pass
    feeds P to the PV product in the storage type alone (no residue term).  Same bound against the CPU checker, and
    within it of the pass that takes its lengths from the device and keeps the term."""
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    dtype = ob.BF16 if dt == "bf16" else ob.F16
    tdt = torch.bfloat16 if dt == "bf16" else torch.float16
    layers, hq, hkv, d, page = 1, 24, 4, 256, 256
    lens = np.array([1500, 3000, 1025, 5000], dtype=np.int32)
    n = len(lens)
    rng = np.random.default_rng(256)
    max_pages = int(sum((int(x) + page - 1) // page for x in lens)) + 4
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype=dt,
                        rotary_dim=64, rope_theta=1e7, max_pages=max_pages, max_seqs=n, max_pages_per_seq=24, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, 64, 1e7)
    try:
        H.shuffled_free_stack(eng, rng)
        seqs = [eng.seq_create() for _ in range(n)]
        for s, x in zip(seqs, lens):
            assert eng.ensure_blocks_for_range(s, 0, int(x))
            eng.set_seq_len(s, int(x))
        eng.sync_block_table()
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        tables = np.stack([eng.table(s) for s in seqs])
        q = H.randn_bits(rng, (n, hq, d), dtype)
        scale = 1.0 / np.sqrt(d)
        eng.plan_decode(seqs, lens.tolist())
        planned = torch.zeros(n, hq, d, dtype=tdt, device="cuda")
        eng.attend_decode_planned(0, H.to_dev(q, dtype), planned, scale)
        rows = torch.tensor(seqs, dtype=torch.int32, device="cuda")
        d_len = torch.from_numpy(lens).cuda()
        plain = torch.zeros_like(planned)
        eng.attend_decode(0, n, rows, d_len, int(lens.max()), H.to_dev(q, dtype), plain, scale)
        torch.cuda.synchronize()
        eng.check_kernels()
        want = np.zeros((n, hq, d), dtype=np.uint16)
        ob.attend_decode(g, pool_host, max_pages, tables, np.arange(n), lens, 0, q, want, scale)
        ref = ob.to_float(want, dtype)
        assert np.abs(ob.to_float(H.torch_bits(planned), dtype) - ref).max() <= TOL
        assert np.abs(ob.to_float(H.torch_bits(plain), dtype) - ref).max() <= TOL
        assert (planned.float() - plain.float()).abs().max().item() <= TOL
    finally:
        eng.close()
