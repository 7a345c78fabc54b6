"""Chunked prefill into the paged cache on the device: RoPE + scatter of a chunk's K/V into newly
allocated pages, then causal attention of the chunk over everything cached so far through the
block table (tcgen05 kernel), against the CPU checker."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu

TOL = 2e-3


def _prefill_case(oracle, *, layers, hq, hkv, page, dtype, theta, chunks, seed, d=128, holes=0, on_decode_kernel=False):
    """chunks: list of chunk lengths processed in order from position 0.  on_decode_kernel: the engine is told to run
    chunk attention as one-token decodes on the split-KV decode kernel instead of the tensor-memory kernel."""
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    rng = np.random.default_rng(seed)
    total = int(sum(chunks))
    n_pages = (total + page - 1) // page
    max_pages = n_pages + 7
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page,
                        dtype="f16" if dtype == ob.F16 else "bf16", rope_theta=theta, max_pages=max_pages,
                        max_seqs=2, max_pages_per_seq=n_pages + 2, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, theta)
    tdt = torch.float16 if dtype == ob.F16 else torch.bfloat16
    try:
        eng.set_prefill_on_decode_kernel(on_decode_kernel)
        H.shuffled_free_stack(eng, rng)
        filler = eng.seq_create()            # so that the sequence under test is not table row 0
        seq = eng.seq_create()
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)   # stale contents everywhere
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        scale = 1.0 / np.sqrt(d)
        pos = 0
        for ci, m in enumerate(chunks):
            assert eng.ensure_blocks_for_range(seq, pos, m)
            if holes and ci == len(chunks) - 1:
                assert eng.evict_blocks(seq, holes) == holes
            eng.sync_block_table()
            table = eng.table(seq)
            for layer in range(layers):
                k = H.randn_bits(rng, (m, hkv, d), dtype)
                v = H.randn_bits(rng, (m, hkv, d), dtype)
                q = H.randn_bits(rng, (m, hq, d), dtype)
                out = torch.full((m, hq, d), 5.0, dtype=tdt, device="cuda")
                eng.append_rope_chunk(layer, seq, pos, m, H.to_dev(k, dtype), H.to_dev(v, dtype))
                eng.attend_prefill_chunk(layer, seq, pos, m, H.to_dev(q, dtype), out, scale)
                torch.cuda.synchronize()
                eng.check_kernels()
                ob.append(g, pool_host, max_pages, table, layer, pos, m, k, v, rope=True)
                want = H.torch_bits(torch.full((m, hq, d), 5.0, dtype=tdt)).copy()
                ob.attend_prefill(g, pool_host, max_pages, table, layer, pos, m, q, want, scale)
                got_f, want_f = ob.to_float(H.torch_bits(out), dtype), ob.to_float(want, dtype)
                tol = np.maximum(TOL, H.ulp(want_f, dtype))
                err = np.abs(got_f - want_f)
                bad = np.argwhere(err > tol)
                assert bad.size == 0, (f"chunk {ci} layer {layer}: {len(bad)} elements off, worst {err.max():.4g} at "
                                       f"{np.unravel_index(err.argmax(), err.shape)}")
                # tokens that already see a few hundred keys must meet the plain 2e-3 bound
                deep = np.arange(m) + pos >= 256
                if deep.any():
                    assert err[deep].max() <= TOL
            got_pool = eng.pool_tensor().cpu().numpy().view(np.uint16)
            assert np.array_equal(got_pool, pool_host), f"chunk {ci}: pool bytes differ after the chunk append"
            pos += m
            eng.set_seq_len(seq, pos)
    finally:
        eng.close()


def test_prefill_group7_two_chunks_bf16(drkv_lib, oracle):
    """28 query / 4 KV heads (GQA 7), head_dim 128, bf16, page 16, 2 layers, 2 chunks of 256."""
    _prefill_case(oracle, layers=2, hq=28, hkv=4, page=16, dtype=oracle.BF16, theta=1e6, chunks=[256, 256], seed=21)


def test_prefill_ragged_chunks_group4(drkv_lib, oracle):
    _prefill_case(oracle, layers=1, hq=32, hkv=8, page=16, dtype=oracle.BF16, theta=1e6, chunks=[1, 37, 100, 333, 64],
                  seed=22)


def test_prefill_group8_page64_fp16(drkv_lib, oracle):
    _prefill_case(oracle, layers=1, hq=64, hkv=8, page=64, dtype=oracle.F16, theta=1e4, chunks=[200, 130], seed=23)


def test_prefill_deep_context(drkv_lib, oracle):
    """A 128-token chunk on top of 3000 cached tokens (odd start position)."""
    _prefill_case(oracle, layers=1, hq=28, hkv=4, page=16, dtype=oracle.BF16, theta=1e6, chunks=[3001, 128], seed=24)


def test_prefill_with_evicted_pages(drkv_lib, oracle):
    _prefill_case(oracle, layers=1, hq=16, hkv=4, page=16, dtype=oracle.BF16, theta=1e4, chunks=[300, 90], seed=25,
                  holes=4)


def test_prefill_reference_model_shape_head_dim_256(drkv_lib, oracle):
    """24 query / 4 KV heads, head_dim 256, 256-key pages, partial rotary 64: the reference's own attention shape
    (src/memoria/block_pool.h:34-40): one 128-row tile per CTA, O in 256 of the 512 tensor-memory columns."""
    _prefill_case(oracle, layers=2, hq=24, hkv=4, page=256, dtype=oracle.F16, theta=1e7, chunks=[300, 77, 1], seed=27,
                  d=256)


def test_prefill_head_dim_64_bf16(drkv_lib, oracle):
    _prefill_case(oracle, layers=1, hq=16, hkv=2, page=32, dtype=oracle.BF16, theta=1e4, chunks=[130, 260], seed=28, d=64)


def test_prefill_batch_of_sequences(drkv_lib, oracle):
    """Three sequences at different depths and chunk lengths in one launch."""
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, d, page, dtype = 1, 28, 4, 128, 16, ob.BF16
    rng = np.random.default_rng(26)
    depth, m = [0, 500, 1300], [200, 64, 37]
    max_pages = sum((a + b + page - 1) // page for a, b in zip(depth, m)) + 6
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=max_pages, max_seqs=3, max_pages_per_seq=100, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        H.shuffled_free_stack(eng, rng)
        seqs = [eng.seq_create() for _ in range(3)]
        for s, a, b in zip(seqs, depth, m):
            assert eng.ensure_blocks_for_range(s, 0, a + b)
            eng.set_seq_len(s, a + b)
        eng.sync_block_table()
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        qs = [H.randn_bits(rng, (b, hq, d), dtype) for b in m]
        d_qs = [H.to_dev(x, dtype) for x in qs]
        outs = [torch.zeros(b, hq, d, dtype=torch.bfloat16, device="cuda") for b in m]
        scale = 1.0 / np.sqrt(d)
        eng.attend_prefill_batch(0, seqs, depth, m, d_qs, outs, scale)
        torch.cuda.synchronize()
        eng.check_kernels()
        for i, s in enumerate(seqs):
            want = np.zeros((m[i], hq, d), dtype=np.uint16)
            ob.attend_prefill(g, pool_host, max_pages, eng.table(s), 0, depth[i], m[i], qs[i], want, scale)
            got_f, want_f = ob.to_float(H.torch_bits(outs[i]), dtype), ob.to_float(want, dtype)
            assert (np.abs(got_f - want_f) <= np.maximum(TOL, H.ulp(want_f, dtype))).all(), f"sequence {i}"
    finally:
        eng.close()


@pytest.mark.parametrize("d,hq,hkv,page", [(256, 24, 4, 256), (128, 8, 2, 16), (64, 16, 2, 32)])
def test_prefill_on_the_decode_kernel(drkv_lib, oracle, d, hq, hkv, page):
    """The path a pool takes that one TMA descriptor cannot address (more than 2^31 head rows), selected here by the
    engine switch: the chunk as a batch of one-token decodes over one block table."""
    _prefill_case(oracle, layers=1, hq=hq, hkv=hkv, page=page, dtype=oracle.BF16, theta=1e6, chunks=[200, 77, 1], seed=41,
                  d=d, on_decode_kernel=True)
