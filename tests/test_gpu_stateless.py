"""The reference's free functions as raw-pointer entry points (paged_kv_cache_write,
paged_kv_cache_write_batch, paged_gqa_decode_attention; src/machina/paged_attention.h:27-71):
one sequence, one table, no RoPE inside the write."""
import ctypes as C

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _run(oracle, drkv_lib, *, hq, hkv, d, page, dtype, seq_len, m_batch, seed, layers=2):
    import torch
    from deusridet_b200 import capi

    ob = oracle
    rng = np.random.default_rng(seed)
    n_pages = (seq_len + m_batch + 1 + page - 1) // page
    max_pages = n_pages + 5
    g = ob.geom(layers, hq, hkv, d, page, dtype, 0, 1e4)
    cg = capi.Geometry(layers, hq, hkv, d, page, dtype, 0, 1e4)
    table = rng.permutation(max_pages)[:n_pages].astype(np.int32)
    pool = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
    tdt = torch.float16 if dtype == ob.F16 else torch.bfloat16
    d_pool = torch.from_numpy(pool.view(np.int16)).cuda()
    d_table = torch.from_numpy(table).cuda()
    layer = layers - 1
    scale = 1.0 / np.sqrt(d)

    # batched write of m_batch tokens at seq_len, then a single-token write with the position on the device
    kb, vb = H.randn_bits(rng, (m_batch, hkv, d), dtype), H.randn_bits(rng, (m_batch, hkv, d), dtype)
    k1, v1 = H.randn_bits(rng, (1, hkv, d), dtype), H.randn_bits(rng, (1, hkv, d), dtype)
    d_kb, d_vb, d_k1, d_v1 = (H.to_dev(x, dtype) for x in (kb, vb, k1, v1))
    rc = drkv_lib.drkv_k_cache_write_batch(C.byref(cg), d_kb.data_ptr(), d_vb.data_ptr(), d_pool.data_ptr(),
                                           d_table.data_ptr(), layer, seq_len, m_batch, max_pages, None)
    assert rc == 0, capi.last_error()
    d_pos = torch.tensor([seq_len + m_batch], dtype=torch.int32, device="cuda")
    rc = drkv_lib.drkv_k_cache_write(C.byref(cg), d_k1.data_ptr(), d_v1.data_ptr(), d_pool.data_ptr(),
                                     d_table.data_ptr(), layer, d_pos.data_ptr(), max_pages, None)
    assert rc == 0, capi.last_error()
    ob.append(g, pool, max_pages, table, layer, seq_len, m_batch, kb, vb, rope=False)
    ob.append(g, pool, max_pages, table, layer, seq_len + m_batch, 1, k1, v1, rope=False)
    torch.cuda.synchronize()
    assert np.array_equal(d_pool.cpu().numpy().view(np.uint16), pool)

    total = seq_len + m_batch + 1
    q = H.randn_bits(rng, (1, hq, d), dtype)
    need = drkv_lib.drkv_k_decode_scratch_bytes(C.byref(cg), total)
    assert need > 0
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    out = torch.zeros(1, hq, d, dtype=tdt, device="cuda")
    want = np.zeros((1, hq, d), dtype=np.uint16)
    ob.attend_decode(g, pool, max_pages, table[None, :], [0], [total], layer, q, want, scale)
    for _ in range(2):   # twice: the scratch header is re-initialised by every call
        out.zero_()
        rc = drkv_lib.drkv_k_decode_attention(C.byref(cg), H.to_dev(q, dtype).data_ptr(), d_pool.data_ptr(),
                                              d_table.data_ptr(), out.data_ptr(), layer, total, max_pages,
                                              scale, scratch.data_ptr(), need, None)
        assert rc == 0, capi.last_error()
        torch.cuda.synchronize()
        err = np.abs(ob.to_float(H.torch_bits(out), dtype) - ob.to_float(want, dtype)).max()
        assert err <= 2e-3, err
    # too little scratch is refused, not overrun
    rc = drkv_lib.drkv_k_decode_attention(C.byref(cg), H.to_dev(q, dtype).data_ptr(), d_pool.data_ptr(),
                                          d_table.data_ptr(), out.data_ptr(), layer, total, max_pages, scale,
                                          scratch.data_ptr(), 1024, None)
    assert rc == capi.ERR_CAPACITY


def test_reference_free_functions_fp16_toy(drkv_lib, oracle):
    _run(oracle, drkv_lib, hq=16, hkv=4, d=128, page=16, dtype=oracle.F16, seq_len=512, m_batch=5, seed=11)


def test_reference_free_functions_model_shape(drkv_lib, oracle):
    """24/4 heads, head_dim 256, block 256: PagedKVConfig's own numbers (src/memoria/block_pool.h:34-40)."""
    _run(oracle, drkv_lib, hq=24, hkv=4, d=256, page=256, dtype=oracle.F16, seq_len=700, m_batch=300, seed=12,
         layers=1)


def test_reference_free_functions_bf16_long(drkv_lib, oracle):
    _run(oracle, drkv_lib, hq=32, hkv=8, d=128, page=16, dtype=oracle.BF16, seq_len=5000, m_batch=17, seed=13)


def test_kernel_error_word_of_the_stateless_path(drkv_lib, oracle):
    """A table entry >= max_pages is refused by the kernel's own range check before any address is formed from it:
    it counts as a hole, and drkv_k_decode_kernel_error reports code 3 for that call only."""
    import torch
    from deusridet_b200 import capi

    ob = oracle
    layers, hq, hkv, d, page, dtype, seq_len = 1, 16, 4, 128, 16, ob.BF16, 900
    rng = np.random.default_rng(14)
    n_pages = (seq_len + page - 1) // page
    max_pages = n_pages + 3
    g = ob.geom(layers, hq, hkv, d, page, dtype, 0, 1e4)
    cg = capi.Geometry(layers, hq, hkv, d, page, dtype, 0, 1e4)
    table = rng.permutation(max_pages)[:n_pages].astype(np.int32)   # exactly ceil(seq_len / page) entries
    pool = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
    d_pool = torch.from_numpy(pool.view(np.int16)).cuda()
    q = H.randn_bits(rng, (1, hq, d), dtype)
    d_q = H.to_dev(q, dtype)
    need = drkv_lib.drkv_k_decode_scratch_bytes(C.byref(cg), seq_len)
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    scale = 1.0 / np.sqrt(d)

    def run(tab, noalloc):
        d_table = torch.from_numpy(tab).cuda()
        out = torch.zeros(1, hq, d, dtype=torch.bfloat16, device="cuda")
        if noalloc:
            rc = drkv_lib.drkv_k_decode_attention_noalloc(C.byref(cg), d_q.data_ptr(), d_pool.data_ptr(),
                                                          d_table.data_ptr(), out.data_ptr(), 0, seq_len, max_pages,
                                                          scale, None)
        else:
            rc = drkv_lib.drkv_k_decode_attention(C.byref(cg), d_q.data_ptr(), d_pool.data_ptr(), d_table.data_ptr(),
                                                  out.data_ptr(), 0, seq_len, max_pages, scale, scratch.data_ptr(),
                                                  need, None)
        assert rc == 0, capi.last_error()
        status = drkv_lib.drkv_k_decode_kernel_error(None if noalloc else scratch.data_ptr(), None)
        return ob.to_float(H.torch_bits(out), dtype), status

    bad = table.copy()
    bad[7] = max_pages + 5                                  # not a page of this pool
    holed = table.copy()
    holed[7] = -1
    want = np.zeros((1, hq, d), dtype=np.uint16)
    ob.attend_decode(g, pool, max_pages, holed[None, :], [0], [seq_len], 0, q, want, scale)
    for noalloc in (False, True):
        got, status = run(bad, noalloc)
        assert status == capi.ERR_CUDA and "code 3" in capi.last_error()
        assert np.abs(got - ob.to_float(want, dtype)).max() <= 2e-3
        _, status = run(table, noalloc)                     # the next call starts clean
        assert status == 0, capi.last_error()


def test_position_written_by_the_kernel_in_front(drkv_lib, oracle):
    """The reference's decode loop uploads / computes d_pos right before paged_kv_cache_write
    (src/conscientia/stream.cpp:304-309): the raw-pointer entry points read the position and the table only after
    every earlier launch on the stream has completed.  A device kernel rewrites both directly in front of each call."""
    import torch
    from deusridet_b200 import capi

    ob = oracle
    layers, hq, hkv, d, page, dtype = 1, 8, 2, 128, 16, ob.BF16
    rng = np.random.default_rng(15)
    max_pages = 12
    g = ob.geom(layers, hq, hkv, d, page, dtype, 0, 1e4)
    cg = capi.Geometry(layers, hq, hkv, d, page, dtype, 0, 1e4)
    pool = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
    d_pool = torch.from_numpy(pool.view(np.int16)).cuda()
    base_table = rng.permutation(max_pages).astype(np.int32)
    d_base = torch.from_numpy(base_table).cuda()
    d_table = torch.full((max_pages,), -1, dtype=torch.int32, device="cuda")
    d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    step = torch.ones(1, dtype=torch.int32, device="cuda")
    table = np.full(max_pages, -1, dtype=np.int32)
    for it in range(40):
        pos = 7 * it % (max_pages * page)
        k1, v1 = H.randn_bits(rng, (1, hkv, d), dtype), H.randn_bits(rng, (1, hkv, d), dtype)
        dk, dv = H.to_dev(k1, dtype), H.to_dev(v1, dtype)
        d_pos.zero_()
        torch.mul(step, pos, out=d_pos)                       # device kernels write the position ...
        d_table.copy_(torch.roll(d_base, it))                 # ... and the table, directly in front of the call
        table = np.roll(base_table, it)
        rc = drkv_lib.drkv_k_cache_write(C.byref(cg), dk.data_ptr(), dv.data_ptr(), d_pool.data_ptr(), d_table.data_ptr(),
                                         0, d_pos.data_ptr(), max_pages, None)
        assert rc == 0, capi.last_error()
        ob.append(g, pool, max_pages, table, 0, pos, 1, k1, v1, rope=False)
    torch.cuda.synchronize()
    assert np.array_equal(d_pool.cpu().numpy().view(np.uint16), pool)
