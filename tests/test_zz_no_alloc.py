"""drkv_k_decode_attention_noalloc: the decode attention entry point for callers that cannot
allocate device memory (a plug-in inside a server that owns all of HBM, a latency-bound decode
thread that must not hit cudaMalloc's synchronisation, a process whose GPU is already full of KV
pages).  It keeps its split-KV partials in a scratch area compiled into the library.

Checked here, through the C ABI: two calls in a row on different inputs give the same result as
drkv_k_decode_attention with caller-provided scratch (same 2e-3 bound as the other attention
tests), the device's free memory does not move across a call, and an over-long sequence is
refused.  The file name sorts last so that a run stopping at the first failure has already run
every other test; the test builds all of its own state, so it also passes alone in a fresh
process."""
import ctypes as C

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu

TOL = 2e-3


def test_noalloc_matches_caller_scratch_entry_point(drkv_lib, oracle):
    import torch
    from deusridet_b200 import capi

    ob = oracle
    layers, hq, hkv, d, page, dtype = 2, 32, 8, 128, 16, ob.BF16
    cg = capi.Geometry(layers, hq, hkv, d, page, dtype, 0, 1e6)
    g = ob.geom(layers, hq, hkv, d, page, dtype, 0, 1e6)
    rng = np.random.default_rng(2024)
    max_len = 6000
    n_pages = (max_len + page - 1) // page
    max_pages = n_pages + 9
    table = rng.permutation(max_pages)[:n_pages].astype(np.int32)
    pool = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
    d_pool = torch.from_numpy(pool.view(np.int16)).cuda()
    d_table = torch.from_numpy(table).cuda()
    scale = 1.0 / np.sqrt(d)
    need = drkv_lib.drkv_k_decode_scratch_bytes(C.byref(cg), max_len)
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")

    # first a long sequence, then a short one on another layer: the second call must not see
    # anything the first one left in the shared scratch
    for call, (seq_len, layer) in enumerate([(max_len, 1), (777, 0)]):
        q = H.to_dev(H.randn_bits(rng, (1, hq, d), dtype), dtype)
        want = torch.zeros(1, hq, d, dtype=torch.bfloat16, device="cuda")
        got = torch.zeros_like(want)
        rc = drkv_lib.drkv_k_decode_attention(C.byref(cg), q.data_ptr(), d_pool.data_ptr(), d_table.data_ptr(),
                                              want.data_ptr(), layer, seq_len, max_pages, scale,
                                              scratch.data_ptr(), need, None)
        assert rc == 0, capi.last_error()
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc = drkv_lib.drkv_k_decode_attention_noalloc(C.byref(cg), q.data_ptr(), d_pool.data_ptr(),
                                                      d_table.data_ptr(), got.data_ptr(), layer, seq_len,
                                                      max_pages, scale, None)
        assert rc == 0, capi.last_error()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        if call > 0:   # the first call may load the module lazily; after that nothing may move
            assert free_after == free_before, "the call changed the device's free memory"
        err = (got.float() - want.float()).abs().max().item()
        assert err <= TOL, f"call {call}: max-abs {err} against the caller-scratch entry point"
        assert want.float().abs().max().item() > 0   # the comparison is not vacuous
        # and both agree with the CPU checker
        ref = np.zeros((1, hq, d), dtype=np.uint16)
        ob.attend_decode(g, pool, max_pages, table[None, :], [0], [seq_len], layer, H.torch_bits(q), ref, scale)
        assert np.abs(ob.to_float(H.torch_bits(got), dtype) - ob.to_float(ref, dtype)).max() <= TOL


def test_noalloc_rejects_what_does_not_fit(drkv_lib):
    import torch
    from deusridet_b200 import capi

    # 64 heads of 256 dims: 66 KB of partials per 4096 keys, so 4 MiB ends near 258k keys
    cg = capi.Geometry(1, 64, 4, 256, 256, capi.F16, 0, 1e4)
    dummy = torch.zeros(1 << 16, dtype=torch.int32, device="cuda")
    rc = drkv_lib.drkv_k_decode_attention_noalloc(C.byref(cg), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                                  dummy.data_ptr(), 0, 1 << 20, 64, 1.0, None)
    assert rc == capi.ERR_CAPACITY
    assert "scratch" in capi.last_error()
    torch.cuda.synchronize()
