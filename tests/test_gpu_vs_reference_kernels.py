"""This repository's CUDA path against outputs recorded from the reference's own CUDA kernels
(tests/golden/paged_attention_reference.npz): the raw-pointer entry points that stand in for
paged_kv_cache_write[_batch] and paged_gqa_decode_attention, and the fused RoPE + append."""
import ctypes as C
import os

import numpy as np
import pytest

from tests import helpers as H
from tests.golden import paged_cases

pytestmark = pytest.mark.gpu

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "paged_attention_reference.npz"))


@pytest.mark.parametrize("name", sorted(paged_cases.CASES))
def test_drop_in_entry_points_match_reference_kernels(drkv_lib, oracle, name):
    import torch
    from deusridet_b200 import capi

    ob = oracle
    c = paged_cases.build(name)
    cg = capi.Geometry(c["layers"], c["hq"], c["hkv"], c["d"], c["page"], capi.F16, c["rot"], c["theta"])
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda()
    pool, table = dev(c["pool"]), torch.from_numpy(c["table"]).cuda()
    pos = c["seq_len"]
    # device copies stay referenced until the kernels that read them have run
    kb, vb, k1, v1, q = (dev(x) for x in (c["kb"], c["vb"], GOLD[name + "_k_roped"], c["v1"], GOLD[name + "_q_roped"]))
    if c["m_batch"]:
        rc = drkv_lib.drkv_k_cache_write_batch(C.byref(cg), kb.data_ptr(), vb.data_ptr(),
                                               pool.data_ptr(), table.data_ptr(), c["layer"], pos, c["m_batch"],
                                               c["max_pages"], None)
        assert rc == 0, capi.last_error()
        pos += c["m_batch"]
    d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    # the reference rotates K before the write: hand over its rotated K, as its caller would
    rc = drkv_lib.drkv_k_cache_write(C.byref(cg), k1.data_ptr(), v1.data_ptr(),
                                     pool.data_ptr(), table.data_ptr(), c["layer"], d_pos.data_ptr(), c["max_pages"], None)
    assert rc == 0, capi.last_error()
    torch.cuda.synchronize()
    ref_pool = c["pool"].copy()
    ref_pool[GOLD[name + "_pool_changed_idx"]] = GOLD[name + "_pool_changed_val"]
    assert np.array_equal(pool.cpu().numpy().view(np.uint16), ref_pool)

    need = drkv_lib.drkv_k_decode_scratch_bytes(C.byref(cg), pos + 1)
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    out = torch.zeros(c["hq"], c["d"], dtype=torch.int16, device="cuda")
    rc = drkv_lib.drkv_k_decode_attention(C.byref(cg), q.data_ptr(), pool.data_ptr(),
                                          table.data_ptr(), out.data_ptr(), c["layer"], pos + 1, c["max_pages"],
                                          1.0 / np.sqrt(c["d"]), scratch.data_ptr(), need, None)
    assert rc == 0, capi.last_error()
    torch.cuda.synchronize()
    err = np.abs(ob.to_float(out.cpu().numpy().view(np.uint16), ob.F16) - ob.to_float(GOLD[name + "_out"], ob.F16)).max()
    assert err <= 2e-3, err


@pytest.mark.parametrize("name", sorted(paged_cases.CASES))
def test_fused_rope_append_against_reference_rope(drkv_lib, oracle, name):
    """drkv_append_rope rotates K itself; its bytes are the checker's bit for bit (tested elsewhere) and must
    sit within the fast-math error of the reference's apply_rope (tests/helpers.py) of what it left in the pool."""
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    c = paged_cases.build(name)
    eng = PagedKVEngine(num_layers=c["layers"], num_q_heads=c["hq"], num_kv_heads=c["hkv"], head_dim=c["d"],
                        page_size=c["page"], dtype="f16", rotary_dim=c["rot"], rope_theta=c["theta"],
                        max_pages=c["max_pages"], max_seqs=1, max_pages_per_seq=len(c["table"]) + 1, device=0)
    try:
        s = eng.seq_create()
        pos = c["seq_len"] + c["m_batch"]
        assert eng.ensure_blocks_for_range(s, 0, pos + 1)
        eng.sync_block_table()
        page = int(eng.table(s)[pos // c["page"]])
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda().view(torch.float16)
        rows = torch.tensor([s], dtype=torch.int32, device="cuda")
        d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
        eng.append_rope(c["layer"], 1, rows, d_pos, dev(c["k1"][None]), dev(c["v1"][None]))
        torch.cuda.synchronize()
        got = eng.pool_tensor().cpu().numpy().view(np.uint16)
        for h in range(c["hkv"]):
            off = ob.pool_elem(c["g"], c["max_pages"], c["layer"], page, 0, h, pos % c["page"])
            a = ob.to_float(got[off:off + c["d"]], ob.F16)
            b = ob.to_float(GOLD[name + "_k_roped"][h], ob.F16)
            tol = H.rope_fastmath_tolerance(c["k1"][h], c["rot"], c["theta"], pos, ob.F16)
            assert (np.abs(a - b) <= tol + 1.01 * H.ulp(np.maximum(np.abs(a), np.abs(b)), ob.F16)).all()
            voff = ob.pool_elem(c["g"], c["max_pages"], c["layer"], page, 1, h, pos % c["page"])
            assert np.array_equal(got[voff:voff + c["d"]], c["v1"][h])
    finally:
        eng.close()
