"""This repository's CUDA path against outputs recorded from the reference's own CUDA kernels
(tests/golden/paged_attention_reference.npz): the raw-pointer entry points that stand in for
paged_kv_cache_write[_batch], paged_gqa_decode_attention and the flat <-> paged copies, the fused RoPE + append,
the prefill attention, and the split-KV partials and merge against the reference's bf16 split-K decode."""
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


def _engine_with_flat_cache(oracle, c, dtype_name, flat, n_tokens, extra_pages=4):
    """An engine whose one sequence holds the cache `flat` ([layers][K|V][token][head][dim]) in pages of its own
    choosing: attention depends on the logical contents only, so a case recorded behind the reference's block
    table can be replayed behind the engine's."""
    import torch
    from deusridet_b200 import PagedKVEngine

    g = c["g"]
    n_pages = (n_tokens + g.page_size - 1) // g.page_size
    eng = PagedKVEngine(num_layers=g.num_layers, num_q_heads=g.num_q_heads, num_kv_heads=g.num_kv_heads,
                        head_dim=g.head_dim, page_size=g.page_size, dtype=dtype_name, rotary_dim=g.rotary_dim,
                        rope_theta=g.rope_theta, max_pages=n_pages + extra_pages, max_seqs=2,
                        max_pages_per_seq=n_pages + 1, device=0)
    H.shuffled_free_stack(eng, np.random.default_rng(n_tokens))
    eng.seq_create()                                     # the sequence under test is not table row 0
    s = eng.seq_create()
    assert eng.ensure_blocks_for_range(s, 0, n_tokens)
    eng.set_seq_len(s, n_tokens)
    eng.sync_block_table()
    eng.pool_tensor().copy_(torch.from_numpy(                # stale values everywhere else
        H.randn_bits(np.random.default_rng(7), eng.total_bytes() // 2, g.dtype).view(np.int16)))
    eng.inject(s, 0, n_tokens, torch.from_numpy(np.ascontiguousarray(flat).view(np.int16)).cuda())
    return eng, s


@pytest.mark.parametrize("name", sorted(paged_cases.PREFILL_CASES))
def test_prefill_path_matches_reference_kernels(drkv_lib, oracle, name):
    """The batched K/V write (bytes exact), the fused RoPE + append (within the reference's fast-math error) and the
    tensor-core prefill attention (2e-3) against paged_kv_cache_write_batch, paged_rope_batch_kernel and
    paged_prefill_attention_kernel as recorded on a B200."""
    import torch
    from deusridet_b200 import capi

    ob = oracle
    c = paged_cases.build_prefill(name)
    g, m, pos0 = c["g"], c["m"], c["pos_start"]
    cg = capi.Geometry(c["layers"], c["hq"], c["hkv"], c["d"], c["page"], capi.F16, c["rot"], c["theta"])
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda()
    pool, table = dev(c["pool"]), torch.from_numpy(c["table"]).cuda()
    k_r, v = dev(GOLD[name + "_k_roped"]), dev(c["v"])
    rc = drkv_lib.drkv_k_cache_write_batch(C.byref(cg), k_r.data_ptr(), v.data_ptr(), pool.data_ptr(), table.data_ptr(),
                                           c["layer"], pos0, m, c["max_pages"], None)
    assert rc == 0, capi.last_error()
    torch.cuda.synchronize()
    ref_pool = pool.cpu().numpy().view(np.uint16)
    assert np.array_equal(paged_cases.digest(ref_pool), GOLD[name + "_pool_sha256"])

    # the same cache behind an engine's own table; the chunk's own K/V go in through the fused RoPE + append
    total = pos0 + m
    flat = ob.extract(g, ref_pool, c["max_pages"], c["table"], 0, total)
    eng, s = _engine_with_flat_cache(ob, c, "f16", flat, total)
    try:
        eng.append_rope_chunk(c["layer"], s, pos0, m, H.to_dev(c["k"], ob.F16), H.to_dev(c["v"], ob.F16))
        torch.cuda.synchronize()
        got_flat = torch.zeros(flat.shape, dtype=torch.int16, device="cuda")
        eng.extract(s, 0, total, got_flat)
        torch.cuda.synchronize()
        got_flat = got_flat.cpu().numpy().view(np.uint16)
        assert np.array_equal(got_flat[:, 1], flat[:, 1])                       # V: copies
        assert np.array_equal(got_flat[:, 0, :pos0], flat[:, 0, :pos0])          # earlier K untouched
        for t in range(m):
            a = ob.to_float(got_flat[c["layer"], 0, pos0 + t], ob.F16)
            b = ob.to_float(GOLD[name + "_k_roped"][t], ob.F16)
            tol = H.rope_fastmath_tolerance(c["k"][t], c["rot"], c["theta"], pos0 + t, ob.F16)
            assert (np.abs(a - b) <= tol + 1.01 * H.ulp(np.maximum(np.abs(a), np.abs(b)), ob.F16)).all(), t
        # attention on exactly the reference's cache (its own rotated K) with its rotated Q
        eng.inject(s, 0, total, torch.from_numpy(flat.view(np.int16)).cuda())
        out = torch.zeros(m, c["hq"], c["d"], dtype=torch.float16, device="cuda")
        eng.attend_prefill_chunk(c["layer"], s, pos0, m, H.to_dev(GOLD[name + "_q_roped"], ob.F16), out,
                                 1.0 / np.sqrt(c["d"]))
        torch.cuda.synchronize()
        eng.check_kernels()
        err = np.abs(ob.to_float(H.torch_bits(out), ob.F16) - ob.to_float(GOLD[name + "_out"], ob.F16)).max()
        assert err <= 2e-3, err
    finally:
        eng.close()


@pytest.mark.parametrize("name", sorted(paged_cases.SPLITK_CASES))
def test_split_kv_matches_reference_bf16_split_k(drkv_lib, oracle, name):
    """drkv_attend_partial over the reference's 128-key partitions, drkv_combine_partials fed the reference's own
    partials, and the batched decode attention, against invoke_causal_gqa_decode (bf16) as recorded on a B200."""
    import torch

    ob = oracle
    c = paged_cases.build_splitk(name)
    hq, d, S, n_parts = c["hq"], c["d"], c["seq_len"], c["n_parts"]
    scale = 1.0 / np.sqrt(d)
    flat = np.stack([c["k_cache"], c["v_cache"]])[None]
    eng, s = _engine_with_flat_cache(ob, c, "bf16", flat, S)
    try:
        d_q = H.to_dev(c["q"], ob.BF16)
        ref_o, ref_m, ref_l = GOLD[name + "_part_o"], GOLD[name + "_part_m"], GOLD[name + "_part_l"]
        nf = eng.partial_floats()
        parts = torch.zeros(n_parts, nf, dtype=torch.float32, device="cuda")
        for p in range(n_parts):
            eng.attend_partial(0, s, 128 * p, min(128 * (p + 1), S), d_q, parts[p], scale)
        torch.cuda.synchronize()
        got = parts.cpu().numpy()
        for p in range(n_parts):
            o, mm, l = got[p, :hq * d].reshape(hq, d), got[p, hq * d:hq * d + hq], got[p, hq * (d + 1):]
            assert np.abs(o / l[:, None] - ref_o[:, p] / ref_l[:, p, None]).max() <= 2e-3, p
            assert np.abs((mm + np.log(l)) - (ref_m[:, p] + np.log(ref_l[:, p]))).max() <= 1e-3, p
        want = ob.to_float(GOLD[name + "_out"], ob.BF16)
        tol = np.maximum(2e-3, H.ulp(want, ob.BF16))
        ext = torch.from_numpy(paged_cases.splitk_parts_external(ref_o, ref_m, ref_l, hq, d, n_parts)).cuda()
        out = torch.zeros(hq, d, dtype=torch.bfloat16, device="cuda")
        eng.combine_partials(n_parts, ext, out)
        torch.cuda.synchronize()
        assert (np.abs(ob.to_float(H.torch_bits(out), ob.BF16) - want) <= tol).all()
        out2 = torch.zeros(1, hq, d, dtype=torch.bfloat16, device="cuda")
        rows = torch.tensor([s], dtype=torch.int32, device="cuda")
        lens = torch.tensor([S], dtype=torch.int32, device="cuda")
        eng.attend_decode(0, 1, rows, lens, S, d_q.view(1, hq, d), out2, scale)
        torch.cuda.synchronize()
        eng.check_kernels()
        assert (np.abs(ob.to_float(H.torch_bits(out2[0]), ob.BF16) - want) <= tol).all()
    finally:
        eng.close()


@pytest.mark.parametrize("name", sorted(paged_cases.FLAT_CASES))
def test_extract_inject_match_reference_kernels(drkv_lib, oracle, name):
    import torch
    from deusridet_b200 import capi

    c = paged_cases.build_flat(name)
    g = c["g"]
    cg = capi.Geometry(c["layers"], g.num_q_heads, c["hkv"], c["d"], c["page"], capi.F16, 0, 1e4)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda()
    pool, table, src = dev(c["pool"]), torch.from_numpy(c["table"]).cuda(), dev(c["src"])
    dst = torch.full((c["layers"], 2, c["num"], c["hkv"], c["d"]), 0x5555, dtype=torch.int16, device="cuda")
    rc = drkv_lib.drkv_k_extract_kv(C.byref(cg), dst.data_ptr(), pool.data_ptr(), table.data_ptr(), c["start"], c["num"],
                                    c["max_pages"], None)
    assert rc == 0, capi.last_error()
    rc = drkv_lib.drkv_k_inject_kv(C.byref(cg), pool.data_ptr(), src.data_ptr(), table.data_ptr(), c["start"], c["num"],
                                   c["max_pages"], None)
    assert rc == 0, capi.last_error()
    torch.cuda.synchronize()
    assert np.array_equal(paged_cases.digest(dst.cpu().numpy().view(np.uint16)), GOLD[name + "_extract_sha256"])
    assert np.array_equal(paged_cases.digest(pool.cpu().numpy().view(np.uint16)), GOLD[name + "_pool_after_inject_sha256"])
