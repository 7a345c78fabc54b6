"""The CPU checker against outputs of the reference's own CUDA kernels (apply_rope, paged_rope_batch_kernel,
paged_kv_cache_write[_batch], paged_gqa_decode_attention, paged_prefill_attention_kernel, the bf16 split-K decode
and merge, the flat <-> paged copies), recorded on a B200 by
tests/golden/make_paged_attention_golden.py into tests/golden/paged_attention_reference.npz.

What is pinned, and how tightly:
  * the K/V writes are copies: the bytes and the places must match exactly;
  * RoPE: the reference evaluates powf/cosf/sinf as fast-math device intrinsics, whose bits no CPU
    reproduces; the checker's rotation must agree to within the documented error of those intrinsics
    at the angle in question plus one fp16 rounding (tests/helpers.py: rope_fastmath_tolerance);
  * decode attention (fp32 accumulate, fast-math exp): max-abs 2e-3 on the fp16 outputs."""
import os

import numpy as np
import pytest

from tests import helpers as H
from tests.golden import paged_cases

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "paged_attention_reference.npz"))


def _rope_close(got_bits, ref_bits, src_bits, c, pos, oracle):
    a, b = oracle.to_float(got_bits, oracle.F16), oracle.to_float(ref_bits, oracle.F16)
    tol = H.rope_fastmath_tolerance(src_bits, c["rot"], c["theta"], pos, oracle.F16)
    tol = tol + 1.01 * H.ulp(np.maximum(np.abs(a), np.abs(b)), oracle.F16)
    return (np.abs(a - b) <= tol).all()


@pytest.mark.parametrize("name", sorted(paged_cases.CASES))
def test_checker_reproduces_reference_kernels(oracle, name):
    ob = oracle
    c = paged_cases.build(name)
    g, pool = c["g"], c["pool"].copy()
    pos = c["seq_len"]
    if c["m_batch"]:
        ob.append(g, pool, c["max_pages"], c["table"], c["layer"], pos, c["m_batch"], c["kb"], c["vb"], rope=False)
        pos += c["m_batch"]
    # RoPE on Q and K at the new position (the reference rotates both, layer_attention.cu:50-68)
    q_r, k_r = c["q"].copy(), c["k1"].copy()
    ob.lib().okv_rope_rows(q_r.ctypes.data, c["hq"], __import__("ctypes").byref(g), pos)
    ob.lib().okv_rope_rows(k_r.ctypes.data, c["hkv"], __import__("ctypes").byref(g), pos)
    assert _rope_close(q_r, GOLD[name + "_q_roped"], c["q"], c, pos, ob)
    assert _rope_close(k_r, GOLD[name + "_k_roped"], c["k1"], c, pos, ob)
    # and it is a rotation of the right pairs, not just something small: most elements did change
    assert (GOLD[name + "_k_roped"][:, :c["rot"]] != c["k1"][:, :c["rot"]]).mean() > 0.9
    # dims beyond the rotary part are untouched, bit for bit
    assert np.array_equal(q_r[:, c["rot"]:], c["q"][:, c["rot"]:])
    assert np.array_equal(GOLD[name + "_q_roped"][:, c["rot"]:], c["q"][:, c["rot"]:])
    # the write itself is a copy: feed it the reference's rotated K so that the bytes must be identical
    ob.append(g, pool, c["max_pages"], c["table"], c["layer"], pos, 1, GOLD[name + "_k_roped"][None], c["v1"][None],
              rope=False)
    ref_pool = c["pool"].copy()
    ref_pool[GOLD[name + "_pool_changed_idx"]] = GOLD[name + "_pool_changed_val"]
    assert np.array_equal(pool, ref_pool), "K/V bytes or their places differ from the reference's writes"
    # attention on the reference's own pool and rotated Q
    out = np.zeros((1, c["hq"], c["d"]), dtype=np.uint16)
    ob.attend_decode(g, ref_pool, c["max_pages"], c["table"][None, :], [0], [pos + 1], c["layer"],
                     GOLD[name + "_q_roped"][None], out, 1.0 / np.sqrt(c["d"]))
    err = np.abs(ob.to_float(out[0], ob.F16) - ob.to_float(GOLD[name + "_out"], ob.F16)).max()
    assert err <= 2e-3, err


def test_importance_update_matches_reference_kernel_record(oracle):
    """score = fma(score, decay, new) against the scores the reference's own ImportanceScorer held after
    each update on a B200 (src/memoria/importance_scorer.cu:27-37, 68-96)."""
    from tests.golden.make_importance_golden import importance_cases
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "importance_reference.npz"))
    for name, (decay, new) in importance_cases().items():
        scores = np.zeros(new.shape[1], dtype=np.float32)
        for k in range(new.shape[0]):
            oracle.importance_update(scores, new[k], decay)
            assert np.array_equal(scores, gold[name][k]), f"{name} step {k}"


@pytest.mark.parametrize("name", sorted(paged_cases.PREFILL_CASES))
def test_checker_reproduces_reference_prefill_kernels(oracle, name):
    """paged_rope_batch_kernel, paged_kv_cache_write_batch and paged_prefill_attention_kernel
    (src/machina/paged_attention.cu:412-451, 123-167, 465-554) as recorded on a B200."""
    import ctypes as C
    ob = oracle
    c = paged_cases.build_prefill(name)
    g, m = c["g"], c["m"]
    q_r, k_r = c["q"].copy(), c["k"].copy()
    for t in range(m):                              # the batch kernel rotates token t at pos_start + t
        ob.lib().okv_rope_rows(q_r[t].ctypes.data, c["hq"], C.byref(g), c["pos_start"] + t)
        ob.lib().okv_rope_rows(k_r[t].ctypes.data, c["hkv"], C.byref(g), c["pos_start"] + t)
        assert _rope_close(q_r[t], GOLD[name + "_q_roped"][t], c["q"][t], c, c["pos_start"] + t, ob), t
        assert _rope_close(k_r[t], GOLD[name + "_k_roped"][t], c["k"][t], c, c["pos_start"] + t, ob), t
    if c["pos_start"] > 0:     # a rotation did happen (the slowest pairs of a large base barely move at these positions)
        assert (GOLD[name + "_k_roped"][:, :, :c["rot"]] != c["k"][:, :, :c["rot"]]).mean() > 0.8
    assert np.array_equal(GOLD[name + "_q_roped"][:, :, c["rot"]:], c["q"][:, :, c["rot"]:])
    # the batched write is a copy: with the reference's rotated K the whole pool must hash to the reference's
    pool = c["pool"].copy()
    ob.append(g, pool, c["max_pages"], c["table"], c["layer"], c["pos_start"], m, GOLD[name + "_k_roped"], c["v"],
              rope=False)
    assert np.array_equal(paged_cases.digest(pool), GOLD[name + "_pool_sha256"])
    # causal attention of the chunk on that pool with the reference's rotated Q
    out = np.zeros((m, c["hq"], c["d"]), dtype=np.uint16)
    ob.attend_prefill(g, pool, c["max_pages"], c["table"], c["layer"], c["pos_start"], m, GOLD[name + "_q_roped"], out,
                      1.0 / np.sqrt(c["d"]))
    got, want = ob.to_float(out, ob.F16), ob.to_float(GOLD[name + "_out"], ob.F16)
    assert np.abs(got - want).max() <= 2e-3


@pytest.mark.parametrize("name", sorted(paged_cases.SPLITK_CASES))
def test_checker_reproduces_reference_split_k_decode(oracle, name):
    """The reference's only bf16 attention (invoke_causal_gqa_decode, src/sensus/auditus/asr/asr_ops_attn.cu:29-132):
    per-partition partials (un-normalised o, m, l; 128-key partitions), their merge, and the final output, against
    the checker's partial / merge / whole-sequence decode on the same values laid out in pages."""
    ob = oracle
    c = paged_cases.build_splitk(name)
    g, hq, d, S, n_parts = c["g"], c["hq"], c["d"], c["seq_len"], c["n_parts"]
    scale = 1.0 / np.sqrt(d)
    ref_o, ref_m, ref_l = GOLD[name + "_part_o"], GOLD[name + "_part_m"], GOLD[name + "_part_l"]
    for p in range(n_parts):
        part = ob.attend_partial(g, c["pool"], c["max_pages"], c["table"], 0, 128 * p, min(128 * (p + 1), S), c["q"], scale)
        o, mm, l = part[:hq * d].reshape(hq, d), part[hq * d:hq * d + hq], part[hq * (d + 1):]
        # (m, l, o) of the two sides may differ by a common factor (running maximum against partition maximum):
        # the normalised partial and the log-sum-exp do not
        assert np.abs(o / l[:, None] - ref_o[:, p] / ref_l[:, p, None]).max() <= 2e-4, p
        assert np.abs((mm + np.log(l)) - (ref_m[:, p] + np.log(ref_l[:, p]))).max() <= 2e-4, p
    want = ob.to_float(GOLD[name + "_out"], ob.BF16)
    tol = np.maximum(2e-3, H.ulp(want, ob.BF16))
    # the checker's merge, fed the reference's own partials, gives the reference's output
    ext = paged_cases.splitk_parts_external(ref_o, ref_m, ref_l, hq, d, n_parts)
    merged = np.zeros((hq, d), dtype=np.uint16)
    ob.combine(g, ext, merged)
    assert (np.abs(ob.to_float(merged, ob.BF16) - want) <= tol).all()
    # and so does the unsplit decode recurrence
    whole = np.zeros((1, hq, d), dtype=np.uint16)
    ob.attend_decode(g, c["pool"], c["max_pages"], c["table"][None, :], [0], [S], 0, c["q"][None], whole, scale)
    assert (np.abs(ob.to_float(whole[0], ob.BF16) - want) <= tol).all()


@pytest.mark.parametrize("name", sorted(paged_cases.FLAT_CASES))
def test_checker_reproduces_reference_extract_inject(oracle, name):
    """invoke_extract_kv_from_pages / invoke_inject_kv_to_pages (src/memoria/cache_kernels.cu:30-187), byte-exact:
    a page missing from the table reads as zeros and is skipped on the way back."""
    ob = oracle
    c = paged_cases.build_flat(name)
    flat = ob.extract(c["g"], c["pool"], c["max_pages"], c["table"], c["start"], c["num"])
    assert np.array_equal(paged_cases.digest(flat), GOLD[name + "_extract_sha256"])
    pool = c["pool"].copy()
    ob.inject(c["g"], pool, c["src"], c["max_pages"], c["table"], c["start"], c["num"])
    assert np.array_equal(paged_cases.digest(pool), GOLD[name + "_pool_after_inject_sha256"])
