"""Records what the reference's own CUDA kernels return for the seeded cases of tests/golden/paged_cases.py.
The kernels are compiled by oracle/ref_build/Makefile from the reference's sources, with the reference's
--use_fast_math, into oracle/_ref/libref_paged.so.  Needs a GPU:

    python tests/golden/make_paged_attention_golden.py OUTPUT.npz

The result is committed as tests/golden/paged_attention_reference.npz.
  * decode cases: as in full_attention_forward_paged (src/machina/paged_attention.cu:353-367): RoPE on Q and K at
    the new position, write of K/V into the page, decode attention over seq_len + 1 keys; before that a batched
    write of m_batch earlier tokens where the case has some;
  * prefill cases: as in full_attention_forward_paged_prefill (paged_attention.cu:604-630): batched RoPE on the
    chunk's Q and K, batched K/V write, causal attention of the chunk through the block table;
  * split-K cases: invoke_causal_gqa_decode (src/sensus/auditus/asr/asr_ops_attn.cu:110-132), bf16: the output and
    the workspace (partial o, m, l per 128-key partition);
  * flat <-> paged cases: invoke_extract_kv_from_pages / invoke_inject_kv_to_pages
    (src/memoria/cache_kernels.cu:147-187); byte-exact results are stored as SHA-256 digests."""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests.golden import paged_cases  # noqa: E402


def main(out_path):
    L = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_paged.so"))
    L.refp_set_model.argtypes = [C.c_int] * 4 + [C.c_float]
    L.refp_apply_rope.argtypes = [C.c_void_p] * 3
    L.refp_cache_write.argtypes = [C.c_void_p] * 4 + [C.c_int, C.c_void_p, C.c_int, C.c_int]
    L.refp_cache_write_batch.argtypes = [C.c_void_p] * 4 + [C.c_int] * 5
    L.refp_decode_attention.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_float]
    L.refp_rope_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
    L.refp_prefill_attention.argtypes = [C.c_void_p] * 4 + [C.c_int] * 5 + [C.c_float]
    L.refp_extract.argtypes = [C.c_void_p] * 3 + [C.c_int] * 5
    L.refp_inject.argtypes = [C.c_void_p] * 3 + [C.c_int] * 5
    L.refp_split_k_decode.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_void_p, C.c_int]
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda()
    host = lambda t: t.cpu().numpy().view(np.uint16)
    out = {}
    for name in paged_cases.CASES:
        c = paged_cases.build(name)
        L.refp_set_model(c["hq"], c["hkv"], c["d"], c["rot"], c["theta"])
        pool, table = dev(c["pool"]), torch.from_numpy(c["table"]).cuda()
        pos = c["seq_len"]
        if c["m_batch"]:
            kb, vb = dev(c["kb"]), dev(c["vb"])
            L.refp_cache_write_batch(kb.data_ptr(), vb.data_ptr(), pool.data_ptr(), table.data_ptr(), c["layer"], pos,
                                     c["m_batch"], c["max_pages"], c["page"])
            pos += c["m_batch"]
        d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
        q, k1, v1 = dev(c["q"]), dev(c["k1"]), dev(c["v1"])
        L.refp_apply_rope(q.data_ptr(), k1.data_ptr(), d_pos.data_ptr())
        L.refp_cache_write(k1.data_ptr(), v1.data_ptr(), pool.data_ptr(), table.data_ptr(), c["layer"], d_pos.data_ptr(),
                           c["max_pages"], c["page"])
        o = torch.zeros(c["hq"], c["d"], dtype=torch.int16, device="cuda")
        L.refp_decode_attention(q.data_ptr(), pool.data_ptr(), table.data_ptr(), o.data_ptr(), c["layer"], pos + 1,
                                c["max_pages"], c["page"], C.c_float(1.0 / np.sqrt(c["d"])))
        assert L.refp_sync() == 0
        out[name + "_q_roped"] = host(q).reshape(c["hq"], c["d"])
        out[name + "_k_roped"] = host(k1).reshape(c["hkv"], c["d"])
        out[name + "_out"] = host(o).reshape(c["hq"], c["d"])
        # the pool after the writes: only the pages of this table matter; store the bytes that changed
        after = host(pool)
        changed = np.nonzero(after != c["pool"])[0].astype(np.int64)
        out[name + "_pool_changed_idx"] = changed
        out[name + "_pool_changed_val"] = after[changed]
        print(name, "changed elements", changed.size, "out[0,:4]", out[name + "_out"][0, :4])

    for name in paged_cases.PREFILL_CASES:
        c = paged_cases.build_prefill(name)
        L.refp_set_model(c["hq"], c["hkv"], c["d"], c["rot"], c["theta"])
        pool, table = dev(c["pool"]), torch.from_numpy(c["table"]).cuda()
        q, k, v = dev(c["q"]), dev(c["k"]), dev(c["v"])
        L.refp_rope_batch(q.data_ptr(), k.data_ptr(), c["pos_start"], c["m"])
        L.refp_cache_write_batch(k.data_ptr(), v.data_ptr(), pool.data_ptr(), table.data_ptr(), c["layer"],
                                 c["pos_start"], c["m"], c["max_pages"], c["page"])
        o = torch.zeros(c["m"], c["hq"], c["d"], dtype=torch.int16, device="cuda")
        L.refp_prefill_attention(q.data_ptr(), pool.data_ptr(), table.data_ptr(), o.data_ptr(), c["layer"],
                                 c["pos_start"], c["m"], c["max_pages"], c["page"], C.c_float(1.0 / np.sqrt(c["d"])))
        assert L.refp_sync() == 0
        out[name + "_q_roped"] = host(q).reshape(c["m"], c["hq"], c["d"])
        out[name + "_k_roped"] = host(k).reshape(c["m"], c["hkv"], c["d"])
        out[name + "_out"] = host(o).reshape(c["m"], c["hq"], c["d"])
        out[name + "_pool_sha256"] = paged_cases.digest(host(pool))
        print(name, "out[0,0,:4]", out[name + "_out"][0, 0, :4])

    for name in paged_cases.SPLITK_CASES:
        c = paged_cases.build_splitk(name)
        hq, d, n_parts = c["hq"], c["d"], c["n_parts"]
        q, kc, vc = dev(c["q"]), dev(c["k_cache"]), dev(c["v_cache"])
        ws = torch.zeros(hq * n_parts * (d + 2), dtype=torch.float32, device="cuda")
        o = torch.zeros(hq, d, dtype=torch.int16, device="cuda")
        L.refp_split_k_decode(o.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), hq, c["hkv"], d, c["seq_len"],
                              ws.data_ptr(), n_parts)
        assert L.refp_sync() == 0
        w = ws.cpu().numpy()
        out[name + "_out"] = host(o).reshape(hq, d)
        out[name + "_part_o"] = w[:hq * n_parts * d].reshape(hq, n_parts, d)
        out[name + "_part_m"] = w[hq * n_parts * d:hq * n_parts * (d + 1)].reshape(hq, n_parts)
        out[name + "_part_l"] = w[hq * n_parts * (d + 1):].reshape(hq, n_parts)
        print(name, "parts", n_parts, "out[0,:4]", out[name + "_out"][0, :4])

    for name in paged_cases.FLAT_CASES:
        c = paged_cases.build_flat(name)
        L.refp_set_model(2 * c["hkv"], c["hkv"], c["d"], 0, 1e4)
        pool, table = dev(c["pool"]), torch.from_numpy(c["table"]).cuda()
        dst = torch.full((c["layers"], 2, c["num"], c["hkv"], c["d"]), 0x5555, dtype=torch.int16, device="cuda")
        L.refp_extract(dst.data_ptr(), pool.data_ptr(), table.data_ptr(), c["start"], c["num"], c["layers"], c["page"],
                       c["max_pages"])
        src = dev(c["src"])
        L.refp_inject(pool.data_ptr(), src.data_ptr(), table.data_ptr(), c["start"], c["num"], c["layers"], c["page"],
                      c["max_pages"])
        assert L.refp_sync() == 0
        out[name + "_extract_sha256"] = paged_cases.digest(host(dst))
        out[name + "_pool_after_inject_sha256"] = paged_cases.digest(host(pool))
        print(name, "extract digest", out[name + "_extract_sha256"][:4])
    np.savez_compressed(out_path, **out)
    print("wrote", out_path)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
