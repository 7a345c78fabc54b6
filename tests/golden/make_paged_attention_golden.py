"""Records what the reference's own CUDA kernels (apply_rope, paged_kv_cache_write[_batch],
paged_gqa_decode_attention; compiled by oracle/ref_build/Makefile into oracle/_ref/libref_paged.so with the
reference's --use_fast_math) return for the seeded cases of tests/golden/paged_cases.py.  Needs a GPU:

    python tests/golden/make_paged_attention_golden.py OUTPUT.npz

The result is committed as tests/golden/paged_attention_reference.npz.  Flow per case, as in
full_attention_forward_paged (src/machina/paged_attention.cu:353-367): RoPE on Q and K at the new position,
write of K/V into the page, decode attention over seq_len + 1 keys; before that a batched write of m_batch
earlier tokens where the case has some."""
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
    np.savez_compressed(out_path, **out)
    print("wrote", out_path)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "gpurun_out", "paged_attention_reference.npz"))
