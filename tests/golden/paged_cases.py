"""Seeded inputs of the cases whose outputs were recorded from the reference's own CUDA kernels
(tests/golden/paged_attention_reference.npz).  Shared by the recorder and by the tests, so that both
rebuild bit-identical inputs from the seed."""
import hashlib

import numpy as np

from oracle import cbind as ob

# Decode step (apply_rope -> paged_kv_cache_write[_batch] -> paged_gqa_decode_attention), fp16.
# name: (hq, hkv, d, rot, theta, page, layers, layer, seq_len (cached tokens), m_batch, seed)
CASES = {
    # config 1 of the benchmark list: 16/4 heads, head_dim 128, fp16, page 16, 512 cached tokens, RoPE base 1e4
    "toy": (16, 4, 128, 128, 1e4, 16, 1, 0, 512, 0, 101),
    # the reference's own model shape: 24/4 heads, head_dim 256, block 256, partial rotary 64
    "model": (24, 4, 256, 64, 1e7, 256, 2, 1, 1000, 37, 102),
    "small_page": (8, 4, 64, 64, 1e4, 32, 1, 0, 77, 5, 103),
    # more than 4096 keys: several split-KV chunks per head and an odd tail in this repository's kernel
    "long": (16, 4, 128, 128, 1e4, 16, 1, 0, 4603, 0, 104),
}

# Chunked prefill (paged_rope_batch_kernel -> paged_kv_cache_write_batch -> paged_prefill_attention_kernel), fp16.
# name: (hq, hkv, d, rot, theta, page, layers, layer, pos_start, m, seed)
PREFILL_CASES = {
    "pf_toy": (16, 4, 128, 128, 1e4, 16, 1, 0, 200, 48, 201),
    # the reference's model shape; the chunk crosses the boundary of its 256-key block
    "pf_model": (24, 4, 256, 64, 1e7, 256, 2, 1, 246, 20, 202),
    "pf_d64": (8, 4, 64, 64, 1e4, 32, 1, 0, 45, 40, 203),
    # first chunk of a sequence (nothing cached), GQA group of 7 as in the chunked-prefill benchmark config
    "pf_first_g7": (28, 4, 128, 128, 1e6, 16, 1, 0, 0, 24, 204),
}

# bf16 split-K decode + merge (invoke_causal_gqa_decode, 128-key partitions, head_dim 128).
# name: (hq, hkv, d, seq_len, seed)
SPLITK_CASES = {
    "sk_c2_shape": (32, 8, 128, 1000, 301),     # the batched-decode benchmark's head shape; last partition partial
    "sk_long": (16, 4, 128, 4500, 302),
    "sk_one_partition": (8, 8, 128, 100, 303),
}

# Flat <-> paged copies (invoke_extract_kv_from_pages / invoke_inject_kv_to_pages), any 16-bit payload.
# name: (layers, hkv, d, page, n_pages, hole_at (logical page or -1), start_token, num_tokens, seed)
FLAT_CASES = {
    "xi_hole": (2, 4, 64, 16, 10, 3, 21, 100, 401),
    "xi_model": (3, 4, 256, 256, 3, -1, 200, 400, 402),
}


def digest(a) -> np.ndarray:
    """SHA-256 of an array's bytes as 32 uint8 values (what the golden file stores for bulky byte-exact results)."""
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), dtype=np.uint8).copy()


def build(name):
    """Returns a dict with geometry, table, initial pool, and the step's K/V/Q (fp16 bit patterns)."""
    hq, hkv, d, rot, theta, page, layers, layer, seq_len, m_batch, seed = CASES[name]
    rng = np.random.default_rng(seed)
    total = seq_len + m_batch + 1
    n_pages = (total + page - 1) // page
    max_pages = max(n_pages + 3, 2 * n_pages if name == "toy" else n_pages + 3)
    g = ob.geom(layers, hq, hkv, d, page, ob.F16, rot, theta)
    table = rng.permutation(max_pages)[:n_pages].astype(np.int32)
    f16 = lambda shape: ob.from_float(rng.standard_normal(shape, dtype=np.float32), ob.F16)
    return dict(name=name, g=g, hq=hq, hkv=hkv, d=d, rot=rot, theta=theta, page=page, layers=layers, layer=layer,
                seq_len=seq_len, m_batch=m_batch, max_pages=max_pages, table=table,
                pool=f16(ob.pool_elems(g, max_pages)), kb=f16((max(m_batch, 1), hkv, d)), vb=f16((max(m_batch, 1), hkv, d)),
                k1=f16((hkv, d)), v1=f16((hkv, d)), q=f16((hq, d)))


def build_prefill(name):
    """One prefill chunk: m tokens at pos_start on top of a pool whose earlier positions hold N(0,1) values."""
    hq, hkv, d, rot, theta, page, layers, layer, pos_start, m, seed = PREFILL_CASES[name]
    rng = np.random.default_rng(seed)
    n_pages = (pos_start + m + page - 1) // page
    max_pages = n_pages + 3
    g = ob.geom(layers, hq, hkv, d, page, ob.F16, rot, theta)
    table = rng.permutation(max_pages)[:n_pages].astype(np.int32)
    f16 = lambda shape: ob.from_float(rng.standard_normal(shape, dtype=np.float32), ob.F16)
    return dict(name=name, g=g, hq=hq, hkv=hkv, d=d, rot=rot, theta=theta, page=page, layers=layers, layer=layer,
                pos_start=pos_start, m=m, max_pages=max_pages, table=table, pool=f16(ob.pool_elems(g, max_pages)),
                q=f16((m, hq, d)), k=f16((m, hkv, d)), v=f16((m, hkv, d)))


def build_splitk(name):
    """A contiguous bf16 cache [seq][Hkv][D] (the layout invoke_causal_gqa_decode reads) and the same values in a
    one-layer paged pool of 16-key pages behind a permuted table."""
    hq, hkv, d, seq_len, seed = SPLITK_CASES[name]
    page = 16
    rng = np.random.default_rng(seed)
    n_pages = (seq_len + page - 1) // page
    max_pages = n_pages + 5
    g = ob.geom(1, hq, hkv, d, page, ob.BF16, 0, 1e4)
    table = rng.permutation(max_pages)[:n_pages].astype(np.int32)
    bf = lambda shape: ob.from_float(rng.standard_normal(shape, dtype=np.float32), ob.BF16)
    k_cache, v_cache, q = bf((seq_len, hkv, d)), bf((seq_len, hkv, d)), bf((hq, d))
    pool = bf(ob.pool_elems(g, max_pages))          # stale values wherever the sequence does not reach
    flat = np.stack([k_cache, v_cache])[None]       # [1 layer][K|V][token][head][dim]
    ob.inject(g, pool, flat, max_pages, table, 0, seq_len)
    return dict(name=name, g=g, hq=hq, hkv=hkv, d=d, page=page, seq_len=seq_len, max_pages=max_pages, table=table,
                pool=pool, k_cache=k_cache, v_cache=v_cache, q=q, n_parts=(seq_len + 127) // 128)


def build_flat(name):
    layers, hkv, d, page, n_pages, hole_at, start, num, seed = FLAT_CASES[name]
    rng = np.random.default_rng(seed)
    max_pages = n_pages + 4
    g = ob.geom(layers, 2 * hkv, hkv, d, page, ob.F16, 0, 1e4)
    table = rng.permutation(max_pages)[:n_pages].astype(np.int32)
    if hole_at >= 0:
        table[hole_at] = -1
    bits = lambda shape: rng.integers(0, 1 << 16, size=shape, dtype=np.uint16)
    return dict(name=name, g=g, layers=layers, hkv=hkv, d=d, page=page, max_pages=max_pages, table=table,
                start=start, num=num, pool=bits(ob.pool_elems(g, max_pages)), src=bits((layers, 2, num, hkv, d)))


def splitk_parts_external(part_o, part_m, part_l, hq, d, n_parts):
    """The reference's split-K workspace ([Hq][parts][D] o, [Hq][parts] m and l) rearranged into this
    repository's external partial layout: per part [Hq*D o | Hq m | Hq l]."""
    out = np.empty((n_parts, hq * (d + 2)), dtype=np.float32)
    out[:, :hq * d] = part_o.reshape(hq, n_parts, d).transpose(1, 0, 2).reshape(n_parts, hq * d)
    out[:, hq * d:hq * d + hq] = part_m.reshape(hq, n_parts).T
    out[:, hq * (d + 1):] = part_l.reshape(hq, n_parts).T
    return out
