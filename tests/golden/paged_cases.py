"""Seeded inputs of the cases whose outputs were recorded from the reference's own CUDA kernels
(tests/golden/paged_attention_reference.npz).  Shared by the recorder and by the tests, so that both
rebuild bit-identical inputs from the seed."""
import numpy as np

from oracle import cbind as ob

# name: (hq, hkv, d, rot, theta, page, layers, layer, seq_len (cached tokens), m_batch, seed)
CASES = {
    # BASELINE.json config 1: 16/4 heads, head_dim 128, fp16, page 16, 512 cached tokens, RoPE base 1e4
    "toy": (16, 4, 128, 128, 1e4, 16, 1, 0, 512, 0, 101),
    # the reference's own model shape: 24/4 heads, head_dim 256, block 256, partial rotary 64
    "model": (24, 4, 256, 64, 1e7, 256, 2, 1, 1000, 37, 102),
    "small_page": (8, 4, 64, 64, 1e4, 32, 1, 0, 77, 5, 103),
}


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
