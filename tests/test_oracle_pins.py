"""Pins on the CPU checker itself (oracle/paged_kv_oracle.c): storage-type conversions against
torch, the sin/cos routine against correctly rounded values, RoPE and attention against
independent numpy fp64 restatements of the reference formulas, partial + merge against the
unsplit attention.  The reference has no golden vectors for this path, so these are the
strongest anchors available on a CPU."""
import numpy as np
import pytest
import torch


def test_storage_conversions_match_torch(oracle):
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-6, 1e-3, 1, 100, 7e4)])
    x = np.concatenate([x, np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8, 6.1e-5], dtype=np.float32)])
    for dt, tdt in ((oracle.F16, torch.float16), (oracle.BF16, torch.bfloat16)):
        want = torch.from_numpy(x).to(tdt).view(torch.int16).numpy().view(np.uint16)
        got = oracle.from_float(x, dt)
        assert np.array_equal(got, want)
        back = torch.from_numpy(want.view(np.int16)).view(tdt).float().numpy()
        assert np.array_equal(oracle.to_float(got, dt), back)


def test_sincos_is_the_correctly_rounded_value(oracle):
    """fp32 sin/cos of fp32 angles up to 6e5 rad (position 524287 x frequency 1)."""
    rng = np.random.default_rng(1)
    ang = np.concatenate([rng.random(30000) * 6e5, rng.random(10000) * 10, np.arange(0, 2000, dtype=np.float64)])
    ang = ang.astype(np.float32)
    s, c = oracle.sincos(ang)
    assert np.array_equal(s, np.sin(ang.astype(np.float64)).astype(np.float32))
    assert np.array_equal(c, np.cos(ang.astype(np.float64)).astype(np.float32))


@pytest.mark.parametrize("dtype_name,theta,rot,d", [("F16", 1e4, 128, 128), ("BF16", 1e6, 128, 128), ("F16", 1e7, 64, 256)])
def test_rope_append_follows_the_reference_formula(oracle, dtype_name, theta, rot, d):
    """src/machina/layer_attention.cu:44-58: pairs (i, i+rot/2), freq = 1/theta^(2i/rot),
    x0' = x0 cos - x1 sin, x1' = x1 cos + x0 sin; dims >= rot and V are copied."""
    dt = getattr(oracle, dtype_name)
    rng = np.random.default_rng(2)
    hkv, page, pages = 2, 16, 6
    g = oracle.geom(1, 4, hkv, d, page, dt, rot, theta)
    pool = np.zeros(oracle.pool_elems(g, pages), dtype=np.uint16)
    table = np.array([3, 1, 4, -1], dtype=np.int32)
    m, pos0 = 20, 9
    k = oracle.from_float(rng.standard_normal((m, hkv, d), dtype=np.float32), dt)
    v = oracle.from_float(rng.standard_normal((m, hkv, d), dtype=np.float32), dt)
    oracle.append(g, pool, pages, table, 0, pos0, m, k, v, rope=True)
    kf = oracle.to_float(k, dt).astype(np.float64)
    half = rot // 2
    inv = oracle.inv_freq(theta, rot).astype(np.float64)
    assert np.allclose(inv, 1.0 / theta ** (2 * np.arange(half) / rot), rtol=1e-6)
    eps = 2.0 ** -10 if dt == oracle.F16 else 2.0 ** -7
    for t in range(m):
        pos = pos0 + t
        ang = np.float32(pos) * inv.astype(np.float32)
        cs, sn = np.cos(ang.astype(np.float64)), np.sin(ang.astype(np.float64))
        for h in range(hkv):
            off = oracle.pool_elem(g, pages, 0, int(table[pos // page]), 0, h, pos % page)
            got = oracle.to_float(pool[off:off + d], dt).astype(np.float64)
            x0, x1 = kf[t, h, :half], kf[t, h, half:rot]
            want = np.concatenate([x0 * cs - x1 * sn, x1 * cs + x0 * sn, kf[t, h, rot:]])
            assert np.all(np.abs(got - want) <= eps * np.maximum(np.abs(want), 1e-3) + 1e-6)
            assert np.array_equal(got[rot:], kf[t, h, rot:])          # non-rotary dims verbatim
            voff = oracle.pool_elem(g, pages, 0, int(table[pos // page]), 1, h, pos % page)
            assert np.array_equal(pool[voff:voff + d], v[t, h])       # V verbatim
    # slots nobody wrote stay zero; the hole (-1) page entry is never touched
    written = np.zeros(pool.shape, dtype=bool)
    for t in range(m):
        pos = pos0 + t
        for kv in (0, 1):
            for h in range(hkv):
                off = oracle.pool_elem(g, pages, 0, int(table[pos // page]), kv, h, pos % page)
                written[off:off + d] = True
    assert not pool[~written].any()


def _numpy_attention(oracle, g, pool, pages, table, layer, q_bits, n, scale):
    hq, d, P = g.num_q_heads, g.head_dim, g.page_size
    group = hq // g.num_kv_heads
    out = np.zeros((hq, d))
    for h in range(hq):
        ks, vs = [], []
        for t in range(n):
            pg = int(table[t // P])
            if pg < 0:
                continue
            ko = oracle.pool_elem(g, pages, layer, pg, 0, h // group, t % P)
            vo = oracle.pool_elem(g, pages, layer, pg, 1, h // group, t % P)
            ks.append(oracle.to_float(pool[ko:ko + d], g.dtype))
            vs.append(oracle.to_float(pool[vo:vo + d], g.dtype))
        if not ks:
            continue
        K, V = np.array(ks, dtype=np.float64), np.array(vs, dtype=np.float64)
        s = K @ oracle.to_float(q_bits[h], g.dtype).astype(np.float64) * scale
        p = np.exp(s - s.max())
        out[h] = (p[:, None] * V).sum(0) / p.sum()
    return out


@pytest.mark.parametrize("dtype_name", ["F16", "BF16"])
def test_decode_attention_against_numpy_fp64(oracle, dtype_name):
    dt = getattr(oracle, dtype_name)
    rng = np.random.default_rng(3)
    layers, hq, hkv, d, page, pages = 2, 8, 2, 128, 16, 40
    g = oracle.geom(layers, hq, hkv, d, page, dt, d, 1e4)
    pool = oracle.from_float(rng.standard_normal(oracle.pool_elems(g, pages), dtype=np.float32), dt)
    tables = np.full((2, 24), -1, dtype=np.int32)
    perm = rng.permutation(pages)
    tables[0, :20] = perm[:20]
    tables[1, :15] = perm[20:35]
    tables[1, 3] = -1                                              # a hole
    lens = np.array([313, 230], dtype=np.int32)
    q = oracle.from_float(rng.standard_normal((2, hq, d), dtype=np.float32), dt)
    out = np.zeros((2, hq, d), dtype=np.uint16)
    scale = 1 / np.sqrt(d)
    oracle.attend_decode(g, pool, pages, tables, [0, 1], lens, 1, q, out, scale)
    f64 = oracle.attend_decode_f64(g, pool, pages, tables, [0, 1], lens, 1, q, scale)
    for b in range(2):
        want = _numpy_attention(oracle, g, pool, pages, tables[b], 1, q[b], int(lens[b]), scale)
        assert np.abs(f64[b] - want).max() < 1e-6
        assert np.abs(oracle.to_float(out[b], dt) - want).max() < 2e-3


def test_no_visible_key_leaves_output_untouched(oracle):
    """src/machina/paged_attention.cu:266-268."""
    g = oracle.geom(1, 4, 2, 64, 16, oracle.BF16, 64, 1e4)
    pool = np.zeros(oracle.pool_elems(g, 4), dtype=np.uint16)
    tables = np.full((1, 4), -1, dtype=np.int32)
    out = np.full((1, 4, 64), 0x1234, dtype=np.uint16)
    q = np.zeros((1, 4, 64), dtype=np.uint16)
    oracle.attend_decode(g, pool, 4, tables, [0], [40], 0, q, out, 0.125)      # every page is a hole
    assert (out == 0x1234).all()
    oracle.attend_decode(g, pool, 4, tables, [0], [0], 0, q, out, 0.125)       # no key at all
    assert (out == 0x1234).all()


def test_prefill_is_decode_per_token(oracle):
    """src/machina/paged_attention.cu:482-484: token t of the chunk sees pos_start + t + 1 keys."""
    rng = np.random.default_rng(4)
    dt = oracle.BF16
    hq, hkv, d, page, pages = 8, 2, 128, 16, 12
    g = oracle.geom(1, hq, hkv, d, page, dt, d, 1e4)
    pool = oracle.from_float(rng.standard_normal(oracle.pool_elems(g, pages), dtype=np.float32), dt)
    table = rng.permutation(pages).astype(np.int32)
    pos0, m = 37, 29
    q = oracle.from_float(rng.standard_normal((m, hq, d), dtype=np.float32), dt)
    out = np.zeros((m, hq, d), dtype=np.uint16)
    oracle.attend_prefill(g, pool, pages, table, 0, pos0, m, q, out, 1 / np.sqrt(d))
    for t in (0, 7, m - 1):
        one = np.zeros((1, hq, d), dtype=np.uint16)
        oracle.attend_decode(g, pool, pages, table[None, :], [0], [pos0 + t + 1], 0, q[t:t + 1], one, 1 / np.sqrt(d))
        assert np.array_equal(one[0], out[t])


def test_partials_merge_to_the_unsplit_result(oracle):
    """src/sensus/auditus/asr/asr_ops_attn.cu:88-108 semantics on paged keys, empty range included."""
    rng = np.random.default_rng(5)
    dt = oracle.BF16
    hq, hkv, d, page, pages = 16, 2, 128, 64, 20
    g = oracle.geom(1, hq, hkv, d, page, dt, d, 1e6)
    pool = oracle.from_float(rng.standard_normal(oracle.pool_elems(g, pages), dtype=np.float32), dt)
    table = rng.permutation(pages).astype(np.int32)
    n = 1111
    q = oracle.from_float(rng.standard_normal((hq, d), dtype=np.float32), dt)
    scale = 1 / np.sqrt(d)
    bounds = [0, 256, 256, 700, n]                                  # the second range is empty
    parts = np.stack([oracle.attend_partial(g, pool, pages, table, 0, bounds[i], bounds[i + 1], q, scale)
                      for i in range(4)])
    assert parts[1][hq * d:hq * d + hq].tolist() == [np.float32(-1e20)] * hq
    assert not parts[1][hq * (d + 1):].any()
    merged = np.zeros((hq, d), dtype=np.uint16)
    oracle.combine(g, parts, merged)
    whole = np.zeros((1, hq, d), dtype=np.uint16)
    oracle.attend_decode(g, pool, pages, table[None, :], [0], [n], 0, q[None], whole, scale)
    assert np.abs(oracle.to_float(merged, dt) - oracle.to_float(whole[0], dt)).max() <= 2e-3
