"""A whole decode step (append + attention, every layer) captured once in a CUDA graph and replayed
for several tokens: positions and lengths live in device arrays, the launch shapes depend only on a
fixed upper bound of the lengths, and page allocation + table sync stay outside the graph.  Each replay
is checked against the CPU checker."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def test_decode_step_replays_from_a_cuda_graph(drkv_lib, oracle):
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, d, page, dtype = 2, 32, 8, 128, 16, ob.BF16
    rng = np.random.default_rng(51)
    lens = np.array([700, 45, 1290, 16], dtype=np.int32)
    n_seq, steps = len(lens), 5
    bound = int(lens.max()) + steps + 1                       # what the grid and the scratch are sized for
    max_pages = int(sum((n + steps + page) // page for n in lens)) + 8
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=max_pages, max_seqs=n_seq, max_pages_per_seq=bound // page + 2, device=0)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    try:
        H.shuffled_free_stack(eng, rng)
        seqs = [eng.seq_create() for _ in range(n_seq)]
        for s, n in zip(seqs, lens):
            assert eng.ensure_blocks_for_range(s, 0, int(n))
            eng.set_seq_len(s, int(n))
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        d_rows = torch.tensor(seqs, dtype=torch.int32, device="cuda")
        d_pos = torch.from_numpy(lens.copy()).cuda()
        d_len = d_pos + 1
        q = torch.zeros(layers, n_seq, hq, d, dtype=torch.bfloat16, device="cuda")
        k = torch.zeros(layers, n_seq, hkv, d, dtype=torch.bfloat16, device="cuda")
        v = torch.zeros_like(k)
        out = torch.zeros_like(q)
        scale = 1.0 / np.sqrt(d)

        def step(stream):
            for l in range(layers):
                eng.append_rope(l, n_seq, d_rows, d_pos, k[l], v[l], stream)
                eng.attend_decode(l, n_seq, d_rows, d_len, bound, q[l], out[l], scale, stream)

        # first calls configure the kernels: they happen before the capture
        eng.reserve_batch(seqs, 1)
        eng.sync_block_table()
        step(torch.cuda.current_stream())
        torch.cuda.synchronize()
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))   # undo the warm-up append
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step(torch.cuda.current_stream())
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))   # capture launches nothing; keep it clean anyway

        cur = lens.copy()
        for it in range(steps):
            if it > 0:
                eng.reserve_batch(seqs, 1)
                eng.sync_block_table()
            hq_, hk_, hv_ = (H.randn_bits(rng, x.shape, dtype) for x in (q, k, v))
            q.copy_(H.to_dev(hq_, dtype)); k.copy_(H.to_dev(hk_, dtype)); v.copy_(H.to_dev(hv_, dtype))
            d_pos.copy_(torch.from_numpy(cur))
            torch.add(d_pos, 1, out=d_len)
            graph.replay()
            torch.cuda.synchronize()
            eng.check_kernels()
            tables = np.stack([eng.table(s) for s in seqs])
            for l in range(layers):
                for i in range(n_seq):
                    ob.append(g, pool_host, max_pages, tables[i], l, int(cur[i]), 1, hk_[l, i], hv_[l, i], rope=True)
                want = np.zeros((n_seq, hq, d), dtype=np.uint16)
                ob.attend_decode(g, pool_host, max_pages, tables, np.arange(n_seq), cur + 1, l, hq_[l], want, scale)
                got_f, want_f = ob.to_float(H.torch_bits(out[l]), dtype), ob.to_float(want, dtype)
                assert (np.abs(got_f - want_f) <= np.maximum(2e-3, H.ulp(want_f, dtype))).all(), f"replay {it} layer {l}"
            assert np.array_equal(eng.pool_tensor().cpu().numpy().view(np.uint16), pool_host), f"replay {it}: pool bytes"
            cur += 1
            eng.advance_batch(seqs, 1)
    finally:
        eng.close()
