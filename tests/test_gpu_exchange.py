"""Cross-GPU merge of split-KV partials by peer stores (drkv_attend_exchange).  On one GPU: a world of one
rank against the per-call path.  With two or more GPUs: one process per GPU merges a sequence split by key
range and is checked against the CPU checker; a peer that stays away makes the bounded wait give up."""
import os
import subprocess
import sys

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_world_of_one_equals_partial_plus_merge(drkv_lib, oracle):
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, d, page, dtype = 2, 32, 8, 128, 16, ob.BF16
    rng = np.random.default_rng(8)
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=80, max_seqs=1, max_pages_per_seq=70, device=0)
    try:
        s = eng.seq_create()
        n_tok = 16 * 60 + 9
        eng.reserve(s, n_tok)
        eng.set_seq_len(s, n_tok)
        eng.pool_tensor().copy_(torch.from_numpy(H.randn_bits(rng, eng.pool_tensor().numel(), dtype).view(np.int16)))
        eng.sync_block_table()
        handle = eng.exchange_create(1, 0)
        assert len(handle) == 64
        eng.exchange_connect([handle])
        part = torch.zeros(eng.partial_floats(), dtype=torch.float32, device="cuda")
        for rep in range(3):
            for layer in range(layers):
                q = H.to_dev(H.randn_bits(rng, (1, hq, d), dtype), dtype)
                a = torch.zeros(hq, d, dtype=torch.bfloat16, device="cuda")
                b = torch.zeros_like(a)
                eng.attend_exchange(layer, s, 0, n_tok, q, a, 0.088)
                eng.attend_partial(layer, s, 0, n_tok, q, part, 0.088)
                eng.combine_partials(1, part, b)
                torch.cuda.synchronize()
                eng.check_kernels()
                assert torch.equal(a, b), f"rep {rep} layer {layer}"
        eng.exchange_destroy()
        with pytest.raises(RuntimeError, match="create and connect"):
            eng.attend_exchange(0, s, 0, n_tok, q, a, 0.088)
    finally:
        eng.close()


def test_absent_peer_ends_the_bounded_wait(drkv_lib, oracle):
    """A world of two in which rank 1 never calls: rank 0's merge kernel pushes its partial, waits for rank 1's flags,
    gives up after the limit (50 ms here) with kernel error 4 and returns; the context stays usable and the next
    call works.  Both areas live on this GPU and are connected by pointer; only rank 0's kernel ever runs, so no
    kernel waits for another kernel of the same GPU."""
    import time
    import torch
    from deusridet_b200 import PagedKVEngine

    ob = oracle
    layers, hq, hkv, d, page, dtype = 1, 16, 4, 128, 16, ob.BF16
    rng = np.random.default_rng(9)
    mk = lambda: PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page,
                               dtype="bf16", rope_theta=1e6, max_pages=40, max_seqs=1, max_pages_per_seq=32, device=0)
    e0, e1 = mk(), mk()
    try:
        s = e0.seq_create()
        n_tok = 300
        e0.reserve(s, n_tok)
        e0.set_seq_len(s, n_tok)
        e0.pool_tensor().copy_(torch.from_numpy(H.randn_bits(rng, e0.pool_tensor().numel(), dtype).view(np.int16)))
        e0.sync_block_table()
        e0.exchange_create(2, 0)
        e1.exchange_create(2, 1)
        areas = [e0.exchange_area(), e1.exchange_area()]
        e0.exchange_connect_local(areas)
        e1.exchange_connect_local(areas)
        e0.exchange_set_wait_ms(50)
        q = H.to_dev(H.randn_bits(rng, (1, hq, d), dtype), dtype)
        out = torch.zeros(hq, d, dtype=torch.bfloat16, device="cuda")
        t0 = time.perf_counter()
        e0.attend_exchange(0, s, 0, n_tok, q, out, 0.088)
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 1.5, "the wait did not end at its limit"
        with pytest.raises(RuntimeError, match="error code 4"):
            e0.check_kernels()
        assert not out.any(), "no output may be written when a peer's partial is missing"
        # the context is usable and the engine still attends
        part = torch.zeros(e0.partial_floats(), dtype=torch.float32, device="cuda")
        e0.attend_partial(0, s, 0, n_tok, q, part, 0.088)
        e0.combine_partials(1, part, out)
        torch.cuda.synchronize()
        e0.check_kernels()
        assert out.float().abs().max().item() > 0
        e0.exchange_destroy()
        e1.exchange_destroy()
    finally:
        e0.close()
        e1.close()


def test_two_ranks_by_peer_stores(drkv_lib, oracle):
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = 2 if n < 4 else 4
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29541", os.path.join(ROOT, "tests", "mp_exchange_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert "EXCHANGE_WORKER OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]
