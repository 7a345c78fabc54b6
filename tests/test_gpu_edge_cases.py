"""Edges of the device path, against the CPU checker: a batch larger than one attention launch takes, empty
calls, single-token chunks at position 0 and deep in a context, and chunk lengths that straddle every tile and
block boundary of the prefill kernel."""
import numpy as np
import pytest

from tests.test_gpu_decode_step import _decode_case
from tests.test_gpu_prefill import _prefill_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fused", [False, True], ids=["separate_append", "fused_append"])
def test_decode_batch_larger_than_one_launch(drkv_lib, oracle, fused):
    """2 118 short sequences: one launch takes 2 048, so the step goes out in two slices whose row, length, Q, K/V
    and output pointers are offset; a wrong offset would show in the pool bytes or the outputs of the tail."""
    lens = np.random.default_rng(21).integers(0 if fused else 1, 40, size=2118)
    _decode_case(oracle, layers=1, hq=8, hkv=2, d=128, page=16, dtype=oracle.BF16, theta=1e4, lens=lens, seed=21,
                 fused=fused)


def test_empty_calls_do_nothing(drkv_lib, oracle):
    import torch
    from deusridet_b200 import PagedKVEngine

    eng = PagedKVEngine(num_layers=1, num_q_heads=8, num_kv_heads=2, head_dim=128, page_size=16, dtype="bf16",
                        rope_theta=1e4, max_pages=8, max_seqs=2, max_pages_per_seq=4, device=0)
    try:
        s = eng.seq_create()
        eng.reserve(s, 20)
        eng.set_seq_len(s, 20)
        eng.sync_block_table()
        pool = eng.pool_tensor()
        pool.fill_(3)
        before = pool.clone()
        rows = torch.tensor([s], dtype=torch.int32, device="cuda")
        lens = torch.tensor([20], dtype=torch.int32, device="cuda")
        kv = torch.zeros(1, 2, 128, dtype=torch.bfloat16, device="cuda")
        q = torch.zeros(1, 8, 128, dtype=torch.bfloat16, device="cuda")
        out = torch.full((1, 8, 128), 9.0, dtype=torch.bfloat16, device="cuda")
        eng.append_rope(0, 0, rows, lens, kv, kv)                          # no sequences
        eng.attend_decode(0, 0, rows, lens, 20, q, out, 0.1)               # no sequences
        eng.attend_decode(0, 1, rows, lens, 0, q, out, 0.1)                # no keys
        eng.append_attend_decode(0, 0, rows, lens, 20, kv, kv, q, out, 0.1)
        eng.append_rope_chunk(0, s, 0, 0, kv, kv)                          # empty chunk
        eng.attend_prefill_chunk(0, s, 0, 0, q, out, 0.1)
        flat = torch.full((1, 2, 4, 2, 128), 9.0, dtype=torch.bfloat16, device="cuda")
        eng.extract(s, 0, 0, flat)
        eng.inject(s, 0, 0, flat)
        torch.cuda.synchronize()
        eng.check_kernels()
        assert torch.equal(pool, before)
        assert (out == 9.0).all() and (flat == 9.0).all()
    finally:
        eng.close()


def test_prefill_single_token_chunks(drkv_lib, oracle):
    """A chunk of one token at position 0 (one visible key), then ordinary chunks, then one token deep in the
    context (a decode step through the prefill call)."""
    _prefill_case(oracle, layers=1, hq=8, hkv=2, page=16, dtype=oracle.BF16, theta=1e4,
                  chunks=[1, 1, 62, 300, 1, 1], seed=31)


def test_prefill_chunk_lengths_across_tile_and_block_boundaries(drkv_lib, oracle):
    """Group 4: a tile holds 32 tokens and a CTA 64; chunk lengths one short of, equal to and one past those, with
    starts that are not multiples of the 64-key block or the 16-token page."""
    _prefill_case(oracle, layers=1, hq=8, hkv=2, page=16, dtype=oracle.F16, theta=1e4,
                  chunks=[31, 32, 33, 63, 64, 65, 127, 129, 7], seed=32)


def test_prefill_group_that_does_not_divide_a_tile(drkv_lib, oracle):
    """Group 6 (24/4 heads as the reference's model, head_dim 128): 21 tokens per tile, 2 of its 128 rows unused."""
    _prefill_case(oracle, layers=1, hq=24, hkv=4, page=32, dtype=oracle.BF16, theta=1e6, chunks=[100, 43, 21, 22],
                  seed=33)


def test_prefill_head_dim_256_across_tile_boundaries(drkv_lib, oracle):
    """The reference's head shape (24/4 heads x 256, 256-key pages): one tile of 21 tokens per CTA; chunk lengths one
    short of, equal to and one past a tile and a few tiles, single tokens, and starts inside a page."""
    _prefill_case(oracle, layers=1, hq=24, hkv=4, page=256, dtype=oracle.BF16, theta=1e7, d=256,
                  chunks=[1, 20, 21, 22, 43, 1, 127, 129, 300], seed=34)


def test_prefill_head_dim_256_with_evicted_pages(drkv_lib, oracle):
    _prefill_case(oracle, layers=1, hq=24, hkv=4, page=64, dtype=oracle.F16, theta=1e7, d=256, chunks=[200, 150, 90],
                  seed=35, holes=2)


def test_prefill_head_dim_64_across_tile_boundaries(drkv_lib, oracle):
    _prefill_case(oracle, layers=1, hq=32, hkv=8, page=16, dtype=oracle.BF16, theta=1e4, d=64,
                  chunks=[1, 31, 32, 33, 63, 65, 200], seed=36, holes=1)
