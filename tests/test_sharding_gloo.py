"""Multi-rank host logic on CPU: page-range partition of one long sequence with an all-gather of
the per-rank partials (gloo, world size 2 and 3), and data-parallel placement of sequences.  The
per-rank arithmetic here is the CPU checker; what is under test is the partition, the gather order
and the merge contract that the GPU path (drkv_attend_partial + NCCL + drkv_combine_partials) uses."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deusridet_b200 import sharding


def test_page_ranges_tile_the_sequence():
    for n_pages in (0, 1, 7, 8, 8192, 8195):
        for world in (1, 2, 3, 4, 8):
            ranges = [sharding.page_range_for_rank(n_pages, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == n_pages
            for a, b in zip(ranges, ranges[1:]):
                assert a[1] == b[0]
            sizes = [hi - lo for lo, hi in ranges]
            assert max(sizes) - min(sizes) <= 1
    # 524288 tokens, page 64, 8 ranks: 1024 pages = 65536 keys each
    assert sharding.key_range_for_rank(524288, 64, 3, 8) == (3 * 65536, 4 * 65536)
    assert sharding.key_range_for_rank(100, 64, 1, 8) == (64, 100)
    assert sharding.key_range_for_rank(100, 64, 5, 8) == (100, 100)       # empty range
    assert sharding.owner_of_position(524288, 524289, 64, 8) == 7
    assert sharding.owner_of_position(0, 524289, 64, 8) == 0


def test_sequences_are_balanced_and_families_stay_together():
    rng = np.random.default_rng(0)
    costs = rng.integers(1024, 8193, size=64).tolist()
    fam = list(range(64))
    fam[10] = fam[11] = fam[12] = 1000                                       # three forks of one prefix
    parts = sharding.shard_sequences(costs, 8, fam)
    assert sorted(sum(parts, [])) == list(range(64))
    owner = {i: r for r, p in enumerate(parts) for i in p}
    assert owner[10] == owner[11] == owner[12]
    loads = [sum(costs[i] for i in p) for p in parts]
    assert max(loads) / min(loads) < 1.25
    assert sharding.shard_sequences([5] * 1024, 8) == [list(range(r, 1024, 8)) for r in range(8)] or \
        all(len(p) == 128 for p in sharding.shard_sequences([5] * 1024, 8))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, seq_len, q_bits, pool, table, geom_args, scale, result):
    from oracle import cbind as ob
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = ob.geom(*geom_args)
    pages = pool.size // (geom_args[0] * 2 * geom_args[2] * geom_args[4] * geom_args[3])
    begin, end = sharding.key_range_for_rank(seq_len, geom_args[4], rank, world)
    part = ob.attend_partial(g, pool, pages, table, 0, begin, end, q_bits, scale)
    mine = torch.from_numpy(part)
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    parts = np.stack([t.numpy() for t in gathered])
    out = np.zeros((geom_args[1], geom_args[3]), dtype=np.uint16)
    ob.combine(g, parts, out)
    if rank == 0:
        result.copy_(torch.from_numpy(out.view(np.int16)))
    # every rank must arrive at the same merged output
    check = torch.from_numpy(out.view(np.int16).astype(np.int32))
    lo, hi = check.clone(), check.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    assert torch.equal(lo, hi)
    dist.destroy_process_group()


@pytest.mark.parametrize("world,seq_len", [(2, 1000), (3, 700), (2, 70)])
def test_split_sequence_allgather_combine(oracle, world, seq_len):
    ob = oracle
    rng = np.random.default_rng(world * 100 + seq_len)
    layers, hq, hkv, d, page = 1, 16, 2, 128, 64
    pages = (seq_len + page - 1) // page + 2
    geom_args = (layers, hq, hkv, d, page, ob.BF16, d, 1e6)
    g = ob.geom(*geom_args)
    pool = ob.from_float(rng.standard_normal(ob.pool_elems(g, pages), dtype=np.float32), ob.BF16)
    table = rng.permutation(pages).astype(np.int32)
    q = ob.from_float(rng.standard_normal((hq, d), dtype=np.float32), ob.BF16)
    scale = 1.0 / np.sqrt(d)
    result = torch.zeros((hq, d), dtype=torch.int16).share_memory_()
    mp.spawn(_rank_main, args=(world, _free_port(), seq_len, q, pool, table, geom_args, scale, result), nprocs=world,
             join=True)
    whole = np.zeros((1, hq, d), dtype=np.uint16)
    ob.attend_decode(g, pool, pages, table[None, :], [0], [seq_len], 0, q[None], whole, scale)
    got = ob.to_float(result.numpy().view(np.uint16), ob.BF16)
    assert np.abs(got - ob.to_float(whole[0], ob.BF16)).max() <= 2e-3


def _rank_with_departure(rank, world, ports, seq_len, q_bits, pool, table, geom_args, scale, result, status):
    """Step 0 with every rank; then the last rank leaves between steps (no collective in flight).  The survivors'
    next gather must end with an error they can turn into a status, not hang; they re-form a smaller world,
    re-split the page ranges over it and the step gives the whole-sequence answer again."""
    import datetime
    from oracle import cbind as ob
    g = ob.geom(*geom_args)
    pages = pool.size // (geom_args[0] * 2 * geom_args[2] * geom_args[4] * geom_args[3])

    def step(r, w):
        begin, end = sharding.key_range_for_rank(seq_len, geom_args[4], r, w)
        mine = torch.from_numpy(ob.attend_partial(g, pool, pages, table, 0, begin, end, q_bits, scale))
        gathered = [torch.empty_like(mine) for _ in range(w)]
        dist.all_gather(gathered, mine)
        out = np.zeros((geom_args[1], geom_args[3]), dtype=np.uint16)
        ob.combine(g, np.stack([t.numpy() for t in gathered]), out)
        return out

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{ports[0]}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=20))
    first = step(rank, world)
    if rank == 0:
        result[0].copy_(torch.from_numpy(first.view(np.int16)))
    dist.barrier()
    if rank == world - 1:                    # leaves between steps, with none of its collectives in flight
        dist.destroy_process_group()
        return
    lost = 0
    try:
        step(rank, world)
    except Exception:                        # RuntimeError / DistBackendError: the peer is gone or the gather timed out
        lost = 1
    status[rank] = lost
    try:
        dist.destroy_process_group()
    except Exception:
        pass
    survivors = world - 1
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{ports[1]}", rank=rank, world_size=survivors,
                            timeout=datetime.timedelta(seconds=20))
    again = step(rank, survivors)
    if rank == 0:
        result[1].copy_(torch.from_numpy(again.view(np.int16)))
    dist.destroy_process_group()


def test_rank_leaves_between_steps_and_the_world_is_reformed(oracle):
    """Failure detection on the host, without a GPU: what is under test is the protocol around the collective
    (an error status instead of a hang, re-partition by sharding.key_range_for_rank over the survivors, the same
    answer afterwards).  Every rank holds the whole cache here; bringing a lost rank's pages back (storage tier,
    re-prefill) is the caller's business."""
    ob = oracle
    rng = np.random.default_rng(77)
    world, seq_len = 3, 900
    layers, hq, hkv, d, page = 1, 8, 2, 128, 64
    pages = (seq_len + page - 1) // page + 2
    geom_args = (layers, hq, hkv, d, page, ob.BF16, d, 1e6)
    g = ob.geom(*geom_args)
    pool = ob.from_float(rng.standard_normal(ob.pool_elems(g, pages), dtype=np.float32), ob.BF16)
    table = rng.permutation(pages).astype(np.int32)
    q = ob.from_float(rng.standard_normal((hq, d), dtype=np.float32), ob.BF16)
    scale = 1.0 / np.sqrt(d)
    result = torch.zeros((2, hq, d), dtype=torch.int16).share_memory_()
    status = torch.full((world,), -1, dtype=torch.int32).share_memory_()
    mp.spawn(_rank_with_departure, args=(world, (_free_port(), _free_port()), seq_len, q, pool, table, geom_args, scale,
                                         result, status), nprocs=world, join=True)
    assert status[:world - 1].tolist() == [1] * (world - 1), "the survivors did not see the departure as an error"
    whole = np.zeros((1, hq, d), dtype=np.uint16)
    ob.attend_decode(g, pool, pages, table[None, :], [0], [seq_len], 0, q[None], whole, scale)
    want = ob.to_float(whole[0], ob.BF16)
    for k in range(2):                       # before the departure (3 ranks) and after it (2 ranks)
        got = ob.to_float(result[k].numpy().view(np.uint16), ob.BF16)
        assert np.abs(got - want).max() <= 2e-3, k
