"""Worker of tests/test_gpu_exchange.py: one process per GPU (launched by torch.distributed.run).  Every rank
holds the whole sequence, attends only its own key range and merges across ranks with drkv_attend_exchange;
rank 0 checks the result against the CPU checker over the whole sequence.  Then one rank stays away from a
call: the other's bounded wait must give up with kernel error 4 and leave the context usable."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from deusridet_b200 import PagedKVEngine, sharding  # noqa: E402
from oracle import cbind as ob  # noqa: E402
from tests import helpers as H  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dist.init_process_group("gloo")                      # host-side plumbing only: handles and barriers
    torch.cuda.set_device(local)
    layers, hq, hkv, d, page, dtype = 2, 16, 4, 128, 16, ob.BF16
    n_tok, max_pages = 16 * 37 + 5, 64
    rng = np.random.default_rng(42)                      # same on every rank
    eng = PagedKVEngine(num_layers=layers, num_q_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, dtype="bf16",
                        rope_theta=1e6, max_pages=max_pages, max_seqs=1, max_pages_per_seq=48, device=local)
    g = ob.geom(layers, hq, hkv, d, page, dtype, d, 1e6)
    failures = []
    try:
        H.shuffled_free_stack(eng, rng)
        s = eng.seq_create()
        eng.reserve(s, n_tok)
        eng.set_seq_len(s, n_tok)
        pool_host = H.randn_bits(rng, ob.pool_elems(g, max_pages), dtype)
        eng.pool_tensor().copy_(torch.from_numpy(pool_host.view(np.int16)))
        eng.sync_block_table()
        table = np.full((1, eng.table_stride()), -1, dtype=np.int32)
        t = eng.table(s)
        table[0, :len(t)] = t
        handle = eng.exchange_create(world, rank)
        handles = [None] * world
        dist.all_gather_object(handles, handle)
        eng.exchange_connect(handles)
        eng.exchange_set_wait_ms(200)                    # a peer that stays away is given up on after 0.2 s
        dist.barrier()
        begin, end = sharding.key_range_for_rank(n_tok, page, rank, world)
        scale = 1.0 / np.sqrt(d)
        for rep in range(3):                             # three rounds: both parities of the area get reused
            for layer in range(layers):
                q = H.randn_bits(rng, (1, hq, d), dtype)
                out = torch.zeros(hq, d, dtype=torch.bfloat16, device="cuda")
                eng.attend_exchange(layer, s, begin, end, H.to_dev(q, dtype), out, scale)
                torch.cuda.synchronize()
                eng.check_kernels()
                want = np.zeros((1, hq, d), dtype=np.uint16)
                ob.attend_decode(g, pool_host, max_pages, table, np.arange(1), np.array([n_tok], dtype=np.int32), layer, q,
                                 want, scale)
                err = np.abs(ob.to_float(H.torch_bits(out), dtype) - ob.to_float(want[0], dtype)).max()
                if err > 2e-3:
                    failures.append(f"rank {rank} rep {rep} layer {layer}: max abs error {err}")
        dist.barrier()
        # ---- a peer that does not arrive: rank 0 calls, the others do not ----
        if world > 1:
            if rank == 0:
                q = H.randn_bits(rng, (1, hq, d), dtype)
                out = torch.zeros(hq, d, dtype=torch.bfloat16, device="cuda")
                eng.attend_exchange(0, s, begin, end, H.to_dev(q, dtype), out, scale)
                torch.cuda.synchronize()
                try:
                    eng.check_kernels()
                    failures.append("rank 0: the wait for an absent peer did not report an error")
                except RuntimeError as e:
                    if "error code 4" not in str(e):
                        failures.append(f"rank 0: unexpected error {e}")
                # the context is still usable
                x = torch.ones(8, device="cuda")
                if float(x.sum().item()) != 8.0:
                    failures.append("rank 0: context unusable after the timed-out wait")
            dist.barrier()
        eng.exchange_destroy()
    finally:
        eng.close()
    all_fail = [None] * world
    dist.all_gather_object(all_fail, failures)
    dist.destroy_process_group()
    flat = [f for fs in all_fail for f in fs]
    if rank == 0:
        print("EXCHANGE_WORKER", "OK" if not flat else "FAILED: " + "; ".join(flat), flush=True)
    sys.exit(1 if flat else 0)


if __name__ == "__main__":
    main()
