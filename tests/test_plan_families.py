"""The shared-prefix decode plan on an engine without a device: families of consecutive batch entries
whose block tables start with the same pages, their blocks of up to 16 query rows, and the chunk at
which every sequence's own items start.  Checked against a restatement over the tables read back and
against the invariant that makes the planned pass the same attention: every (sequence, chunk) of the
batch is covered exactly once, by a family block or by the sequence itself."""
import numpy as np
import pytest


def _engine(hq, hkv, page, max_pages=600, max_seqs=64, width=80):
    from deusridet_b200 import PagedKVEngine
    return PagedKVEngine(num_layers=1, num_q_heads=hq, num_kv_heads=hkv, head_dim=128, page_size=page, dtype="bf16",
                         rope_theta=1e6, max_pages=max_pages, max_seqs=max_seqs, max_pages_per_seq=width, device=-1)


def _grow(eng, s, n):
    eng.reserve(s, n)
    eng.set_seq_len(s, eng.seq_len(s) + n)


def _model(tables, lens, page, per_block, chunk):
    """Families the way the plan is specified: greedy runs from a leader; a neighbour joins while it has
    at least 64 keys and at least half of the run's shared keys in common with the leader."""
    n = len(lens)
    fams, fam_of, i = [], [-1] * n, 0
    while i < n and per_block >= 2:
        shared, j = lens[i], i + 1
        while j < n:
            same = 0
            while same < len(tables[i]) and same < len(tables[j]) and tables[i][same] >= 0 and tables[i][same] == tables[j][same]:
                same += 1
            common = min(same * page, lens[j])
            if common < 64 or common * 2 < shared:
                break
            shared = min(shared, common)
            j += 1
        if j - i >= 2:
            for k in range(i, j):
                fam_of[k] = len(fams)
            fams.append((i, j - i, shared))
        i = j
    first = [fams[f][2] // chunk if f >= 0 else 0 for f in fam_of]
    blocks = []
    for lead, count, shared in fams:
        if shared // chunk == 0:
            continue
        for m0 in range(0, count, per_block):
            blocks.append((lead, shared // chunk, list(range(lead + m0, lead + min(m0 + per_block, count)))))
    return first, blocks


@pytest.mark.parametrize("hq,hkv,page", [(32, 8, 16), (16, 2, 16), (8, 8, 32), (16, 1, 16), (8, 4, 64)])
def test_plan_matches_model_and_covers_every_chunk_once(drkv_lib, hq, hkv, page):
    rng = np.random.default_rng(hq * 100 + hkv + page)
    per_block = 16 // (hq // hkv)
    for trial in range(6):
        eng = _engine(hq, hkv, page)
        try:
            seqs = []
            for _ in range(int(rng.integers(1, 5))):                    # a few fork trees and loners
                root = eng.seq_create()
                _grow(eng, root, int(rng.integers(1, 40 * page)))
                members = [root]
                for _ in range(int(rng.integers(0, 12))):
                    parent = members[int(rng.integers(0, len(members)))] if rng.random() < 0.3 else root
                    child = eng.seq_fork(parent)
                    members.append(child)
                    if rng.random() < 0.8:
                        _grow(eng, child, int(rng.integers(1, 6 * page)))
                    if rng.random() < 0.3:
                        _grow(eng, parent, int(rng.integers(1, 3 * page)))
                seqs += members
            lens = [eng.seq_len(s) for s in seqs]
            tables = [eng.table(s).tolist() for s in seqs]
            chunk = int(rng.choice([64, 128, 256]))
            eng.set_chunk_tokens(chunk)
            info = eng.plan_decode(seqs, lens)
            plan = eng.plan_dump()
            first, blocks = _model(tables, lens, page, per_block, chunk)
            assert plan["rows"].tolist() == seqs and plan["kv_len"].tolist() == lens
            assert plan["first_chunk"].tolist() == first
            assert info["n_blocks"] == len(blocks) and info["chunk_tokens"] == chunk
            for k, (lead, chunks, members) in enumerate(blocks):
                assert plan["fb_row"][k] == seqs[lead] and plan["fb_chunks"][k] == chunks
                assert plan["fb_members"][k].tolist() == members + [-1] * (16 - len(members))
            # every (sequence, chunk) exactly once; a block's chunks lie in pages its members all hold
            cover = [np.zeros(-(-n // chunk), dtype=np.int32) for n in lens]
            for b, n in enumerate(lens):
                cover[b][plan["first_chunk"][b]:] += 1
            keys = sum(max(n - int(f) * chunk, 0) for n, f in zip(lens, plan["first_chunk"]))
            for k in range(info["n_blocks"]):
                sc = int(plan["fb_chunks"][k])
                keys += sc * chunk
                lead_table = eng.table(int(plan["fb_row"][k])).tolist()
                for b in plan["fb_members"][k]:
                    if b < 0:
                        continue
                    cover[b][:sc] += 1
                    assert sc * chunk <= lens[b]
                    n_pages = -(-sc * chunk // page)
                    assert tables[b][:n_pages] == lead_table[:n_pages]
            assert all((c == 1).all() for c in cover)
            assert info["keys_planned_pass"] == keys and info["keys_per_sequence_pass"] == sum(lens)
        finally:
            eng.close()


def test_group_of_sixteen_has_no_families(drkv_lib):
    eng = _engine(16, 1, 16)
    try:
        root = eng.seq_create()
        _grow(eng, root, 500)
        kids = [eng.seq_fork(root) for _ in range(3)]
        info = eng.plan_decode([root] + kids, [500] * 4)
        assert info["n_families"] == 0 and info["n_blocks"] == 0
    finally:
        eng.close()


def test_attention_calls_still_need_a_device(drkv_lib):
    eng = _engine(8, 2, 16)
    try:
        s = eng.seq_create()
        _grow(eng, s, 100)
        eng.plan_decode([s], [100])
        with pytest.raises(RuntimeError, match="without a device"):
            eng.attend_decode_planned(0, 1, 1, 1.0)
    finally:
        eng.close()
