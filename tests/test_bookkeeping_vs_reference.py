"""Host bookkeeping (pool ids, tables, eviction order) of libdrkv.so against the reference's own
BlockPool / CacheManager: against the recorded goldens always, and against the reference objects
compiled in oracle/_ref/ whenever they are present (they are built where the reference tree is
mounted).  Bit-exact: these are integers."""
import json
import os
import subprocess

import pytest

from tests import ref_driver as R

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden")

with open(os.path.join(GOLD, "bookkeeping_traces.json")) as f:
    GOLDEN = json.load(f)


@pytest.mark.parametrize("case", GOLDEN["traces"], ids=lambda c: f"seed{c['seed']}-{c['pages']}pages")
def test_engine_matches_recorded_reference_trace(drkv_lib, case):
    eng = R.EngineAsCacheManager(2, case["pages"], case["page_size"])
    got = R.run_ops(eng, case["ops"], case["pages"])
    eng.close()
    for i, (g, w) in enumerate(zip(got, case["trace"])):
        assert g == w, f"op {i} {case['ops'][i] if i < len(case['ops']) else 'final table'}: {g} != {w}"
    assert len(got) == len(case["trace"])


@pytest.mark.parametrize("case", GOLDEN["traces"], ids=lambda c: f"seed{c['seed']}-{c['pages']}pages")
def test_python_model_matches_recorded_reference_trace(case):
    m = R.ModelAsCacheManager(2, case["pages"], case["page_size"])
    assert R.run_ops(m, case["ops"], case["pages"]) == case["trace"]


@pytest.mark.skipif(not R.ref_available(), reason="oracle/_ref not built (reference tree not mounted)")
@pytest.mark.parametrize("seed", range(100, 112))
def test_engine_matches_live_reference_objects(drkv_lib, seed):
    pages = [4, 7, 16, 40][seed % 4]
    psize = [16, 64, 256][seed % 3]
    ops = R.random_ops(seed, pages, psize, 400)
    ref = R.RefCacheManager(3, pages, psize)
    eng = R.EngineAsCacheManager(3, pages, psize)
    want, got = R.run_ops(ref, ops, pages), R.run_ops(eng, ops, pages)
    ref.close()
    eng.close()
    assert got == want


# ---- CacheManager with an ImportanceScorer attached (cache_manager.cpp:185-205, importance_scorer.cu:75-87) ----
@pytest.mark.parametrize("case", GOLDEN["scored"], ids=lambda c: f"seed{c['seed']}-{c['pages']}pages-decay{c['decay']}")
def test_scored_engine_matches_recorded_reference_trace(drkv_lib, case):
    eng = R.EngineAsCacheManager(2, case["pages"], case["page_size"], decay=case["decay"])
    got = R.run_ops(eng, case["ops"], case["pages"])
    eng.close()
    for i, (g, w) in enumerate(zip(got, case["trace"])):
        assert g == w, f"op {i} {case['ops'][i] if i < len(case['ops']) else 'final table'}: {g} != {w}"
    assert len(got) == len(case["trace"])
    assert any(op[0] == "evict" and rec[0] > 0 for op, rec in zip(case["ops"], case["trace"]))


@pytest.mark.parametrize("case", GOLDEN["scored"], ids=lambda c: f"seed{c['seed']}-{c['pages']}pages-decay{c['decay']}")
def test_scored_python_model_matches_recorded_reference_trace(oracle, case):
    m = R.ModelAsCacheManager(2, case["pages"], case["page_size"], decay=case["decay"])
    assert R.run_ops(m, case["ops"], case["pages"]) == case["trace"]


@pytest.mark.skipif(not R.ref_available(), reason="oracle/_ref not built (reference tree not mounted)")
@pytest.mark.parametrize("seed", range(200, 210))
def test_scored_engine_matches_live_reference_objects(drkv_lib, seed):
    pages = [4, 7, 16, 40][seed % 4]
    psize = [16, 64, 256][seed % 3]
    decay = [0.95, 0.5, 1.0][seed % 3]
    ops = R.random_ops(seed, pages, psize, 400, scored=True)
    ref = R.RefScoredCacheManager(3, pages, psize, decay)
    eng = R.EngineAsCacheManager(3, pages, psize, decay=decay)
    want, got = R.run_ops(ref, ops, pages), R.run_ops(eng, ops, pages)
    ref.close()
    eng.close()
    assert got == want


def test_scored_eviction_differs_from_oldest_first(drkv_lib):
    """The policy matters: with scores attached the victim is the lowest-scored page, not the oldest."""
    import numpy as np
    eng = R.EngineAsCacheManager(1, 8, 16, decay=0.5)
    for pos in range(0, 6 * 16, 16):
        assert eng.ensure(pos)
    eng.score_update(np.array([5, 4, 0.5, 3, 0.5, 9], dtype=np.float32))
    assert eng.evict(2) == 2
    t = eng.table(8)
    assert t[2] == -1 and t[4] == -1 and all(t[i] >= 0 for i in (0, 1, 3, 5))   # ties: allocation order
    eng.close()


@pytest.mark.parametrize("case", GOLDEN["pool"], ids=lambda c: f"{c['layers']}L-{c['pages']}p")
def test_pool_sizing_and_offsets(drkv_lib, oracle, case):
    """max_blocks from the budget by integer division, total_bytes, k/v byte offsets
    (src/memoria/block_pool.cpp:30-41, 89-95) - with the reference's compile-time 4 KV heads x 256 dims."""
    from deusridet_b200 import PagedKVEngine
    layers, pages, ps = case["layers"], case["pages"], case["page_size"]
    budget = layers * 2 * 4 * ps * 256 * 2 * pages + case["extra"]
    e = PagedKVEngine(num_layers=layers, num_q_heads=24, num_kv_heads=4, head_dim=256, page_size=ps, dtype="f16",
                      rotary_dim=64, budget_bytes=budget, max_seqs=1, device=-1)
    assert e.max_blocks() == case["max_blocks"]
    assert e.total_bytes() == case["total_bytes"]
    g = oracle.geom(layers, 24, 4, 256, ps, oracle.F16, 64, 1e7)
    for li, l in enumerate((0, layers - 1)):
        for pi, p in enumerate((0, 1, pages - 1)):
            assert e.k_offset(l, p) == case["k_offsets"][li][pi]
            assert e.v_offset(l, p) == case["v_offsets"][li][pi]
            # the checker's addressing is the same function
            assert 2 * oracle.pool_elem(g, case["max_blocks"], l, p, 0, 0, 0) == case["k_offsets"][li][pi]
            assert 2 * oracle.pool_elem(g, case["max_blocks"], l, p, 1, 0, 0) == case["v_offsets"][li][pi]
    e.close()


def test_pool_below_four_pages_is_refused(drkv_lib):
    from deusridet_b200 import DrkvError, PagedKVEngine
    with pytest.raises(DrkvError):
        PagedKVEngine(num_layers=1, num_q_heads=4, num_kv_heads=4, head_dim=128, page_size=16, max_pages=3,
                      max_seqs=1, device=-1)


def _build_shim_scenario(tmp_path):
    exe = str(tmp_path / "memoria_scenario_shim")
    cuda_inc = "/usr/local/cuda/include"
    cmd = ["g++", "-std=c++17", "-O1", f"-I{ROOT}/include", f"-I{cuda_inc}", f"{ROOT}/tests/cpp/memoria_scenario.cpp",
           "-o", exe, f"-L{ROOT}/deusridet_b200", "-ldrkv", f"-Wl,-rpath,{ROOT}/deusridet_b200"]
    subprocess.run(cmd, check=True)
    return exe


def test_reference_class_scenario_through_the_shim(drkv_lib, tmp_path):
    """tests/cpp/memoria_scenario.cpp is written against the reference's BlockPool / CacheManager
    interface; built on include/deusridet_shim.hpp + libdrkv.so it must print what the build
    against the reference's own sources printed (tests/golden/memoria_scenario.txt)."""
    exe = _build_shim_scenario(tmp_path)
    env = dict(os.environ, DRKV_SHIM_DEVICE="-1")
    got = subprocess.run([exe], check=True, capture_output=True, text=True, env=env).stdout
    with open(os.path.join(GOLD, "memoria_scenario.txt")) as f:
        assert got == f.read()
    if os.path.exists(R.REF_SCENARIO):
        live = subprocess.run([R.REF_SCENARIO], check=True, capture_output=True, text=True).stdout
        assert got == live
