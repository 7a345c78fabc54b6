"""Records what the reference's own BlockPool / CacheManager objects do (compiled from the
mounted reference tree into oracle/_ref/ by oracle/ref_build/Makefile) for seeded operation
sequences, and the text their class-level scenario prints.  Run where the reference tree is
mounted; the outputs are committed so that the tests can use them where it is not.

    python tests/golden/make_bookkeeping_golden.py
"""
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from tests.ref_driver import RefCacheManager, RefBlockPool, RefScoredCacheManager, random_ops, run_ops  # noqa: E402

CASES = [  # (seed, pages, page_size, n_ops)
    (1, 8, 16, 120), (2, 5, 16, 200), (3, 33, 256, 300), (4, 64, 16, 600), (5, 4, 64, 150), (6, 129, 16, 900),
]


SCORED_CASES = [  # (seed, pages, page_size, n_ops, decay): CacheManager with an ImportanceScorer attached
    (11, 8, 16, 200, 0.95), (12, 5, 16, 250, 0.5), (13, 40, 16, 600, 0.9), (14, 17, 64, 400, 0.0),
]


def main():
    subprocess.run(["make", "-C", os.path.join(ROOT, "oracle", "ref_build"), "-s", "all"], check=True)
    traces = []
    for seed, pages, psize, n_ops in CASES:
        ops = random_ops(seed, pages, psize, n_ops)
        ref = RefCacheManager(2, pages, psize)
        traces.append({"seed": seed, "pages": pages, "page_size": psize, "ops": ops,
                       "trace": run_ops(ref, ops, pages)})
        ref.close()
    scored = []
    for seed, pages, psize, n_ops, decay in SCORED_CASES:
        ops = random_ops(seed, pages, psize, n_ops, scored=True)
        ref = RefScoredCacheManager(2, pages, psize, decay)
        scored.append({"seed": seed, "pages": pages, "page_size": psize, "decay": decay, "ops": ops,
                       "trace": run_ops(ref, ops, pages)})
        ref.close()
    pool = []
    for layers, pages, psize, extra in [(1, 4, 16, 0), (16, 9, 256, 12345), (36, 100, 16, 1 << 20)]:
        bp = RefBlockPool(layers, pages, psize, extra)
        pool.append({"layers": layers, "pages": pages, "page_size": psize, "extra": extra,
                     "max_blocks": bp.max_blocks(), "total_bytes": bp.total_bytes(),
                     "k_offsets": [[bp.k_offset(l, p) for p in (0, 1, pages - 1)] for l in (0, layers - 1)],
                     "v_offsets": [[bp.v_offset(l, p) for p in (0, 1, pages - 1)] for l in (0, layers - 1)]})
        bp.close()
    with open(os.path.join(HERE, "bookkeeping_traces.json"), "w") as f:
        json.dump({"traces": traces, "scored": scored, "pool": pool}, f, separators=(",", ":"))
    out = subprocess.run([os.path.join(ROOT, "oracle", "_ref", "memoria_scenario_ref")], check=True,
                         capture_output=True, text=True).stdout
    with open(os.path.join(HERE, "memoria_scenario.txt"), "w") as f:
        f.write(out)
    print("wrote", len(traces), "traces,", len(scored), "scored traces,", len(pool), "pool cases, scenario text", len(out), "bytes")


if __name__ == "__main__":
    main()
