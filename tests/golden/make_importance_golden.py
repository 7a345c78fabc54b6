"""Records what the reference's own ImportanceScorer (src/memoria/importance_scorer.cu, compiled by
oracle/ref_build/Makefile into oracle/_ref/libref_paged.so) holds after seeded sequences of updates.
Needs a GPU:

    python tests/golden/make_importance_golden.py OUTPUT.npz

The result is committed as tests/golden/importance_reference.npz; importance_cases() below is the
seeded input both the recorder and the tests use."""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

CASES = {"decay095": (0.95, 300, 6, 1), "decay05": (0.5, 1000, 4, 2), "decay0": (0.0, 33, 3, 3), "decay1": (1.0, 257, 5, 4)}


def importance_cases():
    """name -> (decay, new_scores float32 [steps][n]): attention-mass-like values of mixed magnitude."""
    out = {}
    for name, (decay, n, steps, seed) in CASES.items():
        rng = np.random.default_rng(seed)
        new = (rng.random((steps, n)) * 10.0 ** rng.integers(-6, 2, size=(steps, n))).astype(np.float32)
        out[name] = (decay, new)
    return out


def main(out_path):
    L = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_paged.so"))
    L.refp_importance_run.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p]
    res = {}
    for name, (decay, new) in importance_cases().items():
        got = np.zeros_like(new)
        rc = L.refp_importance_run(new.ctypes.data, new.shape[0], new.shape[1], decay, got.ctypes.data)
        assert rc == 0, rc
        res[name] = got
        print(name, got[-1, :4])
    np.savez_compressed(out_path, **res)
    print("wrote", out_path)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
