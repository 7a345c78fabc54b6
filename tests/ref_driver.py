"""ctypes drivers for the reference's compiled Memoria objects (oracle/_ref/libref_memoria.so)
and the seeded operation generator shared by the golden recorder and the tests."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_memoria.so")
REF_SCENARIO = os.path.join(ROOT, "oracle", "_ref", "memoria_scenario_ref")

_ref = None


def ref_lib():
    global _ref
    if _ref is None:
        L = C.CDLL(REF_LIB)
        L.ref_cm_create.restype = C.c_void_p
        L.ref_bp_create.restype = C.c_void_p
        L.ref_bp_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_size_t]
        L.ref_scored_create.restype = C.c_void_p
        L.ref_scored_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_float, C.POINTER(C.c_void_p)]
        L.ref_scored_update.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.ref_scored_score.restype = C.c_float
        L.ref_scored_score.argtypes = [C.c_void_p, C.c_int]
        for n in ("ref_bp_total_bytes", "ref_bp_k_offset", "ref_bp_v_offset"):
            getattr(L, n).restype = C.c_size_t
        for n in dir(L):
            pass
        L.ref_quiet(1)
        _ref = L
    return _ref


def ref_available() -> bool:
    return os.path.exists(REF_LIB)


class RefCacheManager:
    def __init__(self, layers, pages, page_size):
        self.L = ref_lib()
        self.h = C.c_void_p(self.L.ref_cm_create(layers, pages, page_size))
        assert self.h.value
    def close(self): self.L.ref_cm_destroy(self.h)
    def ensure(self, pos): return self.L.ref_cm_ensure(self.h, pos)
    def ensure_range(self, pos, m): return self.L.ref_cm_ensure_range(self.h, pos, m)
    def evict(self, n): return self.L.ref_cm_evict(self.h, n)
    def ensure_free(self, n): return self.L.ref_cm_ensure_free(self.h, n)
    def set_len(self, n): self.L.ref_cm_set_seq_len(self.h, n)
    def num_logical(self): return self.L.ref_cm_num_logical_blocks(self.h)
    def free_blocks(self): return self.L.ref_cm_free_blocks(self.h)
    def used(self): return self.L.ref_cm_gpu_blocks_used(self.h)
    def pool_alloc(self): return self.L.ref_cm_pool_alloc(self.h)
    def pool_free(self, p): self.L.ref_cm_pool_free(self.h, p)
    def table(self, n):
        buf = (C.c_int * n)()
        got = self.L.ref_cm_table(self.h, buf, n)
        return list(buf)[:got]


class RefScoredCacheManager(RefCacheManager):
    """The reference's CacheManager with its own ImportanceScorer attached."""
    def __init__(self, layers, pages, page_size, decay):
        self.L = ref_lib()
        cm = C.c_void_p()
        self.owner = C.c_void_p(self.L.ref_scored_create(layers, pages, page_size, decay, C.byref(cm)))
        assert self.owner.value
        self.h = cm
        self.width = 2 * pages
    def close(self): self.L.ref_scored_destroy(self.owner)
    def score_update(self, values):
        arr = np.ascontiguousarray(values, dtype=np.float32)
        self.L.ref_scored_update(self.owner, arr.ctypes.data, len(arr))
    def scores(self):
        return np.array([self.L.ref_scored_score(self.owner, i) for i in range(self.width)], dtype=np.float32)


class RefBlockPool:
    def __init__(self, layers, pages, page_size, extra=0):
        self.L = ref_lib()
        self.h = C.c_void_p(self.L.ref_bp_create(layers, pages, page_size, extra))
        assert self.h.value
    def close(self): self.L.ref_bp_destroy(self.h)
    def max_blocks(self): return self.L.ref_bp_max_blocks(self.h)
    def total_bytes(self): return self.L.ref_bp_total_bytes(self.h)
    def k_offset(self, l, p): return self.L.ref_bp_k_offset(self.h, l, p)
    def v_offset(self, l, p): return self.L.ref_bp_v_offset(self.h, l, p)


class EngineAsCacheManager:
    """The same calls on libdrkv.so (bookkeeping-only engine, one sequence, stream_evict on)."""
    def __init__(self, layers, pages, page_size, decay=None):
        from deusridet_b200 import PagedKVEngine
        self.e = PagedKVEngine(num_layers=layers, num_q_heads=24, num_kv_heads=4, head_dim=256, page_size=page_size,
                               dtype="f16", rotary_dim=64, max_pages=pages, max_seqs=1, device=-1, stream_evict=True)
        if decay is not None:
            self.e.scorer_enable(decay)
        self.s = self.e.seq_create()
        self.held = []
    def score_update(self, values): self.e.scorer_update(self.s, np.asarray(values, dtype=np.float32))
    def scores(self): return self.e.scorer_scores(self.s)
    def close(self): self.e.close()
    def ensure(self, pos): return 1 if self.e.ensure_blocks_for(self.s, pos) else 0
    def ensure_range(self, pos, m): return 1 if self.e.ensure_blocks_for_range(self.s, pos, m) else 0
    def evict(self, n): return self.e.evict_blocks(self.s, n)
    def ensure_free(self, n): return 1 if self.e.ensure_free_blocks(self.s, n) else 0
    def set_len(self, n): self.e.set_seq_len(self.s, n)
    def num_logical(self): return self.e.num_logical_blocks(self.s)
    def free_blocks(self): return self.e.free_count()
    def used(self): return self.e.max_blocks() - self.e.free_count()
    def pool_alloc(self): return self.e.alloc_block()
    def pool_free(self, p): self.e.free_block(p)
    def table(self, n): return self.e.table(self.s, n).tolist()


class ModelAsCacheManager:
    """The same calls on the Python model (oracle/bookkeeping.py)."""
    def __init__(self, layers, pages, page_size, decay=None):
        from oracle.bookkeeping import BookModel
        self.m = BookModel(pages, page_size, 1, 0, True)
        self.s = self.m.seq_create()
        self.decay = decay
        if decay is not None:
            self.m.scores = {self.s: np.zeros(2 * pages, dtype=np.float32)}
    def score_update(self, values):
        from oracle import cbind
        v = np.asarray(values, dtype=np.float32)
        row = self.m.scores[self.s]
        head = np.ascontiguousarray(row[:len(v)])
        cbind.importance_update(head, v, self.decay)
        row[:len(v)] = head
    def scores(self): return self.m.scores[self.s]
    def close(self): pass
    def ensure(self, pos): return 1 if self.m.seq_ensure_pos(self.s, pos) == 0 else 0
    def ensure_range(self, pos, m): return 1 if self.m.seq_ensure_range(self.s, pos, m) == 0 else 0
    def evict(self, n): return self.m.seq_evict(self.s, n)
    def ensure_free(self, n): return self.m.ensure_free(self.s, n)
    def set_len(self, n): self.m.seq_set_len(self.s, n)
    def num_logical(self): return (self.m.seqs[self.s].len + self.m.P - 1) // self.m.P
    def free_blocks(self): return len(self.m.free)
    def used(self): return self.m.n - len(self.m.free)
    def pool_alloc(self): return self.m.pool_alloc()
    def pool_free(self, p): self.m.pool_free(p)
    def table(self, n): return self.m.table(self.s)[:n]


def random_ops(seed, pages, page_size, n_ops, scored=False):
    """Seeded mix of the calls Conscientia makes (ensure / ensure_range / set_seq_len) plus
    evictions, ensure_free and direct pool traffic.  Only valid pool frees are generated: the
    reference's free_block has no double-free check (block_pool.cpp:71-74)."""
    rng = np.random.default_rng(seed)
    ops, pos, held = [], 0, 0
    limit = 2 * pages * page_size
    for _ in range(n_ops):
        r = rng.random()
        if scored and rng.random() < 0.2:
            # new importance values for the first n logical blocks: coarse values make ties, which the
            # policy breaks by allocation order
            ops.append(["score", int(rng.integers(1, 2 * pages + 1)), int(rng.random() < 0.5), int(rng.integers(1 << 30))])
        if r < 0.35:
            ops.append(["ensure", int(pos)])
            pos = min(pos + int(rng.integers(1, 2 * page_size)), limit + page_size)
            ops.append(["set_len", int(min(pos, limit))])
        elif r < 0.55:
            m = int(rng.integers(1, 4 * page_size))
            ops.append(["ensure_range", int(pos), m])
            pos = min(pos + m, limit + page_size)
            ops.append(["set_len", int(min(pos, limit))])
        elif r < 0.65:
            ops.append(["ensure", int(rng.integers(0, limit + 3 * page_size))])   # random access, may exceed the table
        elif r < 0.75:
            ops.append(["evict", int(rng.integers(0, 4))])
        elif r < 0.82:
            ops.append(["ensure_free", int(rng.integers(0, pages + 2))])
        elif r < 0.91:
            ops.append(["pool_alloc"])
        else:
            ops.append(["pool_free_last"])
    return ops


def score_values(op):
    """The values of a ["score", n, coarse, seed] operation."""
    rng = np.random.default_rng(op[3])
    vals = rng.integers(0, 4, size=op[1]) * 0.25 if op[2] else rng.random(op[1])
    return vals.astype(np.float32)


def run_ops(cm, ops, pages):
    """Applies the operations; returns, per operation, [result, free count, used, logical blocks,
    crc32 of the int32 table], and the full table after the last one."""
    import zlib
    out, held = [], []
    width = 2 * pages
    for op in ops:
        k = op[0]
        if k == "ensure":
            r = cm.ensure(op[1])
        elif k == "ensure_range":
            r = cm.ensure_range(op[1], op[2])
        elif k == "set_len":
            cm.set_len(op[1]); r = 0
        elif k == "evict":
            r = cm.evict(op[1])
        elif k == "ensure_free":
            r = cm.ensure_free(op[1])
        elif k == "pool_alloc":
            r = cm.pool_alloc()
            if r >= 0:
                held.append(r)
        elif k == "score":
            cm.score_update(score_values(op)); r = op[1]
        elif k == "pool_free_last":
            r = -9
            if held:
                r = held.pop()
                cm.pool_free(r)
        tab = np.asarray(cm.table(width), dtype=np.int32)
        rec = [int(r), cm.free_blocks(), cm.used(), cm.num_logical(), zlib.crc32(tab.tobytes())]
        if k == "score":
            rec.append(zlib.crc32(np.asarray(cm.scores(), dtype=np.float32).tobytes()))
        out.append(rec)
    out.append([int(x) for x in cm.table(width)])
    return out
