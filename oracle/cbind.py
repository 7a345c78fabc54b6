"""ctypes binding of liboracle.so (oracle/paged_kv_oracle.c) over numpy arrays.

Test infrastructure only.  uint16 arrays carry fp16/bf16 bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")

F16, BF16 = 0, 1


class Geom(C.Structure):
    _fields_ = [("num_layers", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("page_size", C.c_int32), ("dtype", C.c_int32),
                ("rotary_dim", C.c_int32), ("rope_theta", C.c_float)]


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "paged_kv_oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-s", "-B", "liboracle.so"], check=True)
    return LIB


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.okv_pool_elem.restype = C.c_int64
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def geom(layers, hq, hkv, d, page, dtype, rot, theta) -> Geom:
    return Geom(layers, hq, hkv, d, page, dtype, rot, theta)


def to_float(bits: np.ndarray, dtype: int) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().okv_to_float(_p(bits), _p(out), C.c_int64(bits.size), dtype)
    return out


def from_float(x: np.ndarray, dtype: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().okv_from_float(_p(x), _p(out), C.c_int64(x.size), dtype)
    return out


def inv_freq(theta: float, rot: int) -> np.ndarray:
    out = np.empty(rot // 2, dtype=np.float32)
    lib().okv_inv_freq(C.c_float(theta), rot, _p(out))
    return out


def sincos(angles: np.ndarray):
    angles = np.ascontiguousarray(angles, dtype=np.float32)
    s = np.empty_like(angles)
    c = np.empty_like(angles)
    fs, fc = C.c_float(), C.c_float()
    f = lib().okv_sincos
    for i, a in enumerate(angles.ravel()):
        f(C.c_float(float(a)), C.byref(fs), C.byref(fc))
        s.ravel()[i] = fs.value
        c.ravel()[i] = fc.value
    return s, c


def pool_elem(g: Geom, max_pages, layer, page, kv, head, slot) -> int:
    return lib().okv_pool_elem(C.byref(g), max_pages, layer, page, kv, head, slot)


def pool_elems(g: Geom, max_pages: int) -> int:
    return g.num_layers * max_pages * 2 * g.num_kv_heads * g.page_size * g.head_dim


def append(g: Geom, pool, max_pages, table, layer, pos_start, m, k_src, v_src, rope=True):
    lib().okv_append(C.byref(g), _p(pool), max_pages, _p(_i32(table)), layer, pos_start, m, _p(k_src), _p(v_src),
                     1 if rope else 0)


def attend_decode(g: Geom, pool, max_pages, tables, rows, kv_len, layer, q, out, scale):
    tables = _i32(tables)
    rows, kv_len = _i32(rows), _i32(kv_len)
    lib().okv_attend_decode(C.byref(g), _p(pool), max_pages, _p(tables), tables.shape[-1], _p(rows), _p(kv_len),
                            len(rows), layer, _p(q), _p(out), C.c_float(scale))


def attend_decode_f64(g: Geom, pool, max_pages, tables, rows, kv_len, layer, q, scale) -> np.ndarray:
    tables = _i32(tables)
    rows, kv_len = _i32(rows), _i32(kv_len)
    out = np.zeros((len(rows), g.num_q_heads, g.head_dim), dtype=np.float32)
    lib().okv_attend_decode_f64(C.byref(g), _p(pool), max_pages, _p(tables), tables.shape[-1], _p(rows), _p(kv_len),
                                len(rows), layer, _p(q), _p(out), C.c_float(scale))
    return out


def page_mass(g: Geom, pool, max_pages, tables, rows, kv_len, layer, q, mass, scale):
    """Adds the layer's attention mass per (batch entry, logical page) to `mass` (float64 [n_seq][stride])."""
    tables = _i32(tables)
    rows, kv_len = _i32(rows), _i32(kv_len)
    assert mass.dtype == np.float64 and mass.flags.c_contiguous
    lib().okv_page_mass(C.byref(g), _p(pool), max_pages, _p(tables), tables.shape[-1], _p(rows), _p(kv_len), len(rows),
                        layer, _p(q), _p(mass), mass.shape[-1], C.c_float(scale))


def importance_update(scores: np.ndarray, fresh: np.ndarray, decay: float) -> None:
    assert scores.dtype == np.float32 and fresh.dtype == np.float32 and scores.flags.c_contiguous
    fresh = np.ascontiguousarray(fresh)
    lib().okv_importance_update(_p(scores), _p(fresh), scores.size, C.c_float(decay))


def attend_prefill(g: Geom, pool, max_pages, table, layer, pos_start, m, q, out, scale):
    lib().okv_attend_prefill(C.byref(g), _p(pool), max_pages, _p(_i32(table)), layer, pos_start, m, _p(q), _p(out),
                             C.c_float(scale))


def attend_partial(g: Geom, pool, max_pages, table, layer, kv_begin, kv_end, q, scale) -> np.ndarray:
    part = np.zeros(g.num_q_heads * (g.head_dim + 2), dtype=np.float32)
    lib().okv_attend_partial(C.byref(g), _p(pool), max_pages, _p(_i32(table)), layer, kv_begin, kv_end, _p(q),
                             _p(part), C.c_float(scale))
    return part


def combine(g: Geom, parts: np.ndarray, out: np.ndarray):
    parts = np.ascontiguousarray(parts, dtype=np.float32)
    lib().okv_combine(C.byref(g), parts.shape[0], _p(parts), _p(out))


def cow_copy(g: Geom, pool, max_pages, src_page, dst_page, n_slots):
    lib().okv_cow_copy(C.byref(g), _p(pool), max_pages, src_page, dst_page, n_slots)


def extract(g: Geom, pool, max_pages, table, start_token, num_tokens) -> np.ndarray:
    dst = np.empty((g.num_layers, 2, num_tokens, g.num_kv_heads, g.head_dim), dtype=np.uint16)
    lib().okv_extract(C.byref(g), _p(dst), _p(pool), max_pages, _p(_i32(table)), start_token, num_tokens)
    return dst


def inject(g: Geom, pool, src, max_pages, table, start_token, num_tokens):
    src = np.ascontiguousarray(src, dtype=np.uint16)
    lib().okv_inject(C.byref(g), _p(pool), _p(src), max_pages, _p(_i32(table)), start_token, num_tokens)


def num_threads() -> int:
    return lib().okv_num_threads()


def use_all_cores() -> int:
    """Sets the OpenMP team to the cores this process may run on (whatever OMP_NUM_THREADS said); returns it."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().okv_set_num_threads(n)
    return num_threads()
