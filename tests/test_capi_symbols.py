"""The C ABI: every function include/drkv.h declares is exported by libdrkv.so and typed in the
Python binding, nothing C++ leaks through the export table, and a bookkeeping-only engine
refuses compute calls (there is no CPU fallback)."""
import ctypes as C
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    with open(os.path.join(ROOT, "include", "drkv.h")) as f:
        src = f.read()
    return sorted(set(re.findall(r"DRKV_API\s+[\w\s\*]+?\b(drkv_\w+)\s*\(", src)))


def test_every_declared_symbol_is_exported_and_bound(drkv_lib):
    from deusridet_b200 import capi
    names = _declared()
    assert len(names) >= 45
    for n in names:
        assert hasattr(drkv_lib, n), f"{n} is declared in include/drkv.h but not exported"
        assert n in capi.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(capi.SIGNATURES) == names


def test_export_table_is_plain_c(drkv_lib):
    from deusridet_b200 import capi
    out = subprocess.run(["nm", "-D", "--defined-only", capi.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = [ln.split()[-1] for ln in out.splitlines() if " T " in ln]
    ours = [s for s in exported if not s.startswith("_")]
    assert sorted(ours) == _declared()
    assert not [s for s in exported if s.startswith("_Z")], "C++ symbols leak through the export table"


def test_shim_header_compiles_standalone():
    src = '#include "deusridet_shim.hpp"\nint main() { deusridet::CacheManager cm; return cm.free_blocks(); }\n'
    subprocess.run(["g++", "-std=c++17", "-fsyntax-only", f"-I{ROOT}/include", "-I/usr/local/cuda/include", "-x", "c++",
                    "-"], input=src, text=True, check=True)


def test_compute_calls_need_a_device(drkv_lib):
    from deusridet_b200 import capi
    g = capi.Geometry(1, 8, 2, 128, 16, capi.BF16, 128, 1e4)
    cfg = capi.Config(0, 8, 1, 0, -1, 0)
    h = C.c_void_p()
    assert drkv_lib.drkv_create(C.byref(g), C.byref(cfg), C.byref(h)) == 0
    assert drkv_lib.drkv_pool_ptr(h) is None
    assert drkv_lib.drkv_append_rope(h, 0, 1, 8, 8, 8, 8, None) == capi.ERR_NO_DEVICE
    assert drkv_lib.drkv_attend_decode(h, 0, 1, 8, 8, 4, 8, 8, 1.0, None) == capi.ERR_NO_DEVICE
    assert drkv_lib.drkv_attend_partial(h, 0, 0, 0, 4, 8, 8, 1.0, None) == capi.ERR_NO_DEVICE
    assert drkv_lib.drkv_sync_tables(h, None) == capi.ERR_NO_DEVICE
    assert b"device" in drkv_lib.drkv_last_error()
    drkv_lib.drkv_destroy(h)
    bad = capi.Geometry(1, 8, 3, 128, 16, capi.BF16, 128, 1e4)   # 8 query heads over 3 KV heads
    assert drkv_lib.drkv_create(C.byref(bad), C.byref(cfg), C.byref(h)) == capi.ERR_INVALID
