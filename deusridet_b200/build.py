"""Builds libdrkv.so (the CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

Run as ``python -m deusridet_b200.build``.  The library lands next to this file so that it
travels with the source tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libdrkv.so")

CUDA_SOURCES = ["engine.cu", "append.cu", "attend_decode.cu", "stateless.cu", "decode_noalloc.cu", "attend_prefill.cu", "gather_scatter.cu"]
CXX_SOURCES = ["page_book.cpp", "page_store.cpp", "sharding.cpp"]
HEADERS = ["kernels.hpp", "kv_common.cuh", "page_book.hpp", "page_store.hpp", "exchange.cuh", "stateless.hpp", "sm100_primitives.cuh", os.path.join("..", "..", "include", "drkv.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "--expt-relaxed-constexpr",
]


def _extra_flags():
    """Extra nvcc flags for experiments (e.g. -DDRKV_PREFETCH_GROUPS=6), from DRKV_NVCC_EXTRA."""
    return os.environ.get("DRKV_NVCC_EXTRA", "").split()


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built")
    return nvcc


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in CUDA_SOURCES + CXX_SOURCES + HEADERS]
    return any(os.path.getmtime(os.path.normpath(d)) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every source into libdrkv.so; returns the library path."""
    if not force and not _stale():
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in CUDA_SOURCES + CXX_SOURCES:
        obj = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *_extra_flags(), "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src} ---\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see the output above")
    cmd = [nvcc, "-shared", "-o", LIB + ".tmp", *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.run(cmd, check=True)
    os.replace(LIB + ".tmp", LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
