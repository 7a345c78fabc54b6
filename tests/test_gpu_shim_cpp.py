"""The C++ shim's free functions on a GPU, from a C++ program: tests/cpp/shim_paged_gpu.cpp is compiled against
include/deusridet_shim.hpp, linked with libdrkv.so and the CUDA runtime, and replays a case recorded from the
reference's own kernels (tests/golden/paged_attention_reference.npz): paged_kv_cache_write_batch ->
paged_kv_cache_write -> paged_gqa_decode_attention (src/machina/paged_attention.h:27-71)."""
import os
import subprocess

import numpy as np
import pytest

from tests.golden import paged_cases

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = np.load(os.path.join(ROOT, "tests", "golden", "paged_attention_reference.npz"))


@pytest.fixture(scope="module")
def shim_program(drkv_lib, tmp_path_factory):
    out = str(tmp_path_factory.mktemp("shim") / "shim_paged_gpu")
    lib_dir = os.path.join(ROOT, "deusridet_b200")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.run(["g++", "-std=c++17", "-O1", f"-I{ROOT}/include", f"-I{cuda}/include",
                    os.path.join(ROOT, "tests", "cpp", "shim_paged_gpu.cpp"), "-o", out,
                    f"-L{lib_dir}", "-l:libdrkv.so", f"-L{cuda}/lib64", "-lcudart",
                    f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{cuda}/lib64"], check=True)
    return out


@pytest.mark.parametrize("name", ["model", "toy", "small_page"])
def test_shim_free_functions_from_cpp(shim_program, tmp_path, name):
    c = paged_cases.build(name)
    ref_pool = c["pool"].copy()
    ref_pool[GOLD[name + "_pool_changed_idx"]] = GOLD[name + "_pool_changed_val"]
    files = {"pool": c["pool"], "table": c["table"], "kb": c["kb"], "vb": c["vb"], "k1": GOLD[name + "_k_roped"],
             "v1": c["v1"], "q": GOLD[name + "_q_roped"], "want_pool": ref_pool, "want_out": GOLD[name + "_out"]}
    for k, v in files.items():
        np.ascontiguousarray(v).tofile(str(tmp_path / f"{k}.bin"))
    with open(tmp_path / "meta.txt", "w") as f:
        f.write(" ".join(str(x) for x in (c["hq"], c["hkv"], c["d"], c["rot"], c["theta"], c["page"], c["layers"],
                                          c["layer"], c["seq_len"], c["m_batch"], c["max_pages"])) + "\n")
    res = subprocess.run([shim_program, str(tmp_path)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "SHIM_GPU OK" in res.stdout, res.stdout + res.stderr
