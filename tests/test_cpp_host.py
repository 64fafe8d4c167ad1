"""The header-only C++ mirror of the Backend seam compiles against the C ABI
(CPU check) and passes ferro's known answers on a GPU (gpu check)."""
import os
import shutil
import subprocess

import pytest

from ferro_b200 import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "host_backend_test.cpp")
BIN = os.path.join(ROOT, "ferro_b200", "lib", "host_backend_test")


def compile_test():
    build.build()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    lib_dir = os.path.join(ROOT, "ferro_b200", "lib")
    subprocess.run([nvcc, "-std=c++17", "-O1", "-x", "cu", "-gencode", "arch=compute_100a,code=sm_100a", SRC, "-o", BIN,
                    "-L", lib_dir, "-lferro_b200", "-cudart", "shared", "-Xlinker", f"-rpath={lib_dir}"], check=True)
    return BIN


def test_cpp_host_mirror_compiles_and_links():
    assert os.path.exists(compile_test())


@pytest.mark.gpu
def test_cpp_host_mirror_known_answers():
    exe = compile_test()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "host_backend_test ok" in r.stdout
