"""The C++ host-side mirror (include/qb200.hpp): compiles everywhere, and on a GPU its parity
program (tests/cpp/test_mirror.cpp — the reference's own test literals, through the C ABI) passes."""
import os
import subprocess

import pytest

from quanta_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "build", "test_mirror")


def _compile():
    _lib.load()
    os.makedirs(os.path.dirname(BIN), exist_ok=True)
    libdir = os.path.dirname(_lib.lib_path())
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++17", "-O1", "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(cuda, "include"),
           os.path.join(ROOT, "tests", "cpp", "test_mirror.cpp"), "-o", BIN, "-L" + libdir, "-lqb200",
           "-L" + os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath," + libdir]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return BIN


def test_cpp_mirror_compiles_and_links():
    assert os.path.exists(_compile())


@pytest.mark.gpu
def test_cpp_mirror_parity_program():
    r = subprocess.run([_compile()], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all C++ mirror tests passed" in r.stdout
