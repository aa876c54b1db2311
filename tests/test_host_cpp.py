"""The C++ mirror of vai::node::Linear (vai_b200/host/linear.h) compiled against the
C ABI: host logic on CPU, and the node end to end on the GPU."""
import os
import subprocess

import pytest

from vai_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "host_linear_test")


def _build():
    _lib.load()
    lib_dir = os.path.dirname(_lib.LIB_PATH)
    src = os.path.join(ROOT, "tests", "cpp", "host_linear_test.cpp")
    if not os.path.exists(EXE) or os.path.getmtime(EXE) < max(os.path.getmtime(src), os.path.getmtime(_lib.LIB_PATH)):
        subprocess.run(["g++", "-std=c++20", "-O1", "-Wall", "-o", EXE, src, "-L", lib_dir, "-lvaicu",
                        f"-Wl,-rpath,{lib_dir}"], check=True)
    return EXE


def test_cpp_host_logic():
    r = subprocess.run([_build()], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


@pytest.mark.gpu
def test_cpp_node_on_gpu():
    r = subprocess.run([_build(), "--gpu"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
