"""The C++ mirrors of vai::node::Linear and vai::NeuralNet (vai_b200/host/) compiled
against the C ABI: host logic on CPU, and the nodes end to end on the GPU."""
import os
import subprocess

import pytest

from vai_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "tests", "cpp")


def _build(name):
    _lib.load()
    lib_dir = os.path.dirname(_lib.LIB_PATH)
    src = os.path.join(CPP, name + ".cpp")
    exe = os.path.join(CPP, name)
    headers = [os.path.join(ROOT, "vai_b200", "host", h) for h in ("linear.h", "net.h", "norm.h", "gated_mul.h", "safetensors.h")]
    newest = max(os.path.getmtime(f) for f in [src, _lib.LIB_PATH] + headers)
    if not os.path.exists(exe) or os.path.getmtime(exe) < newest:
        subprocess.run(["g++", "-std=c++20", "-O1", "-Wall", "-o", exe, src, "-L", lib_dir, "-lvaicu",
                        f"-Wl,-rpath,{lib_dir}"], check=True)
    return exe


@pytest.mark.parametrize("name", ["host_linear_test", "host_net_test"])
def test_cpp_host_logic(name):
    r = subprocess.run([_build(name)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["host_linear_test", "host_net_test"])
def test_cpp_on_gpu(name):
    r = subprocess.run([_build(name), "--gpu"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
