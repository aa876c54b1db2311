"""CPU: the C-ABI library loads without a GPU, exports exactly what include/vaicu.h
declares, and fails cleanly (no fallback) when there is no device."""
import ctypes
import os
import re
import subprocess

import pytest

from vai_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "vaicu.h")


def declared_functions():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"VAICU_API\s+[\w\s\*]+?\b(vaicu_\w+)\s*\(", text)))


def test_header_declares_functions():
    names = declared_functions()
    assert "vaicu_linear_run" in names and "vaicu_linear_plan_create" in names and len(names) >= 30


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in vaicu.h but not exported"
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = sorted(set(re.findall(r"\b(vaicu_\w+)\b", out)))
    assert exported == declared_functions(), "exported symbols and header declarations differ"


def test_ctypes_table_covers_header():
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_header_compiles_as_c():
    src = '#include "vaicu.h"\nint main(void){ vaicu_linear_desc d; (void)d; return VAICU_OK; }\n'
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-x", "c", "-", "-fsyntax-only"],
                       input=src, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_status_strings_and_version():
    lib = _lib.load()
    assert lib.vaicu_version() >= 1000
    assert lib.vaicu_status_string(0) == b"ok"
    for code in range(1, 9):
        assert lib.vaicu_status_string(code) not in (b"ok", b"unknown status")


def _has_gpu():
    lib = _lib.load()
    h = ctypes.c_void_p()
    rc = lib.vaicu_device_open(0, ctypes.byref(h))
    if rc == 0:
        lib.vaicu_device_close(h)
    return rc == 0


def test_no_device_means_error_not_fallback():
    """Without an sm_100 device the product path refuses to run: opening the device
    reports VAICU_ERR_NO_DEVICE and the host API raises."""
    if _has_gpu():
        pytest.skip("a GPU is present")
    lib = _lib.load()
    h = ctypes.c_void_p()
    assert lib.vaicu_device_open(0, ctypes.byref(h)) in (3, 4)
    import vai_b200
    with pytest.raises(_lib.VaicuError):
        vai_b200.Device(0)


def test_null_arguments_are_rejected():
    lib = _lib.load()
    assert lib.vaicu_device_open(0, None) == 1
    assert lib.vaicu_linear_plan_create(None, None, None) == 1
    assert lib.vaicu_linear_run(None, None, None, None, None, None, None, None) == 1
    assert lib.vaicu_buffer_free(None) == 1


def test_shard_desc_splits_rows_evenly():
    """Column split of the math = contiguous row slabs of W; gate|value splits per half."""
    lib = _lib.load()
    full = _lib.LinearDesc()
    full.M, full.N, full.K = 64, 262144, 2560
    full.i_dtype = full.w_dtype = full.o_dtype = 3
    full.b_dtype = 2
    full.scalar_scale = 1.0
    covered = 0
    for world in (1, 2, 4, 8):
        covered = 0
        for rank in range(world):
            shard = _lib.LinearDesc()
            b, c = ctypes.c_uint32(), ctypes.c_uint32()
            assert lib.vaicu_linear_shard_desc(ctypes.byref(full), rank, world, ctypes.byref(shard), ctypes.byref(b), ctypes.byref(c)) == 0
            assert b.value == covered and shard.N == c.value == full.N // world and shard.K == full.K and shard.M == full.M
            covered += c.value
        assert covered == full.N
    gate = _lib.LinearDesc.from_buffer_copy(bytes(full))
    gate.N, gate.gate_fuse, gate.epilogue = 2 * 10240, 1, 3
    shard = _lib.LinearDesc()
    b, c = ctypes.c_uint32(), ctypes.c_uint32()
    assert lib.vaicu_linear_shard_desc(ctypes.byref(gate), 3, 8, ctypes.byref(shard), ctypes.byref(b), ctypes.byref(c)) == 0
    assert (b.value, c.value, shard.N, shard.gate_fuse) == (3 * 1280, 1280, 2560, 1)
    # uneven split: the first ranks take one extra row
    odd = _lib.LinearDesc.from_buffer_copy(bytes(full))
    odd.N = 50257
    sizes = []
    for rank in range(8):
        assert lib.vaicu_linear_shard_desc(ctypes.byref(odd), rank, 8, ctypes.byref(shard), ctypes.byref(b), ctypes.byref(c)) == 0
        sizes.append(c.value)
    assert sum(sizes) == 50257 and max(sizes) - min(sizes) == 1
    assert lib.vaicu_linear_shard_desc(ctypes.byref(full), 8, 8, ctypes.byref(shard), ctypes.byref(b), ctypes.byref(c)) == 1


def test_static_split_k_rejects_misaligned_operands_before_any_launch():
    """vaicu_linear_splitk_static applies vaicu_linear_run's rule (every operand aligned to
    its element size) before it touches the GPU: an odd pointer is a status code, never a
    kernel argument.  The pointers here are made-up addresses; the call returns before
    anything could read them, which is why this runs without a GPU."""
    lib = _lib.load()
    d = _lib.LinearDesc()
    d.M, d.N, d.K = 4, 8, 64
    d.i_dtype = d.w_dtype = d.o_dtype = 0
    d.b_dtype = 0
    d.has_bias, d.bias_elems = 1, 8
    d.has_residual = 1
    d.scalar_scale = 1.0
    good = 0x10000
    args = dict(I=good, W=good, bias=good, residual=good, O=good)
    for name in args:
        for off in (1, 2, 3):
            a = dict(args)
            a[name] = good + off
            rc = lib.vaicu_linear_splitk_static(ctypes.byref(d), None, a["I"], a["W"], a["bias"], a["residual"], a["O"])
            assert rc == 6, (name, off, rc)
    # 16-bit operands need 2-byte alignment only
    d.w_dtype, d.b_dtype = 3, 1
    assert lib.vaicu_linear_splitk_static(ctypes.byref(d), None, good, good + 1, good, good, good) == 6
    assert lib.vaicu_linear_splitk_static(ctypes.byref(d), None, good, good, good + 1, good, good) == 6
    # an absent operand is not checked
    d.has_bias = d.has_residual = 0
    d.b_dtype = 2
    assert lib.vaicu_linear_splitk_static(ctypes.byref(d), None, good + 2, good, None, None, good) == 6
