"""GPU: vaicu_linear_splitk_static, the split-K Linear for callers that cannot
allocate device memory at call time (hosts that partition the whole device heap at
start-up, or that expose no allocator to plugins).  Its partial sums live in an 8 MiB
array built into the library instead of a caller-provided workspace.

Checked here through the C ABI against the existing entry point (vaicu_linear_run on
the FMA tile kernel with the same K split), on two calls in a row whose shapes differ,
so that the second call runs over what the first one left in the shared array, and
against the float64 oracle over the stored operand values, with fp32, fp16 and bf16
weights.  This file sorts last on purpose: a run that stops at the first failure has already executed
every other test.
"""
import ctypes

import numpy as np
import pytest
from linear_check import BOUND_FP32, assert_close

from oracle import linear_oracle as orc
from vai_b200 import _lib
from vai_b200.engine import DeviceBuffer, Dtype, bits_to_f32, encode

pytestmark = pytest.mark.gpu

KERNEL_FMA_TILE = 2
ERR_TOO_LARGE = 7


def _desc(M, N, K, split, epilogue, has_bias, has_res, order, w_dtype=0):
    d = _lib.LinearDesc()
    d.M, d.N, d.K = M, N, K
    d.i_dtype = d.o_dtype = 0
    d.w_dtype = w_dtype
    d.b_dtype = 0 if has_bias else 2
    d.has_bias, d.bias_elems = (1, N) if has_bias else (0, 0)
    d.has_residual, d.residual_elems = (1, 0) if has_res else (0, 0)
    d.residual_order = order
    d.epilogue = epilogue
    d.scalar_scale = 0.75
    d.split_size = split
    return d


def _both_ways(device, M, N, K, split, epilogue, has_bias, has_res, order, seed, w_dtype=0, with_oracle=False):
    lib = device.lib
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    r = rng.standard_normal((M, N)).astype(np.float32)
    w_dev = encode(w, Dtype(w_dtype))          # what the device holds: fp32, or 16-bit patterns
    w_seen = w if w_dtype == 0 else bits_to_f32(w_dev, Dtype(w_dtype)).reshape(N, K)
    bufs = {}
    for name, arr in (("x", x), ("w", w_dev), ("b", b), ("r", r)):
        bufs[name] = DeviceBuffer(device, arr.nbytes)
        bufs[name].upload(arr)
    out_ref = DeviceBuffer(device, M * N * 4)
    out_new = DeviceBuffer(device, M * N * 4)
    d = _desc(M, N, K, split, epilogue, has_bias, has_res, order, w_dtype)
    bias_p = bufs["b"].ptr if has_bias else None
    res_p = bufs["r"].ptr if has_res else None

    # existing entry point: a plan on the same kernel, workspace from the caller
    plan = ctypes.c_void_p()
    _lib.check(lib.vaicu_linear_plan_create_forced(device.handle, ctypes.byref(d), KERNEL_FMA_TILE, ctypes.byref(plan)), "plan")
    info = _lib.LinearInfo()
    _lib.check(lib.vaicu_linear_plan_info(plan, ctypes.byref(info)), "info")
    ws = DeviceBuffer(device, max(info.workspace_bytes, 256))
    _lib.check(lib.vaicu_linear_run(plan, None, bufs["x"].ptr, bufs["w"].ptr, bias_p, res_p, out_ref.ptr, ws.ptr), "run")

    # new entry point: same operands, no workspace argument at all
    _lib.check(lib.vaicu_linear_splitk_static(ctypes.byref(d), None, bufs["x"].ptr, bufs["w"].ptr, bias_p, res_p, out_new.ptr),
               "vaicu_linear_splitk_static")
    device.synchronize()
    ref = out_ref.download(np.empty((M, N), dtype=np.float32))
    new = out_new.download(np.empty((M, N), dtype=np.float32))
    lib.vaicu_linear_plan_destroy(plan)
    assert info.split_count >= 1
    if with_oracle:
        want = orc.linear_f64(x, w_seen, b if has_bias else None, r if has_res else None, epilogue=epilogue,
                              residual_order=order, scalar_scale=0.75)
        return new, ref, info.split_count, want
    return new, ref, info.split_count


def test_static_scratch_matches_workspace_path_twice(device):
    # first call: 6 K-spans of a 96 x 200 output, bias + GELU(tanh) + residual inside the epilogue
    new, ref, splits = _both_ways(device, 96, 200, 1536, 256, 3, True, True, 1, seed=1)
    assert splits == 6
    assert_close(new, ref, BOUND_FP32, "first call")
    # second call, straight after: a smaller problem with other options; the array still
    # holds the first call's partial sums where this one does not overwrite them
    new2, ref2, splits2 = _both_ways(device, 33, 48, 1000, 100, 1, False, True, 0, seed=2)
    assert splits2 == 10
    assert_close(new2, ref2, BOUND_FP32, "second call")
    assert np.isfinite(new).all() and np.isfinite(new2).all()


def test_static_scratch_default_split_and_size_limit(device):
    lib = device.lib
    # split chosen by the library (split_size 0)
    new, ref, _ = _both_ways(device, 16, 64, 4096, 0, 0, True, False, 0, seed=3)
    assert_close(new, ref, BOUND_FP32, "default split")
    # 4 spans x 1024 x 1024 fp32 = 16 MiB of partial sums: more than the built-in 8 MiB
    d = _desc(1024, 1024, 1024, 256, 0, False, False, 0)
    dummy = DeviceBuffer(device, 1024 * 1024 * 4)
    rc = lib.vaicu_linear_splitk_static(ctypes.byref(d), None, dummy.ptr, dummy.ptr, None, None, dummy.ptr)
    assert rc == ERR_TOO_LARGE
    assert b"8 MiB" in lib.vaicu_last_cuda_error()
    # gate fusion is not offered by this entry point
    g = _desc(16, 64, 256, 0, 4, False, False, 0)
    g.gate_fuse = 1
    assert lib.vaicu_linear_splitk_static(ctypes.byref(g), None, dummy.ptr, dummy.ptr, None, None, dummy.ptr) == 2


@pytest.mark.parametrize("w_dtype", [0, 1, 3], ids=["f32", "f16", "bf16"])
def test_static_scratch_against_the_float64_oracle(w_dtype, device):
    """Not only equal to the other entry point: right.  fp32 activations against fp32,
    fp16 and bf16 weights (the kernel widens 16-bit weights and accumulates in fp32), bias +
    SiLU + residual, 5 K spans; float64 over the values the device holds."""
    new, ref, splits, want = _both_ways(device, 40, 72, 1280, 256, 4, True, True, 0, seed=11 + w_dtype, w_dtype=w_dtype,
                                        with_oracle=True)
    assert splits == 5
    assert_close(new, want, BOUND_FP32, "static entry vs float64")
    assert_close(new, ref, BOUND_FP32, "static entry vs vaicu_linear_run")


def test_static_scratch_misaligned_pointer_is_a_status(device):
    """An operand that is not aligned to its element size comes back as VAICU_ERR_ALIGNMENT
    (6) with nothing launched: the output buffer keeps its canary."""
    lib = device.lib
    d = _desc(8, 16, 64, 0, 0, False, False, 0)
    x = DeviceBuffer(device, 8 * 64 * 4 + 16)
    w = DeviceBuffer(device, 16 * 64 * 4 + 16)
    o = DeviceBuffer(device, 8 * 16 * 4 + 16)
    canary = np.full(8 * 16 + 4, 7.0, dtype=np.float32)
    o.upload(canary)
    for args in ((x.ptr + 2, w.ptr, o.ptr), (x.ptr, w.ptr + 1, o.ptr), (x.ptr, w.ptr, o.ptr + 2)):
        assert lib.vaicu_linear_splitk_static(ctypes.byref(d), None, args[0], args[1], None, None, args[2]) == 6
    device.synchronize()
    np.testing.assert_array_equal(o.download(np.empty_like(canary)), canary)
