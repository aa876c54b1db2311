"""GPU: vaicu_linear_splitk_static, the split-K Linear for callers that cannot
allocate device memory at call time (hosts that partition the whole device heap at
start-up, or that expose no allocator to plugins).  Its partial sums live in an 8 MiB
array built into the library instead of a caller-provided workspace.

Checked here through the C ABI against the existing entry point (vaicu_linear_run on
the FMA tile kernel with the same K split), on two calls in a row whose shapes differ,
so that the second call runs over what the first one left in the shared array.  This
file sorts last on purpose: a run that stops at the first failure has already executed
every other test.
"""
import ctypes

import numpy as np
import pytest
from linear_check import BOUND_FP32, assert_close

from vai_b200 import _lib
from vai_b200.engine import DeviceBuffer

pytestmark = pytest.mark.gpu

KERNEL_FMA_TILE = 2
ERR_TOO_LARGE = 7


def _desc(M, N, K, split, epilogue, has_bias, has_res, order):
    d = _lib.LinearDesc()
    d.M, d.N, d.K = M, N, K
    d.i_dtype = d.w_dtype = d.o_dtype = 0
    d.b_dtype = 0 if has_bias else 2
    d.has_bias, d.bias_elems = (1, N) if has_bias else (0, 0)
    d.has_residual, d.residual_elems = (1, 0) if has_res else (0, 0)
    d.residual_order = order
    d.epilogue = epilogue
    d.scalar_scale = 0.75
    d.split_size = split
    return d


def _both_ways(device, M, N, K, split, epilogue, has_bias, has_res, order, seed):
    lib = device.lib
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    r = rng.standard_normal((M, N)).astype(np.float32)
    bufs = {}
    for name, arr in (("x", x), ("w", w), ("b", b), ("r", r)):
        bufs[name] = DeviceBuffer(device, arr.nbytes)
        bufs[name].upload(arr)
    out_ref = DeviceBuffer(device, M * N * 4)
    out_new = DeviceBuffer(device, M * N * 4)
    d = _desc(M, N, K, split, epilogue, has_bias, has_res, order)
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
