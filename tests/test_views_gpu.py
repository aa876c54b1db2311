"""GPU: operands that are views at an element offset into a larger buffer.

vAi's Tensor is a shape plus an element offset into a dense buffer (vai/engine/tensor.h:228-242,
309-313), so a Linear may be handed I, W, bias, residual or O whose address is only aligned to
the element size.  The fast kernels need 16 bytes (vector loads, TMA); vaicu_linear_run then
takes the element-wise weight-streaming kernel or the FMA tile kernel for that call.  Each
case here runs the same Linear twice through the C ABI — every operand 256-byte aligned, then
one operand shifted by 2, 4 or 8 bytes — and checks

  * which kernel ran (vaicu_linear_plan_last_run): the plan's own the first time, the fallback
    the second time when the shifted operand is one the fast kernel cannot address;
  * both results against float64 over the stored values, at the bound of the kernel family;
  * the canary bytes on both sides of the output, the workspace and every input.

With compute-sanitizer unavailable these canaries are the out-of-bounds check of the suite.
"""
import ctypes

import numpy as np
import pytest
from gpu_util import DT, out_tol, seen
from linear_check import assert_close

from oracle import linear_oracle as orc
from vai_b200 import _lib
from vai_b200.engine import DeviceBuffer, Dtype, dtype_size, encode

pytestmark = pytest.mark.gpu

GUARD = 512
CANARY = 0xA5
GEMV, FMA, TC, SKINNY = 1, 2, 3, 4


class Guarded:
    """`nbytes` at base + GUARD + shift inside a buffer filled with the canary."""

    def __init__(self, device, nbytes, shift=0, host=None):
        self.device, self.nbytes, self.shift = device, nbytes, shift
        self.total = GUARD + shift + nbytes + GUARD
        self.buf = DeviceBuffer(device, self.total)
        image = np.full(self.total, CANARY, dtype=np.uint8)
        if host is not None:
            raw = np.ascontiguousarray(host).view(np.uint8).reshape(-1)
            image[GUARD + shift:GUARD + shift + raw.size] = raw
        self.image = image
        self.buf.upload(image)
        self.ptr = self.buf.ptr + GUARD + shift

    def read(self, np_dtype, shape):
        whole = self.buf.download(np.empty(self.total, dtype=np.uint8))
        lo, hi = whole[:GUARD + self.shift], whole[GUARD + self.shift + self.nbytes:]
        assert (lo == CANARY).all() and (hi == CANARY).all(), "bytes outside the operand were written"
        return whole[GUARD + self.shift:GUARD + self.shift + self.nbytes].view(np_dtype).reshape(shape).copy(), whole

    def untouched(self):
        whole = self.buf.download(np.empty(self.total, dtype=np.uint8))
        return bool((whole == self.image).all())


def _run(device, M, K, N, dts, kernel, shifts, *, epilogue="GELU_TANH", bias=True, residual=True, split_size=0, seed=0):
    """dts = (i, w, o) dtype names; shifts = dict operand -> byte shift.  Returns (got fp32, want f64, ran kernel, vectorized, plan kernel)."""
    lib = device.lib
    i_dt, w_dt, o_dt = (DT[d] for d in dts)
    rng = np.random.default_rng(seed + M * 7 + K + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    r = rng.standard_normal((M, N)).astype(np.float32)
    ops = {"I": Guarded(device, x.size * dtype_size(i_dt), shifts.get("I", 0), encode(x, i_dt)),
           "W": Guarded(device, w.size * dtype_size(w_dt), shifts.get("W", 0), encode(w, w_dt)),
           "bias": Guarded(device, b.size * dtype_size(w_dt), shifts.get("bias", 0), encode(b, w_dt)),
           "res": Guarded(device, r.size * dtype_size(o_dt), shifts.get("res", 0), encode(r, o_dt))}
    out = Guarded(device, M * N * dtype_size(o_dt), shifts.get("O", 0))
    d = _lib.LinearDesc()
    d.M, d.N, d.K = M, N, K
    d.i_dtype, d.w_dtype, d.o_dtype = int(i_dt), int(w_dt), int(o_dt)
    d.b_dtype = int(w_dt) if bias else int(Dtype.NONE)
    d.has_bias, d.bias_elems = (1, N) if bias else (0, 0)
    d.has_residual = 1 if residual else 0
    d.epilogue = orc.EPILOGUES[epilogue]
    d.scalar_scale = 0.5
    d.split_size = split_size
    plan = ctypes.c_void_p()
    if kernel:
        _lib.check(lib.vaicu_linear_plan_create_forced(device.handle, ctypes.byref(d), kernel, ctypes.byref(plan)), "plan")
    else:
        _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(plan)), "plan")
    info = _lib.LinearInfo()
    _lib.check(lib.vaicu_linear_plan_info(plan, ctypes.byref(info)), "info")
    ws = Guarded(device, max(int(info.workspace_bytes), 256))       # GUARD is a multiple of 256: stays 256-byte aligned
    _lib.check(lib.vaicu_linear_run(plan, None, ops["I"].ptr, ops["W"].ptr, ops["bias"].ptr if bias else None,
                                    ops["res"].ptr if residual else None, out.ptr, ws.ptr), "vaicu_linear_run")
    device.synchronize()
    device.check_status()
    ran, vec = ctypes.c_int(), ctypes.c_int()
    _lib.check(lib.vaicu_linear_plan_last_run(plan, ctypes.byref(ran), ctypes.byref(vec)), "last_run")
    raw, _ = out.read(np.float32 if o_dt == Dtype.F32 else np.uint16, (M, N))
    ws.read(np.uint8, (ws.nbytes,))                                   # canaries round the workspace
    for name, op in ops.items():
        assert op.untouched(), f"{name} was written"
    lib.vaicu_linear_plan_destroy(plan)
    got = raw if o_dt == Dtype.F32 else (raw.view(np.float16).astype(np.float32) if o_dt == Dtype.F16
                                         else (raw.astype(np.uint32) << 16).view(np.float32))
    xs = seen(x, i_dt)
    if ran.value in (TC, SKINNY) and i_dt == Dtype.F32:
        xs = seen(xs, w_dt)                 # the tensor-core kernels stage fp32 activations in the weights' type
    want = orc.linear_f64(xs, seen(w, w_dt), seen(b, w_dt) if bias else None, seen(r, o_dt) if residual else None,
                          epilogue=d.epilogue, scalar_scale=0.5)
    return got, want, ran.value, vec.value, info.kernel


# (name, M, K, N, (i, w, o) dtypes, forced kernel): one per kernel family and dtype mix
FAMILIES = [
    ("gemv f32.bf16", 1, 2048, 520, ("f32", "bf16", "f32"), GEMV),
    ("gemv bf16.bf16", 3, 1024, 264, ("bf16", "bf16", "bf16"), GEMV),
    ("gemv f32.f32", 4, 512, 96, ("f32", "f32", "f32"), GEMV),
    ("skinny bf16", 64, 512, 384, ("bf16", "bf16", "bf16"), SKINNY),
    ("skinny f32 in", 24, 256, 136, ("f32", "f16", "f32"), SKINNY),
    ("tc pair bf16", 300, 256, 264, ("bf16", "bf16", "f32"), TC),
    ("tc f32 in", 130, 320, 96, ("f32", "bf16", "bf16"), TC),
    ("fma f32", 40, 200, 72, ("f32", "f32", "f32"), FMA),
]
SHIFTED = ["I", "W", "O", "bias", "res"]


def _needs_fallback(operand, shift, dts, kernel):
    """Does this shifted operand keep the fast form of `kernel` from running?"""
    if shift % 16 == 0 or kernel == FMA:
        return False
    if kernel == GEMV:
        return operand in ("I", "W")                     # 16-byte vector loads of both
    if operand == "W":
        return True                                      # TMA
    if operand == "I":
        return dts[0] != "f32"                           # fp32 activations pass through the cast pass, which takes any alignment
    return False


@pytest.mark.parametrize("shift", [2, 4, 8])
@pytest.mark.parametrize("operand", SHIFTED)
@pytest.mark.parametrize("family", FAMILIES, ids=[f[0] for f in FAMILIES])
def test_shifted_views(family, operand, shift, device):
    name, M, K, N, dts, kernel = family
    esz = {"I": dtype_size(DT[dts[0]]), "W": dtype_size(DT[dts[1]]), "bias": dtype_size(DT[dts[1]]),
           "O": dtype_size(DT[dts[2]]), "res": dtype_size(DT[dts[2]])}[operand]
    if shift % esz:
        pytest.skip("a view starts at a whole element")
    base, want0, ran0, vec0, planned = _run(device, M, K, N, dts, kernel, {})
    assert planned == kernel and ran0 == kernel and (vec0 == 1 or kernel == FMA), "aligned operands take the plan's kernel"
    got, want, ran, vec, _ = _run(device, M, K, N, dts, kernel, {operand: shift})
    if _needs_fallback(operand, shift, dts, kernel):
        assert (ran, vec) == ((GEMV, 0) if kernel == GEMV else (FMA, 0)), f"{name}: shifted {operand} should take the fallback"
    else:
        assert (ran, vec) == (ran0, vec0), f"{name}: shifted {operand} needs no fallback"
    tol = out_tol(dts[2])
    assert_close(base, want0, tol, f"{name} aligned")
    assert_close(got, want, tol, f"{name} {operand}+{shift}")
    # the two runs read the same values: they may differ only by accumulation order / staging
    assert_close(got, base, (2e-2, 2e-2) if "f32" != dts[1] else (1e-4, 1e-5), f"{name} shifted vs aligned")


def test_odd_pointer_is_rejected(device):
    """An address that is not a whole element is an error status, not a launch."""
    lib = device.lib
    d = _lib.LinearDesc()
    d.M, d.N, d.K = 2, 64, 256
    d.i_dtype, d.w_dtype, d.o_dtype, d.b_dtype = 0, 3, 0, 2
    d.scalar_scale = 1.0
    plan = ctypes.c_void_p()
    _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(plan)), "plan")
    x, w, o = Guarded(device, 2 * 256 * 4), Guarded(device, 64 * 256 * 2), Guarded(device, 2 * 64 * 4)
    for args in ((x.ptr + 2, w.ptr, o.ptr), (x.ptr, w.ptr + 1, o.ptr), (x.ptr, w.ptr, o.ptr + 1)):
        assert lib.vaicu_linear_run(plan, None, args[0], args[1], None, None, args[2], None) == 6
    device.synchronize()
    assert o.untouched()
    lib.vaicu_linear_plan_destroy(plan)


def test_plan_keeps_descriptors_for_two_buffers_per_operand(device):
    """One tensor-core plan run over alternating activation buffers (what a caller with double-buffered
    activations does), then a third: every run reads the buffer it was given."""
    lib = device.lib
    rng = np.random.default_rng(3)
    M, K, N = 64, 512, 256
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    xs = [rng.standard_normal((M, K)).astype(np.float32) for _ in range(3)]
    wb = DeviceBuffer(device, N * K * 2)
    wb.upload(encode(w, Dtype.BF16))
    xbs = []
    for x in xs:
        b = DeviceBuffer(device, M * K * 2)
        b.upload(encode(x, Dtype.BF16))
        xbs.append(b)
    out = DeviceBuffer(device, M * N * 4)
    d = _lib.LinearDesc()
    d.M, d.N, d.K = M, N, K
    d.i_dtype = d.w_dtype = int(Dtype.BF16)
    d.o_dtype, d.b_dtype, d.scalar_scale = 0, 2, 1.0
    plan = ctypes.c_void_p()
    _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(plan)), "plan")
    info = _lib.LinearInfo()
    lib.vaicu_linear_plan_info(plan, ctypes.byref(info))
    ws = DeviceBuffer(device, max(int(info.workspace_bytes), 256))
    wants = [orc.linear_f64(seen(x, Dtype.BF16), seen(w, Dtype.BF16)) for x in xs]
    for which in (0, 1, 0, 1, 2, 0, 2, 1):
        _lib.check(lib.vaicu_linear_run(plan, None, xbs[which].ptr, wb.ptr, None, None, out.ptr, ws.ptr), "run")
        device.synchronize()
        got = out.download(np.empty((M, N), dtype=np.float32))
        assert_close(got, wants[which], (2e-4, 5e-5), f"buffer {which}")
    lib.vaicu_linear_plan_destroy(plan)
