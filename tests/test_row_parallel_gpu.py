"""GPU (one device): the pieces of the row-parallel Linear that exchanges its partial sums through
this package's own kernels — the GEMM epilogue that scatters rows to their owners' staging buffers
(vaicu_linear_run_reduce_scatter), the fold that adds the ranks' slabs (vaicu_partial_fold_run) and
the barrier kernel (vaicu_peer_barrier_run).  The ranks are played one after the other on one GPU
with their own K slices and staging buffers in local memory, so that every index of the scheme is
exercised without a second GPU; the two-GPU run of the same code is tests/test_fused_gather_gpu.py."""
import ctypes

import numpy as np
import pytest
from gpu_util import seen
from linear_check import assert_close

from oracle import linear_oracle as orc
from vai_b200 import Dtype, _lib
from vai_b200.engine import DeviceBuffer, bits_to_f32, encode

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,N,world,part", [(512, 1024, 264, 2, Dtype.F32), (1024, 512, 520, 4, Dtype.BF16),
                                              (64, 2048, 136, 2, Dtype.F32), (96, 768, 64, 4, Dtype.BF16),
                                              (256, 512, 100, 2, Dtype.F32)])       # N % 8 != 0: the element-wise fold
def test_reduce_scatter_epilogue_then_fold(M, K, N, world, part, device):
    lib = device.lib
    rng = np.random.default_rng(M + K + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    rows = M // world
    psz = 4 if part == Dtype.F32 else 2
    canary = 0x7FC1 if part != Dtype.F32 else None
    # staging of "GPU" d: [world][rows][N]; all in this GPU's memory here
    staging = [DeviceBuffer(device, world * rows * N * psz) for _ in range(world)]
    for b in staging:
        _lib.check(lib.vaicu_memset(b.ptr, 0xFF, b.nbytes, None), "memset")
    ptrs = (ctypes.c_void_p * world)(*[b.ptr for b in staging])
    kper = K // world
    keep = []
    for r in range(world):                      # rank r: its K slice, its slab in every owner's staging
        xs = np.ascontiguousarray(x[:, r * kper:(r + 1) * kper])
        ws = np.ascontiguousarray(w[:, r * kper:(r + 1) * kper])
        xb, wb = DeviceBuffer(device, xs.size * 2), DeviceBuffer(device, ws.size * 2)
        xb.upload(encode(xs, Dtype.BF16))
        wb.upload(encode(ws, Dtype.BF16))
        d = _lib.LinearDesc()
        d.M, d.N, d.K = M, N, kper
        d.i_dtype = d.w_dtype = int(Dtype.BF16)
        d.o_dtype = int(part)
        d.b_dtype, d.scalar_scale = 2, 1.0
        d.split_size = max(32, kper)
        plan = ctypes.c_void_p()
        _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(plan)), "plan")
        info = _lib.LinearInfo()
        lib.vaicu_linear_plan_info(plan, ctypes.byref(info))
        wsb = DeviceBuffer(device, max(info.workspace_bytes, 256))
        _lib.check(lib.vaicu_linear_run_reduce_scatter(plan, None, xb.ptr, wb.ptr, ptrs, world, r, wsb.ptr), "reduce_scatter")
        keep += [xb, wb, wsb]
        device.synchronize()
        lib.vaicu_linear_plan_destroy(plan)
    # every slab of every owner now holds that rank's partial rows: check one against float64
    raw = staging[1].download(np.empty((world, rows, N), dtype=np.float32 if part == Dtype.F32 else np.uint16))
    slab = raw[0] if part == Dtype.F32 else bits_to_f32(raw[0], Dtype.BF16).reshape(rows, N)
    want_slab = orc.linear_f64(seen(x[rows:2 * rows, :kper], Dtype.BF16), seen(w[:, :kper], Dtype.BF16))
    assert_close(slab, want_slab, (1e-4, 2e-5) if part == Dtype.F32 else (8e-3, 1e-3), "rank 0's slab in owner 1's staging")
    # the fold on each owner, written into two full outputs (its own and a peer's)
    outs = [DeviceBuffer(device, M * N * 2) for _ in range(2)]
    rb = DeviceBuffer(device, M * N * 2)
    rb.upload(encode(res, Dtype.BF16))
    optrs = (ctypes.c_void_p * 2)(outs[0].ptr, outs[1].ptr)
    for owner in range(world):
        _lib.check(lib.vaicu_partial_fold_run(device.handle, None, staging[owner].ptr, world, rows, N, int(part), rb.ptr, 0.5,
                                              int(Dtype.BF16), optrs, 2, owner * rows), "fold")
    device.synchronize()
    device.check_status()
    want = 0.5 * orc.linear_f64(seen(x, Dtype.BF16), seen(w, Dtype.BF16)) + seen(res, Dtype.BF16)
    got = [bits_to_f32(o.download(np.empty((M, N), dtype=np.uint16)), Dtype.BF16).reshape(M, N) for o in outs]
    np.testing.assert_array_equal(got[0], got[1])
    # bf16 output; with bf16 partial sums each of the `world` slabs adds a rounding of up to 2^-9 of its magnitude
    assert_close(got[0], want, (1.2e-2, 2e-3) if part == Dtype.F32 else (2e-2, 8e-3), "folded output")


def test_reduce_scatter_needs_a_plain_plan(device):
    lib = device.lib
    d = _lib.LinearDesc()
    d.M, d.N, d.K = 256, 128, 256
    d.i_dtype = d.w_dtype = d.o_dtype = 3
    d.b_dtype, d.scalar_scale, d.epilogue = 2, 1.0, 4
    plan = ctypes.c_void_p()
    _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(plan)), "plan")
    buf = DeviceBuffer(device, 256 * 256 * 4)
    ptrs = (ctypes.c_void_p * 2)(buf.ptr, buf.ptr)
    assert lib.vaicu_linear_run_reduce_scatter(plan, None, buf.ptr, buf.ptr, ptrs, 2, 0, buf.ptr) == 2     # an epilogue belongs to the fold
    assert lib.vaicu_linear_run_reduce_scatter(plan, None, buf.ptr, buf.ptr, ptrs, 2, 2, buf.ptr) == 1     # slot out of range
    lib.vaicu_linear_plan_destroy(plan)


def test_peer_barrier_alone_on_one_gpu(device):
    """world = 1: the kernel signals and finds itself; twice, so the epoch moves; no time-out."""
    lib = device.lib
    flags, epoch = DeviceBuffer(device, 256), DeviceBuffer(device, 256)
    for b in (flags, epoch):
        _lib.check(lib.vaicu_memset(b.ptr, 0, 256, None), "memset")
    ptrs = (ctypes.c_void_p * 1)(flags.ptr)
    for _ in range(2):
        _lib.check(lib.vaicu_peer_barrier_run(device.handle, None, ptrs, 1, 0, epoch.ptr), "barrier")
    device.synchronize()
    device.check_status()
    assert int(epoch.download(np.empty(1, dtype=np.uint32))[0]) == 2
    assert int(flags.download(np.empty(1, dtype=np.uint32))[0]) == 2
    # a barrier whose peer never arrives gives up after its bounded wait and reports through the status word
    lonely = DeviceBuffer(device, 256)
    _lib.check(lib.vaicu_memset(lonely.ptr, 0, 256, None), "memset")
    two = (ctypes.c_void_p * 2)(flags.ptr, lonely.ptr)        # "rank 1" is a buffer nobody writes
    _lib.check(lib.vaicu_peer_barrier_run(device.handle, None, two, 2, 0, epoch.ptr), "barrier")
    word = ctypes.c_int()
    assert lib.vaicu_device_status(device.handle, ctypes.byref(word)) == 8 and word.value != 0
    assert lib.vaicu_device_status(device.handle, ctypes.byref(word)) == 0


def test_block_chain_replayed_as_one_graph_matches_float64(device):
    """The one-GPU form of the chain that the multi-GPU report times (TensorParallelBlocks, tp off): two
    Gemma-3-4B-shaped blocks at batch 64 captured into one CUDA graph; the replayed output against float64
    over the stored bf16 weights, with the intermediates rounded to bf16 where the chain stores them."""
    torch = pytest.importorskip("torch")
    from vai_b200.sharded import TensorParallelBlocks
    M = 64
    chain = TensorParallelBlocks(device, None, "gemma-3-4b", M, 2, 2, False)
    assert chain.group is not None                     # q / k / v run as one group at this batch
    cuda = torch.device("cuda", device.ordinal)
    x0 = torch.randn(M, 2560, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    xd = x0.to(cuda)
    out = chain.capture(xd)
    for _ in range(3):
        chain.graph.replay()
    torch.cuda.synchronize()
    device.check_status()
    got = out.float().cpu().numpy()

    def r16(t):
        return t.to(torch.bfloat16).double()

    x = x0.double()
    for w in chain.weights:
        wq, wo, wg, wd = (w[k].cpu().double() for k in ("q", "o", "g", "d"))
        q = r16(x @ wq.T)
        h = r16(0.5 * (q @ wo.T) + x0.double())
        acc = h @ wg.T
        H = acc.shape[1] // 2
        g, u = acc[:, :H], acc[:, H:]
        act = 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
        hid = r16(act * u)
        x = r16(0.25 * (hid @ wd.T) + x0.double())
    want = x.numpy()
    # activations are unit-scale by construction (residual = the unit-variance input), and an output is a
    # sum that may cancel: the bound is relative to max(|want|, 1)
    err = np.abs(got - want) / np.maximum(np.abs(want), 1.0)
    assert err.max() < 2e-2, err.max()
    chain.close()
