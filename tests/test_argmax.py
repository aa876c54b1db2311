"""Argmax, the greedy-decode consumer of the lm_head Linear (vAi vai/nodes/argmax.h,
python/tests/nodes/test_argmax.py): CPU oracle against the golden output of the
reference's test, and the CUDA node against both."""
import numpy as np
import pytest
from linear_check import draw_case, load_golden

from oracle import linear_oracle as orc

META, ARRAYS = load_golden()


def test_argmax_oracle_matches_golden():
    _, _, fed = draw_case(META, "argmax")
    want = ARRAYS["argmax"].astype(np.uint32)
    np.testing.assert_array_equal(orc.argmax_c(fed["in0"]), want)
    np.testing.assert_array_equal(fed["in0"].argmax(axis=-1).astype(np.uint32), want)


def test_argmax_oracle_16bit():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 1000)).astype(np.float32)
    for dt in (orc.F16, orc.BF16):
        bits = orc.to_dtype(x, dt)
        vals = orc.to_f32(bits, dt)
        got = orc.argmax_c(bits, dt)
        assert all(vals[r, got[r]] == vals[r].max() for r in range(3))


def _run_node(x, dtype="f32", device=None):
    import vai_b200
    from gpu_util import DT
    from vai_b200 import Tensor, nodes

    class Net(vai_b200.NeuralNet):
        def __init__(self):
            super().__init__()
            self.a = nodes.ArgmaxNode()
            self.input("in0") - self.a - self.output("out0")

    net = Net()
    t = Tensor.from_numpy(x, dtype=DT[dtype])
    first = net(t).to_u32()
    np.testing.assert_array_equal(net(t).to_u32(), first)      # the replay gives the same indices
    return first


@pytest.mark.gpu
def test_argmax_node_reference_case(device):
    """vAi python/tests/nodes/test_argmax.py: [4, 50] standard normal, exact."""
    _, _, fed = draw_case(META, "argmax")
    np.testing.assert_array_equal(_run_node(fed["in0"]), ARRAYS["argmax"].astype(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("M,N", [(1, 128256), (3, 50257), (64, 4099), (2, 1)])
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_argmax_node_sizes(M, N, dtype, device):
    from gpu_util import DT, seen
    rng = np.random.default_rng(M * 7 + N)
    x = rng.standard_normal((M, N)).astype(np.float32)
    vals = seen(x, DT[dtype])
    got = _run_node(x, dtype)
    np.testing.assert_array_equal(got, vals.argmax(axis=-1).astype(np.uint32))    # first occurrence on ties
    if dtype == "f32":
        np.testing.assert_array_equal(got, orc.argmax_c(x))


@pytest.mark.gpu
def test_argmax_ties_go_to_the_lowest_index(device):
    x = np.zeros((2, 5000), dtype=np.float32)
    x[0, [4097, 33, 2048]] = 7.0
    x[1, :] = -1.0
    np.testing.assert_array_equal(_run_node(x), np.array([33, 0], dtype=np.uint32))


def _pairs(device, logits, ld_view, base):
    """vaicu_argmax_pairs_run on a torch tensor [M, N] that may be a column window of a
    wider buffer (row stride ld_view)."""
    import ctypes

    import torch

    from vai_b200 import _lib
    M, N = logits.shape
    dt = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 3}[logits.dtype]
    ws_bytes = ctypes.c_size_t()
    _lib.check(device.lib.vaicu_argmax_workspace_bytes(M, N, ctypes.byref(ws_bytes)), "workspace")
    ws = torch.empty(ws_bytes.value, dtype=torch.uint8, device=logits.device)
    val = torch.empty(M, dtype=torch.float32, device=logits.device)
    idx = torch.empty(M, dtype=torch.int32, device=logits.device)
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(device.lib.vaicu_argmax_pairs_run(stream, logits.data_ptr(), dt, M, N, ld_view, base, ws.data_ptr(),
                                                 val.data_ptr(), idx.data_ptr()), "vaicu_argmax_pairs_run")
    return val, idx


@pytest.mark.gpu
@pytest.mark.parametrize("M,N", [(1, 128256), (64, 262144), (5, 20001), (3, 7)])
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_two_stage_argmax_matches_one_block_per_row(M, N, dtype, device):
    import torch
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[dtype]
    g = torch.Generator(device="cuda").manual_seed(N + M)
    x = torch.randn(M, N, generator=g, device="cuda").to(tdt)
    x[0, N // 2:] = x[0, : N - N // 2].flip(0)            # plant equal maxima in different segments
    val, idx = _pairs(device, x, N, 0)
    torch.cuda.synchronize()
    want_val, _ = x.float().max(dim=1)
    first = (x.float() == want_val[:, None]).int().argmax(dim=1)      # lowest index among equal maxima
    assert torch.equal(idx.long(), first) and torch.equal(val, want_val)


@pytest.mark.gpu
def test_vocabulary_slabs_merge_to_the_global_argmax(device):
    """Four column slabs of one logits matrix (windows of the wide rows, ragged widths),
    candidates per slab with their vocabulary offset, then one merge: the same tokens as the
    argmax over whole rows, with a tie across slabs going to the lower slab."""
    import ctypes

    import torch

    from vai_b200 import _lib
    M, V = 6, 50257
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(M, V, generator=g, device="cuda")
    x[2, 100] = x[2, 40000] = 9.0
    bounds = [0, 12565, 25130, 37694, V]
    vals = torch.empty(4, M, dtype=torch.float32, device="cuda")
    idxs = torch.empty(4, M, dtype=torch.int32, device="cuda")
    for s in range(4):
        window = x[:, bounds[s]:bounds[s + 1]]
        v, i = _pairs(device, window, V, bounds[s])
        vals[s], idxs[s] = v, i
    out = torch.empty(M, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(device.lib.vaicu_argmax_merge_run(stream, vals.data_ptr(), idxs.data_ptr(), 4, M, M, None, out.data_ptr()), "merge")
    torch.cuda.synchronize()
    want = x.argmax(dim=1)
    want[2] = 100
    assert torch.equal(out.long(), want)


# ---- Argmax sharing the lm_head's launch -------------------------------------------------

def _head_net(K, V, w, w_dtype, o_dtype=None, fuse=True, bias=None, second_reader=False):
    import vai_b200
    from gpu_util import DT
    from vai_b200 import Tensor, nodes

    class Net(vai_b200.NeuralNet):
        def __init__(self):
            super().__init__(w_default_dtype=DT[w_dtype], fuse_argmax=fuse)
            self.head = nodes.LinearNode(in_dim=K, out_dim=V)
            if o_dtype:
                self.head.set_o_dtype(DT[o_dtype])
            self.pick = nodes.ArgmaxNode()
            self.input("in0") - self.head - self.pick - self.output("token")
            if second_reader:
                self.head - self.output("logits")

    net = Net()
    net.head["weight"] = Tensor.from_numpy(w, dtype=DT[w_dtype])
    if bias is not None:
        net.head["bias"] = Tensor.from_numpy(bias, dtype=DT[w_dtype])
    return net


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,V", [(1, 2048, 128256), (1, 768, 50257), (3, 512, 4099), (4, 256, 33), (2, 1024, 1000)])
@pytest.mark.parametrize("w_dtype,o_dtype", [("bf16", None), ("f16", "f16"), ("f32", None), ("bf16", "bf16")])
def test_argmax_shares_the_linear_launch(M, K, V, w_dtype, o_dtype, device):
    """lm_head -> Argmax recorded as one launch picks the tokens the two nodes pick when
    recorded separately (same kernel, same sums: equal, ties included), and those are the
    argmax of the float64 logits wherever the top-2 margin exceeds the accumulation error."""
    from gpu_util import DT, seen
    from vai_b200 import Tensor
    if V > 100000 and w_dtype != "bf16":
        pytest.skip("the vocabulary-sized case once per output dtype")
    rng = np.random.default_rng(M + K + V)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((V, K)) / np.sqrt(K)).astype(np.float32)
    w[V // 3] = w[V // 2]                                  # two equal logits in every row
    b = rng.standard_normal(V).astype(np.float32) * 0.1
    b[V // 3] = b[V // 2]
    t = Tensor.from_numpy(x)
    one = _head_net(K, V, w, w_dtype, o_dtype, fuse=True, bias=b)
    two = _head_net(K, V, w, w_dtype, o_dtype, fuse=False, bias=b)
    tok1 = one(t).to_u32()
    tok2 = two(t).to_u32()
    assert one.pick.fused and not two.pick.fused
    rec1, rec2 = next(iter(one._recordings.values())), next(iter(two._recordings.values()))
    assert rec1.kernel_launches == 1 and rec2.kernel_launches in (2, 3)
    np.testing.assert_array_equal(tok1, tok2)
    np.testing.assert_array_equal(one(t).to_u32(), tok1)              # replay: the ticket counter reset itself
    np.testing.assert_array_equal(one(Tensor.from_numpy(x[::-1].copy())).to_u32(), two(Tensor.from_numpy(x[::-1].copy())).to_u32())
    logits = orc.linear_f64(x, seen(w, DT[w_dtype]), seen(b, DT[w_dtype]))
    top2 = np.sort(logits, axis=1)[:, -2:]
    # 16-bit logits tie after rounding (bf16 resolves 1/32 near 4.0): only rows whose top two stay apart count
    clear = (top2[:, 1] - top2[:, 0]) > ({"bf16": 0.07, "f16": 0.01}[o_dtype] if o_dtype else 1e-4)
    np.testing.assert_array_equal(tok1[clear], logits.argmax(axis=1)[clear].astype(np.uint32))


@pytest.mark.gpu
def test_argmax_keeps_its_own_launch_when_it_must(device):
    """A second reader of the logits, or a Linear that is not on the weight-streaming kernel
    (M > 8), leaves Argmax as a node of its own; the tokens are the same either way."""
    from vai_b200 import Tensor
    rng = np.random.default_rng(8)
    K, V = 256, 3000
    w = (rng.standard_normal((V, K)) / 16).astype(np.float32)
    x = rng.standard_normal((2, K)).astype(np.float32)
    net = _head_net(K, V, w, "bf16", second_reader=True)
    out = net(Tensor.from_numpy(x))
    assert not net.pick.fused
    np.testing.assert_array_equal(out["token"].to_u32(), out["logits"].to_numpy().argmax(axis=1).astype(np.uint32))
    big = rng.standard_normal((40, K)).astype(np.float32)
    net = _head_net(K, V, w, "bf16")
    tok = net(Tensor.from_numpy(big)).to_u32()
    assert not net.pick.fused and net.head.info.kernel != 1
    ref = _head_net(K, V, w, "bf16", second_reader=True)(Tensor.from_numpy(big))
    np.testing.assert_array_equal(tok, ref["token"].to_u32())


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 4])
def test_fused_argmax_candidates_of_vocabulary_slabs_merge(M, device):
    """vaicu_linear_run_argmax per vocabulary slab with the slab's index base and maxima out,
    then vaicu_argmax_merge_run: the tokens of the argmax over the whole head, which is how a
    column-split lm_head decodes greedily without gathering logits."""
    import ctypes

    from gpu_util import seen
    from vai_b200 import Dtype, _lib
    from vai_b200.engine import DeviceBuffer, encode
    lib = device.lib
    rng = np.random.default_rng(M)
    K, V, slabs = 512, 10007, 3
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((V, K)) / np.sqrt(K)).astype(np.float32)
    w[9000] = w[17]                                        # a tie across slabs goes to the lower token id
    xb = DeviceBuffer(device, x.nbytes)
    xb.upload(x)
    bounds = [0, 3336, 6672, V]
    vals = DeviceBuffer(device, slabs * M * 4)
    idxs = DeviceBuffer(device, slabs * M * 4)
    keep = []
    for s in range(slabs):
        rows = bounds[s + 1] - bounds[s]
        wb = DeviceBuffer(device, rows * K * 2)
        wb.upload(encode(w[bounds[s]:bounds[s + 1]], Dtype.BF16))
        d = _lib.LinearDesc()
        d.M, d.N, d.K = M, rows, K
        d.i_dtype, d.w_dtype, d.o_dtype, d.b_dtype = 0, 3, 0, 2
        d.scalar_scale = 1.0
        plan = ctypes.c_void_p()
        _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(plan)), "plan")
        n = ctypes.c_size_t()
        _lib.check(lib.vaicu_linear_argmax_workspace_bytes(plan, ctypes.byref(n)), "ws bytes")
        assert n.value >= 512
        ws = DeviceBuffer(device, n.value)
        _lib.check(lib.vaicu_memset(ws.ptr, 0, 256, None), "memset")
        logits = DeviceBuffer(device, M * rows * 4)
        for _ in range(2):                                 # twice: the second call runs on the counter the first one left
            _lib.check(lib.vaicu_linear_run_argmax(plan, None, xb.ptr, wb.ptr, None, None, logits.ptr, ws.ptr, bounds[s],
                                                   vals.ptr + s * M * 4, idxs.ptr + s * M * 4), "vaicu_linear_run_argmax")
        keep += [wb, ws, logits, plan]
    out = DeviceBuffer(device, M * 4)
    _lib.check(lib.vaicu_argmax_merge_run(None, vals.ptr, idxs.ptr, slabs, M, M, None, out.ptr), "merge")
    device.synchronize()
    got = out.download(np.empty(M, dtype=np.uint32))
    logits = orc.linear_f64(x, seen(w, Dtype.BF16))
    want = logits.argmax(axis=1)
    top2 = np.sort(logits, axis=1)[:, -2:]
    for m in range(M):
        if top2[m, 1] - top2[m, 0] > 1e-4 or want[m] in (17, 9000):
            assert got[m] == (17 if want[m] in (17, 9000) else want[m])
    # a gated plan, or a plan on the tensor-core kernel, has no fused form
    g = _lib.LinearDesc()
    g.M, g.N, g.K = 64, 512, 256
    g.i_dtype = g.w_dtype = g.o_dtype = 3
    g.b_dtype, g.scalar_scale = 2, 1.0
    plan = ctypes.c_void_p()
    _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(g), ctypes.byref(plan)), "plan")
    n = ctypes.c_size_t(1)
    _lib.check(lib.vaicu_linear_argmax_workspace_bytes(plan, ctypes.byref(n)), "ws bytes")
    assert n.value == 0
    assert lib.vaicu_linear_run_argmax(plan, None, xb.ptr, xb.ptr, None, None, None, xb.ptr, 0, None, out.ptr) == 2
    lib.vaicu_linear_plan_destroy(plan)
    for p in keep[3::4]:
        lib.vaicu_linear_plan_destroy(p)
