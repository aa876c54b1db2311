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
