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
