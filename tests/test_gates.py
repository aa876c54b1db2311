"""Gates and optional inputs of the engine host layer (vAi vai/nodes/gate.h,
vai/engine/graph-controller.h): which nodes a recording keeps.  The wiring rules run on the
CPU; the recorded graphs run on the GPU."""
import numpy as np
import pytest

import vai_b200
from vai_b200 import Dtype, Epilogue, Tensor, nodes
from vai_b200.engine import GateNode, InputNode


class _NoDevice:
    """Stands in for Device so that graph wiring can be checked without a GPU."""
    lib = None

    def create_stream(self):
        return None


def _net(device=None):
    """x -> gate; then: a (relu) ; else: b (scale -1) ; both -> c; a second input y feeds d."""
    class Net(vai_b200.NeuralNet):
        def __init__(self):
            super().__init__(w_default_dtype=Dtype.F32, device=device)
            self.gate = GateNode()
            self.a = nodes.LinearNode(in_dim=8, out_dim=8, epilogue=Epilogue.RELU)
            self.b = nodes.LinearNode(in_dim=8, out_dim=8, scalar_scale=-1.0)
            self.c = nodes.LinearNode(in_dim=8, out_dim=4)
            self.d = nodes.LinearNode(in_dim=6, out_dim=4)
            self.input("x") - self.gate
            self.gate / "then" - self.a - self.c
            self.gate / "else" - self.b - self.c            # the merge: two producers of c.in0
            self.c - self.output("main")
            self.input("y") - self.d - self.output("side")

    return Net()


def _names(net, live):
    table = {net.gate: "gate", net.a: "a", net.b: "b", net.c: "c", net.d: "d"}
    return sorted(table[n] for n in live if n in table)


def test_live_nodes_follow_the_gate_and_the_inputs_given():
    net = _net(_NoDevice())
    order = net._sorted()
    assert _names(net, net._live(order, {"x", "y"})) == ["a", "c", "d", "gate"]
    net.gate.set_open(False)
    live = net._live(order, {"x", "y"})
    assert _names(net, live) == ["b", "c", "d", "gate"]
    assert live[net.c]["in0"] == (net.b, "out0")                 # the merge point reads the branch that survived
    assert _names(net, net._live(order, {"y"})) == ["d"]         # x left out: nothing that needs it is recorded
    assert _names(net, net._live(order, {"x"})) == ["b", "c", "gate"]
    assert not any(isinstance(n, InputNode) and n.name == "y" for n in net._live(order, {"x"}))


def test_fan_in_outside_a_gate_merge_is_rejected():
    class Bad(vai_b200.NeuralNet):
        def __init__(self):
            super().__init__(w_default_dtype=Dtype.F32, device=_NoDevice())
            self.a = nodes.LinearNode(in_dim=4, out_dim=4)
            self.b = nodes.LinearNode(in_dim=4, out_dim=4)
            self.c = nodes.LinearNode(in_dim=4, out_dim=4)
            self.input("x") - self.a - self.c
            self.input("x") - self.b - self.c
            self.c - self.output("out0")

    with pytest.raises(RuntimeError, match="producers"):
        Bad()._sorted()
    with pytest.raises(KeyError):
        net = _net(_NoDevice())
        net.input("x") - "nope" / net.a


def test_else_left_unwired_drops_the_downstream():
    class Net(vai_b200.NeuralNet):
        def __init__(self):
            super().__init__(w_default_dtype=Dtype.F32, device=_NoDevice())
            self.gate = GateNode()
            self.a = nodes.LinearNode(in_dim=4, out_dim=4)
            self.input("x") - self.gate
            self.gate / "then" - self.a - self.output("out0")

    net = Net()
    order = net._sorted()
    assert net.a in net._live(order, {"x"})
    net.gate.set_open(False)
    assert net.a not in net._live(order, {"x"})


@pytest.mark.gpu
def test_gate_branches_and_optional_input_on_gpu(device):
    rng = np.random.default_rng(0)
    net = _net()
    w = {k: rng.standard_normal(s).astype(np.float32) for k, s in
         {"a": (8, 8), "b": (8, 8), "c": (4, 8), "d": (4, 6)}.items()}
    for k in w:
        getattr(net, k)["weight"] = Tensor.from_numpy(w[k])
    x = rng.standard_normal((3, 8)).astype(np.float32)
    y = rng.standard_normal((3, 6)).astype(np.float32)
    out = net(x=Tensor.from_numpy(x), y=Tensor.from_numpy(y))
    np.testing.assert_allclose(out["main"].to_numpy(), np.maximum(x @ w["a"].T, 0) @ w["c"].T, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(out["side"].to_numpy(), y @ w["d"].T, rtol=1e-5, atol=1e-5)
    net.gate.set_open(False)                                      # flips the branch: the next call records that state
    out = net(x=Tensor.from_numpy(x), y=Tensor.from_numpy(y))
    np.testing.assert_allclose(out["main"].to_numpy(), -(x @ w["b"].T) @ w["c"].T, rtol=1e-5, atol=1e-5)
    only_side = net(y=Tensor.from_numpy(y))                       # x left out: one output, one Linear recorded
    np.testing.assert_allclose(only_side.to_numpy(), y @ w["d"].T, rtol=1e-5, atol=1e-5)
    assert sorted(r.kernel_launches for r in net._recordings.values()) == [1, 3, 3]
    with pytest.raises(ValueError):
        net(z=Tensor.from_numpy(y))


@pytest.mark.gpu
def test_flipping_a_gate_keeps_one_recording_per_state(device):
    """A decode loop that flips a gate every step: two recordings in all, and the page-locked
    staging stays what those two recordings need.  Changing a weight drops the recordings
    together with their staging and returns their device ranges to the pool."""
    rng = np.random.default_rng(4)
    net = _net()
    w = {k: rng.standard_normal(s).astype(np.float32) for k, s in {"a": (8, 8), "b": (8, 8), "c": (4, 8), "d": (4, 6)}.items()}
    for k in w:
        getattr(net, k)["weight"] = Tensor.from_numpy(w[k])
    x = rng.standard_normal((3, 8)).astype(np.float32)
    want = {True: np.maximum(x @ w["a"].T, 0) @ w["c"].T, False: -(x @ w["b"].T) @ w["c"].T}
    pinned = []
    for step in range(12):
        is_open = step % 2 == 0
        net.gate.set_open(is_open)
        got = net(x=Tensor.from_numpy(x)).to_numpy()
        np.testing.assert_allclose(got, want[is_open], rtol=1e-5, atol=1e-5)
        pinned.append(sum(len(r.pinned) for r in net._recordings.values()) + len(net._pinned_ptrs))
    assert len(net._recordings) == 2
    assert pinned[1] == pinned[-1] and pinned[1] <= 2 * pinned[0]
    net.a["weight"] = Tensor.from_numpy(w["a"] * 2)               # a parameter changed: recordings are stale
    got = net(x=Tensor.from_numpy(x)).to_numpy()                  # gate is closed: branch b, unchanged
    np.testing.assert_allclose(got, want[False], rtol=1e-5, atol=1e-5)
    assert len(net._recordings) == 1
    assert sum(len(r.pinned) for r in net._recordings.values()) + len(net._pinned_ptrs) == pinned[0]
    assert sum(len(v) for v in net.pool.free.values()) > 0         # the dropped recordings' ranges are reusable
