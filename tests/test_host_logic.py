"""CPU: host-side logic of the Python mirror — conversions, LinearNode argument
checks, graph wiring, preset shapes."""
import numpy as np
import pytest

from oracle import linear_oracle as orc
from vai_b200 import engine, presets
from vai_b200.engine import Dtype


def test_host_conversions_equal_the_loader_restatement():
    rng = np.random.default_rng(0)
    a = np.concatenate([rng.standard_normal(5000).astype(np.float32) * s for s in (1e-7, 1e-4, 1.0, 300.0, 1e5)])
    a = np.concatenate([a, np.array([0.0, -0.0, np.inf, -np.inf, 65504.0, 65520.0, 2.0 ** -14, 2.0 ** -14 * 0.999], dtype=np.float32)])
    np.testing.assert_array_equal(engine.f32_to_f16_bits(a), orc.to_dtype(a, orc.F16))
    np.testing.assert_array_equal(engine.f32_to_bf16_bits(a), orc.to_dtype(a, orc.BF16))
    for dt, o in ((Dtype.F16, orc.F16), (Dtype.BF16, orc.BF16)):
        bits = engine.encode(a, dt)
        np.testing.assert_array_equal(engine.bits_to_f32(bits, dt), orc.to_f32(bits, o))


def test_preset_counts_match_the_reference_models():
    """Weight element counts of the in-scope nets (vAi models/production/*/net.h)."""
    assert presets.weight_elements("llama-3.2-1b") == 1_235_746_816
    assert presets.weight_elements("gemma-3-4b") == 3_879_731_200
    assert presets.weight_elements("gpt2-small") == 123_532_032
    p = presets.PRESETS["llama-3.2-3b"]
    per_block = sum(k * n for _, k, n, _ in presets.block_linears(p))
    assert per_block == 100_663_296
    assert presets.flops("llama-3.2-3b", 8192) - 2 * 8192 * 3072 * 128256 == 28 * 2 * 8192 * per_block


class _NoDevice:
    """Stands in for Device so that graph wiring can be checked without a GPU."""
    lib = None

    def create_stream(self):
        return None


def _net():
    return engine.NeuralNet(device=_NoDevice())


def test_linear_node_argument_checks():
    from vai_b200 import nodes
    _net()
    with pytest.raises(ValueError):
        nodes.LinearNode(in_dim=8, out_dim=8, split_size=16)      # must be 0 or >= 32 (vAi linear.cpp:27)
    with pytest.raises(ValueError):
        nodes.LinearNode(in_dim=0, out_dim=8)
    with pytest.raises(ValueError):
        nodes.LinearNode(in_dim=8, out_dim=7, gate_fuse=True)
    n = nodes.LinearNode(in_dim=8, out_dim=4, accept_residual=True)
    assert set(n.slots) == {"out0", "in0", "weight", "partial", "bias", "residual"}   # vAi linear.h:2134-2144
    assert not n.has_bias()
    assert set(nodes.LinearNode(in_dim=8, out_dim=4).slots) == {"out0", "in0", "weight", "partial", "bias"}
    with pytest.raises(KeyError):
        n["nope"] = engine.Tensor((1,), Dtype.F32)


def test_wiring_and_topological_order():
    from vai_b200 import nodes
    net = _net()
    a = nodes.LinearNode(in_dim=4, out_dim=4)
    b = nodes.LinearNode(in_dim=4, out_dim=4, accept_residual=True)
    net.input("x") - a - b - net.output("y")
    net.input("x") - "residual" / b
    order = net._sorted()
    assert order.index(a) < order.index(b)
    assert b.links["in0"] == (a, "out0") and b.links["residual"][1] == "out0"
    assert order.index(net._inputs["x"]) < order.index(a) and order.index(b) < order.index(net._outputs["y"])


def test_chain_builder_shapes():
    net = _net()
    nodes_ = presets.build_linear_chain(net, "llama-3.2-1b", layers=2, vocab_rows=1024)
    assert len(nodes_) == 2 * 6 + 1
    assert [(n.in_dim, n.out_dim) for n in nodes_[:6]] == [(2048, 2048), (2048, 512), (2048, 512), (2048, 2048), (2048, 16384), (8192, 2048)]
    assert nodes_[4].gate_fuse and nodes_[3].accept_residual and nodes_[5].accept_residual
    assert nodes_[0]["weight"].shape == (2048, 2048) and nodes_[0]["weight"].dtype == Dtype.BF16
    w = engine.bits_to_f32(nodes_[0]["weight"].host, Dtype.BF16)
    assert abs(float(w.std()) - 0.02) < 1e-3
    net._sorted()
