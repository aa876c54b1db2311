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
    with pytest.raises(TypeError):
        nodes.LinearNode(in_dim=8, out_dim=8, gate_fuse=True)     # not part of the reference's Config (linear.h:270-280)
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
    assert nodes_[4].can_absorb_gate() and nodes_[3].accept_residual and nodes_[5].accept_residual
    # gateValue - gatedMul - out, as vAi's gated feed-forward wires it (gated-feed-forward.h:46)
    gm, gm_slot = nodes_[5].links["in0"]
    from vai_b200.nodes import GatedMulNode
    assert isinstance(gm, GatedMulNode) and gm.links["in0"] == (nodes_[4], "out0") and gm.activation == engine.Epilogue.SILU
    assert nodes_[0]["weight"].shape == (2048, 2048) and nodes_[0]["weight"].dtype == Dtype.BF16
    w = engine.bits_to_f32(nodes_[0]["weight"].host, Dtype.BF16)
    assert abs(float(w.std()) - 0.02) < 1e-3
    net._sorted()


def test_gated_mul_node_and_the_merge_rule():
    """GatedMulNode has the reference's single option and slots (vAi vai/nodes/gated-mul.h:34-54);
    a Linear may carry it in its epilogue only when it ends at acc + bias[row]."""
    from vai_b200 import Epilogue, nodes
    _net()
    g = nodes.GatedMulNode()
    assert g.activation == Epilogue.SILU and set(g.slots) == {"out0", "in0"}
    g = nodes.GatedMulNode(activation=Epilogue.GELU_TANH)
    g.slots["in0"] = engine.Tensor((3, 5, 48), Dtype.F16)
    g.prepare()
    assert g["out0"].shape == (3, 5, 24) and g["out0"].dtype == Dtype.F32      # the net's default output dtype
    g.set_o_dtype(Dtype.F16)
    g.prepare()
    assert g["out0"].dtype == Dtype.F16
    g.slots["in0"] = engine.Tensor((3, 7), Dtype.F32)
    with pytest.raises(ValueError):
        g.prepare()

    plain = nodes.LinearNode(in_dim=8, out_dim=16)
    assert plain.can_absorb_gate() and not plain.gate_fuse
    assert not nodes.LinearNode(in_dim=8, out_dim=15).can_absorb_gate()
    assert not nodes.LinearNode(in_dim=8, out_dim=16, epilogue=Epilogue.RELU).can_absorb_gate()
    assert not nodes.LinearNode(in_dim=8, out_dim=16, accept_residual=True).can_absorb_gate()
    assert not nodes.LinearNode(in_dim=8, out_dim=16, scalar_scale=2.0).can_absorb_gate()
    plain["bias"] = engine.Tensor((2, 16), Dtype.F32)      # a table over rows is not one entry per weight row
    assert not plain.can_absorb_gate()
    plain["bias"] = engine.Tensor((16,), Dtype.F32)
    assert plain.can_absorb_gate()
    g.set_o_dtype(Dtype.BF16)
    assert g.absorb_into_producer(plain, "out0") and g.fused and plain.gate_fuse
    assert plain._gate == Epilogue.GELU_TANH and plain._gate_o_dtype == Dtype.BF16
    g.reset_fusion()
    plain.reset_fusion()
    assert not g.fused and not plain.gate_fuse
    assert not g.absorb_into_producer(nodes.RmsNormNode(), "out0")
