"""LayerNorm, the producer of a Linear's activations in the GPT-2 blocks (vAi
vai/nodes/layer-norm.h, python/tests/nodes/test_layer_norm.py): the CPU oracles against
the golden outputs of the reference's four tests (and the rerun at another row count),
and the CUDA node against both."""
import numpy as np
import pytest
from linear_check import FP32, assert_close, draw_case, load_golden

from oracle import linear_oracle as orc

META, ARRAYS = load_golden()
CASES = sorted(k for k in META if k.startswith("layer_norm"))


def _operands(key):
    cfg, params, fed = draw_case(META, key)
    both = {**params, **fed}
    return cfg, both["in0"], both["scale"], both.get("shift"), both.get("residual")


def test_all_reference_cases_present():
    assert CASES == ["layer_norm_coeffs_as_inputs", "layer_norm_no_shift", "layer_norm_residual", "layer_norm_with_shift",
                     "layer_norm_with_shift__alt"]


@pytest.mark.parametrize("key", CASES)
def test_layer_norm_oracles_match_golden(key):
    cfg, x, scale, shift, res = _operands(key)
    np.testing.assert_allclose(orc.layer_norm_f64(x, scale, shift, res, cfg["eps"]), ARRAYS[key], rtol=1e-11, atol=1e-11)
    for wg in (None, 32, 256):      # the reference's own geometry, and two others: the statistics must not depend on it
        assert_close(orc.layer_norm_c(x, scale, shift, res, cfg["eps"], wg_size=wg), ARRAYS[key], FP32, f"{key} wg {wg}")


def test_layer_norm_oracle_large_offset():
    """Rows with a mean far from zero: the shifted one-pass statistics keep fp32 accuracy
    where a plain sum of squares would cancel."""
    rng = np.random.default_rng(3)
    x = (1000.0 + rng.standard_normal((4, 768))).astype(np.float32)
    scale = np.ones(768, dtype=np.float32)
    want = orc.layer_norm_f64(x, scale)
    assert_close(orc.layer_norm_c(x, scale), want, (2e-3, 2e-3), "offset rows")


def test_layer_norm_wg_size_rule():
    assert [orc.layer_norm_wg_size(f) for f in (50, 96, 128, 129, 768, 2048, 100000)] == [32, 32, 32, 64, 256, 512, 512]


def _net(cfg, slots, o_dtype=None):
    import vai_b200
    from vai_b200 import nodes

    class Net(vai_b200.NeuralNet):
        def __init__(self):
            super().__init__(w_default_dtype=vai_b200.Dtype.F32)
            self.node = nodes.LayerNormNode(eps=cfg["eps"], coeffs_as_inputs=cfg.get("coeffs_as_inputs", False),
                                            accept_residual=cfg.get("accept_residual", False))
            if o_dtype is not None:
                self.node.set_o_dtype(o_dtype)
            self.input(slots[0]) - slots[0] / self.node - self.output("out0")
            for s in slots[1:]:
                self.input(s) - s / self.node

    return Net()


def test_layer_norm_node_needs_scale():
    import vai_b200
    from vai_b200 import Tensor, nodes
    node = nodes.LayerNormNode()
    node.slots["in0"] = Tensor((2, 8), vai_b200.Dtype.F32)
    with pytest.raises(ValueError):
        node.prepare()


@pytest.mark.gpu
@pytest.mark.parametrize("key", [k for k in CASES if not k.endswith("__alt")])
def test_layer_norm_node_reference_cases(key, device):
    from vai_b200 import Tensor
    cfg, params, fed = draw_case(META, key)
    net = _net(cfg, list(fed))
    for name, arr in params.items():
        net.node[name] = Tensor.from_numpy(arr)
    got = net(**{k: Tensor.from_numpy(v) for k, v in fed.items()}).to_numpy()
    assert_close(got, ARRAYS[key], FP32, key)
    np.testing.assert_array_equal(net(**{k: Tensor.from_numpy(v) for k, v in fed.items()}).to_numpy(), got)
    assert_close(got, orc.layer_norm_c(fed["in0"], {**params, **fed}["scale"], {**params, **fed}.get("shift"),
                                       fed.get("residual"), cfg["eps"]), (2e-6, 2e-6), key + " vs the C restatement")
    alt = key + "__alt"
    if alt in META:
        _, _, fed2 = draw_case(META, alt)
        got2 = net(**{k: Tensor.from_numpy(v) for k, v in fed2.items()}).to_numpy()
        assert_close(got2, ARRAYS[alt], FP32, alt)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,feat", [(1, 768), (1024, 768), (7, 5000), (64, 2560), (3, 33)])
@pytest.mark.parametrize("dt", [("f32", "f32", "f32"), ("f32", "f16", "f16"), ("bf16", "bf16", "bf16"), ("f16", "f32", "f32")])
def test_layer_norm_node_sizes_and_dtypes(rows, feat, dt, device):
    from gpu_util import DT, seen
    from vai_b200 import Tensor
    rng = np.random.default_rng(rows + feat)
    x = (rng.standard_normal((rows, feat)) * 3 + 5).astype(np.float32)
    scale = rng.standard_normal(feat).astype(np.float32)
    shift = rng.standard_normal(feat).astype(np.float32)
    res = rng.standard_normal((rows, feat)).astype(np.float32)
    i_dt, w_dt, o_dt = (DT[d] for d in dt)
    net = _net({"eps": 1e-5, "accept_residual": True}, ["in0", "residual"], o_dtype=o_dt)
    net.node["scale"] = Tensor.from_numpy(scale, dtype=w_dt)
    net.node["shift"] = Tensor.from_numpy(shift, dtype=w_dt)
    got = net(in0=Tensor.from_numpy(x, dtype=i_dt), residual=Tensor.from_numpy(res, dtype=i_dt)).to_numpy().astype(np.float32)
    want = orc.layer_norm_f64(seen(x, i_dt), seen(scale, w_dt), seen(shift, w_dt), seen(res, i_dt), 1e-5)
    tol = (2e-5, 2e-5) if dt[2] == "f32" else ((2.0 ** -11 + 1e-5, 1e-4) if dt[2] == "f16" else (2.0 ** -8 + 1e-5, 1e-4))
    assert_close(got, want, tol, f"layer norm {rows}x{feat} {dt}")


@pytest.mark.gpu
def test_layer_norm_feeds_gpt2_fc1(device):
    """LayerNorm -> Linear with bias and GELU(tanh), the head of a GPT-2 feed-forward block
    (768 -> 3072, fp16 weights, 128 rows), against float64 over the stored operands."""
    import vai_b200
    from gpu_util import seen
    from vai_b200 import Dtype, Epilogue, Tensor, nodes
    rng = np.random.default_rng(0)
    M, D, N = 128, 768, 3072
    x = rng.standard_normal((M, D)).astype(np.float32)
    scale = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    shift = (0.1 * rng.standard_normal(D)).astype(np.float32)
    w = (rng.standard_normal((N, D)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(N) * 0.02).astype(np.float32)

    class Net(vai_b200.NeuralNet):
        def __init__(self):
            super().__init__(w_default_dtype=Dtype.F16)
            self.norm = nodes.LayerNormNode(eps=1e-5)
            self.norm.set_o_dtype(Dtype.F16)
            self.lin = nodes.LinearNode(in_dim=D, out_dim=N, epilogue=Epilogue.GELU_TANH)
            self.input("in0") - self.norm - self.lin - self.output("out0")

    net = Net()
    net.norm["scale"] = Tensor.from_numpy(scale)
    net.norm["shift"] = Tensor.from_numpy(shift)
    net.lin["weight"] = Tensor.from_numpy(w, dtype=Dtype.F16)
    net.lin["bias"] = Tensor.from_numpy(b, dtype=Dtype.F16)
    got = net(Tensor.from_numpy(x)).to_numpy()
    normed = seen(orc.layer_norm_f64(x, scale, shift).astype(np.float32), Dtype.F16)
    want = orc.linear_f64(normed, seen(w, Dtype.F16), seen(b, Dtype.F16), epilogue=orc.EPILOGUES["GELU_TANH"])
    # 16-bit activations: no cast pass; a split-K fold is the only possible second launch (none when the splits fold inside clusters)
    assert net.lin.info.launches <= 1 + (net.lin.info.split_count > 1)
    assert_close(got, want, (5e-3, 5e-3), "ln -> fc1")
