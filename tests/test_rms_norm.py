"""RmsNorm, the producer of a Linear's activations in the Llama / Gemma blocks (vAi
vai/nodes/rms-norm.h, python/tests/nodes/test_rms_norm.py): the CPU oracles against the
golden outputs of the reference's tests, and the CUDA node against both — including the
16-bit output that lets the tensor-core Linear skip its fp32 -> 16-bit staging pass."""
import numpy as np
import pytest
from linear_check import FP32, assert_close, draw_case, load_golden

from oracle import linear_oracle as orc

META, ARRAYS = load_golden()
CASES = sorted(k for k in META if k.startswith("rms_norm"))


def _operands(key):
    cfg, params, fed = draw_case(META, key)
    both = {**params, **fed}
    return cfg, both["in0"], both.get("scale"), both.get("shift"), both.get("residual")


@pytest.mark.parametrize("key", CASES)
def test_rms_norm_oracles_match_golden(key):
    cfg, x, scale, shift, res = _operands(key)
    np.testing.assert_allclose(orc.rms_norm_f64(x, scale, shift, res, cfg["eps"]), ARRAYS[key], rtol=1e-12, atol=1e-12)
    for wg in (32, 256):
        assert_close(orc.rms_norm_c(x, scale, shift, res, cfg["eps"], wg_size=wg), ARRAYS[key], FP32, f"{key} wg {wg}")


def _net(cfg, slots, o_dtype=None):
    import vai_b200
    from vai_b200 import nodes

    class Net(vai_b200.NeuralNet):
        def __init__(self):
            super().__init__(w_default_dtype=vai_b200.Dtype.F32)
            self.node = nodes.RmsNormNode(eps=cfg["eps"], coeffs_as_inputs=cfg.get("coeffs_as_inputs", False),
                                          accept_residual=cfg.get("accept_residual", False))
            if o_dtype is not None:
                self.node.set_o_dtype(o_dtype)
            self.input(slots[0]) - slots[0] / self.node - self.output("out0")
            for s in slots[1:]:
                self.input(s) - s / self.node

    return Net()


@pytest.mark.gpu
@pytest.mark.parametrize("key", [k for k in CASES if not k.endswith("__alt")])
def test_rms_norm_node_reference_cases(key, device):
    """The three reference cases (and the rerun at another row count), FP32 tier."""
    from vai_b200 import Tensor
    cfg, params, fed = draw_case(META, key)
    net = _net(cfg, list(fed))
    for name, arr in params.items():
        net.node[name] = Tensor.from_numpy(arr)
    got = net(**{k: Tensor.from_numpy(v) for k, v in fed.items()}).to_numpy()
    assert_close(got, ARRAYS[key], FP32, key)
    np.testing.assert_array_equal(net(**{k: Tensor.from_numpy(v) for k, v in fed.items()}).to_numpy(), got)
    alt = key + "__alt"
    if alt in META:
        _, _, fed2 = draw_case(META, alt)
        got2 = net(**{k: Tensor.from_numpy(v) for k, v in fed2.items()}).to_numpy()
        assert_close(got2, ARRAYS[alt], FP32, alt)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,feat", [(1, 2048), (64, 2560), (7, 5000), (300, 768), (3, 33)])
@pytest.mark.parametrize("dt", [("f32", "f32", "f32"), ("f32", "f32", "bf16"), ("bf16", "bf16", "bf16"), ("f16", "f32", "f16")])
def test_rms_norm_node_sizes_and_dtypes(rows, feat, dt, device):
    from gpu_util import DT, seen
    from vai_b200 import Tensor
    rng = np.random.default_rng(rows + feat)
    x = rng.standard_normal((rows, feat)).astype(np.float32) * 3
    scale = rng.standard_normal(feat).astype(np.float32)
    res = rng.standard_normal((rows, feat)).astype(np.float32)
    i_dt, w_dt, o_dt = (DT[d] for d in dt)
    net = _net({"eps": 1e-6, "accept_residual": True}, ["in0", "residual"], o_dtype=o_dt)
    net.node["scale"] = Tensor.from_numpy(scale, dtype=w_dt)
    got = net(in0=Tensor.from_numpy(x, dtype=i_dt), residual=Tensor.from_numpy(res, dtype=i_dt)).to_numpy().astype(np.float32)
    want = orc.rms_norm_f64(seen(x, i_dt), seen(scale, w_dt), None, seen(res, i_dt), 1e-6)
    tol = (1e-5, 1e-5) if dt[2] == "f32" else ((2.0 ** -11 + 1e-5, 1e-5) if dt[2] == "f16" else (2.0 ** -8 + 1e-5, 1e-5))
    assert_close(got, want, tol, f"rms {rows}x{feat} {dt}")


@pytest.mark.gpu
def test_rms_norm_16bit_output_removes_the_linear_cast_pass(device):
    """RmsNorm -> Linear (64 rows, bf16 weights): with bf16 activations out of the norm the
    Linear runs one kernel instead of cast + GEMM, and the result equals float64 over the
    rounded activations."""
    import vai_b200
    from gpu_util import seen
    from vai_b200 import Dtype, Tensor, nodes
    rng = np.random.default_rng(0)
    M, D, N = 64, 512, 384
    x = rng.standard_normal((M, D)).astype(np.float32)
    scale = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    w = (rng.standard_normal((N, D)) / np.sqrt(D)).astype(np.float32)
    launches = {}
    outs = {}
    for name, norm_out in (("fp32", Dtype.F32), ("bf16", Dtype.BF16)):
        class Net(vai_b200.NeuralNet):
            def __init__(self):
                super().__init__(w_default_dtype=Dtype.BF16)
                self.norm = nodes.RmsNormNode(eps=1e-6)
                self.norm.set_o_dtype(norm_out)
                self.lin = nodes.LinearNode(in_dim=D, out_dim=N)
                self.input("in0") - self.norm - self.lin - self.output("out0")
        net = Net()
        net.norm["scale"] = Tensor.from_numpy(scale)
        net.lin["weight"] = Tensor.from_numpy(w, dtype=Dtype.BF16)
        outs[name] = net(Tensor.from_numpy(x)).to_numpy()
        launches[name] = net.lin.info.launches
    assert launches["fp32"] == launches["bf16"] + 1      # the cast pass is gone (a split-K fold may remain)
    normed = seen(orc.rms_norm_f64(x, scale, eps=1e-6).astype(np.float32), Dtype.BF16)
    want = orc.linear_f64(normed, seen(w, Dtype.BF16))
    for name in outs:
        assert_close(outs[name], want, (5e-3, 5e-3), name)      # the norm's own rounding moves a few activations by one bf16 ulp
    assert np.abs(outs["fp32"] - outs["bf16"]).max() < 2e-2
