"""GatedMul, the consumer of a gate|value Linear (vAi vai/nodes/gated-mul.h,
python/tests/nodes/test_gated_mul.py): out = activation(in0[..., :H]) * in0[..., H:].

The reference's three cases are checked three ways: the two oracles against the golden
outputs (CPU); the node on its own, as the reference's test builds it (one GatedMulNode
between the net's input and output); and the node behind a Linear whose [2H, 2H] weight is
the identity, where the net records the pair as ONE launch (the dot products return in0
exactly, so what is left is the gate arithmetic in the Linear kernel's epilogue).  All at
the reference's tolerance for transcendental epilogues (TRANS).  Then the record-time rule
itself: when the pair merges, when it must not, and that merged and unmerged agree."""
import numpy as np
import pytest
from linear_check import TRANS, assert_close, draw_case, load_golden

from oracle import linear_oracle as orc

META, ARRAYS = load_golden()
CASES = sorted(k for k in META if k.startswith("gated_mul"))


def test_all_reference_cases_present():
    assert CASES == ["gated_mul_GELU_TANH", "gated_mul_RELU", "gated_mul_SILU"]
    assert all(tuple(META[k]["tol"]) == TRANS for k in CASES)


@pytest.mark.parametrize("key", CASES)
def test_gate_epilogue_oracles_match_golden(key):
    cfg, _, fed = draw_case(META, key)
    x = fed["in0"]
    n = x.shape[-1]
    eye = np.eye(n, dtype=np.float32)
    code = orc.EPILOGUES[cfg["activation"]]
    np.testing.assert_allclose(orc.gated_mul_f64(x, code), ARRAYS[key], rtol=1e-12, atol=1e-12)
    assert_close(orc.gated_mul_c(x, code), ARRAYS[key], TRANS, key + " (shader restatement)")
    np.testing.assert_allclose(orc.linear_f64(x, eye, epilogue=code, gate_fuse=True), ARRAYS[key], rtol=1e-12, atol=1e-12)
    d = orc.make_desc(x.shape[0], n, n, epilogue=code, gate_fuse=True)
    assert_close(orc.linear_c(d, x, eye), ARRAYS[key], TRANS, key)


def test_gated_mul_restatement_dtypes():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 5, 24)).astype(np.float32)
    for i_dt in (orc.F32, orc.F16, orc.BF16):
        xs = orc.to_dtype(x, i_dt)
        want = orc.gated_mul_f64(orc.to_f32(xs, i_dt), 4)
        for o_dt, tol in ((orc.F32, 1e-5), (orc.F16, 2e-3), (orc.BF16, 1e-2)):
            got = orc.to_f32(orc.gated_mul_c(xs, 4, i_dt, o_dt), o_dt)
            assert got.shape == (3, 5, 12)
            np.testing.assert_allclose(got, want, rtol=tol, atol=tol)


def _node_net(activation, o_dtype=None, i_shape=None):
    import vai_b200
    from vai_b200 import Epilogue, nodes

    class Net(vai_b200.NeuralNet):
        def __init__(self):
            super().__init__()
            self.gm = nodes.GatedMulNode(activation=getattr(Epilogue, activation))
            if o_dtype is not None:
                self.gm.set_o_dtype(o_dtype)
            self.input("in0") - self.gm - self.output("out0")

    return Net()


@pytest.mark.gpu
@pytest.mark.parametrize("key", CASES)
def test_node_alone_matches_golden(key, device):
    """check_node(lambda: GatedMulNode(activation=...), {"in0": (4, 48)}, ref, tol=TRANS) of the
    reference's test: first forward, rerun on fresh inputs, and a replay."""
    from vai_b200 import Tensor
    cfg, _, fed = draw_case(META, key)
    net = _node_net(cfg["activation"])
    got = net(Tensor.from_numpy(fed["in0"])).to_numpy()
    assert got.shape == (4, 24) and not net.gm.fused
    assert_close(got, ARRAYS[key], TRANS, key)
    np.testing.assert_array_equal(net(Tensor.from_numpy(fed["in0"])).to_numpy(), got)
    rerun = key + "_rerun"
    if rerun in META:
        _, _, fed2 = draw_case(META, rerun)
        assert_close(net(Tensor.from_numpy(fed2["in0"])).to_numpy(), ARRAYS[rerun], TRANS, rerun)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(4, 48), (3, 7, 30), (1, 16384), (64, 20480), (5, 2)])
@pytest.mark.parametrize("dt", [("f32", "f32"), ("bf16", "bf16"), ("f16", "f32"), ("f32", "bf16")])
@pytest.mark.parametrize("activation", ["SILU", "GELU_TANH", "NONE"])
def test_node_alone_shapes_and_dtypes(shape, dt, activation, device):
    """Vector path (H a multiple of the 16-byte width) and element path, every dtype pair,
    against float64 over the stored values and against the shader restatement."""
    from gpu_util import DT, out_tol, seen
    from vai_b200 import Tensor
    if shape == (64, 20480) and activation != "GELU_TANH":
        pytest.skip("the wide case once")
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal(shape).astype(np.float32)
    net = _node_net(activation, o_dtype=DT[dt[1]])
    got = net(Tensor.from_numpy(x, dtype=DT[dt[0]])).to_numpy().astype(np.float32)
    code = orc.EPILOGUES[activation]
    xs = seen(x, DT[dt[0]])
    assert got.shape == tuple(shape[:-1]) + (shape[-1] // 2,)
    assert_close(got, orc.gated_mul_f64(xs, code), out_tol(dt[1], 1e-5, 1e-6), f"{shape} {dt} {activation}")
    i_c, o_c = {"f32": orc.F32, "f16": orc.F16, "bf16": orc.BF16}[dt[0]], {"f32": orc.F32, "f16": orc.F16, "bf16": orc.BF16}[dt[1]]
    c = orc.to_f32(orc.gated_mul_c(orc.to_dtype(x, i_c), code, i_c, o_c), o_c)
    # the device's expf / tanhf and the host's differ in the last fp32 bit now and then, which can move
    # a 16-bit output to the neighbouring value: one unit in the last place of the output dtype is allowed
    ulp = {"f32": 0.0, "f16": 2.0 ** -10, "bf16": 2.0 ** -7}[dt[1]]
    assert_close(got, c, (1e-5 + ulp, 1e-6), f"{shape} {dt} {activation} vs restatement")


@pytest.mark.gpu
@pytest.mark.parametrize("key", CASES)
@pytest.mark.parametrize("kernel", ["auto", "fma"])
def test_gate_epilogue_on_gpu_matches_golden(key, kernel, device):
    """Linear(identity) - GatedMul recorded as one launch."""
    from gpu_util import run_linear
    from vai_b200 import nodes
    cfg, _, fed = draw_case(META, key)
    x = fed["in0"]
    n = x.shape[-1]
    got, want, node = run_linear(x, np.eye(n, dtype=np.float32), epilogue=cfg["activation"], gate_fuse=True,
                                 kernel={"auto": nodes.KERNEL_AUTO, "fma": nodes.KERNEL_FMA_TILE}[kernel])
    assert got.shape == (4, n // 2) and node.info.launches == (2 if kernel == "fma" else 1)
    assert_close(got, ARRAYS[key], TRANS, f"{key} {kernel}")
    assert_close(got, want, TRANS, f"{key} {kernel} vs float64")


@pytest.mark.gpu
@pytest.mark.parametrize("case", [
    # M, K, H, w_dtype, kernel: the weight-streaming kernel, the exact fp32 tile kernel, both tensor-core kernels
    (1, 512, 328, "bf16", 0), (4, 256, 64, "f32", 0), (40, 96, 56, "f32", 0), (64, 512, 384, "bf16", 0), (300, 256, 192, "f16", 0)])
@pytest.mark.parametrize("activation", ["SILU", "GELU_TANH"])
def test_merged_and_unmerged_agree(case, activation, device):
    """The same Linear - GatedMul net recorded as one launch and as two.  With an fp32
    intermediate the two differ only by the activation's evaluation (the tensor-core epilogue
    uses the fast exp / divide units) and by nothing at all on the CUDA-core kernels, whose
    merged epilogue calls the same function as the stand-alone kernel."""
    from gpu_util import run_linear
    from vai_b200 import nodes
    M, K, H, w_dtype, kernel = case
    rng = np.random.default_rng(M + K + H)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((2 * H, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(2 * H).astype(np.float32)
    one, want, node1 = run_linear(x, w, b, w_dtype=w_dtype, b_dtype="f32", epilogue=activation, gate_fuse=True, kernel=kernel)
    two, want2, node2 = run_linear(x, w, b, w_dtype=w_dtype, b_dtype="f32", epilogue=activation, gate_fuse=True, kernel=kernel, fuse=False)
    assert node1.info.kernel == node2.info.kernel
    assert_close(one, want, (1e-4, 2e-5), f"merged {case}")
    assert_close(two, want2, (1e-4, 2e-5), f"unmerged {case}")
    if node1.info.kernel == nodes.KERNEL_FMA_TILE:
        np.testing.assert_array_equal(one, two)         # same sums, same activation code: bit for bit
    else:
        assert_close(one, two, (1e-5, 1e-5), f"merged vs unmerged {case}")


@pytest.mark.gpu
def test_pairs_that_must_not_merge(device):
    """A second reader of the Linear's output, or a Linear with an epilogue / scale / residual
    of its own, keeps the two launches — and the results still follow the two-node arithmetic."""
    import vai_b200
    from vai_b200 import Epilogue, Tensor, nodes
    rng = np.random.default_rng(3)
    K, H = 64, 40
    x = rng.standard_normal((3, K)).astype(np.float32)
    w = (rng.standard_normal((2 * H, K)) / 8).astype(np.float32)

    class TwoReaders(vai_b200.NeuralNet):
        def __init__(self):
            super().__init__(w_default_dtype=vai_b200.Dtype.F32)
            self.lin = nodes.LinearNode(in_dim=K, out_dim=2 * H)
            self.gm = nodes.GatedMulNode(activation=Epilogue.SILU)
            self.input("in0") - self.lin - self.gm - self.output("gated")
            self.lin - self.output("raw")

    net = TwoReaders()
    net.lin["weight"] = Tensor.from_numpy(w)
    out = net(Tensor.from_numpy(x))
    assert not net.lin.gate_fuse and not net.gm.fused
    raw = orc.linear_f64(x, w)
    assert_close(out["raw"].to_numpy(), raw, (1e-5, 1e-5), "raw")
    assert_close(out["gated"].to_numpy(), orc.gated_mul_f64(raw, 4), (1e-4, 1e-5), "gated")

    class OwnEpilogue(vai_b200.NeuralNet):
        def __init__(self, **kw):
            super().__init__(w_default_dtype=vai_b200.Dtype.F32)
            self.lin = nodes.LinearNode(in_dim=K, out_dim=2 * H, **kw)
            self.gm = nodes.GatedMulNode(activation=Epilogue.RELU)
            self.input("in0") - self.lin - self.gm - self.output("out0")

    for kw, ref in (({"epilogue": Epilogue.SIGMOID}, lambda a: orc.epilogue_f64(5, a)), ({"scalar_scale": 0.5}, lambda a: 0.5 * a)):
        net = OwnEpilogue(**kw)
        net.lin["weight"] = Tensor.from_numpy(w)
        got = net(Tensor.from_numpy(x)).to_numpy()
        assert not net.lin.gate_fuse and not net.gm.fused
        assert_close(got, orc.gated_mul_f64(ref(raw), 1), (1e-4, 1e-5), str(kw))
