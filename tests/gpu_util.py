"""Shared helpers of the GPU parity tests: run one Linear through the public host
API (NeuralNet + LinearNode -> C ABI) and build the float64 expectation from the
values the device actually sees."""
import numpy as np

import vai_b200
from vai_b200 import Dtype, Epilogue, ResidualOrder, Tensor, nodes
from vai_b200.engine import bits_to_f32, encode

from oracle import linear_oracle as orc

DT = {"f32": Dtype.F32, "f16": Dtype.F16, "bf16": Dtype.BF16}


def seen(a, dt):
    """Values of fp32 array `a` after storage in dtype `dt`."""
    if dt == Dtype.F32:
        return np.asarray(a, dtype=np.float32)
    return bits_to_f32(encode(a, dt), dt).reshape(np.shape(a))


class OneLinear(vai_b200.NeuralNet):
    """The one-node net of the reference's node tests (node_check.py:103-118); with `gated`
    (an Epilogue) a GatedMul node follows the Linear, wired as vAi's gated feed-forward
    wires gateValue - gatedMul (vai/groups/gated-feed-forward.h:46)."""

    def __init__(self, make, slots, w_dtype=Dtype.F32, use_graph=True, gated=None, o_dtype=None, fuse=True):
        # every activation, output and workspace range sits between 512-byte canary zones
        super().__init__(w_default_dtype=w_dtype, use_graph=use_graph, fuse_gated_mul=fuse, guard_bytes=512)
        self.node = make()
        self.gm = None
        if gated is None:
            self.input(slots[0]) - slots[0] / self.node - self.output("out0")
        else:
            self.gm = nodes.GatedMulNode(activation=gated)
            if o_dtype is not None:
                self.gm.set_o_dtype(o_dtype)
            self.input(slots[0]) - slots[0] / self.node - self.gm - self.output("out0")
        for slot in slots[1:]:
            self.input(slot) - slot / self.node


def run_linear(x, w, bias=None, residual=None, *, i_dtype="f32", w_dtype="f32", o_dtype="f32", b_dtype=None,
               epilogue="NONE", residual_order="AFTER_EPILOGUE", scalar_scale=1.0, split_size=0, gate_fuse=False,
               kernel=0, use_graph=True, fuse=True, tuning=None):
    """Returns (out float32 array, expected float64 array, node).  gate_fuse=True builds
    Linear -> GatedMul(epilogue) and expects the net to record the pair as one launch
    (fuse=False keeps the two launches and the [M, 2H] intermediate in o_dtype)."""
    i_dt, w_dt, o_dt = DT[i_dtype], DT[w_dtype], DT[o_dtype]
    b_dt = DT[b_dtype] if b_dtype else w_dt
    N, K = w.shape
    slots = ["in0"] + (["residual"] if residual is not None else [])

    def make():
        n = nodes.LinearNode(in_dim=K, out_dim=N, accept_residual=residual is not None,
                             residual_order=getattr(ResidualOrder, residual_order),
                             epilogue=Epilogue.NONE if gate_fuse else getattr(Epilogue, epilogue),
                             scalar_scale=scalar_scale, split_size=split_size, kernel=kernel, tuning=tuning)
        n.set_o_dtype(o_dt)
        return n

    net = OneLinear(make, slots, w_dtype=w_dt, use_graph=use_graph, gated=getattr(Epilogue, epilogue) if gate_fuse else None,
                    o_dtype=o_dt, fuse=fuse)
    net.node["weight"] = Tensor.from_numpy(w, dtype=w_dt)
    if bias is not None:
        net.node["bias"] = Tensor.from_numpy(bias, dtype=b_dt)
    fed = {"in0": Tensor.from_numpy(x, dtype=i_dt)}
    if residual is not None:
        fed["residual"] = Tensor.from_numpy(residual, dtype=o_dt)
    out = net(**fed)
    got = out.to_numpy().astype(np.float32)
    if gate_fuse:
        assert net.node.gate_fuse == fuse and net.gm.fused == fuse, "the Linear -> GatedMul pair was not recorded as asked"
    again = net(**fed).to_numpy().astype(np.float32)
    np.testing.assert_array_equal(again, got, err_msg="the replayed forward differs from the first")
    assert net.pool.check_guards() >= 1      # the input, and every output or workspace larger than a host-mapped token
    # the expectation: float64 over the values the kernels read
    xs = seen(x, i_dt)
    if net.node.info.kernel in (nodes.KERNEL_TC_GEMM, nodes.KERNEL_TC_SKINNY) and i_dt == Dtype.F32:
        xs = seen(xs, w_dt)          # the cast pre-pass stages fp32 activations in the weights' type
    want = orc.linear_f64(xs, seen(w, w_dt), None if bias is None else seen(bias, b_dt),
                          None if residual is None else seen(residual, o_dt),
                          epilogue=orc.EPILOGUES[epilogue], residual_order=1 if residual_order == "BEFORE_EPILOGUE" else 0,
                          scalar_scale=scalar_scale, gate_fuse=gate_fuse)
    want = want.reshape(got.shape)
    return got, want, net.node


def out_tol(o_dtype, acc_rtol=1e-4, acc_atol=1e-5):
    """Accumulation tolerance plus one rounding of the output dtype."""
    if o_dtype == "f32":
        return (acc_rtol, acc_atol)
    ulp = 2.0 ** -11 if o_dtype == "f16" else 2.0 ** -8
    return (acc_rtol + ulp, acc_atol + 1e-6)
