"""GatedMul, the consumer of a gate|value Linear (vAi vai/nodes/gated-mul.h,
python/tests/nodes/test_gated_mul.py): out = activation(in0[..., :H]) * in0[..., H:].
This repository folds the node into the Linear's epilogue (gate_fuse), so the reference's
three cases are run through a Linear whose [2H, 2H] weight is the identity: the dot
products return in0 exactly and what is left is the gate arithmetic, compared with the
golden outputs at the reference's own tolerance for transcendental epilogues."""
import numpy as np
import pytest
from linear_check import assert_close, draw_case, load_golden

from oracle import linear_oracle as orc

META, ARRAYS = load_golden()
CASES = sorted(k for k in META if k.startswith("gated_mul"))


def test_all_reference_cases_present():
    assert CASES == ["gated_mul_GELU_TANH", "gated_mul_RELU", "gated_mul_SILU"]


@pytest.mark.parametrize("key", CASES)
def test_gate_epilogue_oracles_match_golden(key):
    cfg, _, fed = draw_case(META, key)
    x = fed["in0"]
    n = x.shape[-1]
    eye = np.eye(n, dtype=np.float32)
    code = orc.EPILOGUES[cfg["activation"]]
    np.testing.assert_allclose(orc.linear_f64(x, eye, epilogue=code, gate_fuse=True), ARRAYS[key], rtol=1e-12, atol=1e-12)
    d = orc.make_desc(x.shape[0], n, n, epilogue=code, gate_fuse=True)
    assert_close(orc.linear_c(d, x, eye), ARRAYS[key], tuple(META[key]["tol"]), key)


@pytest.mark.gpu
@pytest.mark.parametrize("key", CASES)
@pytest.mark.parametrize("kernel", ["auto", "fma"])
def test_gate_epilogue_on_gpu_matches_golden(key, kernel, device):
    from gpu_util import run_linear
    from vai_b200 import nodes
    cfg, _, fed = draw_case(META, key)
    x = fed["in0"]
    n = x.shape[-1]
    got, want, node = run_linear(x, np.eye(n, dtype=np.float32), epilogue=cfg["activation"], gate_fuse=True,
                                 kernel={"auto": nodes.KERNEL_AUTO, "fma": nodes.KERNEL_FMA_TILE}[kernel])
    assert got.shape == (4, n // 2)
    assert_close(got, ARRAYS[key], tuple(META[key]["tol"]), f"{key} {kernel}")
    assert_close(got, want, tuple(META[key]["tol"]), f"{key} {kernel} vs float64")
