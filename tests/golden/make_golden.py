"""Generate tests/golden/linear_golden.npz from the reference's own Linear tests.

Run once in a container that has the vAi source tree:

    python tests/golden/make_golden.py /path/to/vAi

The reference's tests (python/tests/nodes/test_linear.py, python/tests/node_check.py,
python/tests/test_nodes.py:28-41) cannot execute their GPU half here (the `pyvai`
extension needs Vulkan), but their seeded draw order and their float64 torch
reference functions are plain Python.  This script imports those two files with
a stand-in `pyvai` module, lets check_node() run, and records for every case:
the node's Config kwargs, the arrays it drew (as a SHA-256, they are re-drawn
from the seed by the tests) and the expected float64 output of the reference's
`ref` function.  Nothing of the reference's source is copied into the fixture.
"""
import hashlib
import json
import os
import sys
import types

import numpy as np


def _stub_pyvai():
    pyvai = types.ModuleType("pyvai")

    class _Names:
        def __init__(self, *names):
            for n in names:
                setattr(self, n, n)

    pyvai.Epilogue = _Names("NONE", "RELU", "GELU", "GELU_TANH", "SILU", "SIGMOID")
    pyvai.ResidualOrder = _Names("AFTER_EPILOGUE", "BEFORE_EPILOGUE")
    pyvai.Dtype = _Names("F32", "F16")
    pyvai.NeuralNet = object
    pyvai.Tensor = object
    nodes = types.ModuleType("pyvai.nodes")
    nodes.LinearNode = lambda **kw: dict(kw)
    nodes.ArgmaxNode = lambda **kw: {"node": "argmax", **kw}
    nodes.RmsNormNode = lambda **kw: {"node": "rms_norm", **kw}
    nodes.LayerNormNode = lambda **kw: {"node": "layer_norm", **kw}
    nodes.GatedMulNode = lambda **kw: {"node": "gated_mul", **kw}
    pyvai.nodes = nodes
    sys.modules["pyvai"] = pyvai
    sys.modules["pyvai.nodes"] = nodes


def main(ref_root):
    _stub_pyvai()
    sys.path.insert(0, os.path.join(ref_root, "python", "tests"))
    sys.path.insert(0, os.path.join(ref_root, "python", "tests", "nodes"))
    import node_check
    import test_argmax
    import test_gated_mul
    import test_layer_norm
    import test_rms_norm
    import test_linear

    records = {}
    arrays = {}
    state = {}

    def fake_net(make, slots, params):
        state["config"] = make()
        return None

    def fake_forward(net, fed, out):
        return np.zeros(1, dtype=np.float32)

    real_expected = node_check._expected

    def spy_expected(ref, fed, params):
        want = real_expected(ref, fed, params)
        state.setdefault("calls", []).append((fed, params, want))
        return want

    node_check._net = fake_net
    node_check._forward = fake_forward
    node_check._expected = spy_expected
    node_check._compare = lambda got, want, tol, out, what: state.setdefault("tols", []).append(tol)

    def digest(d):
        h = hashlib.sha256()
        for k in sorted(d):
            h.update(k.encode())
            h.update(np.ascontiguousarray(d[k], dtype=np.float32).tobytes())
        return h.hexdigest()

    def record(case_id):
        # Draw recipe (node_check.py:75-78, 92-93): one default_rng(0) stream; params
        # in dict order, then inputs in dict order, then the rerun's inputs. Every
        # array is standard normal except the weight, scaled by 1/sqrt(K)
        # (test_linear.py:30, 81).
        for i, (fed, params, want) in enumerate(state["calls"]):
            key = case_id if i == 0 else f"{case_id}__alt"
            tol = state["tols"][i]
            records[key] = {
                "config": state["config"],
                "param_order": list(params),
                "input_order": list(fed),
                "input_shapes": {k: list(v.shape) for k, v in fed.items()},
                "param_shapes": {k: list(v.shape) for k, v in params.items()},
                "inputs_sha256": digest(fed),
                "params_sha256": digest(params),
                "tol": list(tol),
                "rerun_of": None if i == 0 else case_id,
            }
            arrays[key] = np.asarray(want, dtype=np.float64)
        state.clear()

    for mark in test_linear.test_linear.pytestmark:
        if mark.name != "parametrize":
            continue
        for p in mark.args[1]:
            test_linear.test_linear(*p.values)
            record(f"linear_{p.id}")
    for mark in test_linear.test_linear_residual.pytestmark:
        if mark.name != "parametrize":
            continue
        for p in mark.args[1]:
            test_linear.test_linear_residual(*p.values)
            record(f"residual_{p.id}")

    # the lm_head's consumer: Argmax (python/tests/nodes/test_argmax.py), exact uint32 indices
    test_argmax.test_argmax()
    record("argmax")

    # the producer of a Linear's activations: RmsNorm (python/tests/nodes/test_rms_norm.py)
    for fn in ("test_rms_norm", "test_rms_norm_scale_shift_residual", "test_rms_norm_coeffs_as_inputs"):
        getattr(test_rms_norm, fn)()
        record(fn.replace("test_", ""))

    # GPT-2's producer: LayerNorm (python/tests/nodes/test_layer_norm.py)
    for fn in ("test_layer_norm_with_shift", "test_layer_norm_no_shift", "test_layer_norm_residual",
               "test_layer_norm_coeffs_as_inputs"):
        getattr(test_layer_norm, fn)()
        record(fn.replace("test_", ""))

    # the consumer of a gate|value Linear: GatedMul (python/tests/nodes/test_gated_mul.py); this
    # repository folds it into the Linear's epilogue (gate_fuse), so the cases pin that epilogue
    for mark in test_gated_mul.test_gated_mul.pytestmark:
        if mark.name != "parametrize":
            continue
        for activation in mark.args[1]:
            test_gated_mul.test_gated_mul(activation)
            record(f"gated_mul_{activation}")

    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "linear_golden.npz"), **arrays)
    with open(os.path.join(here, "linear_golden.json"), "w") as f:
        json.dump(records, f, indent=1, sort_keys=True)
    print(f"wrote {len(records)} cases")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/vAi")
    main(sys.argv[1])
