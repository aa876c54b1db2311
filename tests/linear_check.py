"""check_node() for this repo: the four checks of the reference's node tests
(vAi python/tests/node_check.py:1-12) against the committed golden outputs.

Draw recipe (node_check.py:75-78, 92-93): one np.random.default_rng(0) stream;
parameters in dict order, then inputs in dict order, then the rerun's inputs; the
weight is scaled by 1/sqrt(K), everything else is standard normal; all float32.
"""
import hashlib
import json
import os

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

FP32 = (1e-5, 1e-5)      # node_check.py:23
TRANS = (1e-4, 1e-5)     # node_check.py:24
FP16 = (1e-3, 5e-3)      # node_check.py:28
# Bounds this repo holds itself to: fp32 operands 1e-4 relative; 16-bit operands
# with fp32 accumulation 2e-2 relative against float64.
BOUND_FP32 = (1e-4, 1e-5)
BOUND_16 = (2e-2, 2e-2)


def load_golden():
    with open(os.path.join(GOLDEN_DIR, "linear_golden.json")) as f:
        meta = json.load(f)
    arrays = np.load(os.path.join(GOLDEN_DIR, "linear_golden.npz"))
    return meta, arrays


def digest(d):
    h = hashlib.sha256()
    for k in sorted(d):
        h.update(k.encode())
        h.update(np.ascontiguousarray(d[k], dtype=np.float32).tobytes())
    return h.hexdigest()


def draw_case(meta, key):
    """Re-draw the arrays of golden case `key`; returns (config, params, fed)."""
    rec = meta[key]
    base = meta[rec["rerun_of"]] if rec["rerun_of"] else rec
    rng = np.random.default_rng(0)
    k = base["config"].get("in_dim", 1)
    params = {}
    for slot in base["param_order"]:
        shape = tuple(base["param_shapes"][slot])
        scale = 1.0 / np.sqrt(k) if slot == "weight" else 1.0
        params[slot] = np.ascontiguousarray(scale * rng.standard_normal(shape), dtype=np.float32)
    fed = {slot: np.ascontiguousarray(rng.standard_normal(tuple(base["input_shapes"][slot])), dtype=np.float32)
           for slot in base["input_order"]}
    if rec["rerun_of"]:
        fed = {slot: np.ascontiguousarray(rng.standard_normal(tuple(rec["input_shapes"][slot])), dtype=np.float32)
               for slot in rec["input_order"]}
    assert digest(params) == rec["params_sha256"], "parameter draw differs from the fixture's"
    assert digest(fed) == rec["inputs_sha256"], "input draw differs from the fixture's"
    return rec["config"], params, fed


def assert_close(got, want, tol, what):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all(), f"{what}: NaN or Inf in the output"
    err = np.abs(got - want)
    lim = tol[1] + tol[0] * np.abs(want)
    bad = err > lim
    if bad.any():
        i = np.unravel_index(np.argmax(err - lim), err.shape)
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} elements off; worst at {i}: got {got[i]!r} want {want[i]!r} "
                             f"(rtol {tol[0]}, atol {tol[1]})")
