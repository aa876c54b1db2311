"""CPU: the C restatement (oracle/linear_oracle.c) and the float64 oracle against
the golden outputs generated from the reference's own test files."""
import numpy as np
import pytest
from linear_check import BOUND_FP32, FP16, FP32, assert_close, draw_case, load_golden

from oracle import linear_oracle as orc

ALL_META, ARRAYS = load_golden()
META = {k: v for k, v in ALL_META.items() if "in_dim" in v["config"]}   # the Linear cases


def _desc_and_arrays(cfg, params, fed):
    x = fed["in0"]
    M, K = x.shape
    N = cfg["out_dim"]
    bias = params.get("bias")
    res = fed.get("residual")
    d = orc.make_desc(M, N, K, b_dtype=orc.F32, bias_elems=bias.size if bias is not None else None,
                      residual_elems=res.size if res is not None else None,
                      residual_order=1 if cfg.get("residual_order") == "BEFORE_EPILOGUE" else 0,
                      epilogue=orc.EPILOGUES[cfg["epilogue"]], split_size=cfg.get("split_size", 0))
    return d, x, params["weight"], bias, res


@pytest.mark.parametrize("key", sorted(META))
def test_f64_oracle_reproduces_golden(key):
    cfg, params, fed = draw_case(META, key)
    got = orc.linear_f64(fed["in0"], params["weight"], params.get("bias"), fed.get("residual"),
                         epilogue=orc.EPILOGUES[cfg["epilogue"]],
                         residual_order=1 if cfg.get("residual_order") == "BEFORE_EPILOGUE" else 0)
    np.testing.assert_allclose(got, ARRAYS[key], rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("key", sorted(META))
def test_c_oracle_matches_golden(key):
    """fp32 operands: slab cases within the reference's FP32 tier, tile cases within
    1e-4 (the fp32 staging of linear-tile.comp, not the fp16 staging the FP16 tier
    allows for)."""
    cfg, params, fed = draw_case(META, key)
    d, x, w, b, r = _desc_and_arrays(cfg, params, fed)
    path = "slab" if d.M <= 8 else "tile"
    got = orc.linear_c(d, x, w, b, r, path=path, wg_size=128, stage16=False)
    assert_close(got, ARRAYS[key], FP32 if d.M <= 8 else BOUND_FP32, key)


@pytest.mark.parametrize("key", [k for k in sorted(META) if META[k]["input_shapes"]["in0"][0] > 8])
def test_c_oracle_fp16_staging_within_reference_tier(key):
    """The cooperative-matrix kernel's fp16 staging stays within the tier the
    reference grants it (node_check.py:25-28)."""
    cfg, params, fed = draw_case(META, key)
    d, x, w, b, r = _desc_and_arrays(cfg, params, fed)
    got = orc.linear_c(d, x, w, b, r, path="tile", stage16=True, stage_dtype=orc.F16)
    assert_close(got, ARRAYS[key], FP16, key)


def test_slab_workgroup_sizes_agree():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 1030)).astype(np.float32)
    w = (rng.standard_normal((17, 1030)) / 32).astype(np.float32)
    d = orc.make_desc(3, 17, 1030)
    a = orc.linear_c(d, x, w, path="slab", wg_size=32)
    b = orc.linear_c(d, x, w, path="slab", wg_size=128)
    assert_close(a, b, FP32, "slab wg 32 vs 128")
    assert_close(a, orc.linear_f64(x, w), FP32, "slab vs f64")


def test_conversions_match_numpy_and_torch():
    import torch
    rng = np.random.default_rng(1)
    a = np.concatenate([rng.standard_normal(4096).astype(np.float32) * s for s in (1e-6, 1e-3, 1.0, 1e3, 7e4)])
    a = np.concatenate([a, np.array([0.0, -0.0, np.inf, -np.inf, 65504.0, 65520.0, 6.1e-5, 6.0e-5, -3e-8], dtype=np.float32)])
    h = orc.to_dtype(a, orc.F16)
    with np.errstate(over="ignore"):
        ref = a.astype(np.float16)
    ref = np.where(np.abs(a) < 2.0 ** -14, np.copysign(np.float16(0), a).astype(np.float16), ref)   # tensor.cpp:66 flush
    np.testing.assert_array_equal(h, ref.view(np.uint16))
    np.testing.assert_array_equal(orc.to_f32(h, orc.F16), ref.astype(np.float32))
    b = orc.to_dtype(a, orc.BF16)
    tb = torch.from_numpy(a).to(torch.bfloat16)
    np.testing.assert_array_equal(b, tb.view(torch.int16).numpy().view(np.uint16))
    np.testing.assert_array_equal(orc.to_f32(b, orc.BF16), tb.float().numpy())


@pytest.mark.parametrize("name,code", sorted(orc.EPILOGUES.items()))
def test_epilogues_match_torch(name, code):
    """activation.h's fp32 functions against torch float64 (the table of node_check.py:31-38)."""
    import torch
    import torch.nn.functional as F
    table = {"NONE": lambda t: t, "RELU": F.relu, "GELU": F.gelu,
             "GELU_TANH": lambda t: F.gelu(t, approximate="tanh"), "SILU": F.silu, "SIGMOID": torch.sigmoid}
    xs = np.linspace(-12, 12, 4001).astype(np.float32)
    got = np.array([orc.lib().vai_oracle_epilogue(code, float(v)) for v in xs])
    want = table[name](torch.from_numpy(xs.astype(np.float64))).numpy()
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=2e-6)


def test_gated_oracle_matches_f64():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((4, 64)).astype(np.float32)
    w = (rng.standard_normal((96, 64)) / 8).astype(np.float32)
    d = orc.make_desc(4, 96, 64, epilogue=orc.EPILOGUES["SILU"], gate_fuse=True)
    got = orc.linear_c(d, x, w)
    want = orc.linear_f64(x, w, epilogue=4, gate_fuse=True)
    assert_close(got, want, (1e-4, 1e-5), "gated")
