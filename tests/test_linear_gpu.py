"""GPU parity: the CUDA kernels, through the public host API and the C ABI,
against the golden outputs of the reference's tests, the float64 oracle and the C
restatement of the shaders."""
import numpy as np
import pytest
from gpu_util import out_tol, run_linear, seen
from linear_check import BOUND_FP32, FP32, assert_close, draw_case, load_golden

from oracle import linear_oracle as orc
from vai_b200 import Dtype, nodes

pytestmark = pytest.mark.gpu

ALL_META, ARRAYS = load_golden()
META = {k: v for k, v in ALL_META.items() if "in_dim" in v["config"]}   # the Linear cases
PRIMARY = [k for k in sorted(META) if not META[k]["rerun_of"]]


def _kw(cfg):
    return dict(epilogue=cfg["epilogue"], residual_order=cfg.get("residual_order", "AFTER_EPILOGUE"),
                split_size=cfg.get("split_size", 0))


@pytest.mark.parametrize("key", sorted(META))
def test_reference_cases_fp32(key, device):
    """The reference's Linear cases (test_linear.py:11-27, 54-84) with fp32 weights,
    kernel chosen by shape: slab cases at the reference's FP32 tier, tile cases at
    1e-4 (fp32 staging, tighter than the FP16 tier the reference allows)."""
    cfg, params, fed = draw_case(META, key)
    got, want, node = run_linear(fed["in0"], params["weight"], params.get("bias"), fed.get("residual"), **_kw(cfg))
    M = fed["in0"].shape[0]
    assert node.info.kernel == (nodes.KERNEL_GEMV if M <= 8 else nodes.KERNEL_FMA_TILE)
    assert_close(got, ARRAYS[key], FP32 if M <= 8 else BOUND_FP32, key)
    assert_close(want, ARRAYS[key], (1e-12, 1e-12), key + " (oracle vs golden)")


@pytest.mark.parametrize("key", PRIMARY)
@pytest.mark.parametrize("kernel", ["fma", "tc", "skinny"])
@pytest.mark.parametrize("w_dtype", ["f16", "bf16"])
def test_reference_cases_16bit_weights(key, kernel, w_dtype, device):
    """Same cases with the weights stored in 16 bits (the deployment default is fp16,
    vAi neural-net.h:279), every kernel family forced in turn.  Against float64 over
    the stored values the only error left is fp32 accumulation."""
    cfg, params, fed = draw_case(META, key)
    K = cfg["in_dim"]
    kid = {"fma": nodes.KERNEL_FMA_TILE, "tc": nodes.KERNEL_TC_GEMM, "skinny": nodes.KERNEL_TC_SKINNY}[kernel]
    if kernel != "fma" and K % 8:
        pytest.skip("tensor-core path needs K % 8 == 0; the plan falls back (covered by the fma run)")
    got, want, node = run_linear(fed["in0"], params["weight"], params.get("bias"), fed.get("residual"),
                                 w_dtype=w_dtype, b_dtype="f32", kernel=kid, **_kw(cfg))
    assert node.info.kernel == kid
    assert_close(got, want, (1e-4, 2e-5), f"{key}/{kernel}/{w_dtype}")
    # and within the reference's own tier of the float64 result on unrounded operands
    golden_tol = (1e-3, 5e-3) if w_dtype == "f16" else (2e-2, 2e-2)
    assert_close(got, ARRAYS[key], golden_tol, f"{key}/{kernel}/{w_dtype} vs golden")


def test_identity_weight_plus_bias(device):
    """vAi python/tests/test_nodes.py:28-41: identity weight + bias, exact."""
    x = np.array([[1.0, 2.0, 3.0, 4.0]], dtype=np.float32)
    got, _, _ = run_linear(x, np.eye(4, dtype=np.float32), np.array([10.0, 20.0, 30.0, 40.0], dtype=np.float32))
    np.testing.assert_array_equal(got, [[11.0, 22.0, 33.0, 44.0]])


SHAPES = [
    # M, K, N
    (1, 2048, 512), (1, 768, 2304), (2, 1024, 300), (3, 512, 64), (4, 8192, 256), (5, 640, 130), (7, 264, 97),
    (8, 3072, 768), (1, 100, 33), (6, 101, 50),
]


@pytest.mark.parametrize("M,K,N", SHAPES)
@pytest.mark.parametrize("dt", [("f32", "f32", "f32"), ("f32", "f16", "f32"), ("bf16", "bf16", "bf16"),
                                ("f16", "f16", "f16"), ("f32", "bf16", "f32"), ("bf16", "bf16", "f32")])
def test_gemv_dtypes(M, K, N, dt, device):
    rng = np.random.default_rng(M * 1000 + K + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    r = rng.standard_normal((M, N)).astype(np.float32)
    got, want, node = run_linear(x, w, b, r, i_dtype=dt[0], w_dtype=dt[1], o_dtype=dt[2], epilogue="GELU_TANH",
                                 scalar_scale=0.5, kernel=nodes.KERNEL_GEMV)
    assert node.info.kernel == nodes.KERNEL_GEMV
    assert_close(got, want, out_tol(dt[2]), f"gemv {M}x{K}x{N} {dt}")


@pytest.mark.parametrize("M", [1, 2, 4, 5, 8])
@pytest.mark.parametrize("w_dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("act", ["SILU", "GELU_TANH", "RELU"])
def test_gemv_gate_fuse(M, w_dtype, act, device):
    """Linear + GatedMul in one pass against the two-node arithmetic
    (vAi nodes/test_gated_mul.py: TRANS tier)."""
    rng = np.random.default_rng(17 + M)
    K, H = 512, 328
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((2 * H, K)) / np.sqrt(K)).astype(np.float32)
    got, want, node = run_linear(x, w, w_dtype=w_dtype, epilogue=act, gate_fuse=True)
    assert got.shape == (M, H)
    assert_close(got, want, (1e-4, 1e-5), f"gate {M} {w_dtype} {act}")


GEMM_SHAPES = [
    # M, K, N: skinny and tiled, with ragged M / N / K-block tails
    (16, 256, 64), (33, 1000, 100), (64, 2560, 512), (100, 512, 384), (128, 768, 3072), (129, 320, 264),
    (300, 1024, 520), (1024, 768, 768), (200, 72, 40), (512, 4096, 256),
]


@pytest.mark.parametrize("M,K,N", GEMM_SHAPES)
@pytest.mark.parametrize("dt", [("f32", "f16", "f32"), ("bf16", "bf16", "bf16"), ("f16", "f16", "f32"),
                                ("f32", "bf16", "bf16")])
@pytest.mark.parametrize("kernel", ["auto", "tc", "skinny"])
def test_tensor_core_dtypes(M, K, N, dt, kernel, device):
    rng = np.random.default_rng(M + K + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    r = rng.standard_normal((M, N)).astype(np.float32)
    kid = {"auto": 0, "tc": nodes.KERNEL_TC_GEMM, "skinny": nodes.KERNEL_TC_SKINNY}[kernel]
    if kernel == "skinny" and M > 256:
        pytest.skip("skinny kernel is offered up to M = 256")
    got, want, node = run_linear(x, w, b, r, i_dtype=dt[0], w_dtype=dt[1], o_dtype=dt[2], epilogue="SILU",
                                 residual_order="BEFORE_EPILOGUE", kernel=kid)
    assert node.info.kernel in (nodes.KERNEL_TC_GEMM, nodes.KERNEL_TC_SKINNY)
    assert_close(got, want, out_tol(dt[2], 2e-4, 5e-5), f"tc {M}x{K}x{N} {dt} {kernel}")


@pytest.mark.parametrize("M,K,H", [(16, 512, 256), (64, 2560, 640), (200, 1024, 384), (1024, 512, 1000), (130, 264, 72)])
@pytest.mark.parametrize("kernel", ["auto", "tc", "skinny", "fma"])
@pytest.mark.parametrize("act", ["SILU", "GELU_TANH"])
def test_gemm_gate_fuse(M, K, H, kernel, act, device):
    rng = np.random.default_rng(M + K + H)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((2 * H, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(2 * H).astype(np.float32)
    kid = {"auto": 0, "tc": nodes.KERNEL_TC_GEMM, "skinny": nodes.KERNEL_TC_SKINNY, "fma": nodes.KERNEL_FMA_TILE}[kernel]
    if kernel == "skinny" and M > 256:
        pytest.skip("skinny kernel is offered up to M = 256")
    got, want, node = run_linear(x, w, b, i_dtype="bf16", w_dtype="bf16", o_dtype="bf16", b_dtype="bf16", epilogue=act,
                                 gate_fuse=True, kernel=kid)
    assert got.shape == (M, H)
    assert_close(got, want, out_tol("bf16", 2e-4, 5e-5), f"gate {M}x{K}x{H} {kernel} {act}")


@pytest.mark.parametrize("M,K,N,split", [(64, 4096, 128, 0), (16, 2050, 64, 0), (33, 1024, 48, 128), (256, 8192, 128, 0),
                                          (64, 10240, 2560, 0)])
@pytest.mark.parametrize("kernel", ["auto", "fma"])
def test_split_k(M, K, N, split, kernel, device):
    rng = np.random.default_rng(K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    kid = {"auto": 0, "fma": nodes.KERNEL_FMA_TILE}[kernel]
    got, want, node = run_linear(x, w, b, w_dtype="bf16", epilogue="RELU", split_size=split, kernel=kid)
    if split or (kernel == "auto" and K >= 4096 and K % 8 == 0):
        assert node.info.split_count > 1
    assert_close(got, want, (2e-4, 5e-5), f"split {M}x{K}x{N}")


def test_bias_table_and_residual_rows(device):
    """bias / residual as rows that repeat over M (vAi linear.h:2333-2338): a
    per-image [rows, N] table under a batch."""
    rng = np.random.default_rng(9)
    M, K, N, rows = 48, 128, 72, 12
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal((rows, N)).astype(np.float32)
    r = rng.standard_normal((rows * 2, N)).astype(np.float32)
    for w_dtype, kid in (("f32", 0), ("bf16", 0), ("bf16", nodes.KERNEL_TC_GEMM), ("bf16", nodes.KERNEL_FMA_TILE)):
        got, want, _ = run_linear(x, w, b, r, w_dtype=w_dtype, b_dtype="f32", epilogue="SIGMOID", kernel=kid)
        assert_close(got, want, (2e-4, 5e-5), f"tables {w_dtype} {kid}")
    got, want, _ = run_linear(x[:4], w, b[:4], r[:2], epilogue="SIGMOID")
    assert_close(got, want, (1e-5, 1e-5), "tables gemv")


@pytest.mark.parametrize("M,K,N", [(4, 1024, 512), (64, 512, 256), (256, 1024, 512)])
def test_cuda_matches_c_restatement(M, K, N, device):
    """CUDA path vs oracle/linear_oracle.c on the same seeded inputs (fp32, and fp16
    weights with the cooperative-matrix staging restated)."""
    rng = np.random.default_rng(M)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    d = orc.make_desc(M, N, K, b_dtype=orc.F32, bias_elems=N, epilogue=3)
    got, _, _ = run_linear(x, w, b, epilogue="GELU_TANH")
    assert_close(got, orc.linear_c(d, x, w, b), BOUND_FP32, "fp32 vs C")
    d16 = orc.make_desc(M, N, K, w_dtype=orc.F16, b_dtype=orc.F32, bias_elems=N, epilogue=3)
    got, _, _ = run_linear(x, w, b, w_dtype="f16", b_dtype="f32", epilogue="GELU_TANH")
    assert_close(got, orc.to_f32(orc.linear_c(d16, x, orc.to_dtype(w, orc.F16), b), orc.F32), (2e-4, 5e-5), "fp16 W vs C")


def test_scalar_scale_negative(device):
    """scalarScale = -1/steps as pi0's Euler step uses it (vAi models/production/pi0/net.h:154-159)."""
    rng = np.random.default_rng(2)
    x = rng.standard_normal((10, 64)).astype(np.float32)
    w = (rng.standard_normal((32, 64)) / 8).astype(np.float32)
    r = rng.standard_normal((10, 32)).astype(np.float32)
    got, want, _ = run_linear(x, w, None, r, scalar_scale=-0.1, epilogue="SILU", residual_order="BEFORE_EPILOGUE")
    assert_close(got, want, BOUND_FP32, "scale")


def test_chain_parallel_branches_match_serial(device):
    """Independent nodes of one level (q / k / v) recorded on side streams give the
    same logits as the one-stream recording, replayed or not."""
    import vai_b200
    from vai_b200 import Tensor, presets
    x = Tensor.from_numpy(np.random.default_rng(4).standard_normal((1, 2048), dtype=np.float32))
    outs = []
    for parallel, graph, grouped in ((False, True, False), (True, True, False), (True, False, False), (True, True, True),
                                     (False, False, True)):
        net = vai_b200.NeuralNet(w_default_dtype=Dtype.BF16, device=device, parallel_branches=parallel, use_graph=graph,
                                 group_siblings=grouped)
        presets.build_linear_chain(net, "llama-3.2-1b", layers=2, vocab_rows=4096, seed=7)
        a = net(x).to_numpy()
        b = net(x).to_numpy()
        np.testing.assert_array_equal(a, b)
        outs.append(a)
    assert np.isfinite(outs[0]).all() and np.abs(outs[0]).max() > 0
    for other in outs[1:]:
        np.testing.assert_array_equal(outs[0], other)


@pytest.mark.parametrize("M,K,w_dtype,expect", [(1, 512, "bf16", "gemv"), (4, 512, "bf16", "gemv"), (5, 512, "bf16", "skinny"),
                                                 (8, 512, "f16", "skinny"), (8, 512, "f32", "gemv"), (6, 500, "bf16", "gemv"),
                                                 (9, 512, "bf16", "skinny"), (200, 512, "bf16", "tc"), (9, 500, "bf16", "fma"),
                                                 (64, 512, "f32", "fma")])
def test_kernel_choice_by_shape(M, K, w_dtype, expect, device):
    """Plan selection (the place of Linear::prepare's slab / tile choice, vAi linear.h:2355,2395)."""
    rng = np.random.default_rng(M + K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((96, K)) / np.sqrt(K)).astype(np.float32)
    got, want, node = run_linear(x, w, w_dtype=w_dtype)
    ids = {"gemv": nodes.KERNEL_GEMV, "skinny": nodes.KERNEL_TC_SKINNY, "tc": nodes.KERNEL_TC_GEMM, "fma": nodes.KERNEL_FMA_TILE}
    assert node.info.kernel == ids[expect]
    assert_close(got, want, (2e-4, 5e-5), f"choice {M} {K} {w_dtype}")


@pytest.mark.parametrize("M,K,N", [(1300, 320, 520), (512, 1024, 256), (2048, 192, 1000)])
@pytest.mark.parametrize("gate", [False, True])
@pytest.mark.parametrize("mode,bn", [("wide", 256), ("pair", 256), ("pair", 192), ("pair", 128), ("pair", 64)])
def test_256_row_tiles(M, K, N, gate, mode, bn, device):
    """256-row tiles of the unswapped tensor-core kernel, forced on small shapes with
    ragged M, N and K tails, bias + residual, gate.  "wide": one CTA, two accumulators,
    one TMEM buffer.  "pair": two CTAs of a cluster share the tile through
    tcgen05.mma.cta_group::2, each staging half of the weights' rows."""
    tuning = dict(tc_pair=int(mode == "pair"), tc_wide=int(mode == "wide"), tc_bn=bn)
    rng = np.random.default_rng(M + N)
    rows = 2 * N if gate else N
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((rows, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(rows).astype(np.float32)
    r = None if gate else rng.standard_normal((M, N)).astype(np.float32)
    got, want, node = run_linear(x, w, b, r, i_dtype="bf16", w_dtype="bf16", o_dtype="f32", b_dtype="f32",
                                 epilogue="SILU", gate_fuse=gate, kernel=nodes.KERNEL_TC_GEMM, tuning=tuning)
    assert node.info.tile_m == 256 and node.info.tile_n == (bn // 2 if gate else bn)
    assert_close(got, want, (2e-4, 5e-5), f"{mode} {M}x{K}x{N} gate={gate} bn={bn}")


@pytest.mark.parametrize("w_dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("tuning", [dict(gemv_unroll=2), dict(gemv_unroll=4), dict(gemv_unroll=4, gemv_rows=2),
                                    dict(gemv_unroll=4, gemv_k_warps=4), dict(gemv_unroll=2, gemv_k_warps=8, gemv_grid=5),
                                    dict(gemv_unroll=4, gemv_grid=3)])
@pytest.mark.parametrize("variant", ["bias_res", "gate"])
def test_weight_streaming_geometries_at_batch_1(w_dtype, tuning, variant, device):
    """Both depths of the batch-1 weight-streaming kernel (two or four k-steps of weight vectors in flight
    per lane), with K splits over the warps and grids small enough that every block takes several tasks
    (the next task's first trip is then requested before the current task's sums are folded): ragged N and
    a K that leaves partial trips, bias + residual read ahead of the dot product, or the fused gate."""
    rng = np.random.default_rng(7 + len(w_dtype))
    K, N = 1096, 203
    gate = variant == "gate"
    rows = 2 * N if gate else N
    x = rng.standard_normal((1, K)).astype(np.float32)
    w = (rng.standard_normal((rows, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(rows).astype(np.float32)
    r = None if gate else rng.standard_normal((1, N)).astype(np.float32)
    got, want, node = run_linear(x, w, b, r, w_dtype=w_dtype, epilogue="SILU", gate_fuse=gate, residual_order="BEFORE_EPILOGUE" if not gate else "AFTER_EPILOGUE",
                                 scalar_scale=1.0 if gate else 0.5, kernel=nodes.KERNEL_GEMV, tuning=tuning)
    assert node.info.kernel == nodes.KERNEL_GEMV
    assert_close(got, want, (1e-5, 1e-5) if w_dtype == "f32" else (2e-4, 5e-5), f"{variant} {w_dtype} {tuning}")


def test_large_batch_1_layers_take_the_deeper_form(device):
    """A 32 MB layer at batch 1 is planned with four k-steps in flight (the planner's threshold is what the
    resident blocks request in one trip); the result is the same as with two, bit for bit, when K is split
    over the warps the same way."""
    rng = np.random.default_rng(3)
    K, N = 8192, 2048
    x = rng.standard_normal((1, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    r = rng.standard_normal((1, N)).astype(np.float32)
    auto, want, node = run_linear(x, w, None, r, w_dtype="bf16")
    assert node.info.kernel == nodes.KERNEL_GEMV
    assert_close(auto, want, (2e-4, 5e-5), "auto")
    four, _, _ = run_linear(x, w, None, r, w_dtype="bf16", tuning=dict(gemv_unroll=4, gemv_k_warps=4))
    two, _, _ = run_linear(x, w, None, r, w_dtype="bf16", tuning=dict(gemv_unroll=2, gemv_k_warps=4))
    np.testing.assert_array_equal(four, two)


@pytest.mark.parametrize("M", [9, 64, 100])
@pytest.mark.parametrize("rows,N,gate,splits", [(72, 1000, False, 0), (40, 520, True, 0), (8, 136, False, 0), (120, 777, True, 0),
                                                (56, 600, False, 3), (96, 264, True, 2)])
def test_short_weight_tiles_of_the_swapped_kernel(M, rows, N, gate, splits, device):
    """Weight tiles of fewer than 128 rows (tc_tile_rows) on the swapped tensor-core kernel: the copy fills
    `rows` rows of a 128-row slot, the MMA spans the slot, and the lanes past `rows` are never stored -
    every output row must come from exactly one tile.  Ragged N, bias + residual or the fused gate, with
    and without a K split."""
    rng = np.random.default_rng(M + rows + N)
    K = 576
    n_w = 2 * N if gate else N
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((n_w, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(n_w).astype(np.float32)
    r = None if gate else rng.standard_normal((M, N)).astype(np.float32)
    got, want, node = run_linear(x, w, b, r, i_dtype="bf16", w_dtype="bf16", o_dtype="f32", b_dtype="f32",
                                 epilogue="SILU", gate_fuse=gate, kernel=nodes.KERNEL_TC_SKINNY,
                                 tuning=dict(tc_tile_rows=rows, tc_splits=max(splits, 1)))
    assert node.info.tile_n == rows and node.info.split_count == max(splits, 1)
    assert_close(got, want, (2e-4, 5e-5), f"tile rows {rows} M={M} N={N} gate={gate} splits={splits}")
    # the same result, bit for bit, as full 128-row tiles: K is walked in the same order
    full, _, _ = run_linear(x, w, b, r, i_dtype="bf16", w_dtype="bf16", o_dtype="f32", b_dtype="f32",
                            epilogue="SILU", gate_fuse=gate, kernel=nodes.KERNEL_TC_SKINNY,
                            tuning=dict(tc_tile_rows=128, tc_splits=max(splits, 1)))
    np.testing.assert_array_equal(got, full)


def test_planner_spreads_a_layer_with_few_weight_tiles_over_the_sms(device):
    """A gate|value layer at batch 64 whose 128-row tiles would occupy a third of the SMs is planned with
    shorter tiles, one per SM, and without a K split."""
    rng = np.random.default_rng(5)
    H = 40 * device.sm_count
    x = rng.standard_normal((64, 256)).astype(np.float32)
    w = (rng.standard_normal((2 * H, 256)) / 16.0).astype(np.float32)
    got, want, node = run_linear(x, w, i_dtype="bf16", w_dtype="bf16", o_dtype="bf16", epilogue="GELU_TANH", gate_fuse=True)
    assert node.info.kernel == nodes.KERNEL_TC_SKINNY and node.info.split_count == 1
    assert node.info.tile_n == 40
    assert_close(got, want, (2e-2, 2e-2), "planned short tiles")


@pytest.mark.parametrize("M,K,N,splits", [(256, 4096, 256, 4), (520, 2048, 300, 3)])
def test_pair_tiles_split_k_match_single_cta(M, K, N, splits, device):
    """Split-K on CTA pairs (raw partials + fold) against the float64 expectation, and the
    unsplit pair kernel bit-identical to the single-CTA kernel (same order of K)."""
    rng = np.random.default_rng(K + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    got, want, node = run_linear(x, w, i_dtype="bf16", w_dtype="bf16", o_dtype="f32", kernel=nodes.KERNEL_TC_GEMM,
                                 tuning=dict(tc_pair=1, tc_splits=splits))
    assert node.info.split_count == splits and node.info.tile_m == 256
    assert_close(got, want, (2e-4, 5e-5), f"pair split-K {M}x{K}x{N}")
    one, _, _ = run_linear(x, w, i_dtype="bf16", w_dtype="bf16", o_dtype="f32", kernel=nodes.KERNEL_TC_GEMM,
                           tuning=dict(tc_pair=1, tc_splits=1))
    single, _, node = run_linear(x, w, i_dtype="bf16", w_dtype="bf16", o_dtype="f32", kernel=nodes.KERNEL_TC_GEMM,
                                 tuning=dict(tc_pair=0, tc_splits=1))
    assert node.info.tile_m == 128
    np.testing.assert_array_equal(one, single)


@pytest.mark.parametrize("M", [1, 3])
@pytest.mark.parametrize("w_dtype", ["bf16", "f32"])
def test_grouped_siblings_match_separate_runs(M, w_dtype, device):
    """vaicu_linear_run_group: q / k / v-like Linears with ragged row counts in one launch."""
    import ctypes

    from vai_b200 import _lib
    from vai_b200.engine import DeviceBuffer, encode
    from gpu_util import DT
    lib = device.lib
    rng = np.random.default_rng(M)
    K, rows = 512, [203, 64, 37]
    dt = DT[w_dtype]
    x = rng.standard_normal((M, K)).astype(np.float32)
    xb = DeviceBuffer(device, x.nbytes)
    xb.upload(x)
    plans, wbufs, obufs, wants = [], [], [], []
    for n in rows:
        w = (rng.standard_normal((n, K)) / np.sqrt(K)).astype(np.float32)
        wb = DeviceBuffer(device, n * K * (4 if w_dtype == "f32" else 2))
        wb.upload(encode(w, dt))
        d = _lib.LinearDesc()
        d.M, d.N, d.K = M, n, K
        d.i_dtype, d.w_dtype, d.o_dtype, d.b_dtype = 0, int(dt), 0, 2
        d.scalar_scale = 1.0
        h = ctypes.c_void_p()
        _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(h)), "plan")
        plans.append(h)
        wbufs.append(wb)
        obufs.append(DeviceBuffer(device, M * n * 4))
        wants.append(orc.linear_f64(x, seen(w, dt)))
    n = len(rows)
    _lib.check(lib.vaicu_linear_run_group((ctypes.c_void_p * n)(*plans), n, None, xb.ptr,
                                          (ctypes.c_void_p * n)(*[b.ptr for b in wbufs]),
                                          (ctypes.c_void_p * n)(*[b.ptr for b in obufs]), None), "group")
    device.synchronize()
    for nrows, ob, want in zip(rows, obufs, wants):
        got = ob.download(np.empty((M, nrows), dtype=np.float32))
        assert_close(got, want, (1e-5, 1e-5), f"group {nrows}")
    # a Linear with an epilogue cannot join a group
    d.epilogue = 1
    h = ctypes.c_void_p()
    _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(h)), "plan")
    rc = lib.vaicu_linear_run_group((ctypes.c_void_p * 2)(plans[0], h), 2, None, xb.ptr,
                                    (ctypes.c_void_p * 2)(wbufs[0].ptr, wbufs[2].ptr), (ctypes.c_void_p * 2)(obufs[0].ptr, obufs[2].ptr), None)
    assert rc == 2


@pytest.mark.parametrize("M,K,rows,i_dtype,o_dtype,splits", [
    (64, 2560, [2048, 1024, 1024], "bf16", "bf16", 0),      # Gemma-3-4B q / k / v
    (64, 512, [256, 128], "bf16", "f32", 0),
    (100, 1024, [128, 384, 128], "f32", "f16", 0),          # fp32 activations: rounded once for the group
    (16, 320, [128, 128, 256], "f16", "f16", 1),            # one split: the fold still stores the outputs
    (128, 2048, [1280, 256, 256], "bf16", "bf16", 5),
])
def test_grouped_siblings_on_the_tensor_core_kernel(M, K, rows, i_dtype, o_dtype, splits, device):
    """vaicu_linear_run_group for 8 < M <= 128: one swapped GEMM over the members' weight rows side by
    side and one fold, bit-identical to the members' own runs when those split K the same way, and
    within the 16-bit bounds of float64 otherwise."""
    import ctypes

    from vai_b200 import _lib
    from vai_b200.engine import DeviceBuffer, bits_to_f32, encode
    from gpu_util import DT
    lib = device.lib
    rng = np.random.default_rng(M + K)
    w_dtype = "bf16" if i_dtype == "f32" else i_dtype
    dt, it, ot = DT[w_dtype], DT[i_dtype], DT[o_dtype]
    x = rng.standard_normal((M, K)).astype(np.float32)
    xb = DeviceBuffer(device, M * K * (4 if i_dtype == "f32" else 2))
    xb.upload(encode(x, it))
    xs = seen(seen(x, it), dt)
    plans, wbufs, obufs, wants, singles = [], [], [], [], []
    for n in rows:
        w = (rng.standard_normal((n, K)) / np.sqrt(K)).astype(np.float32)
        wb = DeviceBuffer(device, n * K * 2)
        wb.upload(encode(w, dt))
        d = _lib.LinearDesc()
        d.M, d.N, d.K = M, n, K
        d.i_dtype, d.w_dtype, d.o_dtype, d.b_dtype = int(it), int(dt), int(ot), 2
        d.scalar_scale = 1.0
        h = ctypes.c_void_p()
        t = _lib.LinearTuning(tc_splits=splits)
        _lib.check(lib.vaicu_linear_plan_create_tuned(device.handle, ctypes.byref(d), ctypes.byref(t), ctypes.byref(h)), "plan")
        info = _lib.LinearInfo()
        _lib.check(lib.vaicu_linear_plan_info(h, ctypes.byref(info)), "info")
        assert info.kernel == 4
        plans.append(h)
        wbufs.append(wb)
        osz = 4 if o_dtype == "f32" else 2
        obufs.append(DeviceBuffer(device, M * n * osz))
        wants.append(orc.linear_f64(xs, seen(w, dt)))
        if splits:
            # the member alone, same K split: the same partial sums in the same order
            ws1 = DeviceBuffer(device, max(int(info.workspace_bytes), 256))
            o1 = DeviceBuffer(device, M * n * osz)
            _lib.check(lib.vaicu_linear_run(h, None, xb.ptr, wb.ptr, None, None, o1.ptr, ws1.ptr), "run")
            device.synchronize()
            singles.append(o1.download(np.empty((M, n), dtype=np.float32 if o_dtype == "f32" else np.uint16)))
    n = len(rows)
    parr = (ctypes.c_void_p * n)(*plans)
    need = ctypes.c_size_t()
    _lib.check(lib.vaicu_linear_group_workspace_bytes(parr, n, ctypes.byref(need)), "group workspace")
    # room for the rounded activations (fp32 input) and for the partial sums, unless the K splits fold inside clusters
    cast_bytes = -(-M * K * 2 // 256) * 256 if i_dtype == "f32" else 0
    assert need.value >= cast_bytes and (need.value > cast_bytes or splits == 0)
    guard = 512
    ws = DeviceBuffer(device, need.value + 2 * guard)
    _lib.check(lib.vaicu_memset(ws.ptr, 0xA5, need.value + 2 * guard, None), "memset")
    warr = (ctypes.c_void_p * n)(*[b.ptr for b in wbufs])
    oarr = (ctypes.c_void_p * n)(*[b.ptr for b in obufs])
    if need.value:
        # without a workspace the call is refused before anything is launched
        assert lib.vaicu_linear_run_group(parr, n, None, xb.ptr, warr, oarr, None) != 0
    for _ in range(2):          # the second call reuses the cached descriptors
        _lib.check(lib.vaicu_linear_run_group(parr, n, None, xb.ptr, warr, oarr, ws.ptr + guard if need.value else None), "group")
    device.synchronize()
    device.check_status()
    edge = ws.download(np.empty(need.value + 2 * guard, dtype=np.uint8))
    assert (edge[:guard] == 0xA5).all() and (edge[-guard:] == 0xA5).all()
    tol = (1e-4, 1e-4) if o_dtype == "f32" else (2e-2, 2e-2)
    for i, (nrows, ob, want) in enumerate(zip(rows, obufs, wants)):
        raw = ob.download(np.empty((M, nrows), dtype=np.float32 if o_dtype == "f32" else np.uint16))
        got = raw if o_dtype == "f32" else bits_to_f32(raw, ot)
        assert_close(got, want, tol, f"group member {i}")
        if splits:
            np.testing.assert_array_equal(raw, singles[i])
    # members that are not whole weight tiles are declined
    d.N = 200
    h = ctypes.c_void_p()
    _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(h)), "plan")
    assert lib.vaicu_linear_group_workspace_bytes((ctypes.c_void_p * 2)(plans[0], h), 2, ctypes.byref(need)) == 2


@pytest.mark.parametrize("M,K,rows,o_dtype", [(300, 512, [512, 256, 256], "bf16"), (1024, 320, [768, 256], "f32"), (2600, 192, [256, 256, 1024], "f16")])
def test_grouped_siblings_on_the_cta_pair_kernel(M, K, rows, o_dtype, device):
    """vaicu_linear_run_group for M > 128: one CTA-pair GEMM over the members' 256-column tiles, each tile stored
    to its member; no workspace; bit-identical to the members' own runs (same tiles, same order of K) and within the
    16-bit bounds of float64."""
    import ctypes

    from vai_b200 import _lib
    from vai_b200.engine import DeviceBuffer, bits_to_f32, encode
    from gpu_util import DT
    lib = device.lib
    rng = np.random.default_rng(M + K)
    w_dtype = "f16" if o_dtype == "f16" else "bf16"
    dt, ot = DT[w_dtype], DT[o_dtype]
    x = rng.standard_normal((M, K)).astype(np.float32)
    xb = DeviceBuffer(device, M * K * 2)
    xb.upload(encode(x, dt))
    xs = seen(x, dt)
    osz = 4 if o_dtype == "f32" else 2
    plans, wbufs, obufs, wants, singles = [], [], [], [], []
    for n in rows:
        w = (rng.standard_normal((n, K)) / np.sqrt(K)).astype(np.float32)
        wb = DeviceBuffer(device, n * K * 2)
        wb.upload(encode(w, dt))
        d = _lib.LinearDesc()
        d.M, d.N, d.K = M, n, K
        d.i_dtype, d.w_dtype, d.o_dtype, d.b_dtype = int(dt), int(dt), int(ot), 2
        d.scalar_scale = 1.0
        h = ctypes.c_void_p()
        t = _lib.LinearTuning(tc_splits=1)          # one K span, as in the group: the same order of addition
        _lib.check(lib.vaicu_linear_plan_create_tuned(device.handle, ctypes.byref(d), ctypes.byref(t), ctypes.byref(h)), "plan")
        info = _lib.LinearInfo()
        _lib.check(lib.vaicu_linear_plan_info(h, ctypes.byref(info)), "info")
        assert info.kernel == 3
        plans.append(h)
        wbufs.append(wb)
        obufs.append(DeviceBuffer(device, M * n * osz + 512))
        _lib.check(lib.vaicu_memset(obufs[-1].ptr, 0x5A, M * n * osz + 512, None), "memset")
        wants.append(orc.linear_f64(xs, seen(w, dt)))
        ws1 = DeviceBuffer(device, max(int(info.workspace_bytes), 256))
        o1 = DeviceBuffer(device, M * n * osz)
        _lib.check(lib.vaicu_linear_run(h, None, xb.ptr, wb.ptr, None, None, o1.ptr, ws1.ptr), "run")
        device.synchronize()
        singles.append(o1.download(np.empty((M, n), dtype=np.float32 if o_dtype == "f32" else np.uint16)))
    n = len(rows)
    parr = (ctypes.c_void_p * n)(*plans)
    need = ctypes.c_size_t(7)
    _lib.check(lib.vaicu_linear_group_workspace_bytes(parr, n, ctypes.byref(need)), "group workspace")
    assert need.value == 0
    warr = (ctypes.c_void_p * n)(*[b.ptr for b in wbufs])
    oarr = (ctypes.c_void_p * n)(*[b.ptr for b in obufs])
    for _ in range(2):
        _lib.check(lib.vaicu_linear_run_group(parr, n, None, xb.ptr, warr, oarr, None), "group")
    device.synchronize()
    device.check_status()
    tol = (1e-4, 1e-4) if o_dtype == "f32" else (2e-2, 2e-2)
    for i, (nrows, ob, want) in enumerate(zip(rows, obufs, wants)):
        raw8 = ob.download(np.empty(M * nrows * osz + 512, dtype=np.uint8))
        assert (raw8[M * nrows * osz:] == 0x5A).all()
        raw = raw8[:M * nrows * osz].view(np.float32 if o_dtype == "f32" else np.uint16).reshape(M, nrows)
        got = raw if o_dtype == "f32" else bits_to_f32(raw, ot)
        assert_close(got, want, tol, f"pair group member {i}")
        np.testing.assert_array_equal(raw, singles[i])


@pytest.mark.parametrize("M,K,N,gate", [(64, 512, 384, False), (33, 256, 200, False), (300, 512, 520, False), (64, 512, 256, True)])
def test_scatter_run_writes_slabs_into_wider_outputs(M, K, N, gate, device):
    """vaicu_linear_run_scatter on one GPU: the plan's output lands as a column slab at col0
    inside two wider buffers (what a column-split rank does to its own and its peers'
    outputs), bit-identical to the dense run, and nothing outside the slab is touched."""
    import ctypes

    from vai_b200 import _lib
    from vai_b200.engine import DeviceBuffer, encode
    from vai_b200 import Dtype
    lib = device.lib
    rng = np.random.default_rng(M + N)
    rows = 2 * N if gate else N
    x = encode(rng.standard_normal((M, K)).astype(np.float32), Dtype.BF16)
    w = encode((rng.standard_normal((rows, K)) / np.sqrt(K)).astype(np.float32), Dtype.BF16)
    xb, wb = DeviceBuffer(device, x.nbytes), DeviceBuffer(device, w.nbytes)
    xb.upload(x)
    wb.upload(w)
    d = _lib.LinearDesc()
    d.M, d.N, d.K = M, rows, K
    d.i_dtype = d.w_dtype = d.o_dtype = int(Dtype.BF16)
    d.b_dtype = 2
    d.scalar_scale = 1.0
    d.gate_fuse = 1 if gate else 0
    d.epilogue = 4 if gate else 0
    d.split_size = 0
    plan = ctypes.c_void_p()
    _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(plan)), "plan")
    info = _lib.LinearInfo()
    lib.vaicu_linear_plan_info(plan, ctypes.byref(info))
    ws = DeviceBuffer(device, max(info.workspace_bytes, 256))
    dense = DeviceBuffer(device, M * N * 2)
    _lib.check(lib.vaicu_linear_run(plan, None, xb.ptr, wb.ptr, None, None, dense.ptr, ws.ptr), "run")
    ldo, col0 = N + 3 * 16 + 8, 24              # col0 keeps 16-byte alignment of the rows only when ldo does too
    wide = [DeviceBuffer(device, M * ldo * 2) for _ in range(2)]
    canary = np.full((M, ldo), 0x7FC1, dtype=np.uint16)
    for b in wide:
        b.upload(canary)
    ptrs = (ctypes.c_void_p * 2)(wide[0].ptr, wide[1].ptr)
    rc = lib.vaicu_linear_run_scatter(plan, None, xb.ptr, wb.ptr, None, ptrs, 2, ldo, col0, ws.ptr)
    if info.split_count > 1:
        assert rc == 2          # plans with a split-K fold do not scatter
        return
    _lib.check(rc, "scatter")
    device.synchronize()
    want = dense.download(np.empty((M, N), dtype=np.uint16))
    for b in wide:
        got = b.download(np.empty((M, ldo), dtype=np.uint16))
        np.testing.assert_array_equal(got[:, col0:col0 + N], want)
        np.testing.assert_array_equal(got[:, :col0], canary[:, :col0])
        np.testing.assert_array_equal(got[:, col0 + N:], canary[:, col0 + N:])


@pytest.mark.parametrize("rows,K,N", [(160, 512, 520), (48, 256, 264), (256, 320, 1000)])
def test_broadcast_run_assembles_row_blocks_with_residual(rows, K, N, device):
    """vaicu_linear_run_broadcast on one GPU: two "ranks" run the same Linear (bias, residual, scale) on their
    own rows of the activations and each writes its block of rows into BOTH full-height outputs (what the o
    projection of a sequence-parallel block does to its own and its peers' hidden state); the assembled
    outputs equal the dense run over all rows, bit for bit."""
    import ctypes

    from vai_b200 import _lib
    from vai_b200.engine import DeviceBuffer, encode
    from vai_b200 import Dtype
    lib = device.lib
    rng = np.random.default_rng(rows + N)
    M = 2 * rows
    x = encode(rng.standard_normal((M, K)).astype(np.float32), Dtype.BF16)
    w = encode((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32), Dtype.BF16)
    b = encode(rng.standard_normal(N).astype(np.float32), Dtype.BF16)
    r = encode(rng.standard_normal((M, N)).astype(np.float32), Dtype.BF16)
    bufs = {}
    for name, arr in (("x", x), ("w", w), ("b", b), ("r", r)):
        bufs[name] = DeviceBuffer(device, arr.nbytes)
        bufs[name].upload(arr)

    def plan_for(m):
        d = _lib.LinearDesc()
        d.M, d.N, d.K = m, N, K
        d.i_dtype = d.w_dtype = d.o_dtype = d.b_dtype = int(Dtype.BF16)
        d.has_bias, d.bias_elems, d.has_residual = 1, N, 1
        d.scalar_scale = 0.5
        d.split_size = max(32, K)          # one K span: the outputs leave through the GEMM's epilogue
        h = ctypes.c_void_p()
        _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(h)), "plan")
        info = _lib.LinearInfo()
        lib.vaicu_linear_plan_info(h, ctypes.byref(info))
        return h, DeviceBuffer(device, max(info.workspace_bytes, 256))

    whole, ws_whole = plan_for(M)
    dense = DeviceBuffer(device, M * N * 2)
    _lib.check(lib.vaicu_linear_run(whole, None, bufs["x"].ptr, bufs["w"].ptr, bufs["b"].ptr, bufs["r"].ptr, dense.ptr, ws_whole.ptr), "run")
    part, ws_part = plan_for(rows)
    outs = [DeviceBuffer(device, M * N * 2 + 512) for _ in range(2)]
    for o in outs:
        _lib.check(lib.vaicu_memset(o.ptr, 0xC3, M * N * 2 + 512, None), "memset")
    for rank in range(2):
        off = rank * rows
        dsts = (ctypes.c_void_p * 2)(*[o.ptr + off * N * 2 for o in outs])
        _lib.check(lib.vaicu_linear_run_broadcast(part, None, bufs["x"].ptr + off * K * 2, bufs["w"].ptr, bufs["b"].ptr,
                                                  bufs["r"].ptr + off * N * 2, dsts, 2, ws_part.ptr), "broadcast")
    device.synchronize()
    device.check_status()
    want = dense.download(np.empty((M, N), dtype=np.uint16))
    for o in outs:
        raw = o.download(np.empty(M * N + 256, dtype=np.uint16))
        np.testing.assert_array_equal(raw[:M * N].reshape(M, N), want)
        assert (raw[M * N:] == 0xC3C3).all()
    # a plan that folds K splits in a second launch cannot broadcast
    d = _lib.LinearDesc()
    d.M, d.N, d.K = 64, 128, 4096
    d.i_dtype = d.w_dtype = d.o_dtype = int(Dtype.BF16)
    d.b_dtype, d.scalar_scale = 2, 1.0
    h = ctypes.c_void_p()
    _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(h)), "plan")
    info = _lib.LinearInfo()
    lib.vaicu_linear_plan_info(h, ctypes.byref(info))
    if info.split_count > 1:
        assert lib.vaicu_linear_run_broadcast(h, None, bufs["x"].ptr, bufs["w"].ptr, None, None, (ctypes.c_void_p * 1)(outs[0].ptr), 1, ws_part.ptr) == 2


def test_config_1_gpt2_mlp_linear_fp32(device):
    """The single-node configuration of the benchmark list at its exact size: X [128, 768] fp32
    ~N(0, 1) seed 0, W [3072, 768] fp32 ~N(0, 0.02), bias ~N(0, 0.02), fused GELU(tanh), output
    [128, 3072] fp32 (GPT-2 small's fc1, vAi models/production/gpt2/net.h:51).  fp32 operands keep
    the exact fp32 kernel; bound: |got - ref| <= 1e-4 * max(|ref|, 0.1) against float64."""
    import torch
    def draw(seed, shape, std):
        g = torch.Generator(device="cpu").manual_seed(seed)
        return (torch.randn(shape, generator=g, dtype=torch.float32) * std).numpy()
    x, w, b = draw(0, (128, 768), 1.0), draw(1, (3072, 768), 0.02), draw(2, (3072,), 0.02)
    got, want, node = run_linear(x, w, b, epilogue="GELU_TANH")
    assert node.info.kernel == nodes.KERNEL_FMA_TILE and got.shape == (128, 3072)
    rel = np.abs(got - want) / np.maximum(np.abs(want), 0.1)
    assert rel.max() <= 1e-4, f"worst relative error {rel.max():.3g}"
    # the C restatement of the reference's scalar tile shader on the same operands
    d = orc.make_desc(128, 3072, 768, b_dtype=orc.F32, bias_elems=3072, epilogue=3)
    assert_close(got, orc.linear_c(d, x, w, b), BOUND_FP32, "config 1 vs the shader restatement")


@pytest.mark.parametrize("M,K,N,kernel", [(64, 10240, 2560, "skinny"), (64, 2560, 2048, "skinny"), (33, 4096, 200, "skinny"),
                                          (128, 4096, 136, "skinny"), (100, 8192, 96, "tc1"), (300, 4096, 264, "tc1")])
@pytest.mark.parametrize("variant", ["plain", "bias_res_gelu", "gate"])
def test_split_k_folded_inside_the_kernel(M, K, N, kernel, variant, device):
    """Split-K on the single-CTA tensor-core kernels without a second launch (an option,
    vaicu_linear_tuning.tc_fold = 1; the default is a dependent fold launch): the CTAs that hold a
    tile's splits publish their partial sums, wait (bounded) for each other, and each folds a slice
    of the tile in split order with bias / epilogue / residual.  Against float64, and bit for bit
    against the same plan with the separate fold launch (same partial sums, same order of addition,
    same epilogue code); replayed through one recording, so the per-tile counters have to come
    back to zero."""
    rng = np.random.default_rng(M + K + N)
    gate = variant == "gate"
    rows = 2 * N if gate else N
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((rows, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(rows).astype(np.float32) if variant != "plain" else None
    r = rng.standard_normal((M, N)).astype(np.float32) if variant == "bias_res_gelu" else None
    kid = nodes.KERNEL_TC_SKINNY if kernel == "skinny" else nodes.KERNEL_TC_GEMM
    base = dict(tc_pair=0) if kernel == "tc1" else {}
    kw = dict(i_dtype="bf16", w_dtype="bf16", o_dtype="bf16" if variant == "plain" else "f32", b_dtype="f32",
              epilogue="GELU_TANH" if variant != "plain" else "NONE", gate_fuse=gate, kernel=kid)
    got, want, node = run_linear(x, w, b, r, tuning=dict(base, tc_splits=4, tc_fold=1), **kw)
    assert node.info.split_count == 4 and node.info.launches == 1
    assert_close(got, want, out_tol(kw["o_dtype"], 2e-4, 5e-5), f"fold {M}x{K}x{N} {variant}")
    two, _, node2 = run_linear(x, w, b, r, tuning=dict(base, tc_splits=4, tc_fold=2), **kw)
    assert node2.info.split_count == 4 and node2.info.launches == 2
    np.testing.assert_array_equal(got, two)


@pytest.mark.parametrize("M,K,N,S", [(64, 2048, 2560, 4), (64, 2560, 2048, 2), (32, 4096, 200, 2), (128, 4096, 136, 8),
                                     (128, 2048, 520, 4), (90, 1024, 1000, 2), (17, 1536, 264, 2)])
@pytest.mark.parametrize("variant", ["plain", "bias_res_gelu"])
def test_split_k_folded_inside_clusters(M, K, N, S, variant, device):
    """Split-K of the swapped tensor-core kernel with the S splits of a tile as one cluster
    (vaicu_linear_tuning.tc_fold = 3): the accumulators cross through distributed shared memory, each
    CTA finishes bn / S activation rows, in one launch.  Against float64, and bit for bit
    against the same K split folded by the second launch (same partial sums added in the same order, same
    epilogue code) for the plain case; replayed through one recording."""
    rng = np.random.default_rng(M + K + N + S)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32) if variant != "plain" else None
    r = rng.standard_normal((M, N)).astype(np.float32) if variant != "plain" else None
    kw = dict(i_dtype="bf16", w_dtype="bf16", o_dtype="bf16" if variant == "plain" else "f32", b_dtype="f32",
              epilogue="GELU_TANH" if variant != "plain" else "NONE", kernel=nodes.KERNEL_TC_SKINNY)
    got, want, node = run_linear(x, w, b, r, tuning=dict(tc_splits=S, tc_fold=3), **kw)
    assert node.info.split_count == S and node.info.launches == 1
    assert_close(got, want, out_tol(kw["o_dtype"], 2e-4, 5e-5), f"cluster fold {M}x{K}x{N} S={S} {variant}")
    two, _, node2 = run_linear(x, w, b, r, tuning=dict(tc_splits=S, tc_fold=2), **kw)
    assert node2.info.split_count == S and node2.info.launches == 2
    if variant == "plain":
        np.testing.assert_array_equal(got, two)
    else:
        # same sums; the GEMM epilogue and the fold kernel evaluate GELU with differently ordered fp32 operations
        np.testing.assert_allclose(got, two, rtol=1e-5, atol=2e-6)


@pytest.mark.parametrize("M,K,N,gate,residual", [(2560, 256, 2048, False, True), (2560, 320, 2048, True, False), (2600, 192, 2000, False, False)])
@pytest.mark.parametrize("strips", [0, 2, 4])
def test_tail_round_in_column_strips(M, K, N, gate, residual, strips, device):
    """CTA-pair kernel when the tile count leaves a partial last round (80 tiles of 256 x 256 on 74
    clusters here): the leftover tiles are cut into column strips of 128 or 64, one work item each.
    Same dot products in the same order as whole tiles, so the outputs equal the unstripped run bit for
    bit; against float64 as well.  With a residual, whose chunks the epilogue requests ahead of use."""
    rng = np.random.default_rng(M + N + strips)
    rows = 2 * N if gate else N
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((rows, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(rows).astype(np.float32)
    r = rng.standard_normal((M, N)).astype(np.float32) if residual else None
    kw = dict(i_dtype="bf16", w_dtype="bf16", o_dtype="bf16" if residual else "f32", b_dtype="f32", epilogue="SILU", gate_fuse=gate,
              kernel=nodes.KERNEL_TC_GEMM)
    got, want, node = run_linear(x, w, b, r, tuning=dict(tc_pair=1, tc_bn=256, tc_tail_strips=strips), **kw)
    assert node.info.tile_m == 256
    assert_close(got, want, out_tol(kw["o_dtype"], 2e-4, 5e-5), f"strips {strips} {M}x{K}x{N}")
    whole, _, _ = run_linear(x, w, b, r, tuning=dict(tc_pair=1, tc_bn=256, tc_tail_strips=1), **kw)
    np.testing.assert_array_equal(got, whole)
