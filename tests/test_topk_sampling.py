"""TopKSampling, the sampling consumer of the lm_head Linear (vAi vai/nodes/topk-sampling.h,
vai/shaders/topk-sampling.comp).  The reference ships no test or golden vector for this node,
so the C restatement of the shader is checked against an independent float64 formulation of
the same distribution (parity unpinned), and the CUDA node against the restatement, exactly:
the sample is an index.  Two anchors to the reference do exist and are checked here: with k = 1 the
node returns the golden output of the reference's Argmax test, and equal logits rank by index.  The
vocabulary-split form (candidates per slab with the slab's offset, then merge + sample) must return
the same token as the node over the whole row."""
import numpy as np
import pytest

from oracle import linear_oracle as orc

US = [0.0, 0.013, 0.25, 0.5, 0.77, 0.93, 0.9990234]


def _expected_from_f64(x, k, temperature, u):
    """Index by float64 CDF lookup, or None where u * Z falls within rounding of a CDF step."""
    idx, p = orc.topk_probabilities_f64(x, k, temperature)
    cdf = np.cumsum(p, axis=1)
    out = []
    for r in range(x.shape[0]):
        j = int(np.searchsorted(cdf[r], u, side="left"))
        j = min(j, idx.shape[1] - 1)
        near = np.abs(cdf[r] - u).min() < 1e-5
        out.append(None if near else int(idx[r, j]))
    return out


@pytest.mark.parametrize("k,temperature", [(40, 1.0), (5, 0.7), (128, 1.5), (1, 1.0)])
def test_oracle_samples_the_float64_distribution(k, temperature):
    rng = np.random.default_rng(k)
    x = (rng.standard_normal((4, 3000)) * 2).astype(np.float32)
    for u in US:
        got = orc.topk_sample_c(x, k, temperature, u)
        for r, want in enumerate(_expected_from_f64(x, k, temperature, u)):
            if want is not None:
                assert int(got[r]) == want, (k, temperature, u, r)


def test_oracle_edge_rules():
    x = np.zeros((2, 20), dtype=np.float32)
    x[0, [3, 11, 7]] = 5.0                          # equal logits rank by index: 3, 7, 11
    x[1, 4] = 1.0
    assert list(orc.topk_sample_c(x, 3, 1.0, 0.0)) == [3, 4]
    assert int(orc.topk_sample_c(x, 3, 1.0, 0.5)[0]) == 7          # three equal thirds: 0.5 lands in the second
    assert int(orc.topk_sample_c(x, 3, 1.0, 0.9)[0]) == 11
    assert int(orc.topk_sample_c(x, 40, 1e-9, 0.99)[1]) == 4        # temperature floor (1e-6): all mass on the maximum
    assert int(orc.topk_sample_c(x, 40, 1e-9, 0.99)[0]) == 11       # ... shared equally by equal maxima
    rng = np.random.default_rng(1)
    y = rng.standard_normal((3, 7)).astype(np.float32)
    np.testing.assert_array_equal(orc.topk_sample_c(y, 128, 1.0, 0.0), y.argmax(axis=1))   # k > N uses N
    np.testing.assert_array_equal(orc.topk_sample_c(y, 1, 1.0, 0.999), y.argmax(axis=1))


def _net(k, temperature):
    import vai_b200
    from vai_b200 import nodes

    class Net(vai_b200.NeuralNet):
        def __init__(self):
            super().__init__()
            self.s = nodes.TopKSamplingNode(k=k, temperature=temperature)
            self.input("in0") - self.s - self.output("out0")

    return Net()


@pytest.mark.gpu
@pytest.mark.parametrize("M,N", [(1, 128256), (3, 50257), (4, 50), (2, 2048), (2, 2050), (1, 262144)])
@pytest.mark.parametrize("k,temperature", [(40, 1.0), (128, 0.8), (1, 1.0)])
def test_topk_node_matches_restatement(M, N, k, temperature, device):
    """Single-launch rows (N <= 2048) and two-stage rows, several uniforms through ONE
    recording: set_uniform between replays changes the sample as the restatement says."""
    from vai_b200 import Tensor
    rng = np.random.default_rng(M + N + k)
    x = (rng.standard_normal((M, N)) * 2).astype(np.float32)
    x[0, N // 3] = x[0, N // 2] = x[0].max() + 1.0          # a tie at the top, in different slices
    net = _net(k, temperature)
    t = Tensor.from_numpy(x)
    for u in US:
        net.s.set_uniform(u)
        got = net(t).to_u32()
        np.testing.assert_array_equal(got, orc.topk_sample_c(x, k, temperature, u), err_msg=f"u={u}")
    assert len(net._recordings) == 1


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_topk_node_16bit_logits(dtype, device):
    from gpu_util import DT, seen
    from vai_b200 import Tensor
    rng = np.random.default_rng(9)
    x = (rng.standard_normal((2, 20000)) * 3).astype(np.float32)
    vals = seen(x, DT[dtype])            # many ties after rounding: the index rule decides
    net = _net(40, 1.0)
    for u in (0.1, 0.6, 0.95):
        net.s.set_uniform(u)
        np.testing.assert_array_equal(net(Tensor.from_numpy(x, dtype=DT[dtype])).to_u32(), orc.topk_sample_c(vals, 40, 1.0, u))


def test_topk_node_rejects_bad_k():
    from vai_b200 import nodes
    with pytest.raises(ValueError):
        nodes.TopKSamplingNode(k=0)
    with pytest.raises(ValueError):
        nodes.TopKSamplingNode(k=129)


# ---- the two anchors the reference does give -------------------------------------------
# (1) With k = 1 the node is greedy decoding whatever the uniform, so it must return the golden
#     output of the reference's Argmax test (python/tests/nodes/test_argmax.py) on that test's
#     seeded input.  (2) topk-sampling.h:33-57 ranks by value descending, then index ascending,
#     and samples by inverse CDF: on a row with three equal maxima and k = 3 the unit interval
#     splits into thirds in index order.  Expected values below are written out by hand; the
#     restatement is not consulted.

def _argmax_case():
    from linear_check import draw_case, load_golden
    meta, arrays = load_golden()
    _, _, fed = draw_case(meta, "argmax")
    return fed["in0"], arrays["argmax"].astype(np.uint32)


def test_restatement_with_k1_returns_the_reference_argmax_case():
    x, want = _argmax_case()
    for u in US:
        np.testing.assert_array_equal(orc.topk_sample_c(x, 1, 1.0, u), want)
        np.testing.assert_array_equal(orc.topk_sample_c(x, 1, 0.3, u), want)


@pytest.mark.gpu
def test_topk_node_with_k1_returns_the_reference_argmax_case(device):
    from vai_b200 import Tensor
    x, want = _argmax_case()
    net = _net(1, 1.0)
    for u in US:
        net.s.set_uniform(u)
        np.testing.assert_array_equal(net(Tensor.from_numpy(x)).to_u32(), want, err_msg=f"u={u}")


TIE_ROWS = [
    # (row length, positions of the equal maxima, k, u, expected index)
    (20, [3, 11, 7], 3, 0.0, 3), (20, [3, 11, 7], 3, 0.2, 3), (20, [3, 11, 7], 3, 0.5, 7), (20, [3, 11, 7], 3, 0.9, 11),
    # ties across the 2048-column slices of the two-stage form
    (9000, [8100, 17, 4000], 3, 0.1, 17), (9000, [8100, 17, 4000], 3, 0.5, 4000), (9000, [8100, 17, 4000], 3, 0.95, 8100),
    # k smaller than the number of equal maxima keeps the lowest indices
    (9000, [8100, 17, 4000, 6000], 2, 0.25, 17), (9000, [8100, 17, 4000, 6000], 2, 0.75, 4000),
]


@pytest.mark.parametrize("n,pos,k,u,want", TIE_ROWS)
def test_restatement_ranks_ties_by_index(n, pos, k, u, want):
    x = np.zeros((1, n), dtype=np.float32)
    x[0, pos] = 5.0
    assert int(orc.topk_sample_c(x, k, 1e-3, u)[0]) == want       # low temperature: all the mass on the maxima


@pytest.mark.gpu
@pytest.mark.parametrize("n,pos,k,u,want", TIE_ROWS)
def test_topk_node_ranks_ties_by_index(n, pos, k, u, want, device):
    from vai_b200 import Tensor
    x = np.zeros((1, n), dtype=np.float32)
    x[0, pos] = 5.0
    net = _net(k, 1e-3)
    net.s.set_uniform(u)
    assert int(net(Tensor.from_numpy(x)).to_u32()[0]) == want


@pytest.mark.gpu
@pytest.mark.parametrize("M,V,bounds", [(2, 9000, [0, 1500, 4700, 9000]), (1, 128256, [0, 32064, 64128, 96192, 128256]),
                                        (3, 60, [0, 7, 30, 60])])
@pytest.mark.parametrize("k", [1, 40, 128])
def test_vocabulary_slabs_merge_to_the_nodes_sample(M, V, bounds, k, device):
    """vaicu_topk_candidates_run per vocabulary slab (windows of the wide rows, with the slab's offset;
    one of them narrower than k in the small case), then vaicu_topk_merge_sample_run: the token of the
    unsplit node (restatement) for several uniforms, and the candidate lists equal to the restatement's."""
    import ctypes

    from vai_b200 import _lib
    from vai_b200.engine import DeviceBuffer
    lib = device.lib
    rng = np.random.default_rng(M + V + k)
    x = (rng.standard_normal((M, V)) * 2).astype(np.float32)
    x[0, bounds[1] - 1] = x[0, bounds[-1] - 1] = x[0].max() + 1.0          # a tie across slabs
    xb = DeviceBuffer(device, x.nbytes)
    xb.upload(x)
    groups = len(bounds) - 1
    pairs = DeviceBuffer(device, groups * M * k * 8)
    keep = []
    for g in range(groups):
        n = bounds[g + 1] - bounds[g]
        nbytes = ctypes.c_size_t()
        _lib.check(lib.vaicu_topk_workspace_bytes(M, n, k, ctypes.byref(nbytes)), "ws")
        ws = DeviceBuffer(device, max(nbytes.value, 256))
        keep.append(ws)
        _lib.check(lib.vaicu_topk_candidates_run(None, xb.ptr + bounds[g] * 4, 0, M, n, V, k, bounds[g], ws.ptr,
                                                 pairs.ptr + g * M * k * 8), "vaicu_topk_candidates_run")
    device.synchronize()
    raw = pairs.download(np.empty((groups, M, k, 2), dtype=np.uint32))
    for g in range(groups):
        vals, idxs = orc.topk_candidates_c(x[:, bounds[g]:bounds[g + 1]], k, bounds[g])
        np.testing.assert_array_equal(raw[g, :, :, 1], idxs)
        np.testing.assert_array_equal(raw[g, :, :, 0], vals.view(np.uint32))
    ub, out = DeviceBuffer(device, 4), DeviceBuffer(device, M * 4)
    for u in US:
        ub.upload(np.array([u], dtype=np.float32))
        _lib.check(lib.vaicu_topk_merge_sample_run(None, pairs.ptr, groups, M * k, M, k, min(k, V), 1.3, ub.ptr, out.ptr), "merge")
        device.synchronize()
        np.testing.assert_array_equal(out.download(np.empty(M, dtype=np.uint32)), orc.topk_sample_c(x, k, 1.3, u), err_msg=f"u={u}")
