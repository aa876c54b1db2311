"""CPU, world_size > 1 over gloo: the column split of a Linear (vai_b200/sharded.py) —
row ranges, gate|value slicing, all-gather layout and reassembly — with the per-rank
Linear computed by the CPU oracle.  The GPU path uses the same split code with
vaicu_linear_run in place of the oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import linear_oracle as orc
from vai_b200 import sharded


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _full_problem(gate):
    rng = np.random.default_rng(11)
    M, K = 5, 96
    N = 2 * 164 if gate else 203        # 203 columns over 2 or 3 ranks: uneven slabs
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    return M, K, N, x, w, b


def _worker(rank, world, port, gate, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K, N, x, w, b = _full_problem(gate)
        n_out = N // 2 if gate else N
        ws = sharded.slice_weight(w, rank, world, gate)
        bs = sharded.slice_bias(b, rank, world, gate)
        begin, count = sharded.shard_rows(n_out, world, rank)
        d = orc.make_desc(M, ws.shape[0], K, b_dtype=orc.F32, bias_elems=ws.shape[0], epilogue=4, gate_fuse=gate)
        local = orc.linear_c(d, x, np.ascontiguousarray(ws), np.ascontiguousarray(bs))
        assert local.shape == (M, count)
        shape = sharded.gathered_shape(M, n_out, world)
        padded = np.zeros(shape[1:], dtype=np.float32)
        padded[:, :count] = local
        gathered = [torch.empty(shape[1:], dtype=torch.float32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(padded))
        full = sharded.assemble(torch.stack(gathered).numpy(), n_out)
        np.save(os.path.join(out_dir, f"rank{rank}.npy"), full)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("gate", [False, True])
def test_column_split_matches_unsplit(world, gate, tmp_path):
    mp.spawn(_worker, args=(world, _free_port(), gate, str(tmp_path)), nprocs=world, join=True)
    M, K, N, x, w, b = _full_problem(gate)
    d = orc.make_desc(M, N, K, b_dtype=orc.F32, bias_elems=N, epilogue=4, gate_fuse=gate)
    want = orc.linear_c(d, x, w, b)
    for rank in range(world):
        got = np.load(tmp_path / f"rank{rank}.npy")
        assert got.shape == want.shape
        # the same fp32 arithmetic per column, so the split is exact
        np.testing.assert_array_equal(got, want)


def test_shard_rows_agree_with_the_library():
    from vai_b200 import _lib
    full = _lib.LinearDesc()
    full.M, full.N, full.K = 64, 50257, 768
    full.i_dtype, full.w_dtype, full.o_dtype, full.b_dtype = 0, 1, 0, 2
    full.scalar_scale = 1.0
    for world in (1, 2, 4, 8):
        for rank in range(world):
            _, b, c = sharded.shard_desc(full, rank, world)
            assert (b, c) == sharded.shard_rows(50257, world, rank)


def _row_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)
        M, K, N = 4, 200, 24                     # 200 = 25 units of 8: uneven over 2 and 3 ranks
        x = rng.standard_normal((M, K)).astype(np.float32)
        w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
        r = rng.standard_normal((M, N)).astype(np.float32)
        kb, kc = sharded.shard_k(K, world, rank)
        ws = sharded.slice_weight_k(w, rank, world)
        assert ws.shape == (N, kc) and ws.flags["C_CONTIGUOUS"]
        d = orc.make_desc(M, N, kc)
        partial = orc.linear_c(d, np.ascontiguousarray(x[:, kb:kb + kc]), ws)
        t = torch.from_numpy(partial.copy())
        dist.all_reduce(t)
        np.save(os.path.join(out_dir, f"row{rank}.npy"), 0.25 * t.numpy() + r)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_row_parallel_split_matches_unsplit(world, tmp_path):
    """K-split `down` (vai_b200.sharded.RowParallelLinear's host arithmetic): slices of the
    reduction axis in 16-byte units, partial products per rank, one all-reduce, then scale and
    residual: equals the unsplit Linear up to fp32 summation order."""
    slices = [sharded.shard_k(200, world, r) for r in range(world)]
    assert slices[0][0] == 0 and sum(c for _, c in slices) == 200
    assert all(b % 8 == 0 for b, _ in slices) and all(slices[i][0] + slices[i][1] == slices[i + 1][0] for i in range(world - 1))
    assert sharded.shard_k(203, 2, 1) == (104, 99)          # the ragged tail goes to the last rank
    port = _free_port()
    mp.spawn(_row_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(5)
    M, K, N = 4, 200, 24
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    r = rng.standard_normal((M, N)).astype(np.float32)
    want = orc.linear_f64(x, w, residual=r, scalar_scale=0.25)
    for rank in range(world):
        got = np.load(os.path.join(str(tmp_path), f"row{rank}.npy"))
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)


def _topk_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, V, k, temperature, logits, us = _topk_problem()
        begin, count = sharded.shard_rows(V, world, rank)
        vals, idxs = orc.topk_candidates_c(logits[:, begin:begin + count], k, begin)     # this rank's slab only
        mine = torch.from_numpy(np.stack([vals.view(np.int32), idxs.view(np.int32)], axis=-1).copy())     # [M, k, 2]: 8 k bytes per row
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        allv = np.stack([g.numpy()[..., 0].copy().view(np.float32) for g in gathered])
        alli = np.stack([g.numpy()[..., 1].copy().view(np.uint32) for g in gathered])
        tokens = np.stack([orc.topk_merge_sample_c(allv, alli, min(k, V), temperature, float(u)) for u in us])
        np.save(os.path.join(out_dir, f"topk{rank}.npy"), tokens)
    finally:
        dist.destroy_process_group()


def _topk_problem():
    rng = np.random.default_rng(21)
    M, V, k, temperature = 2, 5003, 40, 0.8
    logits = (rng.standard_normal((M, V)) * 2).astype(np.float32)
    logits[0, 100] = logits[0, 4000] = logits[0].max() + 0.5        # equal maxima in different slabs
    us = np.random.default_rng(22).random(1000, dtype=np.float32)
    return M, V, k, temperature, logits, us


@pytest.mark.parametrize("world", [2, 3])
def test_vocabulary_split_topk_draws_the_single_gpu_token(world, tmp_path):
    """TopKSampling over vocabulary slabs (vai_b200.sharded.ShardedTopKHead's arithmetic, with the C
    restatement standing in for the kernels): per-rank k candidates with their vocabulary offset, an
    all-gather of 8 k bytes per row and rank, the same merge + sample on every rank — the token the
    unsplit node draws, for 1000 seeded uniforms, ties across slabs included."""
    mp.spawn(_topk_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    M, V, k, temperature, logits, us = _topk_problem()
    want = np.stack([orc.topk_sample_c(logits, k, temperature, float(u)) for u in us])
    for rank in range(world):
        np.testing.assert_array_equal(np.load(tmp_path / f"topk{rank}.npy"), want)
    assert len(np.unique(want[:, 0])) > 10          # the uniforms do reach many ranks of the distribution


def test_destination_order_spreads_the_ranks_over_the_peers():
    """Every rank starts with its right-hand neighbour and ends with itself, so that at step i the
    `world` ranks store to `world` different GPUs."""
    for world in (1, 2, 4, 8):
        orders = [sharded.destination_order(r, world) for r in range(world)]
        for r, o in enumerate(orders):
            assert sorted(o) == list(range(world)) and o[-1] == r
        for step in range(world):
            assert sorted(o[step] for o in orders) == list(range(world))
