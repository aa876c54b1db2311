"""GPU, 2 ranks on 2 GPUs (skipped on a one-GPU box): the column-split Linear whose
tensor-core epilogue stores its slab into every rank's output over NVLink
(vaicu_linear_run_scatter + CUDA IPC) gives bit-identical results to the NCCL all-gather
of the same plan's dense output, and the vocabulary-split greedy head (per-GPU argmax
candidates merged after an 8-byte-per-row exchange) picks the same tokens as the argmax over
the gathered logits.  Runs vai_b200.sharded under torch.distributed.run."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_fused_gather_matches_nccl_on_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", "-m", "vai_b200.sharded", "--M", "64"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1]
    res = json.loads(line)
    for name in ("lm_head", "gate_up"):
        layer = res["layers"][name]
        assert layer["fused_gather_matches_nccl"] is True, name
        assert layer["fused_gather_us"] > 0 and layer["t1_us"] > 0
        # against float64 on sampled outputs, not only against the NCCL path
        assert all(v <= 2e-2 for v in layer["max_rel_err_vs_float64"].values()), layer["max_rel_err_vs_float64"]
    mlp = res["layers"]["mlp_column_then_row_parallel"]
    assert all(v is not None and v <= 2e-2 for v in mlp["max_rel_err_vs_float64"].values()), mlp["max_rel_err_vs_float64"]
    assert mlp["fused_reduce_scatter_us"] > 0
    # vocabulary-split greedy head: candidates instead of logits cross the link
    head = res["layers"]["lm_head"]
    assert head["greedy_head_matches_argmax_of_gathered_logits"] is True
    assert head["greedy_exchange_bytes_per_gpu"] == 8 * 64


def _nodes_check(nproc, port):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    if nproc == 1:
        cmd = [sys.executable, "-m", "vai_b200.sharded", "--nodes-check", "--M", "64"]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr", "127.0.0.1",
               "--master-port", str(port), "-m", "vai_b200.sharded", "--nodes-check", "--M", "64"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])["tp_nodes"]


def test_row_parallel_node_in_a_recorded_net_one_rank():
    """The tensor-parallel MLP as nodes of the engine (plain Linear over this rank's gate|value rows ->
    GatedMul -> RowParallelLinearNode + residual), two blocks recorded into one graph and replayed, with a
    process group of one rank: every kernel of the exchange runs, against float64."""
    res = _nodes_check(1, 0)
    assert res["max_rel_err_vs_float64"] < 2e-2, res
    # the vocabulary-split lm_head node + Argmax node of the same check
    assert res["head_max_rel_err_vs_float64"] < 1e-3 and res["head_token_mismatches"] == 0, res
    # per block: gate|value with the GatedMul merged (1, or 2 with a split-K fold), down GEMM, barrier, fold, barrier
    assert 2 * 5 <= res["launches_recorded"] <= 2 * 6, res


def test_row_parallel_node_in_a_recorded_net_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = _nodes_check(2, 29543)
    assert res["world"] == 2 and res["max_rel_err_vs_float64"] < 2e-2, res
    assert res["head_max_rel_err_vs_float64"] < 1e-3 and res["head_token_mismatches"] == 0, res
