#!/usr/bin/env python
"""Benchmark of the Linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1 and every N): the Linear nodes of one Llama-3.2-1B-shaped decode step,
batch 1 (M = 1): 16 blocks of q / k / v / o(+R) / gate|value (SiLU gate fused) /
down(+R), then the 128256-row lm_head; bf16 weights ~N(0, 0.02) (synthetic, seeded),
fp32 activations.  97 Linear nodes (65 kernel launches: q / k / v of a block share one)
and 2.47 GB of weights per step, replayed as one recorded CUDA graph — the analogue of
the reference's resubmitted command buffer.
Attention, norms and rope are other operators and are not part of the step.

`value` is decode tokens/s with everything resident in HBM (device-timed with events);
`e2e` is the same step driven through the public host API with the step's input copied
from pinned host memory and the logits copied back, every step.  With N > 1 every rank
runs its own token stream on its own GPU (weak scaling, no collective on the data
path); the time is the max over ranks.

`--impl reference` times the CPU restatement of the reference's shader arithmetic
(oracle/linear_oracle.c, all host threads) on a bounded sample of the same step; the
reference itself has no CPU code for this path and its Vulkan build cannot run here.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PRESET = "llama-3.2-1b"
FALLBACK_HBM_GBS = 6650.0


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return json.load(f), "measured"
    except Exception:
        return {"hbm_gbs": FALLBACK_HBM_GBS}, "fallback"


class ClockSampler:
    """SM clock and throttle reasons while the timed region runs: NVML polled from a thread
    every few milliseconds (read-only queries), nvidia-smi as the fallback."""
    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index):
        self.index = index
        self.sm, self.bits = [], 0
        self.max_mhz = None
        self.stop_flag = False
        self.thread = None
        self.how = None

    def _poll_nvml(self):
        import pynvml
        h = self.handle
        while not self.stop_flag:
            try:
                self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                self.bits |= int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            try:     # the CUDA ordinal is not NVML's index when CUDA_VISIBLE_DEVICES reorders
                import torch
                uuid = "GPU-" + str(torch.cuda.get_device_properties(self.index).uuid)
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.how = "nvml"
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
        except Exception:
            self.how = None

    def stop(self):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=1.0)
        if not self.sm:      # NVML unavailable: one nvidia-smi reading right after the region
            try:
                out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
                                      "clocks_event_reasons.sw_power_cap,clocks_event_reasons.sw_thermal_slowdown,"
                                      "clocks_event_reasons.hw_thermal_slowdown", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=10).stdout
                parts = [q.strip() for q in out.strip().split(",")]
                self.sm = [float(parts[0])]
                self.max_mhz = float(parts[1])
                for name, v in zip(["hw_slowdown", "sw_power_cap", "sw_thermal_slowdown", "hw_thermal_slowdown"], parts[2:6]):
                    if v.lower().startswith("active"):
                        self.bits |= self.REASONS[name]
                self.how = "nvidia-smi after the region"
            except Exception:
                return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["clock query unavailable"]}
        reasons = sorted(n for n, bit in self.REASONS.items() if self.bits & bit)
        return {"sm_mhz": statistics.median(self.sm), "sm_max_mhz": self.max_mhz, "samples": len(self.sm),
                "reasons": reasons, "source": self.how}


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist_mod.init_process_group(backend="nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    return rank, world, local, dist


def barrier_and_sync(dist, dev):
    if dist is not None:
        import torch
        dist.barrier()
        torch.cuda.synchronize()
    dev.synchronize()


def max_over_ranks(dist, value):
    if dist is None:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class Events:
    def __init__(self, lib):
        self.lib = lib
        self.a, self.b = ctypes.c_void_p(), ctypes.c_void_p()
        from vai_b200 import _lib
        _lib.check(lib.vaicu_event_create(ctypes.byref(self.a)), "event")
        _lib.check(lib.vaicu_event_create(ctypes.byref(self.b)), "event")

    def start(self, stream):
        self.lib.vaicu_event_record(self.a, stream)

    def stop_ms(self, stream):
        self.lib.vaicu_event_record(self.b, stream)
        self.lib.vaicu_event_synchronize(self.b)
        ms = ctypes.c_float()
        self.lib.vaicu_event_elapsed_ms(self.a, self.b, ctypes.byref(ms))
        return float(ms.value)


def cpu_sample(steps, warmup):
    """The C restatement on one transformer block's Linears plus 1/16 of the lm_head
    rows, all host threads; scaled to a whole step by weight bytes."""
    from oracle import linear_oracle as orc
    from vai_b200 import presets
    p = presets.PRESETS[PRESET]
    rng = np.random.default_rng(0)
    jobs = []
    sample_elems = 0
    shapes = [(k, n, ex) for _, k, n, ex in presets.block_linears(p)] + [(p["d"], p["vocab"] // 16, {})]
    for k, n, ex in shapes:
        w = orc.to_dtype((rng.standard_normal((n, k), dtype=np.float32) * 0.02), orc.BF16)
        x = rng.standard_normal((1, k), dtype=np.float32)
        gate = bool(ex.get("gate"))
        out_n = n // 2 if gate else n
        r = rng.standard_normal((1, out_n), dtype=np.float32) if ex.get("residual") else None
        d = orc.make_desc(1, n, k, w_dtype=orc.BF16, residual_elems=out_n if r is not None else None,
                          epilogue=4 if gate else 0, gate_fuse=gate)
        jobs.append((d, x, w, r))
        sample_elems += n * k
    total_elems = presets.weight_elements(PRESET)

    def one():
        t0 = time.perf_counter()
        for d, x, w, r in jobs:
            orc.linear_c(d, x, w, None, r)
        return time.perf_counter() - t0

    for _ in range(warmup):
        one()
    times = [one() for _ in range(steps)]
    t = sum(times) / len(times)
    tok_s = 1.0 / (t * total_elems / sample_elems)
    return tok_s, orc.num_threads(), t, f"1 of {p['layers']} blocks + 1/16 of the lm_head rows per step ({sample_elems * 2 / 1e6:.0f} MB of " \
        f"bf16 weights), scaled to the whole step by weight bytes"


def run_reference(args, rank):
    if rank != 0:
        return
    steps = max(1, min(args.steps, 20))
    tok_s, cores, t, sample = cpu_sample(steps, min(args.warmup, 2))
    from vai_b200 import presets
    line = {
        "impl": "reference", "metric": "llama-3.2-1b decode tokens/s (Linear path)", "value": tok_s, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 2), "ms_per_step": 1000.0 / tok_s,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample,
                         "note": "CPU restatement of the reference's shader arithmetic; the reference has no CPU code for "
                                 "this path and its Vulkan build is unavailable on this box"},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config():
    from vai_b200 import presets
    return {"workload": "Llama-3.2-1B-shaped decode step, batch 1 (M=1): 16 blocks x {q,k,v,o,gate|value,down} + lm_head "
                        "128256; bf16 weights N(0,0.02), fp32 activations; 97 Linear nodes, 65 kernel launches per step",
            "weight_bytes_per_step": presets.weight_elements(PRESET) * 2,
            "l2": "weights per step (2.47 GB) exceed L2 (126 MB); no flush needed",
            "parallelism": "one token stream per GPU"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    args.warmup = max(args.warmup, 3)

    rank, world, local, dist = dist_setup(args.gpus)
    import vai_b200
    from vai_b200 import Device, Dtype, Tensor, _lib, presets

    dev = Device(local)
    lib = dev.lib
    net = vai_b200.NeuralNet(w_default_dtype=Dtype.BF16, device=dev)
    nodes = presets.build_linear_chain(net, PRESET, w_dtype=Dtype.BF16, seed=rank)
    p = presets.PRESETS[PRESET]
    rng = np.random.default_rng(100 + rank)
    x = Tensor.from_numpy(rng.standard_normal((1, p["d"]), dtype=np.float32))
    # first call: uploads the weights, records the step, replays it once
    out = net(x)
    assert out.shape == (1, p["vocab"]) and np.isfinite(out.to_numpy()).all()
    rec = next(iter(net._recordings.values()))
    launches_per_step = rec.kernel_launches     # q / k / v of a block share one launch
    kernels = sorted({n.info.kernel for n in nodes})
    assert kernels == [vai_b200.nodes.KERNEL_GEMV], kernels

    ev = Events(lib)
    # ---- device-resident timing: graph replays back to back --------------------
    for _ in range(args.warmup):
        lib.vaicu_graph_launch(rec.graph, net.stream)
    barrier_and_sync(dist, dev)
    sampler = ClockSampler(local)
    sampler.start()
    ev.start(net.stream)
    for _ in range(args.steps):
        lib.vaicu_graph_launch(rec.graph, net.stream)
    ms = ev.stop_ms(net.stream)
    barrier_and_sync(dist, dev)
    clocks = sampler.stop()
    dev.check_status()
    ms = max_over_ranks(dist, ms)
    tok_s = world * args.steps / (ms / 1e3)

    # ---- end to end through the host API, as a decode loop runs it: every step copies the
    # step's input from pinned host memory, replays the recording (the same Linears on the
    # same weight buffers, followed by the Argmax node that consumes the logits) and copies
    # the sampled token back, then synchronises
    net2 = vai_b200.NeuralNet(w_default_dtype=Dtype.BF16, device=dev)
    presets.build_linear_chain(net2, PRESET, w_dtype=Dtype.BF16, argmax=True, share_weights=nodes)
    tok = net2(x).to_u32()
    assert int(tok[0]) == int(np.argmax(out.to_numpy()[0])), "argmax node disagrees with the logits"
    for _ in range(args.warmup):
        net2(x)
    barrier_and_sync(dist, dev)
    ev.start(net2.stream)
    for _ in range(args.steps):
        tok = net2(x)
    e2e_ms = ev.stop_ms(net2.stream)
    net_e2e = net2
    barrier_and_sync(dist, dev)
    e2e_ms = max_over_ranks(dist, e2e_ms)
    e2e_tok_s = world * args.steps / (e2e_ms / 1e3)

    # Column split of the large-N layers over the GPUs (Gemma-3-4B-shaped lm_head and gate|value
    # Linear at batch 64; Llama-3.2-3B-shaped ones at M = 8192): local slab, NCCL all-gather,
    # gather fused into the GEMM epilogue, greedy head, column-then-row-parallel MLP.  Reported
    # beside the headline, never part of it.
    sharded = None
    if world > 1:
        try:
            from vai_b200 import sharded as sharded_mod
            sharded = {"decode_gemma3_4b_m64": sharded_mod.bench_sharded(dev, dist, "gemma-3-4b", 64, iters=10, warmup=3),
                       "prefill_llama32_3b_m8192": sharded_mod.bench_sharded(dev, dist, "llama-3.2-3b", 8192, iters=5, warmup=2)}
        except Exception as e:   # a report only
            sharded = {"error": str(e)[:200]}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    pk, pk_kind = peaks()
    alg_bytes = presets.algorithmic_bytes(PRESET, 1)
    step_s = ms / 1e3 / args.steps
    achieved = alg_bytes / step_s / 1e9
    line = {
        "metric": "llama-3.2-1b decode tokens/s (Linear path)", "value": tok_s, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 weights, f32 accumulate", "data": "synthetic",
        "config": workload_config(),
        "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": net_e2e.h2d_bytes, "d2h_bytes_per_step": net_e2e.d2h_bytes,
                "ms_per_step": e2e_ms / args.steps,
                "path": "NeuralNet call: one graph submission (H2D of x from pinned memory, 97 Linear nodes + Argmax, the token stored by its kernel into page-locked host memory), then a sync"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "gemv_kernel<bf16, M=1, R> (every launch of the step)",
                     "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                     "peak_kind": f"of {pk_kind}",
                     # DRAM bytes per step: ncu captures of the lm_head and gate|value launches read
                     # 1.006 x their algorithmic bytes; the other launches are the same kernel, scaled
                     "traffic": int(alg_bytes * 1.006),
                     "algorithmic_bytes_per_step": alg_bytes, "launches_per_step": launches_per_step,
                     "avg_launch_us": step_s / launches_per_step * 1e6},
    }
    if sharded is not None:
        line["sharded"] = sharded
    if world == 1 and not args.no_cpu_baseline:
        try:
            v, cores, t, sample = cpu_sample(5, 1)
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
        except Exception as e:   # the baseline is a report, never a reason to lose the GPU number
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
