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

The K-step timed region is repeated until at least half a second has been timed (every
repeat bracketed by a barrier and a synchronize, max over ranks); `value` comes from the
median repeat, the fastest is reported beside it, and the clock sampler runs over all of them.

Beside the headline the line carries, inside `roofline`:
  secondary (N = 1)  the other parts of the metric: the Llama-3.2-3B-shaped prefill blocks at
                     M = 8192 (TFLOP/s, per layer and as a recorded 28-block step), the
                     Gemma-3-4B-shaped batched decode step at M = 64 (GB/s, per layer and whole
                     step) and the fp32 GPT-2 MLP Linear;
  sharded (N > 1)    the column / row split of the large-N layers over the N GPUs: per layer the
                     same layer on one GPU, on N, speed-up, efficiency, fraction of N x roofline
                     and the collective's share, with sampled outputs checked against float64.

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
    # every core this process may run on, whatever OMP_NUM_THREADS the launcher exported
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    orc.set_num_threads(cores)
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


def timed_repeats(region, dist, dev, min_total_ms=500.0, max_repeats=400):
    """Runs region() -> milliseconds (one K-step region, device-timed) between barriers until
    at least min_total_ms has been timed; every rank repeats the same number of times because the
    count is derived from the first region's max-over-ranks time.  Returns the list of per-region
    times, each the max over ranks."""
    barrier_and_sync(dist, dev)
    first = max_over_ranks(dist, region())
    barrier_and_sync(dist, dev)
    repeats = int(min(max_repeats, max(1, np.ceil(min_total_ms / max(first, 1e-3)))))
    times = [first]
    for _ in range(repeats - 1):
        t = max_over_ranks(dist, region())
        barrier_and_sync(dist, dev)
        times.append(t)
    return times


def replay_ms(lib, graph, stream, ev, steps, warmup):
    for _ in range(warmup):
        lib.vaicu_graph_launch(graph, stream)
    lib.vaicu_stream_sync(stream)
    ev.start(stream)
    for _ in range(steps):
        lib.vaicu_graph_launch(graph, stream)
    return ev.stop_ms(stream) / steps


def secondary_reports(dev, pk):
    """The parts of the metric the headline workload does not show, on this GPU: prefill GEMM
    TFLOP/s (Llama-3.2-3B shapes, M = 8192), skinny-GEMM / batched-decode GB/s (Gemma-3-4B
    shapes, M = 64), and the fp32 single-node case.  Per layer in isolation (weights rotated
    over more than L2) and as a recorded step of the whole model's Linear nodes."""
    import gc

    import vai_b200
    from vai_b200 import Dtype, Tensor, microbench, presets
    lib = dev.lib
    ev = Events(lib)
    burst, sustained, hbm = pk.get("bf16_tflops", 1590.0), pk.get("bf16_tflops_sustained", 1400.0), pk["hbm_gbs"]
    out = []

    def layers_of(preset, M, iters):
        p = presets.PRESETS[preset]
        rows = []
        for name, k, n, ex in presets.block_linears(p) + [("lm_head", p["d"], p["vocab"], {})]:
            r = microbench.run(M, k, n, "bf16", "bf16", "bf16", epilogue=p["act"] if ex.get("gate") else "NONE",
                               gate=bool(ex.get("gate")), residual=bool(ex.get("residual")), iters=iters, warmup=3, device=dev)
            rows.append({"layer": name, "K": k, "N": n, "us": round(r["us_per_call"], 2), "TFLOPs": round(r["TFLOPs"], 1),
                         "GBps": round(r["GBps"], 1), "launches": r["launches"], "tile": r["tile"], "splits": r["split_count"]})
        return rows

    # ---- Llama-3.2-3B-shaped prefill, batch 4 x 2048 tokens (M = 8192), bf16 in / out
    M = 8192
    rows = layers_of("llama-3.2-3b", M, 10)
    for r in rows:
        r["frac_of_burst"] = round(r["TFLOPs"] / burst, 3)
        r.pop("GBps")
    net = vai_b200.NeuralNet(w_default_dtype=Dtype.BF16, o_default_dtype=Dtype.BF16, device=dev)
    presets.build_linear_chain(net, "llama-3.2-3b", w_dtype=Dtype.BF16, lm_head=False, seed=3)
    x = Tensor.from_numpy(np.random.default_rng(4).standard_normal((M, 3072), dtype=np.float32), dtype=Dtype.BF16)
    net(x)
    rec = next(iter(net._recordings.values()))
    ms = replay_ms(lib, rec.graph, net.stream, ev, 5, 2)
    dev.check_status()
    fl = presets.flops("llama-3.2-3b", M) - 2.0 * M * 3072 * 128256
    tf = fl / (ms * 1e-3) / 1e12
    out.append({"config": "Llama-3.2-3B-shaped prefill, M = 8192 (4 x 2048 tokens), bf16: the 28 blocks' Linear nodes "
                          "(q, k, v, o + residual, gate|value with the SiLU gate fused, down + residual) as one recorded step; "
                          "lm_head listed per layer only (the reference slices the last row before it)",
                "bound": "tensor", "ms_per_step": round(ms, 3), "flops_per_step": fl, "launches_per_step": rec.kernel_launches,
                "TFLOPs": round(tf, 1), "frac_of_burst_peak": round(tf / burst, 3), "frac_of_sustained_peak": round(tf / sustained, 3),
                "frac_of_nominal_2250": round(tf / 2250.0, 3), "peaks": {"burst": burst, "sustained": sustained}, "per_layer": rows})
    del net, rec, x
    gc.collect()

    # ---- Gemma-3-4B-shaped batched decode, batch 64 (M = 64), bf16 in / out
    M = 64
    rows = layers_of("gemma-3-4b", M, 20)
    for r in rows:
        r["frac_of_hbm"] = round(r["GBps"] / hbm, 3)
        r.pop("TFLOPs")
    net = vai_b200.NeuralNet(w_default_dtype=Dtype.BF16, o_default_dtype=Dtype.BF16, device=dev)
    presets.build_linear_chain(net, "gemma-3-4b", w_dtype=Dtype.BF16, seed=5)
    x = Tensor.from_numpy(np.random.default_rng(6).standard_normal((M, 2560), dtype=np.float32), dtype=Dtype.BF16)
    net(x)
    rec = next(iter(net._recordings.values()))
    ms = replay_ms(lib, rec.graph, net.stream, ev, 10, 3)
    dev.check_status()
    ab = presets.algorithmic_bytes("gemma-3-4b", M, w_bytes=2, io_bytes=2)
    gbs = ab / (ms * 1e-3) / 1e9
    out.append({"config": "Gemma-3-4B-shaped batched decode step, batch 64 (M = 64), bf16: 34 blocks + lm_head 262144 as one recorded step",
                "bound": "hbm", "ms_per_step": round(ms, 3), "algorithmic_bytes_per_step": ab, "launches_per_step": rec.kernel_launches,
                "GBps": round(gbs, 1), "frac_of_measured_hbm": round(gbs / hbm, 3), "steps_per_s": round(1e3 / ms, 1),
                "tokens_per_s": round(64e3 / ms, 1), "per_layer": rows})
    del net, rec, x
    gc.collect()

    # ---- the single fp32 node (GPT-2 small fc1: M 128, K 768, N 3072, bias + GELU-tanh)
    r = microbench.run(128, 768, 3072, "f32", "f32", "f32", epilogue="GELU_TANH", bias=True, iters=50, warmup=5, device=dev)
    out.append({"config": "GPT-2-small MLP Linear, fp32: X [128, 768], W [3072, 768], bias, GELU(tanh)", "bound": "latency-sized (0.6 GFLOP)",
                "us": round(r["us_per_call"], 2), "TFLOPs": round(r["TFLOPs"], 2), "kernel": r["kernel"]})
    return out


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
    ap.add_argument("--no-secondary", action="store_true", help="skip the prefill / batched-decode / fp32 reports (N = 1)")
    ap.add_argument("--min-timed-ms", type=float, default=500.0,
                    help="the K-step region is repeated until this much has been timed (0: once; for profiler runs)")
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

    def resident_region():
        ev.start(net.stream)
        for _ in range(args.steps):
            lib.vaicu_graph_launch(rec.graph, net.stream)
        return ev.stop_ms(net.stream)

    sampler = ClockSampler(local)
    sampler.start()
    regions = timed_repeats(resident_region, dist, dev, args.min_timed_ms)
    clocks = sampler.stop()
    dev.check_status()
    ms = statistics.median(regions)             # one K-step region, max over ranks, median of the repeats
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

    def e2e_region():
        ev.start(net2.stream)
        for _ in range(args.steps):
            net2(x)
        return ev.stop_ms(net2.stream)

    e2e_regions = timed_repeats(e2e_region, dist, dev, args.min_timed_ms)
    net_e2e = net2
    e2e_ms = statistics.median(e2e_regions)
    e2e_tok_s = world * args.steps / (e2e_ms / 1e3)

    # Column split of the large-N layers over the GPUs (Gemma-3-4B-shaped lm_head and gate|value
    # Linear at batch 64; Llama-3.2-3B-shaped ones at M = 8192): local slab, NCCL all-gather,
    # gather fused into the GEMM epilogue, greedy head, column-then-row-parallel MLP.  Reported
    # beside the headline, never part of it.
    sharded = None
    if world > 1:
        # no try / except: a split that fails or computes something wrong fails the run
        from vai_b200 import sharded as sharded_mod
        pk_sh, _ = peaks()
        sharded = sharded_mod.sharded_report(dev, dist, pk_sh)

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
        "timing": {"repeats": len(regions), "timed_ms_total": round(sum(regions), 1), "ms_per_step_median": ms / args.steps,
                   "ms_per_step_min": min(regions) / args.steps, "ms_per_step_max": max(regions) / args.steps,
                   "e2e_repeats": len(e2e_regions), "e2e_ms_per_step_min": min(e2e_regions) / args.steps},
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
        line["roofline"]["sharded"] = sharded
    if world == 1 and not args.no_secondary:
        line["roofline"]["secondary"] = secondary_reports(dev, pk)
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
