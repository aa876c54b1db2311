"""Time one Linear shape in isolation through the C ABI.

    python -m vai_b200.microbench --M 1 --K 2048 --N 128256 --w-dtype bf16 [--gate] [--kernel 0]
    python -m vai_b200.microbench --M 64 --K 2560 --group 2048,1024,1024 --i-dtype bf16 --o-dtype bf16

The weights rotate over `--copies` distinct device buffers (chosen so that the set is
larger than the 126 MB L2 unless --copies is given), so every launch streams its
weights from HBM.  Prints one JSON line: microseconds per launch, algorithmic GB/s and
TFLOP/s.  Also the small-case target for `ncu` captures of a single kernel.
"""
import argparse
import ctypes
import json

import numpy as np

from . import _lib
from .engine import Device, DeviceBuffer, Dtype, Epilogue, dtype_size, encode

DT = {"f32": Dtype.F32, "f16": Dtype.F16, "bf16": Dtype.BF16}


def algorithmic_bytes(M, N, K, i_dt, w_dt, o_dt, bias, residual, gate):
    out_n = N // 2 if gate else N
    b = N * K * dtype_size(w_dt) + M * K * dtype_size(i_dt) + M * out_n * dtype_size(o_dt)
    if bias:
        b += N * dtype_size(w_dt)
    if residual:
        b += M * out_n * dtype_size(o_dt)
    return b


def run(M, K, N, i_dtype="f32", w_dtype="bf16", o_dtype="f32", epilogue="NONE", gate=False, bias=False,
        residual=False, kernel=0, copies=0, iters=50, warmup=5, split_size=0, device=None, graph=False, clocks=False,
        tuning=None):
    dev = device or Device.default()
    lib = dev.lib
    i_dt, w_dt, o_dt = DT[i_dtype], DT[w_dtype], DT[o_dtype]
    out_n = N // 2 if gate else N
    w_bytes = N * K * dtype_size(w_dt)
    if copies <= 0:
        copies = max(2, min(64, int(np.ceil(300e6 / w_bytes))))
    rng = np.random.default_rng(0)
    w_host = encode((rng.standard_normal((N, K), dtype=np.float32) * 0.02), w_dt)
    x_host = encode(rng.standard_normal((M, K), dtype=np.float32), i_dt)
    weights = []
    for _ in range(copies):
        b = DeviceBuffer(dev, w_bytes)
        b.upload(w_host)
        weights.append(b)
    xb = DeviceBuffer(dev, x_host.nbytes)
    xb.upload(x_host)
    ob = DeviceBuffer(dev, M * out_n * dtype_size(o_dt))
    bb = rb = None
    if bias:
        bb = DeviceBuffer(dev, N * dtype_size(w_dt))
        bb.upload(encode(rng.standard_normal(N, dtype=np.float32), w_dt))
    if residual:
        rb = DeviceBuffer(dev, M * out_n * dtype_size(o_dt))
        rb.upload(encode(rng.standard_normal((M, out_n), dtype=np.float32), o_dt))
    d = _lib.LinearDesc()
    d.M, d.N, d.K = M, N, K
    d.i_dtype, d.w_dtype, d.o_dtype = int(i_dt), int(w_dt), int(o_dt)
    d.b_dtype = int(w_dt) if bias else int(Dtype.NONE)
    d.has_bias, d.bias_elems = (1, N) if bias else (0, 0)
    d.has_residual, d.residual_elems = (1, 0) if residual else (0, 0)
    d.epilogue = int(getattr(Epilogue, epilogue))
    d.scalar_scale = 1.0
    d.split_size = split_size
    d.gate_fuse = 1 if gate else 0
    plans = []
    info = _lib.LinearInfo()
    for _ in range(copies):   # one plan per weight copy: each keeps its own tensor maps
        h = ctypes.c_void_p()
        if tuning:
            t = _lib.LinearTuning(kernel=kernel, **tuning)
            _lib.check(lib.vaicu_linear_plan_create_tuned(dev.handle, ctypes.byref(d), ctypes.byref(t), ctypes.byref(h)), "plan")
        elif kernel:
            _lib.check(lib.vaicu_linear_plan_create_forced(dev.handle, ctypes.byref(d), kernel, ctypes.byref(h)), "plan")
        else:
            _lib.check(lib.vaicu_linear_plan_create(dev.handle, ctypes.byref(d), ctypes.byref(h)), "plan")
        plans.append(h)
    _lib.check(lib.vaicu_linear_plan_info(plans[0], ctypes.byref(info)), "info")
    ws = DeviceBuffer(dev, info.workspace_bytes) if info.workspace_bytes else None
    stream = dev.create_stream()
    e0, e1 = ctypes.c_void_p(), ctypes.c_void_p()
    lib.vaicu_event_create(ctypes.byref(e0))
    lib.vaicu_event_create(ctypes.byref(e1))

    def launch(i):
        c = i % copies
        _lib.check(lib.vaicu_linear_run(plans[c], stream, xb.ptr, weights[c].ptr, bb.ptr if bb else None,
                                        rb.ptr if rb else None, ob.ptr, ws.ptr if ws else None), "run")

    for i in range(max(warmup, copies)):
        launch(i)
    lib.vaicu_stream_sync(stream)
    sampler = None
    if clocks:
        import subprocess
        sampler = subprocess.Popen(["nvidia-smi", "--query-gpu=clocks.sm,power.draw,clocks_event_reasons.sw_power_cap,"
                                    "clocks_event_reasons.hw_slowdown,clocks_event_reasons.sw_thermal_slowdown",
                                    "--format=csv,noheader,nounits", "-lms", "100", "-i", str(dev.ordinal)],
                                   stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    if graph:
        # record `iters` launches once and replay the recording: no host launch cost
        # between kernels, as in a net's replayed step
        _lib.check(lib.vaicu_graph_capture_begin(stream), "capture")
        for i in range(iters):
            launch(i)
        g = ctypes.c_void_p()
        _lib.check(lib.vaicu_graph_capture_end(stream, ctypes.byref(g)), "capture end")
        _lib.check(lib.vaicu_graph_launch(g, stream), "graph launch")
        lib.vaicu_stream_sync(stream)
        lib.vaicu_event_record(e0, stream)
        _lib.check(lib.vaicu_graph_launch(g, stream), "graph launch")
    else:
        lib.vaicu_event_record(e0, stream)
        for i in range(iters):
            launch(i)
    lib.vaicu_event_record(e1, stream)
    lib.vaicu_event_synchronize(e1)
    ms = ctypes.c_float()
    lib.vaicu_event_elapsed_ms(e0, e1, ctypes.byref(ms))
    dev.check_status()
    clock_info = None
    if sampler is not None:
        import statistics
        import time
        time.sleep(0.15)
        sampler.terminate()
        rows = [ln.split(",") for ln in sampler.stdout.read().strip().splitlines() if ln.strip()]
        mhz = [float(r[0]) for r in rows if r[0].strip().replace(".", "").isdigit()]
        watts = [float(r[1]) for r in rows if len(r) > 1 and r[1].strip().replace(".", "").isdigit()]
        clock_info = {"sm_mhz_median": statistics.median(mhz) if mhz else None, "sm_mhz_min": min(mhz) if mhz else None,
                      "power_w_max": max(watts) if watts else None, "samples": len(mhz),
                      "power_cap_seen": any("Active" in r[2] for r in rows if len(r) > 2),
                      "slowdown_seen": any("Active" in c and "Not" not in c for r in rows for c in r[3:5])}
    us = ms.value * 1e3 / iters
    ab = algorithmic_bytes(M, N, K, i_dt, w_dt, o_dt, bias, residual, gate)
    res = {"M": M, "K": K, "N": N, "dtypes": [i_dtype, w_dtype, o_dtype], "gate": gate, "kernel": info.kernel,
           "split_count": info.split_count, "tile": [info.tile_m, info.tile_n], "launches": info.launches,
           "us_per_call": us, "GBps": ab / us / 1e3, "TFLOPs": 2.0 * M * N * K / us / 1e6, "copies": copies,
           "algorithmic_bytes": ab}
    if clock_info:
        res["clocks"] = clock_info
    for h in plans:
        lib.vaicu_linear_plan_destroy(h)
    for b in weights:
        b.free()
    return res


def run_group(M, K, rows, i_dtype="bf16", w_dtype="bf16", o_dtype="bf16", copies=0, iters=50, warmup=5, device=None, graph=False,
              tuning=None):
    """2-3 plain Linears over the same activations through vaicu_linear_run_group (q / k / v of a block)."""
    dev = device or Device.default()
    lib = dev.lib
    i_dt, w_dt, o_dt = DT[i_dtype], DT[w_dtype], DT[o_dtype]
    n = len(rows)
    w_bytes = sum(rows) * K * dtype_size(w_dt)
    if copies <= 0:
        copies = max(2, min(64, int(np.ceil(300e6 / w_bytes))))
    rng = np.random.default_rng(0)
    x_host = encode(rng.standard_normal((M, K), dtype=np.float32), i_dt)
    xb = DeviceBuffer(dev, x_host.nbytes)
    xb.upload(x_host)
    sets = []
    info = _lib.LinearInfo()
    for _ in range(copies):
        plans, weights = [], []
        for r in rows:
            wb = DeviceBuffer(dev, r * K * dtype_size(w_dt))
            wb.upload(encode(rng.standard_normal((r, K), dtype=np.float32) * 0.02, w_dt))
            d = _lib.LinearDesc()
            d.M, d.N, d.K = M, r, K
            d.i_dtype, d.w_dtype, d.o_dtype, d.b_dtype = int(i_dt), int(w_dt), int(o_dt), int(Dtype.NONE)
            d.scalar_scale = 1.0
            h = ctypes.c_void_p()
            t = _lib.LinearTuning(**(tuning or {}))
            _lib.check(lib.vaicu_linear_plan_create_tuned(dev.handle, ctypes.byref(d), ctypes.byref(t), ctypes.byref(h)), "plan")
            plans.append(h)
            weights.append(wb)
        sets.append(((ctypes.c_void_p * n)(*plans), (ctypes.c_void_p * n)(*[b.ptr for b in weights]), weights))
    _lib.check(lib.vaicu_linear_plan_info(sets[0][0][0], ctypes.byref(info)), "info")
    outs = [DeviceBuffer(dev, M * r * dtype_size(o_dt)) for r in rows]
    oarr = (ctypes.c_void_p * n)(*[b.ptr for b in outs])
    need = ctypes.c_size_t()
    _lib.check(lib.vaicu_linear_group_workspace_bytes(sets[0][0], n, ctypes.byref(need)), "vaicu_linear_group_workspace_bytes")
    ws = DeviceBuffer(dev, need.value) if need.value else None
    stream = dev.create_stream()
    e0, e1 = ctypes.c_void_p(), ctypes.c_void_p()
    lib.vaicu_event_create(ctypes.byref(e0))
    lib.vaicu_event_create(ctypes.byref(e1))

    def launch(i):
        plans, warr, _ = sets[i % copies]
        _lib.check(lib.vaicu_linear_run_group(plans, n, stream, xb.ptr, warr, oarr, ws.ptr if ws else None), "vaicu_linear_run_group")

    for i in range(max(warmup, copies)):
        launch(i)
    lib.vaicu_stream_sync(stream)
    if graph:
        _lib.check(lib.vaicu_graph_capture_begin(stream), "capture")
        for i in range(iters):
            launch(i)
        g = ctypes.c_void_p()
        _lib.check(lib.vaicu_graph_capture_end(stream, ctypes.byref(g)), "capture end")
        _lib.check(lib.vaicu_graph_launch(g, stream), "graph launch")
        lib.vaicu_stream_sync(stream)
        lib.vaicu_event_record(e0, stream)
        _lib.check(lib.vaicu_graph_launch(g, stream), "graph launch")
    else:
        lib.vaicu_event_record(e0, stream)
        for i in range(iters):
            launch(i)
    lib.vaicu_event_record(e1, stream)
    lib.vaicu_event_synchronize(e1)
    ms = ctypes.c_float()
    lib.vaicu_event_elapsed_ms(e0, e1, ctypes.byref(ms))
    dev.check_status()
    us = ms.value * 1e3 / iters
    ab = sum(algorithmic_bytes(M, r, K, i_dt, w_dt, o_dt, False, False, False) for r in rows) - (n - 1) * M * K * dtype_size(i_dt)
    res = {"M": M, "K": K, "group": list(rows), "dtypes": [i_dtype, w_dtype, o_dtype], "kernel": info.kernel,
           "us_per_call": us, "GBps": ab / us / 1e3, "TFLOPs": 2.0 * M * sum(rows) * K / us / 1e6, "copies": copies,
           "algorithmic_bytes": ab}
    for plans, _, weights in sets:
        for h in plans:
            lib.vaicu_linear_plan_destroy(h)
        for b in weights:
            b.free()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, required=True)
    ap.add_argument("--K", type=int, required=True)
    ap.add_argument("--N", type=int, default=0)
    ap.add_argument("--group", default="", help="rows of 2-3 sibling Linears, e.g. 2048,1024,1024: one vaicu_linear_run_group")
    ap.add_argument("--i-dtype", default="f32")
    ap.add_argument("--w-dtype", default="bf16")
    ap.add_argument("--o-dtype", default="f32")
    ap.add_argument("--epilogue", default="NONE")
    ap.add_argument("--gate", action="store_true")
    ap.add_argument("--bias", action="store_true")
    ap.add_argument("--residual", action="store_true")
    ap.add_argument("--kernel", type=int, default=0)
    ap.add_argument("--copies", type=int, default=0)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--split-size", type=int, default=0)
    ap.add_argument("--graph", action="store_true", help="time a replayed recording of the launches")
    ap.add_argument("--clocks", action="store_true", help="sample nvidia-smi SM clock and power during the timed loop")
    ap.add_argument("--tune", default="", help="vaicu_linear_tuning fields, e.g. tc_bn=192,tc_pair=1")
    a = ap.parse_args()
    tuning = {k: int(v) for k, v in (kv.split("=") for kv in a.tune.split(",") if kv)} or None
    if a.group:
        rows = [int(r) for r in a.group.split(",")]
        print(json.dumps(run_group(a.M, a.K, rows, a.i_dtype, a.w_dtype, a.o_dtype, a.copies, a.iters, a.warmup, graph=a.graph, tuning=tuning)))
        return
    if a.N <= 0:
        ap.error("--N or --group is required")
    print(json.dumps(run(a.M, a.K, a.N, a.i_dtype, a.w_dtype, a.o_dtype, a.epilogue, a.gate, a.bias, a.residual,
                         a.kernel, a.copies, a.iters, a.warmup, a.split_size, graph=a.graph, clocks=a.clocks, tuning=tuning)))


if __name__ == "__main__":
    main()
