"""ctypes binding of libvaicu.so (the C ABI declared in include/vaicu.h).

The library is the product path; there is no fallback.  If the shared object is
missing, load() raises with the command that builds it.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libvaicu.so")

c_void_pp = ctypes.POINTER(ctypes.c_void_p)


class LinearDesc(ctypes.Structure):
    """struct vaicu_linear_desc."""
    _fields_ = [("M", ctypes.c_uint32), ("N", ctypes.c_uint32), ("K", ctypes.c_uint32),
                ("i_dtype", ctypes.c_int32), ("w_dtype", ctypes.c_int32), ("o_dtype", ctypes.c_int32),
                ("b_dtype", ctypes.c_int32), ("has_bias", ctypes.c_int32), ("bias_elems", ctypes.c_uint32),
                ("has_residual", ctypes.c_int32), ("residual_elems", ctypes.c_uint32),
                ("residual_order", ctypes.c_int32), ("epilogue", ctypes.c_int32),
                ("scalar_scale", ctypes.c_float), ("split_size", ctypes.c_uint32), ("gate_fuse", ctypes.c_int32)]


class LinearInfo(ctypes.Structure):
    """struct vaicu_linear_info."""
    _fields_ = [("kernel", ctypes.c_int32), ("split_count", ctypes.c_uint32), ("tile_m", ctypes.c_uint32),
                ("tile_n", ctypes.c_uint32), ("launches", ctypes.c_uint32), ("workspace_bytes", ctypes.c_size_t)]


class LinearTuning(ctypes.Structure):
    """struct vaicu_linear_tuning; a fresh instance means "the library's choice" everywhere."""
    _fields_ = [("kernel", ctypes.c_int32), ("tc_pair", ctypes.c_int32), ("tc_wide", ctypes.c_int32),
                ("tc_bn", ctypes.c_uint32), ("tc_splits", ctypes.c_uint32), ("gemv_rows", ctypes.c_int32),
                ("gemv_k_warps", ctypes.c_int32), ("gemv_unroll", ctypes.c_int32), ("gemv_grid", ctypes.c_int32),
                ("gemv_plain_launch", ctypes.c_int32), ("tc_fold", ctypes.c_int32),
                ("tc_tail_strips", ctypes.c_int32), ("tc_tile_rows", ctypes.c_uint32),
                ("tc_stages", ctypes.c_uint32)]

    def __init__(self, **kw):
        super().__init__()
        self.tc_pair = self.tc_wide = -1
        for k, v in kw.items():
            if k not in dict(self._fields_):
                raise TypeError(f"no tuning field {k}")
            setattr(self, k, int(v))


# name -> (restype, argtypes); every function include/vaicu.h declares
SIGNATURES = {
    "vaicu_device_open": (ctypes.c_int, [ctypes.c_int, c_void_pp]),
    "vaicu_device_close": (ctypes.c_int, [ctypes.c_void_p]),
    "vaicu_device_sm_count": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]),
    "vaicu_device_synchronize": (ctypes.c_int, [ctypes.c_void_p]),
    "vaicu_device_status": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]),
    "vaicu_device_selftest_wait_expiry": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "vaicu_buffer_alloc": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_size_t, c_void_pp]),
    "vaicu_buffer_free": (ctypes.c_int, [ctypes.c_void_p]),
    "vaicu_buffer_ptr": (ctypes.c_void_p, [ctypes.c_void_p]),
    "vaicu_buffer_size": (ctypes.c_size_t, [ctypes.c_void_p]),
    "vaicu_memcpy_h2d": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "vaicu_memcpy_d2h": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "vaicu_memset": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_void_p]),
    "vaicu_host_alloc_pinned": (ctypes.c_int, [ctypes.c_size_t, c_void_pp]),
    "vaicu_host_free_pinned": (ctypes.c_int, [ctypes.c_void_p]),
    "vaicu_stream_create": (ctypes.c_int, [ctypes.c_void_p, c_void_pp]),
    "vaicu_stream_sync": (ctypes.c_int, [ctypes.c_void_p]),
    "vaicu_stream_destroy": (ctypes.c_int, [ctypes.c_void_p]),
    "vaicu_stream_wait_stream": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "vaicu_event_create": (ctypes.c_int, [c_void_pp]),
    "vaicu_event_record": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "vaicu_event_synchronize": (ctypes.c_int, [ctypes.c_void_p]),
    "vaicu_event_elapsed_ms": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)]),
    "vaicu_event_destroy": (ctypes.c_int, [ctypes.c_void_p]),
    "vaicu_graph_capture_begin": (ctypes.c_int, [ctypes.c_void_p]),
    "vaicu_graph_capture_end": (ctypes.c_int, [ctypes.c_void_p, c_void_pp]),
    "vaicu_graph_launch": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "vaicu_graph_destroy": (ctypes.c_int, [ctypes.c_void_p]),
    "vaicu_linear_plan_create": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(LinearDesc), c_void_pp]),
    "vaicu_linear_plan_create_forced": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(LinearDesc), ctypes.c_int, c_void_pp]),
    "vaicu_linear_plan_create_tuned": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(LinearDesc), ctypes.POINTER(LinearTuning), c_void_pp]),
    "vaicu_linear_plan_destroy": (ctypes.c_int, [ctypes.c_void_p]),
    "vaicu_linear_plan_info": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(LinearInfo)]),
    "vaicu_linear_plan_last_run": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]),
    "vaicu_linear_workspace_bytes": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_size_t)]),
    "vaicu_linear_run": (ctypes.c_int, [ctypes.c_void_p] * 8),
    "vaicu_linear_argmax_workspace_bytes": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_size_t)]),
    "vaicu_linear_run_argmax": (ctypes.c_int, [ctypes.c_void_p] * 8 + [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p]),
    "vaicu_linear_group_workspace_bytes": (ctypes.c_int, [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                                          ctypes.POINTER(ctypes.c_size_t)]),
    "vaicu_linear_run_group": (ctypes.c_int, [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                              ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]),
    "vaicu_linear_run_scatter": (ctypes.c_int, [ctypes.c_void_p] * 5 + [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                                                        ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p]),
    "vaicu_linear_run_broadcast": (ctypes.c_int, [ctypes.c_void_p] * 6 + [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_void_p]),
    "vaicu_linear_run_reduce_scatter": (ctypes.c_int, [ctypes.c_void_p] * 4 + [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "vaicu_partial_fold_run": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32,
                                              ctypes.c_int, ctypes.c_void_p, ctypes.c_float, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                              ctypes.c_int, ctypes.c_uint32]),
    "vaicu_peer_barrier_run": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "vaicu_ipc_export": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    "vaicu_ipc_open": (ctypes.c_int, [ctypes.c_void_p, c_void_pp]),
    "vaicu_ipc_close": (ctypes.c_int, [ctypes.c_void_p]),
    "vaicu_linear_splitk_static": (ctypes.c_int, [ctypes.POINTER(LinearDesc)] + [ctypes.c_void_p] * 6),
    "vaicu_rms_norm_run": (ctypes.c_int, [ctypes.c_void_p] * 7 + [ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int, ctypes.c_int,
                                                                   ctypes.c_int, ctypes.c_float]),
    "vaicu_layer_norm_run": (ctypes.c_int, [ctypes.c_void_p] * 7 + [ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int, ctypes.c_int,
                                                                   ctypes.c_int, ctypes.c_float]),
    "vaicu_gated_mul_run": (ctypes.c_int, [ctypes.c_void_p] * 4 + [ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int, ctypes.c_int, ctypes.c_int]),
    "vaicu_argmax_run": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p]),
    "vaicu_argmax_workspace_bytes": (ctypes.c_int, [ctypes.c_uint32, ctypes.c_uint32, ctypes.POINTER(ctypes.c_size_t)]),
    "vaicu_argmax_pairs_run": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32,
                                              ctypes.c_size_t, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "vaicu_argmax_merge_run": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_size_t,
                                              ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p]),
    "vaicu_topk_workspace_bytes": (ctypes.c_int, [ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.POINTER(ctypes.c_size_t)]),
    "vaicu_topk_sample_run": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32,
                                             ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "vaicu_topk_candidates_run": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_size_t,
                                                 ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p]),
    "vaicu_topk_merge_sample_run": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_size_t, ctypes.c_uint32,
                                                   ctypes.c_uint32, ctypes.c_uint32, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]),
    "vaicu_linear_shard_desc": (ctypes.c_int, [ctypes.POINTER(LinearDesc), ctypes.c_int, ctypes.c_int,
                                               ctypes.POINTER(LinearDesc), ctypes.POINTER(ctypes.c_uint32),
                                               ctypes.POINTER(ctypes.c_uint32)]),
    "vaicu_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "vaicu_last_cuda_error": (ctypes.c_char_p, []),
    "vaicu_version": (ctypes.c_int, []),
}

_lib = None


class VaicuError(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        detail = _lib.vaicu_last_cuda_error().decode() if _lib is not None else ""
        text = _lib.vaicu_status_string(status).decode() if _lib is not None else str(status)
        super().__init__(f"{where}: {text} (status {status})" + (f" [{detail}]" if detail and status in (3, 4) else ""))


def load():
    """Load libvaicu.so and attach the signatures.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m vai_b200.build` "
                           "(there is no CPU or PyTorch fallback for this path)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status, where):
    if status != 0:
        raise VaicuError(status, where)
