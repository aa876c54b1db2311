"""Python face of the CPU oracle (test infrastructure; see linear_oracle.c).

Two oracles:
  * linear_f64(): the reference's own test oracle — float64 linear + epilogue
    (vAi python/tests/node_check.py:31-38,128-131; nodes/test_linear.py:34-35,
    66-70), written with numpy.
  * linear_c(): the C restatement of the shader arithmetic in fp32
    (linear_oracle.c), which is also the timed CPU baseline.
"""
import ctypes
import math
import os

import numpy as np

from . import build_oracle

F32, F16, NONE, BF16 = 0, 1, 2, 3
EPILOGUES = {"NONE": 0, "RELU": 1, "GELU": 2, "GELU_TANH": 3, "SILU": 4, "SIGMOID": 5}

_erf = np.vectorize(math.erf, otypes=[np.float64])


def epilogue_f64(code, x):
    """float64 epilogues, the functions torch computes in the reference's tests
    (node_check.py:31-38)."""
    x = np.asarray(x, dtype=np.float64)
    if code == 0:
        return x
    if code == 1:
        return np.maximum(x, 0.0)
    if code == 2:
        return 0.5 * x * (1.0 + _erf(x / math.sqrt(2.0)))
    if code == 3:
        return 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))
    if code == 4:
        return x / (1.0 + np.exp(-x))
    if code == 5:
        return 1.0 / (1.0 + np.exp(-x))
    raise ValueError(code)


def linear_f64(x, w, bias=None, residual=None, *, epilogue=0, residual_order=0, scalar_scale=1.0,
               gate_fuse=False):
    """O = s*ep(x w^T + b) + R  (order 0)  or  s*ep(x w^T + b + R)  (order 1), in float64.
    Operands may be any float arrays (already holding the values the device sees)."""
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(w, dtype=np.float64)
    acc = x.reshape(-1, x.shape[-1]) @ w.T
    if bias is not None:
        b = np.asarray(bias, dtype=np.float64).reshape(-1)
        acc = (acc.reshape(-1) + np.resize(b, acc.size)).reshape(acc.shape)
    if gate_fuse:
        h = acc.shape[1] // 2
        out = scalar_scale * (epilogue_f64(epilogue, acc[:, :h]) * acc[:, h:])
        return out
    r = None
    if residual is not None:
        r = np.resize(np.asarray(residual, dtype=np.float64).reshape(-1), acc.size).reshape(acc.shape)
    if r is not None and residual_order == 1:
        return scalar_scale * epilogue_f64(epilogue, acc + r)
    out = scalar_scale * epilogue_f64(epilogue, acc)
    return out + r if r is not None else out


class _Desc(ctypes.Structure):
    _fields_ = [("M", ctypes.c_uint32), ("N", ctypes.c_uint32), ("K", ctypes.c_uint32),
                ("i_dtype", ctypes.c_int32), ("w_dtype", ctypes.c_int32), ("o_dtype", ctypes.c_int32),
                ("b_dtype", ctypes.c_int32), ("has_bias", ctypes.c_int32), ("bias_elems", ctypes.c_uint32),
                ("has_residual", ctypes.c_int32), ("residual_elems", ctypes.c_uint32),
                ("residual_order", ctypes.c_int32), ("epilogue", ctypes.c_int32),
                ("scalar_scale", ctypes.c_float), ("split_size", ctypes.c_uint32), ("gate_fuse", ctypes.c_int32)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build_oracle.build())
        _lib.vai_oracle_f32_to_f16.restype = ctypes.c_uint16
        _lib.vai_oracle_f32_to_f16.argtypes = [ctypes.c_float]
        _lib.vai_oracle_f16_to_f32.restype = ctypes.c_float
        _lib.vai_oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.vai_oracle_f32_to_bf16.restype = ctypes.c_uint16
        _lib.vai_oracle_f32_to_bf16.argtypes = [ctypes.c_float]
        _lib.vai_oracle_bf16_to_f32.restype = ctypes.c_float
        _lib.vai_oracle_bf16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.vai_oracle_epilogue.restype = ctypes.c_float
        _lib.vai_oracle_epilogue.argtypes = [ctypes.c_int, ctypes.c_float]
        _lib.vai_oracle_convert_f32.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t]
        _lib.vai_oracle_widen_f32.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t]
        _lib.vai_oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads():
    return int(lib().vai_oracle_num_threads())


def set_num_threads(n):
    """Use n OpenMP threads whatever OMP_NUM_THREADS said when the process started."""
    lib().vai_oracle_set_num_threads(ctypes.c_int(int(n)))
    return num_threads()


def to_dtype(a, dtype):
    """fp32 array -> device representation (np.float32, or uint16 bit patterns for
    fp16/bf16) using the loader's conversions (vAi vai/engine/tensor.cpp:46-85)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    if dtype == F32:
        return a.copy()
    out = np.empty(a.shape, dtype=np.uint16)
    lib().vai_oracle_convert_f32(a.ctypes.data, out.ctypes.data, dtype, a.size)
    return out


def to_f32(a, dtype):
    """Device representation -> fp32 values."""
    if dtype == F32:
        return np.ascontiguousarray(a, dtype=np.float32)
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().vai_oracle_widen_f32(a.ctypes.data, dtype, out.ctypes.data, a.size)
    return out


def _ptr(a):
    return None if a is None else ctypes.c_void_p(a.ctypes.data)


def make_desc(M, N, K, *, i_dtype=F32, w_dtype=F32, o_dtype=F32, b_dtype=NONE, bias_elems=None,
              residual_elems=None, residual_order=0, epilogue=0, scalar_scale=1.0, split_size=0,
              gate_fuse=False):
    out_elems = M * (N // 2 if gate_fuse else N)
    return _Desc(M, N, K, i_dtype, w_dtype, o_dtype, b_dtype if bias_elems else NONE,
                 1 if bias_elems else 0, 0 if (not bias_elems or bias_elems == M * N) else bias_elems,
                 1 if residual_elems else 0,
                 0 if (not residual_elems or residual_elems == out_elems) else residual_elems,
                 residual_order, epilogue, scalar_scale, split_size, 1 if gate_fuse else 0)


def linear_c(desc, I, W, bias=None, residual=None, path="auto", wg_size=128, stage16=None, stage_dtype=F16):
    """Run the C restatement. Arrays are device representations (float32 / uint16).
    Returns O in its device representation."""
    L = lib()
    n_out = desc.N // 2 if desc.gate_fuse else desc.N
    O = np.empty((desc.M, n_out), dtype=np.float32 if desc.o_dtype == F32 else np.uint16)
    I = np.ascontiguousarray(I)
    W = np.ascontiguousarray(W)
    bias = None if bias is None else np.ascontiguousarray(bias)
    residual = None if residual is None else np.ascontiguousarray(residual)
    if path == "auto":
        rc = L.vai_oracle_linear(ctypes.byref(desc), _ptr(I), _ptr(W), _ptr(bias), _ptr(residual), _ptr(O))
    elif path == "slab":
        rc = L.vai_oracle_linear_slab(ctypes.byref(desc), _ptr(I), _ptr(W), _ptr(bias), _ptr(residual), _ptr(O),
                                      ctypes.c_uint32(wg_size))
    elif path == "tile":
        if stage16 is None:
            stage16 = not (desc.i_dtype == F32 and desc.w_dtype == F32)
        rc = L.vai_oracle_linear_tile(ctypes.byref(desc), _ptr(I), _ptr(W), _ptr(bias), _ptr(residual), _ptr(O),
                                      ctypes.c_int(1 if stage16 else 0), ctypes.c_int(stage_dtype))
    else:
        raise ValueError(path)
    if rc != 0:
        raise RuntimeError(f"oracle returned {rc}")
    return O


def gated_mul_f64(x, epilogue):
    """float64 GLU gating as the reference's test states it (vAi
    python/tests/nodes/test_gated_mul.py:10-13): activation(first half) * second half."""
    x = np.asarray(x, dtype=np.float64)
    h = x.shape[-1] // 2
    return epilogue_f64(epilogue, x[..., :h]) * x[..., h:]


def gated_mul_c(x, epilogue, i_dtype=F32, o_dtype=F32):
    """The C restatement of vAi's gated-mul shader; x [..., 2H] in device representation."""
    x = np.ascontiguousarray(x)
    h = x.shape[-1] // 2
    rows = int(np.prod(x.shape[:-1])) if x.ndim > 1 else 1
    out = np.empty(tuple(x.shape[:-1]) + (h,), dtype=np.float32 if o_dtype == F32 else np.uint16)
    rc = lib().vai_oracle_gated_mul(_ptr(x), _ptr(out), ctypes.c_uint32(rows), ctypes.c_uint32(h), ctypes.c_int(i_dtype),
                                    ctypes.c_int(o_dtype), ctypes.c_int(epilogue))
    if rc != 0:
        raise RuntimeError(f"oracle returned {rc}")
    return out


def argmax_c(logits, dtype=F32):
    """The C restatement of vAi's argmax shader on a [M, N] array in device representation."""
    a = np.ascontiguousarray(logits)
    out = np.empty(a.shape[0], dtype=np.uint32)
    rc = lib().vai_oracle_argmax(ctypes.c_void_p(a.ctypes.data), ctypes.c_int(dtype), ctypes.c_uint32(a.shape[0]),
                                 ctypes.c_uint32(a.shape[1]), ctypes.c_void_p(out.ctypes.data))
    if rc != 0:
        raise RuntimeError(f"oracle returned {rc}")
    return out


def rms_norm_f64(x, scale=None, shift=None, residual=None, eps=1e-5):
    """float64 RMS norm, what torch.nn.functional.rms_norm computes in the reference's tests
    (vAi python/tests/nodes/test_rms_norm.py)."""
    x = np.asarray(x, dtype=np.float64)
    out = x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    if scale is not None:
        out = out * np.asarray(scale, dtype=np.float64).reshape(-1)
    if shift is not None:
        out = out + np.asarray(shift, dtype=np.float64).reshape(-1)
    if residual is not None:
        out = out + np.asarray(residual, dtype=np.float64)
    return out


def rms_norm_c(x, scale=None, shift=None, residual=None, eps=1e-5, i_dtype=F32, w_dtype=F32, o_dtype=F32, wg_size=32):
    """The C restatement of vAi's rms-norm shader; arrays in device representation."""
    x = np.ascontiguousarray(x)
    rows, feat = int(np.prod(x.shape[:-1])), x.shape[-1]
    out = np.empty(x.shape, dtype=np.float32 if o_dtype == F32 else np.uint16)
    keep = [None if a is None else np.ascontiguousarray(a) for a in (scale, shift, residual)]
    rc = lib().vai_oracle_rms_norm(_ptr(x), _ptr(keep[0]), _ptr(keep[1]), _ptr(keep[2]), _ptr(out), ctypes.c_uint32(rows),
                                   ctypes.c_uint32(feat), ctypes.c_int(i_dtype), ctypes.c_int(w_dtype), ctypes.c_int(o_dtype),
                                   ctypes.c_float(eps), ctypes.c_uint32(wg_size))
    if rc != 0:
        raise RuntimeError(f"oracle returned {rc}")
    return out


def layer_norm_f64(x, scale, shift=None, residual=None, eps=1e-5):
    """float64 layer norm, what torch.nn.functional.layer_norm computes in the reference's
    tests (vAi python/tests/nodes/test_layer_norm.py): biased variance over the last axis."""
    x = np.asarray(x, dtype=np.float64)
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    out = (x - mean) / np.sqrt(var + eps) * np.asarray(scale, dtype=np.float64).reshape(-1)
    if shift is not None:
        out = out + np.asarray(shift, dtype=np.float64).reshape(-1)
    if residual is not None:
        out = out + np.asarray(residual, dtype=np.float64)
    return out


def layer_norm_wg_size(feat, subgroup=32):
    """Threads per row the reference picks (vAi vai/nodes/layer-norm.h:73-88)."""
    cap = min(16 * subgroup, 1024)
    wg = subgroup
    while wg * 4 < feat and wg < cap:
        wg *= 2
    return wg


def layer_norm_c(x, scale, shift=None, residual=None, eps=1e-5, i_dtype=F32, w_dtype=F32, o_dtype=F32, wg_size=None):
    """The C restatement of vAi's layer-norm shader; arrays in device representation."""
    x = np.ascontiguousarray(x)
    rows, feat = int(np.prod(x.shape[:-1])), x.shape[-1]
    out = np.empty(x.shape, dtype=np.float32 if o_dtype == F32 else np.uint16)
    keep = [None if a is None else np.ascontiguousarray(a) for a in (scale, shift, residual)]
    wg = wg_size or layer_norm_wg_size(feat)
    rc = lib().vai_oracle_layer_norm(_ptr(x), _ptr(keep[0]), _ptr(keep[1]), _ptr(keep[2]), _ptr(out), ctypes.c_uint32(rows),
                                     ctypes.c_uint32(feat), ctypes.c_int(i_dtype), ctypes.c_int(w_dtype), ctypes.c_int(o_dtype),
                                     ctypes.c_float(eps), ctypes.c_uint32(wg))
    if rc != 0:
        raise RuntimeError(f"oracle returned {rc}")
    return out


def topk_sample_c(logits, k, temperature, u):
    """The C restatement of vAi's top-k sampling shader on fp32 logits [M, N]; returns uint32 [M]."""
    a = np.ascontiguousarray(logits, dtype=np.float32)
    out = np.empty(a.shape[0], dtype=np.uint32)
    rc = lib().vai_oracle_topk_sample(_ptr(a), ctypes.c_uint32(a.shape[0]), ctypes.c_uint32(a.shape[1]), ctypes.c_uint32(k),
                                      ctypes.c_float(temperature), ctypes.c_float(u), _ptr(out))
    if rc != 0:
        raise RuntimeError(f"oracle returned {rc}")
    return out


def topk_candidates_c(logits, k, index_base=0):
    """Per-slab step of the vocabulary-split top-k: (values [M, k] fp32, indices [M, k] uint32), the k
    best of each row in rank order with index_base added; short slabs pad with (lowest, 0xFFFFFFFF)."""
    a = np.ascontiguousarray(logits, dtype=np.float32)
    vals = np.empty((a.shape[0], k), dtype=np.float32)
    idxs = np.empty((a.shape[0], k), dtype=np.uint32)
    rc = lib().vai_oracle_topk_candidates(_ptr(a), ctypes.c_uint32(a.shape[0]), ctypes.c_uint32(a.shape[1]), ctypes.c_uint32(k),
                                          ctypes.c_uint32(index_base), _ptr(vals), _ptr(idxs))
    if rc != 0:
        raise RuntimeError(f"oracle returned {rc}")
    return vals, idxs


def topk_merge_sample_c(vals, idxs, k, temperature, u):
    """Merge step: vals / idxs [groups, M, list_len] candidate lists -> sampled uint32 [M]."""
    v = np.ascontiguousarray(vals, dtype=np.float32)
    i = np.ascontiguousarray(idxs, dtype=np.uint32)
    groups, M, list_len = v.shape
    out = np.empty(M, dtype=np.uint32)
    rc = lib().vai_oracle_topk_merge_sample(_ptr(v), _ptr(i), ctypes.c_uint32(groups), ctypes.c_size_t(M * list_len), ctypes.c_uint32(M),
                                            ctypes.c_uint32(list_len), ctypes.c_uint32(k), ctypes.c_float(temperature), ctypes.c_float(u),
                                            _ptr(out))
    if rc != 0:
        raise RuntimeError(f"oracle returned {rc}")
    return out


def topk_probabilities_f64(logits, k, temperature):
    """float64 view of the same distribution: (indices [M, k] in rank order, probabilities
    [M, k]); ties rank the lower index first."""
    a = np.asarray(logits, dtype=np.float64)
    k = min(k, a.shape[1])
    order = np.lexsort((np.arange(a.shape[1])[None, :].repeat(a.shape[0], 0), -a), axis=1)[:, :k]
    top = np.take_along_axis(a, order, axis=1)
    e = np.exp((top - top[:, :1]) / max(temperature, 1e-6))
    return order.astype(np.uint32), e / e.sum(axis=1, keepdims=True)
