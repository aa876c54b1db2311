"""Run this package's Linear kernels on torch CUDA tensors.

A thin adapter for harnesses that keep the rest of a model in PyTorch (attention, norms,
embeddings are other operators): one plan per (shape, dtype) set, launched with
vaicu_linear_run on torch's current stream, reading and writing torch tensors in place.
torch supplies memory and streams only; the arithmetic is the library's.

Mirrors the Linear formula of vAi (vai/nodes/linear.h:49-52):
    out = scalar_scale * epilogue(x W^T + bias) + residual      (AFTER_EPILOGUE)
"""
import ctypes

from . import _lib
from .engine import Device, Dtype, Epilogue, ResidualOrder


def _dtype_of(t):
    import torch
    return {torch.float32: Dtype.F32, torch.float16: Dtype.F16, torch.bfloat16: Dtype.BF16}[t.dtype]


class TorchLinear:
    """weight [N, K] (fp16 / bf16 / fp32 torch CUDA tensor, row-major), optional bias [N].
    gate_fuse: weight is [2H, K] gate rows first, output [.., H] = epilogue(gate) * value."""

    def __init__(self, weight, bias=None, *, epilogue=Epilogue.NONE, residual_order=ResidualOrder.AFTER_EPILOGUE,
                 scalar_scale=1.0, split_size=0, gate_fuse=False, out_dtype=None, device=None, kernel=0):
        import torch
        assert weight.is_cuda and weight.is_contiguous() and weight.dim() == 2
        self.torch = torch
        self.dev = device or Device(weight.device.index or 0)
        self.w, self.b = weight, bias
        self.N, self.K = weight.shape
        self.epilogue, self.residual_order = Epilogue(epilogue), ResidualOrder(residual_order)
        self.scalar_scale, self.split_size, self.gate_fuse, self.kernel = float(scalar_scale), int(split_size), bool(gate_fuse), kernel
        self.out_dtype = out_dtype
        self.plans = {}

    def _plan(self, M, x, residual, out_dtype):
        key = (M, x.dtype, out_dtype, residual is not None)
        hit = self.plans.get(key)
        if hit is not None:
            return hit
        torch = self.torch
        d = _lib.LinearDesc()
        d.M, d.N, d.K = M, self.N, self.K
        d.i_dtype, d.w_dtype = int(_dtype_of(x)), int(_dtype_of(self.w))
        d.o_dtype = int({torch.float32: Dtype.F32, torch.float16: Dtype.F16, torch.bfloat16: Dtype.BF16}[out_dtype])
        d.b_dtype = int(Dtype.NONE)
        if self.b is not None:
            d.has_bias, d.b_dtype, d.bias_elems = 1, int(_dtype_of(self.b)), self.N
        if residual is not None:
            d.has_residual, d.residual_elems = 1, 0
        d.residual_order, d.epilogue = int(self.residual_order), int(self.epilogue)
        d.scalar_scale, d.split_size, d.gate_fuse = self.scalar_scale, self.split_size, 1 if self.gate_fuse else 0
        h = ctypes.c_void_p()
        lib = self.dev.lib
        if self.kernel:
            _lib.check(lib.vaicu_linear_plan_create_forced(self.dev.handle, ctypes.byref(d), self.kernel, ctypes.byref(h)), "plan")
        else:
            _lib.check(lib.vaicu_linear_plan_create(self.dev.handle, ctypes.byref(d), ctypes.byref(h)), "plan")
        info = _lib.LinearInfo()
        _lib.check(lib.vaicu_linear_plan_info(h, ctypes.byref(info)), "info")
        ws = torch.empty(max(info.workspace_bytes, 256), dtype=torch.uint8, device=self.w.device)
        hit = (h, info, ws)
        self.plans[key] = hit
        return hit

    def __call__(self, x, residual=None, out=None):
        torch = self.torch
        assert x.is_cuda and x.is_contiguous() and x.shape[-1] == self.K
        M = x.numel() // self.K
        out_dtype = self.out_dtype or (torch.float32 if x.dtype == torch.float32 else x.dtype)
        n_out = self.N // 2 if self.gate_fuse else self.N
        if out is None:
            out = torch.empty(tuple(x.shape[:-1]) + (n_out,), dtype=out_dtype, device=x.device)
        if residual is not None:
            assert residual.is_contiguous() and residual.dtype == out_dtype and residual.numel() == M * n_out
        plan, info, ws = self._plan(M, x, residual, out_dtype)
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(self.dev.lib.vaicu_linear_run(plan, stream, x.data_ptr(), self.w.data_ptr(),
                                                 self.b.data_ptr() if self.b is not None else None,
                                                 residual.data_ptr() if residual is not None else None,
                                                 out.data_ptr(), ws.data_ptr()), "vaicu_linear_run")
        self.last_info = info
        return out

    def __del__(self):
        try:
            for h, _, _ in self.plans.values():
                self.dev.lib.vaicu_linear_plan_destroy(h)
        except Exception:
            pass
