"""Column split of a large-N Linear across the GPUs of one host.

Output columns are independent (O[:, n0:n1] = ep(I . W[n0:n1, :]^T + b[n0:n1])) and W is
stored [N, K] row-major, so rank r of g simply owns a contiguous row slab of W and the
matching bias slice; the activations are replicated.  With a fused gate|value weight
([2H, K], gate rows first, vAi vai/groups/gated-feed-forward.h:38) the split is per
half, so the gate epilogue stays local: rank r holds gate rows [b, b+c) and value rows
[H+b, H+b+c) stacked as a private [2c, K] copy.  After the local Linear the output
slabs [M, c_r] are all-gathered over NVLink (NCCL) and laid side by side.

The reference is single-device; nothing here has a counterpart in it.  The row
arithmetic comes from the C ABI (vaicu_linear_shard_desc) so that C++ hosts split
identically.  torch is used for what it is here for: device tensors that
torch.distributed can gather.  `ShardedLinear.forward` launches this package's kernels
through vaicu_linear_run on the current torch stream; no TMA descriptor ever points at
another GPU's memory (remote slabs arrive through the all-gather first).
"""
import ctypes

import numpy as np

from . import _lib


def shard_rows(n_out, world, rank):
    """(begin, count) of rank's output columns when n_out columns are split as evenly as
    possible (the first n_out % world ranks take one more).  Mirrors
    vaicu_linear_shard_desc."""
    base, extra = divmod(n_out, world)
    return rank * base + min(rank, extra), base + (1 if rank < extra else 0)


def shard_desc(full, rank, world):
    """Ask the library for rank's desc; returns (LinearDesc, begin, count)."""
    lib = _lib.load()
    out = _lib.LinearDesc()
    b, c = ctypes.c_uint32(), ctypes.c_uint32()
    _lib.check(lib.vaicu_linear_shard_desc(ctypes.byref(full), rank, world, ctypes.byref(out), ctypes.byref(b), ctypes.byref(c)),
               "vaicu_linear_shard_desc")
    return out, b.value, c.value


def slice_weight(w, rank, world, gate_fuse=False):
    """Rank's rows of W [N, K] (any array type with numpy-style slicing).  For a
    gate|value weight: its gate rows followed by its value rows."""
    n = w.shape[0]
    if not gate_fuse:
        b, c = shard_rows(n, world, rank)
        return w[b:b + c]
    h = n // 2
    b, c = shard_rows(h, world, rank)
    if hasattr(w, "numpy") or not isinstance(w, np.ndarray):   # torch tensor
        import torch
        return torch.cat([w[b:b + c], w[h + b:h + b + c]], dim=0)
    return np.concatenate([w[b:b + c], w[h + b:h + b + c]], axis=0)


def slice_bias(bias, rank, world, gate_fuse=False):
    return None if bias is None else slice_weight(bias, rank, world, gate_fuse)


def gathered_shape(m, n_out, world):
    """Shape of the all-gather target: every rank contributes [M, cmax] (slabs narrower
    than cmax are padded on the right)."""
    return (world, m, shard_rows(n_out, world, 0)[1])


def assemble(gathered, n_out):
    """[world, M, cmax] slabs -> O [M, n_out]."""
    world, m = gathered.shape[0], gathered.shape[1]
    parts = []
    for r in range(world):
        _, c = shard_rows(n_out, world, r)
        parts.append(gathered[r, :, :c])
    if isinstance(gathered, np.ndarray):
        return np.concatenate(parts, axis=1)
    import torch
    return torch.cat(parts, dim=1)


class ShardedLinear:
    """Rank-local slab of a column-split Linear on the GPU, plus the all-gather.

    x: torch CUDA tensor [M, K]; returns O [M, n_out] on every rank.  Weights are given
    as the FULL [N, K] torch tensor on the host (or device); only this rank's rows are
    kept."""

    def __init__(self, device, dist, full_desc, weight, bias=None):
        import torch
        self.torch = torch
        self.dist = dist
        self.dev = device
        self.rank = dist.get_rank() if dist is not None else 0
        self.world = dist.get_world_size() if dist is not None else 1
        self.full = full_desc
        self.gate = bool(full_desc.gate_fuse)
        self.n_out = full_desc.N // 2 if self.gate else full_desc.N
        self.desc, self.begin, self.count = shard_desc(full_desc, self.rank, self.world)
        cuda = torch.device("cuda", device.ordinal)
        self.w = slice_weight(weight, self.rank, self.world, self.gate).contiguous().to(cuda)
        self.b = None if bias is None else slice_bias(bias, self.rank, self.world, self.gate).contiguous().to(cuda)
        lib = device.lib
        h = ctypes.c_void_p()
        _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(self.desc), ctypes.byref(h)), "plan")
        self.plan = h
        self.info = _lib.LinearInfo()
        _lib.check(lib.vaicu_linear_plan_info(h, ctypes.byref(self.info)), "info")
        self.ws = torch.empty(max(self.info.workspace_bytes, 256), dtype=torch.uint8, device=cuda)
        o_dt = {0: torch.float32, 1: torch.float16, 3: torch.bfloat16}[self.desc.o_dtype]
        cmax = gathered_shape(self.desc.M, self.n_out, self.world)[2]
        self.local = torch.zeros((self.desc.M, cmax), dtype=o_dt, device=cuda)
        self.slab = self.local if cmax == self.count else torch.empty((self.desc.M, self.count), dtype=o_dt, device=cuda)
        self.gathered = torch.empty((self.world, self.desc.M, cmax), dtype=o_dt, device=cuda)

    def local_forward(self, x):
        """This rank's slab only: one vaicu_linear_run on the current torch stream."""
        stream = self.torch.cuda.current_stream().cuda_stream
        _lib.check(self.dev.lib.vaicu_linear_run(self.plan, stream, x.data_ptr(), self.w.data_ptr(),
                                                 self.b.data_ptr() if self.b is not None else None, None,
                                                 self.slab.data_ptr(), self.ws.data_ptr()), "vaicu_linear_run")
        if self.slab is not self.local:
            self.local[:, :self.count].copy_(self.slab)
        return self.local

    def forward(self, x, assemble_output=True):
        local = self.local_forward(x)
        if self.world == 1:
            return local[:, :self.count]
        self.dist.all_gather_into_tensor(self.gathered, local)
        return assemble(self.gathered, self.n_out) if assemble_output else self.gathered
