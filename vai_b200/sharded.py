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


def destination_order(rank, world):
    """Ranks in the order rank `rank` stores to them: its right-hand neighbour first, itself
    last, so that at any moment the `world` ranks write to `world` different GPUs."""
    return [(rank + 1 + i) % world for i in range(world)]


class _CudaView:
    """A [rows, cols] view of a device range for torch.as_tensor (CUDA array interface)."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 3}


def share_buffer(device, dist, nbytes, zero=False):
    """One cudaMalloc'ed range per rank, opened by every other rank through CUDA IPC.  Returns
    (own DeviceBuffer, [pointer to rank r's range for r in range(world)], [opened pointers to close])."""
    from .engine import DeviceBuffer
    lib = device.lib
    rank, world = dist.get_rank(), dist.get_world_size()
    own = DeviceBuffer(device, nbytes)
    if zero:
        _lib.check(lib.vaicu_memset(own.ptr, 0, nbytes, None), "vaicu_memset")
        device.synchronize()
    handle = (ctypes.c_uint8 * 64)()
    _lib.check(lib.vaicu_ipc_export(own.ptr, handle), "vaicu_ipc_export")
    handles = [None] * world
    dist.all_gather_object(handles, bytes(handle))
    by_rank, opened = [], []
    for r, raw in enumerate(handles):
        if r == rank:
            by_rank.append(own.ptr)
            continue
        p = ctypes.c_void_p()
        _lib.check(lib.vaicu_ipc_open((ctypes.c_uint8 * 64).from_buffer_copy(raw), ctypes.byref(p)), "vaicu_ipc_open")
        opened.append(p)
        by_rank.append(p.value)
    return own, by_rank, opened


class PeerBarrier:
    """Barrier between the ranks' streams without a library collective: one single-warp kernel per
    GPU that signals every peer through flag words in their memory and waits, bounded, for theirs
    (vaicu_peer_barrier_run).  What a rank stored into its peers' buffers before the barrier is
    visible to them after it.  A few microseconds, where a 4-byte NCCL all-reduce costs tens.
    The wait is bounded (about half a second): ranks are expected to enqueue their steps together, as
    the ranks of a serving job do; a rank that finds no peer within the limit records the device
    status word (vaicu_device_status -> VAICU_ERR_TIMEOUT) and carries on."""

    def __init__(self, device, dist):
        from .engine import DeviceBuffer
        self.dev, self.rank, self.world = device, dist.get_rank(), dist.get_world_size()
        self.flags, by_rank, self._opened = share_buffer(device, dist, 256, zero=True)
        self.ptrs = (ctypes.c_void_p * self.world)(*by_rank)
        self.epoch = DeviceBuffer(device, 256)
        _lib.check(device.lib.vaicu_memset(self.epoch.ptr, 0, 256, None), "vaicu_memset")
        device.synchronize()
        dist.barrier()          # every rank's flags are zero and mapped before the first kernel signals

    def run(self, stream):
        _lib.check(self.dev.lib.vaicu_peer_barrier_run(self.dev.handle, stream, self.ptrs, self.world, self.rank, self.epoch.ptr),
                   "vaicu_peer_barrier_run")

    def close(self):
        for p in self._opened:
            self.dev.lib.vaicu_ipc_close(p)
        self._opened = []


class FusedGatherLinear(ShardedLinear):
    """Column-split Linear whose tensor-core epilogue writes this rank's slab straight into
    every rank's [M, n_out] output (vaicu_linear_run_scatter): the all-gather happens
    tile by tile as plain stores over NVLink, followed by a barrier kernel (PeerBarrier) that
    tells every rank that all slabs have landed; no library collective is left on the path.

    The outputs are cudaMalloc'ed ranges shared through CUDA IPC handles; no TMA descriptor
    and no multicast load touches peer memory — peers are only ever stored to.

    Two hazards of writing into other ranks' memory are handled here.  (1) Every rank would
    otherwise walk the destinations in the same order and all of them would store to rank 0
    at once, then to rank 1, ...: each rank's destination list starts with its right-hand
    neighbour and ends with itself.  (2) A fast rank may start call n + 1 while a slow rank's
    consumers of call n still read its output; two outputs alternate by call parity, so a
    store of call n + 1 lands in the buffer nobody has read since call n - 1, and the flag
    barrier of call n (which every rank passes only after its readers of call n - 1 were
    enqueued ahead of it on the same stream) orders that reuse."""

    def __init__(self, device, dist, full_desc, w_local, bias_local=None):
        import torch
        self.torch, self.dist, self.dev = torch, dist, device
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.full = full_desc
        self.gate = bool(full_desc.gate_fuse)
        self.n_out = full_desc.N // 2 if self.gate else full_desc.N
        self.desc, self.begin, self.count = shard_desc(full_desc, self.rank, self.world)
        self.desc.split_size = max(32, full_desc.K)     # one K span: a split-K fold cannot scatter
        self.w, self.b = w_local, bias_local
        lib = device.lib
        h = ctypes.c_void_p()
        _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(self.desc), ctypes.byref(h)), "plan")
        self.plan = h
        self.info = _lib.LinearInfo()
        _lib.check(lib.vaicu_linear_plan_info(h, ctypes.byref(self.info)), "info")
        cuda = torch.device("cuda", device.ordinal)
        self.ws = torch.empty(max(self.info.workspace_bytes, 256), dtype=torch.uint8, device=cuda)
        from .engine import DeviceBuffer
        esz = 4 if self.desc.o_dtype == 0 else 2
        self._opened = []
        self.outs, self.ptrs, self.results = [], [], []
        typestr = {0: "<f4", 1: "<f2", 3: "<u2"}[self.desc.o_dtype]
        for parity in range(2):
            out = DeviceBuffer(device, self.desc.M * self.n_out * esz)      # a gathered [M, n_out] of this rank
            handle = (ctypes.c_uint8 * 64)()
            _lib.check(lib.vaicu_ipc_export(out.ptr, handle), "vaicu_ipc_export")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle))
            by_rank = []
            for r, raw in enumerate(handles):
                if r == self.rank:
                    by_rank.append(out.ptr)
                    continue
                p = ctypes.c_void_p()
                _lib.check(lib.vaicu_ipc_open((ctypes.c_uint8 * 64).from_buffer_copy(raw), ctypes.byref(p)), "vaicu_ipc_open")
                self._opened.append(p)
                by_rank.append(p.value)
            order = destination_order(self.rank, self.world)
            self.outs.append(out)
            self.ptrs.append((ctypes.c_void_p * self.world)(*[by_rank[r] for r in order]))
            view = torch.as_tensor(_CudaView(out.ptr, (self.desc.M, self.n_out), typestr), device=cuda)
            self.results.append(view.view(torch.bfloat16) if self.desc.o_dtype == 3 else view)
        self.calls = 0
        self.barrier = PeerBarrier(device, dist)

    def forward(self, x):
        stream = self.torch.cuda.current_stream().cuda_stream
        parity = self.calls & 1
        self.calls += 1
        _lib.check(self.dev.lib.vaicu_linear_run_scatter(self.plan, stream, x.data_ptr(), self.w.data_ptr(),
                                                         self.b.data_ptr() if self.b is not None else None,
                                                         self.ptrs[parity], self.world, self.n_out, self.begin,
                                                         self.ws.data_ptr()), "vaicu_linear_run_scatter")
        # every rank's kernel precedes its signal on the stream: behind the barrier all slabs
        # are in this rank's output
        self.barrier.run(stream)
        return self.results[parity]

    def close(self):
        self.barrier.close()
        for p in self._opened:
            self.dev.lib.vaicu_ipc_close(p)
        self._opened = []


def shard_k(k, world, rank, align=8):
    """(begin, count) of rank's slice of the reduction axis K, in multiples of `align`
    elements (16 bytes of a 16-bit weight row) so that every slice keeps the fast kernels."""
    units = k // align
    base, extra = divmod(units, world)
    begin = (rank * base + min(rank, extra)) * align
    count = (base + (1 if rank < extra else 0)) * align
    if rank == world - 1:
        count = k - begin          # a tail that is not a multiple of `align` goes to the last rank
    return begin, count


def slice_weight_k(w, rank, world):
    """Rank's columns W[:, k0:k1] of W [N, K] as a contiguous array (row-parallel split)."""
    b, c = shard_k(w.shape[1], world, rank)
    part = w[:, b:b + c]
    return part.contiguous() if hasattr(part, "contiguous") else np.ascontiguousarray(part)


class RowParallelLinear:
    """The second half of a tensor-parallel MLP: `down` split along K.  After a column-split
    gate|value Linear every rank already holds columns [k0, k1) of the hidden state, which
    are exactly the activations its K slice of `down` needs, so the hidden state is never
    gathered: each rank multiplies its slice (fp32 partial output [M, N]) and one all-reduce
    sums the partials (48 MiB at M = 8192, d = 3072, against 128 MiB for gathering the hidden
    state).  Bias, residual, epilogue and scale apply after the sum, on every rank alike; only
    the plain `O = sum + R` form that the models' down projections use is provided here."""

    def __init__(self, device, dist, M, N, K, w_local, w_dtype, residual=False, scalar_scale=1.0):
        import torch

        from .engine import Dtype
        self.torch, self.dist, self.dev = torch, dist, device
        self.rank = dist.get_rank() if dist is not None else 0
        self.world = dist.get_world_size() if dist is not None else 1
        self.k_begin, self.k_count = shard_k(K, self.world, self.rank)
        d = _lib.LinearDesc()
        d.M, d.N, d.K = M, N, self.k_count
        d.i_dtype = d.w_dtype = int(w_dtype)
        d.o_dtype = int(Dtype.F32)               # partial sums stay fp32 until after the reduction
        d.b_dtype = int(Dtype.NONE)
        d.scalar_scale = 1.0
        self.desc, self.scale, self.residual = d, float(scalar_scale), residual
        self.w = w_local
        h = ctypes.c_void_p()
        _lib.check(device.lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(h)), "plan")
        self.plan = h
        self.info = _lib.LinearInfo()
        _lib.check(device.lib.vaicu_linear_plan_info(h, ctypes.byref(self.info)), "info")
        cuda = torch.device("cuda", device.ordinal)
        self.ws = torch.empty(max(self.info.workspace_bytes, 256), dtype=torch.uint8, device=cuda)
        self.partial = torch.empty((M, N), dtype=torch.float32, device=cuda)

    def local_forward(self, x_slice):
        stream = self.torch.cuda.current_stream().cuda_stream
        _lib.check(self.dev.lib.vaicu_linear_run(self.plan, stream, x_slice.data_ptr(), self.w.data_ptr(), None, None,
                                                 self.partial.data_ptr(), self.ws.data_ptr()), "vaicu_linear_run")
        return self.partial

    def forward(self, x_slice, residual=None):
        """x_slice: this rank's columns [k0, k1) of the activations, contiguous [M, k_count]."""
        out = self.local_forward(x_slice)
        if self.world > 1:
            self.dist.all_reduce(out)
        if self.scale != 1.0:
            out.mul_(self.scale)
        if residual is not None:
            out.add_(residual)
        return out

    def close(self):
        if self.plan:
            self.dev.lib.vaicu_linear_plan_destroy(self.plan)
            self.plan = None


class FusedRowParallelLinear:
    """`down` split along K with the reduction done by this package's kernels over NVLink instead
    of an all-reduce after the GEMM:

      1. the GEMM's epilogue stores every finished tile of partial sums straight into the staging
         buffer of the GPU that owns those rows (vaicu_linear_run_reduce_scatter): the
         reduce-scatter traffic overlaps the remaining tiles;
      2. barrier; each GPU adds the `world` slabs it received for its M / world rows, applies scale and
         residual, and stores the finished rows into every GPU's output (vaicu_partial_fold_run): that
         is the all-gather;
      3. barrier; the [M, N] output is complete everywhere.

    Partial sums cross the link in `part_dtype` and are added in fp32.  fp32 is the default of the
    callers here: 16-bit partials halve the bytes but lose accuracy where the ranks' partial sums
    cancel (the rounding is relative to the partials, not to their sum).
    Two barriers per call order every reuse of the staging and output buffers across calls."""

    def __init__(self, device, dist, M, N, K, w_local, w_dtype, part_dtype=0, scalar_scale=1.0):
        import torch

        from .engine import Dtype
        self.torch, self.dist, self.dev = torch, dist, device
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        if M % self.world:
            raise ValueError("M must be divisible by the number of ranks")
        self.M, self.N, self.rows = M, N, M // self.world
        self.k_begin, self.k_count = shard_k(K, self.world, self.rank)
        self.part_dtype = Dtype(part_dtype)
        self.o_dtype = Dtype(w_dtype)
        d = _lib.LinearDesc()
        d.M, d.N, d.K = M, N, self.k_count
        d.i_dtype = d.w_dtype = int(w_dtype)
        d.o_dtype = int(self.part_dtype)
        d.b_dtype = int(Dtype.NONE)
        d.scalar_scale = 1.0
        d.split_size = max(32, self.k_count)         # one K span: the partials leave through the epilogue
        self.desc, self.scale, self.w = d, float(scalar_scale), w_local
        lib = device.lib
        h = ctypes.c_void_p()
        _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(h)), "plan")
        self.plan = h
        self.info = _lib.LinearInfo()
        _lib.check(lib.vaicu_linear_plan_info(h, ctypes.byref(self.info)), "info")
        cuda = torch.device("cuda", device.ordinal)
        self.ws = torch.empty(max(self.info.workspace_bytes, 256), dtype=torch.uint8, device=cuda)
        psz = 4 if self.part_dtype == Dtype.F32 else 2
        osz = 4 if self.o_dtype == Dtype.F32 else 2
        self._opened = []
        self.staging, by_rank, opened = share_buffer(device, dist, self.world * self.rows * N * psz)
        self._opened += opened
        self.staging_ptrs = (ctypes.c_void_p * self.world)(*by_rank)
        self.out, by_rank, opened = share_buffer(device, dist, M * N * osz)
        self._opened += opened
        order = destination_order(self.rank, self.world)
        self.out_ptrs = (ctypes.c_void_p * self.world)(*[by_rank[r] for r in order])
        typestr = {0: "<f4", 1: "<f2", 3: "<u2"}[int(self.o_dtype)]
        view = torch.as_tensor(_CudaView(self.out.ptr, (M, N), typestr), device=cuda)
        self.result = view.view(torch.bfloat16) if self.o_dtype == Dtype.BF16 else view
        self.barrier = PeerBarrier(device, dist)

    def forward(self, x_slice, residual=None):
        """x_slice: this rank's columns [k0, k1) of the activations, contiguous [M, k_count];
        residual: the full [M, N] residual in the output dtype (every rank holds it), or None."""
        lib = self.dev.lib
        stream = self.torch.cuda.current_stream().cuda_stream
        _lib.check(lib.vaicu_linear_run_reduce_scatter(self.plan, stream, x_slice.data_ptr(), self.w.data_ptr(), self.staging_ptrs,
                                                       self.world, self.rank, self.ws.data_ptr()), "vaicu_linear_run_reduce_scatter")
        self.barrier.run(stream)
        _lib.check(lib.vaicu_partial_fold_run(self.dev.handle, stream, self.staging.ptr, self.world, self.rows, self.N,
                                              int(self.part_dtype), residual.data_ptr() if residual is not None else None, self.scale,
                                              int(self.o_dtype), self.out_ptrs, self.world, self.rank * self.rows), "vaicu_partial_fold_run")
        self.barrier.run(stream)
        return self.result

    def close(self):
        self.barrier.close()
        for p in self._opened:
            self.dev.lib.vaicu_ipc_close(p)
        self._opened = []
        if self.plan:
            self.dev.lib.vaicu_linear_plan_destroy(self.plan)
            self.plan = None


class ShardedGreedyHead:
    """Vocabulary-split lm_head followed by greedy sampling without gathering logits: every
    rank runs its slab of the head, reduces it to one (max, token) candidate per row with
    the token's vocabulary offset (vaicu_argmax_pairs_run), the ranks exchange 8 bytes per
    row, and each folds the candidates (vaicu_argmax_merge_run).  The same tokens as
    Argmax over the gathered [M, vocab] logits, ties to the lowest token id."""

    def __init__(self, device, dist, full_desc, w_local):
        import torch
        self.torch, self.dist, self.dev = torch, dist, device
        self.rank = dist.get_rank() if dist is not None else 0
        self.world = dist.get_world_size() if dist is not None else 1
        self.desc, self.begin, self.count = shard_desc(full_desc, self.rank, self.world)
        self.w = w_local
        lib = device.lib
        h = ctypes.c_void_p()
        _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(self.desc), ctypes.byref(h)), "plan")
        self.plan = h
        self.info = _lib.LinearInfo()
        _lib.check(lib.vaicu_linear_plan_info(h, ctypes.byref(self.info)), "info")
        cuda = torch.device("cuda", device.ordinal)
        M = self.desc.M
        o_dt = {0: torch.float32, 1: torch.float16, 3: torch.bfloat16}[self.desc.o_dtype]
        self.ws = torch.empty(max(self.info.workspace_bytes, 256), dtype=torch.uint8, device=cuda)
        self.logits = torch.empty((M, self.count), dtype=o_dt, device=cuda)
        n = ctypes.c_size_t()
        _lib.check(lib.vaicu_argmax_workspace_bytes(M, self.count, ctypes.byref(n)), "vaicu_argmax_workspace_bytes")
        self.arg_ws = torch.empty(n.value, dtype=torch.uint8, device=cuda)
        # up to 4 rows the slab runs on the weight-streaming kernel, whose blocks can keep the best
        # logit themselves: slab and candidates in one launch, the logits never stored
        n = ctypes.c_size_t()
        _lib.check(lib.vaicu_linear_argmax_workspace_bytes(h, ctypes.byref(n)), "vaicu_linear_argmax_workspace_bytes")
        self.fused_ws = torch.zeros(n.value, dtype=torch.uint8, device=cuda) if n.value else None
        # one buffer [2, M] per rank: row 0 the maxima (fp32), row 1 the token ids (uint32 bits)
        self.mine = torch.empty((2, M), dtype=torch.float32, device=cuda)
        self.all = torch.empty((self.world, 2, M), dtype=torch.float32, device=cuda)
        self.tokens = torch.empty(M, dtype=torch.int32, device=cuda)

    def forward(self, x):
        lib, M = self.dev.lib, self.desc.M
        stream = self.torch.cuda.current_stream().cuda_stream
        if self.fused_ws is not None and x.data_ptr() % 16 == 0 and self.w.data_ptr() % 16 == 0:
            _lib.check(lib.vaicu_linear_run_argmax(self.plan, stream, x.data_ptr(), self.w.data_ptr(), None, None, None,
                                                   self.fused_ws.data_ptr(), self.begin, self.mine[0].data_ptr(),
                                                   self.mine[1].data_ptr()), "vaicu_linear_run_argmax")
        else:
            _lib.check(lib.vaicu_linear_run(self.plan, stream, x.data_ptr(), self.w.data_ptr(), None, None, self.logits.data_ptr(),
                                            self.ws.data_ptr()), "vaicu_linear_run")
            _lib.check(lib.vaicu_argmax_pairs_run(stream, self.logits.data_ptr(), self.desc.o_dtype, M, self.count, self.count,
                                                  self.begin, self.arg_ws.data_ptr(), self.mine[0].data_ptr(), self.mine[1].data_ptr()),
                       "vaicu_argmax_pairs_run")
        if self.world == 1:
            return self.mine[1].view(self.torch.int32)
        self.dist.all_gather_into_tensor(self.all, self.mine)
        _lib.check(lib.vaicu_argmax_merge_run(stream, self.all.data_ptr(), self.all[0, 1].data_ptr(), self.world, 2 * M, M, None,
                                              self.tokens.data_ptr()), "vaicu_argmax_merge_run")
        return self.tokens

    def close(self):
        if self.plan:
            self.dev.lib.vaicu_linear_plan_destroy(self.plan)
            self.plan = None


class ShardedTopKHead:
    """Vocabulary-split lm_head followed by top-k sampling without gathering logits (vAi's
    TopKSampling node, vai/nodes/topk-sampling.h:33-57, in two steps): every rank runs its slab of
    the head and reduces it to its k best (value, token) pairs per row in rank order
    (vaicu_topk_candidates_run, tokens offset by the slab's first vocabulary entry), the ranks
    all-gather those lists (8 k bytes per row and GPU), and each merges them and samples with the
    same uniform (vaicu_topk_merge_sample_run).  The token is the one the single-GPU node draws
    from the whole row: the top-k of a union lies within the union of the parts' top-k."""

    def __init__(self, device, dist, full_desc, w_local, k=40, temperature=1.0):
        import torch
        self.torch, self.dist, self.dev = torch, dist, device
        self.rank = dist.get_rank() if dist is not None else 0
        self.world = dist.get_world_size() if dist is not None else 1
        self.desc, self.begin, self.count = shard_desc(full_desc, self.rank, self.world)
        self.w, self.k, self.temperature, self.vocab = w_local, int(k), float(temperature), int(full_desc.N)
        lib = device.lib
        h = ctypes.c_void_p()
        _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(self.desc), ctypes.byref(h)), "plan")
        self.plan = h
        self.info = _lib.LinearInfo()
        _lib.check(lib.vaicu_linear_plan_info(h, ctypes.byref(self.info)), "info")
        cuda = torch.device("cuda", device.ordinal)
        M = self.desc.M
        o_dt = {0: torch.float32, 1: torch.float16, 3: torch.bfloat16}[self.desc.o_dtype]
        self.ws = torch.empty(max(self.info.workspace_bytes, 256), dtype=torch.uint8, device=cuda)
        self.logits = torch.empty((M, self.count), dtype=o_dt, device=cuda)
        n = ctypes.c_size_t()
        _lib.check(lib.vaicu_topk_workspace_bytes(M, self.count, self.k, ctypes.byref(n)), "vaicu_topk_workspace_bytes")
        self.topk_ws = torch.empty(max(n.value, 256), dtype=torch.uint8, device=cuda)
        self.mine = torch.empty((M, self.k, 2), dtype=torch.int32, device=cuda)            # (value bits, token) pairs
        self.all = torch.empty((self.world, M, self.k, 2), dtype=torch.int32, device=cuda)
        self.uniform = torch.zeros(1, dtype=torch.float32, device=cuda)
        self.tokens = torch.empty(M, dtype=torch.int32, device=cuda)

    def set_uniform(self, u):
        """The uniform in [0, 1) of the next forward: the same value on every rank."""
        self.uniform.fill_(float(u))

    def forward(self, x):
        lib, M = self.dev.lib, self.desc.M
        stream = self.torch.cuda.current_stream().cuda_stream
        _lib.check(lib.vaicu_linear_run(self.plan, stream, x.data_ptr(), self.w.data_ptr(), None, None, self.logits.data_ptr(),
                                        self.ws.data_ptr()), "vaicu_linear_run")
        _lib.check(lib.vaicu_topk_candidates_run(stream, self.logits.data_ptr(), self.desc.o_dtype, M, self.count, self.count, self.k,
                                                 self.begin, self.topk_ws.data_ptr(), self.mine.data_ptr()), "vaicu_topk_candidates_run")
        if self.world > 1:
            self.dist.all_gather_into_tensor(self.all, self.mine)
            lists = self.all
        else:
            lists = self.mine
        _lib.check(lib.vaicu_topk_merge_sample_run(stream, lists.data_ptr(), self.world, M * self.k, M, self.k, min(self.k, self.vocab),
                                                   self.temperature, self.uniform.data_ptr(), self.tokens.data_ptr()),
                   "vaicu_topk_merge_sample_run")
        return self.tokens

    def close(self):
        if self.plan:
            self.dev.lib.vaicu_linear_plan_destroy(self.plan)
            self.plan = None


def _node_base():
    from .engine import Node
    return Node


class RowParallelLinearNode(_node_base()):
    """The down projection of a tensor-parallel MLP as a node of the engine, so that a whole block
    records into one CUDA graph per rank like any other chain of nodes.

    Slots: in0 = this rank's K slice of the activations [.., K / world] (what its column-split
    gate|value Linear + GatedMul produced), weight = its [N, K / world] slice, residual (optional) = the
    full [.., N] residual, out0 = the full [.., N] result on EVERY rank.  The formula is the Linear's
    with no bias or epilogue: out0 = s * (in0 . W^T summed over the ranks) + residual.

    run() enqueues, all on the net's stream and all kernels of this package: the GEMM whose epilogue
    stores every finished tile of partial sums (fp32) into the staging buffer of the GPU that owns those
    rows; a barrier kernel; the fold of this GPU's rows, which stores the finished rows into every GPU's
    out0; a second barrier kernel.  out0 and the staging buffer are allocated by the node (they are
    shared with the other ranks through CUDA IPC), not by the net's pool.  The ranks must record and
    run their nets in step, as the ranks of one job do.  M (the product of in0's leading axes) must be
    a multiple of the number of ranks and larger than 8 (the tensor-core kernels), weights 16-bit."""

    def __init__(self, in_dim, out_dim, dist, accept_residual=False, scalar_scale=1.0):
        from .engine import INPUT, OUTPUT, PERSISTENT, TEMPORARY
        super().__init__()
        self.in_dim, self.out_dim, self.dist = in_dim, out_dim, dist
        self.accept_residual, self.scalar_scale = accept_residual, float(scalar_scale)
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.add_slot("in0", INPUT)
        self.add_slot("out0", OUTPUT)
        self.add_slot("weight", PERSISTENT)
        self.add_slot("partial", TEMPORARY)
        if accept_residual:
            self.add_slot("residual", INPUT)
        self._plans = {}
        self._shared = {}
        self._plan = self.info = None

    def _device(self):
        from .engine import Device
        return self.net.device if self.net is not None else Device.default()

    def prepare(self):
        from .engine import Dtype, Tensor
        x, w = self["in0"], self["weight"]
        if x.shape[-1] != self.in_dim or tuple(w.shape) != (self.out_dim, self.in_dim):
            raise ValueError("in0 / weight do not match this rank's K slice")
        if w.dtype not in (Dtype.F16, Dtype.BF16) or x.dtype != w.dtype:
            raise ValueError("the row-parallel node takes 16-bit weights and activations of the same type")
        o_dtype = self.o_dtype if self.o_dtype != Dtype.NONE else (self.net.o_default_dtype if self.net else Dtype.F32)
        M = 1
        for s_ in x.shape[:-1]:
            M *= s_
        if M % self.world or M <= 8:
            raise ValueError("M must be a multiple of the number of ranks and larger than 8")
        dev = self._device()
        d = _lib.LinearDesc()
        d.M, d.N, d.K = M, self.out_dim, self.in_dim
        d.i_dtype = d.w_dtype = int(w.dtype)
        d.o_dtype, d.b_dtype = int(Dtype.F32), int(Dtype.NONE)      # fp32 partial sums cross the link
        d.scalar_scale = 1.0
        d.split_size = max(32, self.in_dim)                         # one K span: the partials leave through the epilogue
        key = bytes(d)
        if key not in self._plans:
            h = ctypes.c_void_p()
            _lib.check(dev.lib.vaicu_linear_plan_create(dev.handle, ctypes.byref(d), ctypes.byref(h)), "vaicu_linear_plan_create")
            info = _lib.LinearInfo()
            _lib.check(dev.lib.vaicu_linear_plan_info(h, ctypes.byref(info)), "vaicu_linear_plan_info")
            self._plans[key] = (h, info)
        self._plan, self.info = self._plans[key]
        skey = (M, int(o_dtype))
        if skey not in self._shared:
            rows = M // self.world
            osz = 4 if o_dtype == Dtype.F32 else 2
            staging, st_ptrs, opened1 = share_buffer(dev, self.dist, self.world * rows * self.out_dim * 4)
            out, out_ptrs, opened2 = share_buffer(dev, self.dist, M * self.out_dim * osz)
            order = destination_order(self.rank, self.world)
            self._shared[skey] = dict(rows=rows, staging=staging, out=out, opened=opened1 + opened2,
                                      staging_ptrs=(ctypes.c_void_p * self.world)(*st_ptrs),
                                      out_ptrs=(ctypes.c_void_p * self.world)(*[out_ptrs[r] for r in order]),
                                      barrier=PeerBarrier(dev, self.dist))
        self._live = self._shared[skey]
        ws = self.info.workspace_bytes
        self.slots["partial"] = Tensor((ws // 4,), Dtype.F32) if ws else Tensor()
        out_t = Tensor(tuple(x.shape[:-1]) + (self.out_dim,), o_dtype)
        out_t.buffer = self._live["out"]            # bound here: the net's pool leaves it alone
        self.slots["out0"] = out_t
        if self.accept_residual and self["residual"].dtype != o_dtype:
            raise ValueError("residual dtype must equal the output dtype")

    def bind(self):
        dev, lib = self._device(), self._device().lib
        sh = self._live
        x, w = self["in0"].ptr, self["weight"].ptr
        r = self["residual"].ptr if self.accept_residual else None
        ws = self["partial"].ptr if self["partial"].valid_shape() else None
        plan, world, rank, N, scale = self._plan, self.world, self.rank, self.out_dim, self.scalar_scale
        o_dtype = int(self["out0"].dtype)
        barrier = sh["barrier"]

        def launch(stream):
            _lib.check(lib.vaicu_linear_run_reduce_scatter(plan, stream, x, w, sh["staging_ptrs"], world, rank, ws),
                       "vaicu_linear_run_reduce_scatter")
            barrier.run(stream)
            _lib.check(lib.vaicu_partial_fold_run(dev.handle, stream, sh["staging"].ptr, world, sh["rows"], N, 0, r, scale,
                                                  o_dtype, sh["out_ptrs"], world, rank * sh["rows"]), "vaicu_partial_fold_run")
            barrier.run(stream)

        launch.kernel_launches = int(self.info.launches) + 3
        return launch

    def close(self):
        lib = self._device().lib
        for sh in self._shared.values():
            sh["barrier"].close()
            for p in sh["opened"]:
                lib.vaicu_ipc_close(p)
        self._shared = {}
        for h, _ in self._plans.values():
            lib.vaicu_linear_plan_destroy(h)
        self._plans = {}


class ColumnParallelLinearNode(_node_base()):
    """A Linear split by output columns (rows of W) over the ranks whose full output appears on every rank,
    as a node of the engine: in0 = the activations [.., K] (every rank holds them), weight = this rank's
    rows [count, K] of the full [N, K] weight (vaicu_linear_shard_desc / shard_rows say which), bias
    (optional) = its entries for those rows, out0 = the full [.., N] result on EVERY rank.

    run() enqueues on the net's stream: a barrier kernel (every rank's readers of the previous run's out0
    were enqueued ahead of it), the GEMM whose epilogue stores this rank's column slab into every rank's out0
    over NVLink (vaicu_linear_run_scatter), and a second barrier kernel (all slabs have landed).  out0 is
    allocated by the node (it is shared with the other ranks through CUDA IPC), not by the net's pool.  The
    ranks record and run their nets in step.  More than 8 rows of activations, 16-bit weights."""

    def __init__(self, in_dim, out_dim_full, dist, epilogue=0, scalar_scale=1.0):
        from .engine import INPUT, OUTPUT, PERSISTENT, TEMPORARY
        super().__init__()
        self.in_dim, self.out_dim, self.dist = in_dim, out_dim_full, dist
        self.epilogue, self.scalar_scale = int(epilogue), float(scalar_scale)
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.begin, self.count = shard_rows(out_dim_full, self.world, self.rank)
        for name, kind in (("in0", INPUT), ("out0", OUTPUT), ("weight", PERSISTENT), ("bias", PERSISTENT), ("partial", TEMPORARY)):
            self.add_slot(name, kind)
        self._plans = {}
        self._shared = {}
        self._plan = self.info = None

    def _device(self):
        from .engine import Device
        return self.net.device if self.net is not None else Device.default()

    def prepare(self):
        from .engine import Dtype, Tensor
        x, w = self["in0"], self["weight"]
        if x.shape[-1] != self.in_dim or tuple(w.shape) != (self.count, self.in_dim):
            raise ValueError("weight must hold this rank's rows of the full weight")
        if w.dtype not in (Dtype.F16, Dtype.BF16):
            raise ValueError("the column-parallel node takes 16-bit weights")
        o_dtype = self.o_dtype if self.o_dtype != Dtype.NONE else (self.net.o_default_dtype if self.net else Dtype.F32)
        M = 1
        for s_ in x.shape[:-1]:
            M *= s_
        if M <= 8:
            raise ValueError("the slab leaves through a tensor-core epilogue: more than 8 rows of activations")
        has_bias = self["bias"].valid_shape()
        dev = self._device()
        d = _lib.LinearDesc()
        d.M, d.N, d.K = M, self.count, self.in_dim
        d.i_dtype, d.w_dtype, d.o_dtype = int(x.dtype), int(w.dtype), int(o_dtype)
        d.b_dtype = int(self["bias"].dtype) if has_bias else int(Dtype.NONE)
        d.has_bias, d.bias_elems = (1, self.count) if has_bias else (0, 0)
        d.epilogue, d.scalar_scale = self.epilogue, self.scalar_scale
        d.split_size = max(32, self.in_dim)                         # one K span: a split-K fold cannot scatter
        key = bytes(d)
        if key not in self._plans:
            h = ctypes.c_void_p()
            _lib.check(dev.lib.vaicu_linear_plan_create(dev.handle, ctypes.byref(d), ctypes.byref(h)), "vaicu_linear_plan_create")
            info = _lib.LinearInfo()
            _lib.check(dev.lib.vaicu_linear_plan_info(h, ctypes.byref(info)), "vaicu_linear_plan_info")
            self._plans[key] = (h, info)
        self._plan, self.info = self._plans[key]
        skey = (M, int(o_dtype))
        if skey not in self._shared:
            osz = 4 if o_dtype == Dtype.F32 else 2
            out, out_ptrs, opened = share_buffer(dev, self.dist, M * self.out_dim * osz)
            order = destination_order(self.rank, self.world)
            self._shared[skey] = dict(out=out, opened=opened, barrier=PeerBarrier(dev, self.dist),
                                      out_ptrs=(ctypes.c_void_p * self.world)(*[out_ptrs[r] for r in order]))
        self._live = self._shared[skey]
        ws = self.info.workspace_bytes
        self.slots["partial"] = Tensor((ws // 4,), Dtype.F32) if ws else Tensor()
        out_t = Tensor(tuple(x.shape[:-1]) + (self.out_dim,), o_dtype)
        out_t.buffer = self._live["out"]            # bound here: the net's pool leaves it alone
        self.slots["out0"] = out_t

    def bind(self):
        lib = self._device().lib
        sh = self._live
        x, w = self["in0"].ptr, self["weight"].ptr
        b = self["bias"].ptr if self["bias"].valid_shape() else None
        ws = self["partial"].ptr if self["partial"].valid_shape() else None
        plan, world, N, begin, barrier = self._plan, self.world, self.out_dim, self.begin, sh["barrier"]

        def launch(stream):
            barrier.run(stream)
            _lib.check(lib.vaicu_linear_run_scatter(plan, stream, x, w, b, sh["out_ptrs"], world, N, begin, ws), "vaicu_linear_run_scatter")
            barrier.run(stream)

        launch.kernel_launches = int(self.info.launches) + 2
        return launch

    def close(self):
        lib = self._device().lib
        for sh in self._shared.values():
            sh["barrier"].close()
            for p in sh["opened"]:
                lib.vaicu_ipc_close(p)
        self._shared = {}
        for h, _ in self._plans.values():
            lib.vaicu_linear_plan_destroy(h)
        self._plans = {}


def column_parallel_head_check(device, dist, M=64, d=512, vocab=4096 + 264, seed=1):
    """A vocabulary-split lm_head as a node (ColumnParallelLinearNode) followed by the engine's Argmax
    node, one net per rank, run three times (two replays): the gathered logits against float64 on
    sampled columns and the tokens against the float64 argmax where the top-2 margin allows.  Returns
    the worst relative logit error and the number of token mismatches."""
    import vai_b200
    from .engine import Dtype, Tensor
    from .nodes import ArgmaxNode
    rank, world = dist.get_rank(), dist.get_world_size()
    rng = np.random.default_rng(seed)
    enc = lambda a: np.asarray(vai_b200.engine.bits_to_f32(vai_b200.engine.encode(a.astype(np.float32), Dtype.BF16), Dtype.BF16))
    x = enc(rng.standard_normal((M, d)))
    w = enc(rng.standard_normal((vocab, d)) / np.sqrt(d))
    net = vai_b200.NeuralNet(w_default_dtype=Dtype.BF16, o_default_dtype=Dtype.F32, device=device)
    head = ColumnParallelLinearNode(d, vocab, dist)
    head["weight"] = Tensor.from_numpy(np.ascontiguousarray(w[head.begin:head.begin + head.count]), dtype=Dtype.BF16)
    net.input("x") - head - net.output("logits")
    vai_b200.engine.Flow(head) - ArgmaxNode() - net.output("token")
    outs = None
    for _ in range(3):
        outs = net(Tensor.from_numpy(x, dtype=Dtype.BF16))
    device.check_status()
    logits = outs["logits"].to_numpy()
    tokens = outs["token"].to_u32().reshape(-1)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    err = float(np.max(np.abs(logits - want) / np.maximum(np.abs(want), 1.0)))
    order = np.sort(want, axis=1)
    clear = (order[:, -1] - order[:, -2]) > 1e-3
    wrong = int(np.sum((tokens != np.argmax(want, axis=1)) & clear))
    head.close()
    return err, wrong


def tensor_parallel_mlp_check(device, dist, M=64, d=512, ffn=1024, blocks=2, seed=0):
    """Builds `blocks` gated MLPs (gate|value column split as a plain LinearNode over this rank's weight
    rows -> GatedMulNode -> RowParallelLinearNode + residual) as ONE net per rank, runs it twice (the second
    call replays the recorded graph) and compares with float64 on rank 0's host.  Returns the worst error
    relative to max(|want|, 1) and the number of launches recorded."""
    import vai_b200
    from .engine import Dtype, Epilogue, Tensor
    from .nodes import GatedMulNode, LinearNode
    rank, world = dist.get_rank(), dist.get_world_size()
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, d)).astype(np.float32)
    x = np.asarray(vai_b200.engine.bits_to_f32(vai_b200.engine.encode(x, Dtype.BF16), Dtype.BF16))     # bf16-exact input
    net = vai_b200.NeuralNet(w_default_dtype=Dtype.BF16, o_default_dtype=Dtype.BF16, device=device)
    begin, count = shard_rows(ffn, world, rank)
    flow = x0 = net.input("x")
    weights, nodes_rp = [], []
    for _ in range(blocks):
        wg = (rng.standard_normal((2 * ffn, d)) / np.sqrt(d)).astype(np.float32)
        wd = (rng.standard_normal((d, ffn)) / np.sqrt(ffn)).astype(np.float32)
        weights.append((wg, wd))
        gate_up = LinearNode(in_dim=d, out_dim=2 * count)
        gate_up["weight"] = Tensor.from_numpy(slice_weight(wg, rank, world, True), dtype=Dtype.BF16)
        down = RowParallelLinearNode(count, d, dist, accept_residual=True, scalar_scale=0.25)
        down["weight"] = Tensor.from_numpy(np.ascontiguousarray(wd[:, begin:begin + count]), dtype=Dtype.BF16)
        flow - gate_up - GatedMulNode(activation=Epilogue.SILU) - down
        x0 - "residual" / down
        flow = vai_b200.engine.Flow(down)
        nodes_rp.append(down)
    flow - net.output("y")
    got = net(Tensor.from_numpy(x, dtype=Dtype.BF16)).to_numpy()
    again = net(Tensor.from_numpy(x, dtype=Dtype.BF16)).to_numpy()
    rec = next(iter(net._recordings.values()))
    device.check_status()
    if not np.array_equal(got, again):
        raise RuntimeError("the replayed tensor-parallel net differs from its first run")

    def r16(a):
        return np.asarray(vai_b200.engine.bits_to_f32(vai_b200.engine.encode(a.astype(np.float32), Dtype.BF16), Dtype.BF16), dtype=np.float64)

    cur = x.astype(np.float64)
    for wg, wd in weights:
        acc = cur @ r16(wg).T
        g, u = acc[:, :ffn], acc[:, ffn:]
        hid = r16(g / (1.0 + np.exp(-g)) * u)
        cur = r16(0.25 * (hid @ r16(wd).T) + x)
    err = float(np.max(np.abs(got - cur) / np.maximum(np.abs(cur), 1.0)))
    for n in nodes_rp:
        n.close()
    return err, rec.kernel_launches


class _LocalLinear:
    """One plan with its workspace, run on torch tensors on the current torch stream."""

    def __init__(self, device, M, N, K, gate=False, epilogue=0, residual=False, scale=1.0, split_size=0):
        import torch

        from .engine import Dtype
        self.dev = device
        d = _lib.LinearDesc()
        d.M, d.N, d.K = M, N, K
        d.split_size = split_size
        d.i_dtype = d.w_dtype = d.o_dtype = int(Dtype.BF16)
        d.b_dtype = int(Dtype.NONE)
        d.has_residual = 1 if residual else 0
        d.gate_fuse = 1 if gate else 0
        d.epilogue = int(epilogue)
        d.scalar_scale = scale
        h = ctypes.c_void_p()
        _lib.check(device.lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(h)), "vaicu_linear_plan_create")
        self.plan = h
        info = _lib.LinearInfo()
        _lib.check(device.lib.vaicu_linear_plan_info(h, ctypes.byref(info)), "vaicu_linear_plan_info")
        self.launches = int(info.launches)
        self.ws = torch.empty(max(int(info.workspace_bytes), 256), dtype=torch.uint8, device=torch.device("cuda", device.ordinal))

    def run(self, stream, x, w, out, residual=None):
        _lib.check(self.dev.lib.vaicu_linear_run(self.plan, stream, x.data_ptr(), w.data_ptr(), None,
                                                 residual.data_ptr() if residual is not None else None, out.data_ptr(),
                                                 self.ws.data_ptr()), "vaicu_linear_run")

    def close(self):
        if self.plan:
            self.dev.lib.vaicu_linear_plan_destroy(self.plan)
            self.plan = None


class TensorParallelBlocks:
    """The Linear nodes of `n_blocks` transformer blocks of a preset at batch M, wired as the one-GPU
    bench wires them (q, k, v; o + residual; gate|value with the gate fused; down + residual), either
    whole on this GPU (tp=False) or tensor-parallel over the ranks (tp=True): q / k / v / o replicated,
    gate|value split by columns, `down` split along K with the reduce-scatter in its epilogue and the
    all-gather in its fold (FusedRowParallelLinear) - every launch is one of this package's kernels, so
    the whole chain is captured into ONE CUDA graph per rank and replayed.  Blocks rotate over `copies`
    weight sets (seeded; the two forms draw the same values) so that weights come from HBM, not L2.

    seq=True (with tp, M / world > 128) is the sequence-parallel form of the same block: every rank runs
    q / k / v / o on its own M / world rows only; the epilogue of its o GEMM stores those rows of the
    hidden state into every rank's [M, d] buffer (vaicu_linear_run_broadcast: the all-gather along rows
    rides in the GEMM); gate|value runs on all rows over this rank's columns; down's reduce-scatter
    delivers the partial sums of a rank's rows to that rank, whose fold writes only its own rows.  The
    exchange moves the same bytes as the tensor-parallel form, but the four "replicated" layers now scale
    with the number of GPUs.  step() then takes and returns this rank's rows."""

    def __init__(self, device, dist, preset, M, n_blocks, copies, tp, seq=False):
        import torch

        from . import presets
        from .engine import Dtype, Epilogue
        p = presets.PRESETS[preset]
        self.torch, self.dev, self.M, self.n_blocks = torch, device, M, n_blocks
        self.tp = bool(tp) and dist is not None and dist.get_world_size() > 1
        world = dist.get_world_size() if self.tp else 1
        rank = dist.get_rank() if self.tp else 0
        self.seq = bool(seq) and self.tp
        self.rank, self.world = rank, world
        if self.seq and (M % world or M // world <= 128):
            raise ValueError("the sequence-parallel form needs more than 128 rows per rank")
        rows = M // world if self.seq else M        # rows of the activations that q / k / v / o see on this rank
        self.rows = rows
        d, q, kv, ffn = p["d"], p["q"], p["kv"], p["ffn"]
        act = int(getattr(Epilogue, p["act"]))
        cuda = torch.device("cuda", device.ordinal)
        begin, count = shard_rows(ffn, world, rank)
        kb, kc = shard_k(ffn, world, rank)
        if (kb, kc) != (begin, count):
            raise ValueError("hidden columns and K slices of the ranks do not line up")
        self.Lq, self.Lk, self.Lv = (_LocalLinear(device, rows, n, d) for n in (q, kv, kv))
        self.Lo = _LocalLinear(device, rows, d, q, residual=True, scale=0.5, split_size=max(32, q) if self.seq else 0)
        self.Lg = _LocalLinear(device, M, 2 * count, d, gate=True, epilogue=act)
        self.Ld = self.rp = None
        if self.tp:
            self.rp = FusedRowParallelLinear(device, dist, M, d, ffn, None, Dtype.BF16, part_dtype=Dtype.F32, scalar_scale=0.25)
        else:
            self.Ld = _LocalLinear(device, M, d, ffn, residual=True, scale=0.25)
        self.weights = []
        for c in range(copies):
            gen = torch.Generator(device=cuda).manual_seed(4000 + c)

            def draw(rows, cols):
                return (torch.randn((rows, cols), generator=gen, device=cuda, dtype=torch.float32) * 0.02).to(torch.bfloat16)

            w = {"q": draw(q, d), "k": draw(kv, d), "v": draw(kv, d), "o": draw(d, q)}
            g_full = draw(2 * ffn, d)
            w["g"] = slice_weight(g_full, rank, world, True).contiguous() if self.tp else g_full
            d_full = draw(d, ffn)
            w["d"] = d_full[:, kb:kb + kc].contiguous() if self.tp else d_full
            del g_full, d_full
            self.weights.append(w)
        bf = dict(dtype=torch.bfloat16, device=cuda)
        self.q, self.k, self.v = torch.empty((rows, q), **bf), torch.empty((rows, kv), **bf), torch.empty((rows, kv), **bf)
        self.slab, self.y = torch.empty((M, count), **bf), torch.empty((rows, d), **bf)
        self._opened = []
        if self.seq:
            # the hidden state [M, d] of every rank, shared: each rank's o GEMM writes its rows into all of them
            self.h_buf, by_rank, self._opened = share_buffer(device, dist, M * d * 2)
            self.h = torch.as_tensor(_CudaView(self.h_buf.ptr, (M, d), "<u2"), device=cuda).view(torch.bfloat16)
            order = destination_order(rank, world)
            self.h_dsts = (ctypes.c_void_p * world)(*[by_rank[r] + rank * rows * d * 2 for r in order])
            self.y_dst = (ctypes.c_void_p * 1)(self.y.data_ptr())
        else:
            self.h = torch.empty((M, d), **bf)
        # q / k / v as one launch where the library takes the group (8 < M <= 128, or the weight-streaming kernel)
        self.group = None
        plans = (ctypes.c_void_p * 3)(self.Lq.plan, self.Lk.plan, self.Lv.plan)
        need = ctypes.c_size_t()
        if device.lib.vaicu_linear_group_workspace_bytes(plans, 3, ctypes.byref(need)) == 0:
            self.group = (plans, torch.empty(max(need.value, 256), dtype=torch.uint8, device=cuda), (ctypes.c_void_p * 3)(
                self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr()))
        group_launches = 1 if need.value == 0 else 2       # GEMM alone, or GEMM + the fold of its K splits
        per_block = (group_launches if self.group else 3 * self.Lq.launches) + self.Lo.launches + self.Lg.launches
        per_block += (4 if self.seq else 4) if self.tp else self.Ld.launches      # tp: GEMM, barrier, fold, barrier; seq: barrier, GEMM, barrier, fold
        self.launches = per_block * n_blocks
        self.bytes_per_gpu_block = 2 * (d * (q + 2 * kv) + d * q + 3 * d * count)
        self.graph = None

    def step(self, x0):
        """Enqueues all blocks on the current torch stream; returns the last block's output."""
        lib, stream = self.dev.lib, self.torch.cuda.current_stream().cuda_stream
        if self.seq and x0.shape[0] != self.rows:
            x0 = x0[self.rank * self.rows:(self.rank + 1) * self.rows]          # this rank's rows (a contiguous view)
        x = x0
        for b in range(self.n_blocks):
            w = self.weights[b % len(self.weights)]
            if self.group:
                plans, work, outs = self.group
                ws3 = (ctypes.c_void_p * 3)(w["q"].data_ptr(), w["k"].data_ptr(), w["v"].data_ptr())
                _lib.check(lib.vaicu_linear_run_group(plans, 3, stream, x.data_ptr(), ws3, outs, work.data_ptr()), "vaicu_linear_run_group")
            else:
                self.Lq.run(stream, x, w["q"], self.q)
                self.Lk.run(stream, x, w["k"], self.k)
                self.Lv.run(stream, x, w["v"], self.v)
            if self.seq:
                rp = self.rp
                _lib.check(lib.vaicu_linear_run_broadcast(self.Lo.plan, stream, self.q.data_ptr(), w["o"].data_ptr(), None, x0.data_ptr(),
                                                          self.h_dsts, self.world, self.Lo.ws.data_ptr()), "vaicu_linear_run_broadcast")
                rp.barrier.run(stream)          # every rank's rows of the hidden state are in this rank's buffer
                self.Lg.run(stream, self.h, w["g"], self.slab)
                _lib.check(lib.vaicu_linear_run_reduce_scatter(rp.plan, stream, self.slab.data_ptr(), w["d"].data_ptr(), rp.staging_ptrs,
                                                               self.world, self.rank, rp.ws.data_ptr()), "vaicu_linear_run_reduce_scatter")
                rp.barrier.run(stream)          # the partial sums of this rank's rows have arrived from every rank
                _lib.check(lib.vaicu_partial_fold_run(self.dev.handle, stream, rp.staging.ptr, self.world, self.rows, rp.N, int(rp.part_dtype),
                                                      x0.data_ptr(), rp.scale, int(rp.o_dtype), self.y_dst, 1, 0), "vaicu_partial_fold_run")
                x = self.y
                continue
            self.Lo.run(stream, self.q, w["o"], self.h, residual=x0)
            self.Lg.run(stream, self.h, w["g"], self.slab)
            if self.tp:
                self.rp.w = w["d"]
                x = self.rp.forward(self.slab, residual=x0)
            else:
                self.Ld.run(stream, self.slab, w["d"], self.y, residual=x0)
                x = self.y
        return x

    def capture(self, x0):
        """One eager pass (descriptors, attributes), then the same pass captured; returns the output tensor."""
        torch = self.torch
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.step(x0)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            out = self.step(x0)
        return out

    def close(self):
        self.graph = None
        for lin in (self.Lq, self.Lk, self.Lv, self.Lo, self.Lg, self.Ld):
            if lin is not None:
                lin.close()
        if self.rp is not None:
            self.rp.close()
        for p in self._opened:
            self.dev.lib.vaicu_ipc_close(p)
        self._opened = []


def bench_blocks(device, dist, preset, M, n_blocks, iters=10, warmup=3):
    """`n_blocks` blocks' Linear nodes as one replayed CUDA graph: on one GPU (every rank measures that itself),
    tensor-parallel over all ranks (t N), and - with more than 128 rows per rank - sequence-parallel (t S);
    device-timed, max over ranks.  The outputs (same seeded weights and input) are compared on every rank."""
    import torch

    from . import presets
    world = dist.get_world_size() if dist is not None else 1
    cuda = torch.device("cuda", device.ordinal)
    gen = torch.Generator(device="cpu").manual_seed(77)
    x0 = torch.randn(M, presets.PRESETS[preset]["d"], generator=gen).to(torch.bfloat16).to(cuda)
    res = {"preset": preset, "M": M, "blocks": n_blocks, "world": world}
    outs = {}
    # both forms rotate over the same weight sets (the chains must compute the same function): as many as
    # the form with the fewest bytes per GPU needs to exceed L2 (126 MB) well
    probe = TensorParallelBlocks(device, dist, preset, M, 1, 1, world > 1)
    copies = max(2, min(n_blocks, -(-320_000_000 // probe.bytes_per_gpu_block)))
    probe.close()
    del probe
    forms = [("t1", False, False)]
    if world > 1:
        forms.append(("tN", True, False))
        if M % world == 0 and M // world > 128:
            forms.append(("tS", True, True))          # sequence-parallel: q / k / v / o on this rank's rows only
    for key, tp, seq in forms:
        chain = TensorParallelBlocks(device, dist, preset, M, n_blocks, copies, tp, seq)
        _host_align(torch, dist)
        out = chain.capture(x0)
        ms = _timed(torch, dist, cuda, chain.graph.replay, iters, warmup)
        torch.cuda.synchronize()
        outs[key] = out.float().cpu()
        res[key + "_us_per_block"] = round(ms * 1e3 / n_blocks, 2)
        res[key + "_launches_per_block"] = chain.launches // n_blocks
        res[key + "_weight_sets"] = copies
        _check_status(device, f"{preset} blocks: a barrier between the ranks gave up waiting")
        chain.close()
        del chain
        torch.cuda.empty_cache()
    if world > 1:
        a, b = outs["tN"], outs["t1"]
        # unit-scale activations whose sums may cancel: relative to max(|one-GPU value|, 1)
        res["max_rel_diff_vs_one_gpu"] = float(((a - b).abs() / b.abs().clamp_min(1.0)).max())
        res["speedup"] = round(res["t1_us_per_block"] / res["tN_us_per_block"], 2)
        res["efficiency"] = round(res["speedup"] / world, 3)
        if "tS" in outs:
            rank, rows = dist.get_rank(), M // world
            mine = b[rank * rows:(rank + 1) * rows]               # the sequence-parallel chain returns this rank's rows
            diff = float(((outs["tS"] - mine).abs() / mine.abs().clamp_min(1.0)).max())
            res["max_rel_diff_vs_one_gpu"] = max(res["max_rel_diff_vs_one_gpu"], diff)
            res["sequence_parallel_speedup"] = round(res["t1_us_per_block"] / res["tS_us_per_block"], 2)
            res["sequence_parallel_efficiency"] = round(res["sequence_parallel_speedup"] / world, 3)
    return res


def _tiled_weight(torch, rows, k, seed):
    """[rows, k] bf16 ~N(0, 0.02) on the host, the same on every rank: one seeded pool of 2^24 + 977
    values repeated (the odd length keeps rows from lining up), so that a 1.3 GB matrix takes a
    second to make."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    pool = (torch.randn((1 << 24) + 977, generator=gen) * 0.02).to(torch.bfloat16)
    total = rows * k
    reps = (total + pool.numel() - 1) // pool.numel()
    return pool.repeat(reps)[:total].view(rows, k)


def _host_align(torch, dist):
    """Brings the ranks' host threads together.  The barrier kernels between the ranks' streams wait
    for about half a second at most: a rank must not enqueue one while another rank is still busy on
    its host (the float64 checks run on rank 0 only)."""
    if dist is not None:
        torch.cuda.synchronize()
        dist.barrier()


def _check_status(device, where):
    """Raises if a kernel on this GPU gave up a bounded wait since the last check."""
    _lib.check(device.lib.vaicu_device_status(device.handle, ctypes.byref(ctypes.c_int())), where)


def _timed(torch, dist, cuda, fn, iters, warmup):
    """Device-timed milliseconds per call of fn, max over ranks."""
    _host_align(torch, dist)
    for _ in range(warmup):
        fn()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    if dist is not None:
        t = torch.tensor([ms], dtype=torch.float64, device=cuda)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def _act_f64(code, v):
    """The gate activations of the presets in float64 (4: SiLU, 3: GELU-tanh)."""
    v = np.asarray(v, dtype=np.float64)
    if code == 4:
        return v / (1.0 + np.exp(-v))
    if code == 3:
        return 0.5 * v * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (v + 0.044715 * v ** 3)))
    if code == 0:
        return v
    raise ValueError(code)


def _sampled_error(torch, got, x_host, w_host, gate, epilogue, samples=4096, seed=99):
    """Largest |got - float64| / max(|float64|, 0.05) over `samples` random outputs: float64 dot
    products of the bf16 values both sides hold, the gate applied as the node pair does."""
    rng = np.random.default_rng(seed)
    M, n_out = got.shape
    ms = rng.integers(0, M, samples)
    ns = rng.integers(0, n_out, samples)
    xs = x_host[ms].double().numpy()
    if gate:
        g = (xs * w_host[ns].double().numpy()).sum(axis=1)
        u = (xs * w_host[ns + n_out].double().numpy()).sum(axis=1)
        want = _act_f64(epilogue, g) * u
    else:
        want = (xs * w_host[ns].double().numpy()).sum(axis=1)
    have = got[torch.as_tensor(ms), torch.as_tensor(ns)].double().cpu().numpy()
    return float(np.max(np.abs(have - want) / np.maximum(np.abs(want), 0.05)))


def bench_sharded(device, dist, preset="gemma-3-4b", M=64, iters=20, warmup=5, peaks=None):
    """The large-N layers of `preset` at batch M split over the ranks' GPUs, each beside the same
    layer on ONE GPU measured in the same run (every rank holds the full weight for that):

      lm_head, gate|value   column split; the slab alone, then gathered three ways — NCCL all-gather
                            + re-layout, the gather fused into the GEMM epilogue (peer stores), and
                            for the lm_head the greedy head that exchanges candidates, not logits;
      mlp                   gate|value column split feeding `down` split along K (row parallel),
                            summed by one all-reduce.

    Device-timed, max over ranks.  Gathered outputs are compared with float64 on sampled elements
    (rank 0's copy) and, bit for bit, with the NCCL path.  Returns a dict; rank 0 reports it."""
    import torch

    from . import presets
    from .engine import Dtype, Epilogue
    p = presets.PRESETS[preset]
    world = dist.get_world_size() if dist is not None else 1
    rank = dist.get_rank() if dist is not None else 0
    cuda = torch.device("cuda", device.ordinal)
    peaks = peaks or {}
    hbm, burst = peaks.get("hbm_gbs", 6650.0), peaks.get("bf16_tflops", 1590.0)
    compute_bound = M >= 1024
    lib = device.lib
    gen = torch.Generator(device="cpu").manual_seed(1234)
    x_host = torch.randn(M, p["d"], generator=gen).to(torch.bfloat16)
    x = x_host.to(cuda)
    act = int(getattr(Epilogue, p["act"]))
    out = {"preset": preset, "M": M, "world": world, "layers": {}}

    def desc_of(n_rows, k, gate, o_dtype=Dtype.BF16):
        d = _lib.LinearDesc()
        d.M, d.N, d.K = M, n_rows, k
        d.i_dtype = d.w_dtype = int(Dtype.BF16)
        d.o_dtype = int(o_dtype)
        d.b_dtype = int(Dtype.NONE)
        d.scalar_scale = 1.0
        d.gate_fuse = 1 if gate else 0
        d.epilogue = act if gate else 0
        return d

    def plan_of(d):
        h = ctypes.c_void_p()
        _lib.check(lib.vaicu_linear_plan_create(device.handle, ctypes.byref(d), ctypes.byref(h)), "plan")
        info = _lib.LinearInfo()
        _lib.check(lib.vaicu_linear_plan_info(h, ctypes.byref(info)), "info")
        return h, info

    def one_gpu_us(d, w_dev, x_dev):
        """The whole layer on this GPU alone."""
        h, info = plan_of(d)
        ws = torch.empty(max(info.workspace_bytes, 256), dtype=torch.uint8, device=cuda)
        n_out = d.N // 2 if d.gate_fuse else d.N
        o = torch.empty((M, n_out), dtype=torch.bfloat16 if d.o_dtype == 3 else torch.float32, device=cuda)

        def run():
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.vaicu_linear_run(h, stream, x_dev.data_ptr(), w_dev.data_ptr(), None, None, o.data_ptr(), ws.data_ptr()), "run")

        ms = _timed(torch, dist, cuda, run, iters, warmup)
        lib.vaicu_linear_plan_destroy(h)
        return ms * 1e3, o

    def figures(name, flops_all, bytes_all, t1_us, tn_us, local_us, collective):
        """Speed-up over one GPU, efficiency, and the fraction of world x the roofline of one GPU."""
        agg = flops_all / (tn_us * 1e-6) / 1e12 if compute_bound else bytes_all / (tn_us * 1e-6) / 1e9
        one = burst if compute_bound else hbm
        return {"layer": name, "bound": "tensor" if compute_bound else "hbm", "t1_us": round(t1_us, 1), "tN_us": round(tn_us, 1),
                "local_us": round(local_us, 1), "speedup": round(t1_us / tn_us, 2), "efficiency": round(t1_us / tn_us / world, 3),
                ("aggregate_TFLOPs" if compute_bound else "aggregate_GBps"): round(agg, 1),
                "frac_of_N_x_roofline": round(agg / (world * one), 3), "collective": collective,
                "collective_share": round(max(0.0, 1.0 - local_us / tn_us), 3)}

    cases = [("lm_head", p["vocab"], False), ("gate_up", 2 * p["ffn"], True)]
    kept = {}
    for name, n_rows, gate in cases:
        full = desc_of(n_rows, p["d"], gate)
        n_out = n_rows // 2 if gate else n_rows
        w_host = _tiled_weight(torch, n_rows, p["d"], 7 + len(name))
        w_full = w_host.to(cuda)
        t1_us, o_full = one_gpu_us(full, w_full, x)
        err_one = _sampled_error(torch, o_full.float(), x_host, w_host, gate, act) if rank == 0 else 0.0
        del w_full, o_full
        w_local = slice_weight(w_host, rank, world, gate).contiguous().to(cuda)

        lin = ShardedLinear.__new__(ShardedLinear)
        lin.torch, lin.dist, lin.dev, lin.rank, lin.world = torch, dist, device, rank, world
        lin.full, lin.gate, lin.n_out = full, gate, n_out
        lin.desc, lin.begin, lin.count = shard_desc(full, rank, world)
        lin.w, lin.b = w_local, None
        lin.plan, lin.info = plan_of(lin.desc)
        lin.ws = torch.empty(max(lin.info.workspace_bytes, 256), dtype=torch.uint8, device=cuda)
        cmax = gathered_shape(M, n_out, world)[2]
        lin.local = torch.zeros((M, cmax), dtype=torch.bfloat16, device=cuda)
        lin.slab = lin.local if cmax == lin.count else torch.empty((M, lin.count), dtype=torch.bfloat16, device=cuda)
        lin.gathered = torch.empty((world, M, cmax), dtype=torch.bfloat16, device=cuda)

        local_ms = _timed(torch, dist, cuda, lambda: lin.local_forward(x), iters, warmup)
        nccl_ms = _timed(torch, dist, cuda, lambda: lin.forward(x, assemble_output=True), iters, warmup)
        ref = lin.forward(x, assemble_output=True)
        err_nccl = _sampled_error(torch, ref.float(), x_host, w_host, gate, act) if rank == 0 else 0.0
        fused_ms, fused_equal, err_fused = None, None, None
        if dist is not None and world > 1:
            fused = FusedGatherLinear(device, dist, full, lin.w, None)
            _host_align(torch, dist)
            got = fused.forward(x)
            # the same plan run densely on this rank and gathered by NCCL: must be bit-identical
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.vaicu_linear_run(fused.plan, stream, x.data_ptr(), lin.w.data_ptr(), None, None,
                                            lin.slab.data_ptr(), fused.ws.data_ptr()), "vaicu_linear_run")
            if lin.slab is not lin.local:
                lin.local[:, :lin.count].copy_(lin.slab)
            dist.all_gather_into_tensor(lin.gathered, lin.local)
            same_plan = assemble(lin.gathered, n_out)
            torch.cuda.synchronize()
            dist.barrier()
            fused_equal = bool(torch.equal(got.view(torch.int16), same_plan.view(torch.int16)))
            err_fused = _sampled_error(torch, got.float(), x_host, w_host, gate, act) if rank == 0 else 0.0
            fused_ms = _timed(torch, dist, cuda, lambda: fused.forward(x), iters, warmup)
            torch.cuda.synchronize()
            dist.barrier()
            fused.close()
        flops_all = 2.0 * M * n_rows * p["d"]
        bytes_all = n_rows * p["d"] * 2 + M * p["d"] * 2 + M * n_out * 2
        best_ms, how = nccl_ms, "NCCL all-gather + re-layout"
        if fused_ms is not None and fused_ms < nccl_ms:
            best_ms, how = fused_ms, "all-gather fused into the GEMM epilogue (peer stores) + a 4-byte all-reduce"
        entry = figures(name, flops_all, bytes_all, t1_us, best_ms * 1e3, local_ms * 1e3, how)
        entry.update({"rows": n_rows, "rows_per_gpu": int(w_local.shape[0]), "kernel": int(lin.info.kernel),
                      "tile": [int(lin.info.tile_m), int(lin.info.tile_n)], "nccl_allgather_us": round(nccl_ms * 1e3, 1),
                      "fused_gather_us": None if fused_ms is None else round(fused_ms * 1e3, 1),
                      "fused_gather_matches_nccl": fused_equal, "allgather_bytes_per_gpu": M * cmax * 2,
                      "max_rel_err_vs_float64": {"one_gpu": err_one, "nccl": err_nccl, "fused": err_fused}})
        if name == "lm_head":
            # greedy sampling without gathering logits: 8 bytes per row and GPU are exchanged
            head = ShardedGreedyHead(device, dist, full, lin.w)
            tok = head.forward(x).clone()
            logits = ref.float()
            top = logits.max(dim=1, keepdim=True).values
            want = (logits == top).int().argmax(dim=1)             # lowest token id among equal maxima
            torch.cuda.synchronize()
            greedy_ms = _timed(torch, dist, cuda, lambda: head.forward(x), iters, warmup)
            g = figures("lm_head + greedy sampling", flops_all, bytes_all, t1_us, greedy_ms * 1e3, local_ms * 1e3,
                        "all-gather of one (max, token) candidate per row and GPU (8 bytes), then a merge kernel")
            g.update({"greedy_head_us": round(greedy_ms * 1e3, 1), "greedy_exchange_bytes_per_gpu": 8 * M,
                      "greedy_head_matches_argmax_of_gathered_logits": bool(torch.equal(tok.long(), want)),
                      "note": "t1_us is the one-GPU lm_head without its argmax pass"})
            # top-k sampling without the logits: k candidates per row and GPU are exchanged
            tk = ShardedTopKHead(device, dist, full, lin.w, k=40, temperature=0.8)
            full_logits = torch.empty_like(ref).copy_(ref).float().contiguous()
            n_ws = ctypes.c_size_t()
            _lib.check(lib.vaicu_topk_workspace_bytes(M, n_rows, 40, ctypes.byref(n_ws)), "vaicu_topk_workspace_bytes")
            ws_full = torch.empty(max(n_ws.value, 256), dtype=torch.uint8, device=cuda)
            one = torch.empty(M, dtype=torch.int32, device=cuda)
            same = True
            for uu in (0.0, 0.21, 0.5, 0.77, 0.98):
                tk.set_uniform(uu)
                got_tok = tk.forward(x).clone()
                stream = torch.cuda.current_stream().cuda_stream
                _lib.check(lib.vaicu_topk_sample_run(stream, ref.data_ptr(), int(Dtype.BF16), M, n_rows, 40, 0.8, tk.uniform.data_ptr(),
                                                     ws_full.data_ptr(), one.data_ptr()), "vaicu_topk_sample_run")
                torch.cuda.synchronize()
                same = same and bool(torch.equal(got_tok, one))
            topk_ms = _timed(torch, dist, cuda, lambda: tk.forward(x), iters, warmup)
            g["topk_head_us"] = round(topk_ms * 1e3, 1)
            g["topk_head_matches_single_gpu_node"] = same
            g["topk_exchange_bytes_per_gpu"] = 8 * 40 * M
            del full_logits
            tk.close()
            out["layers"]["lm_head_greedy"] = g
            entry["greedy_head_us"] = g["greedy_head_us"]
            entry["greedy_head_matches_argmax_of_gathered_logits"] = g["greedy_head_matches_argmax_of_gathered_logits"]
            entry["greedy_exchange_bytes_per_gpu"] = 8 * M
            head.close()
        out["layers"][name] = entry
        if name == "gate_up":
            kept = {"lin": lin, "w_host": w_host, "t1_us": t1_us}
        else:
            lib.vaicu_linear_plan_destroy(lin.plan)
            del lin, w_host

    # the natural tensor-parallel MLP: this rank's hidden columns feed its K slice of `down`
    # directly; one all-reduce of [M, d] replaces the all-gather of the hidden state
    lin = kept["lin"]
    kb, kc = shard_k(p["ffn"], world, rank)
    if kc == lin.count and kb == lin.begin:
        wd_host = _tiled_weight(torch, p["d"], p["ffn"], 31)
        wd_full = wd_host.to(cuda)
        h_full = torch.empty((M, p["ffn"]), dtype=torch.bfloat16, device=cuda).normal_(0, 0.5)
        down_t1_us, _ = one_gpu_us(desc_of(p["d"], p["ffn"], False), wd_full, h_full)
        del wd_full, h_full
        w_down = wd_host[:, kb:kb + kc].contiguous().to(cuda)
        down = RowParallelLinear(device, dist, M, p["d"], p["ffn"], w_down, Dtype.BF16)

        def mlp_local():
            lin.local_forward(x)
            down.local_forward(lin.slab)

        def mlp():
            lin.local_forward(x)
            down.forward(lin.slab)

        local_ms = _timed(torch, dist, cuda, mlp_local, iters, warmup)
        total_ms = _timed(torch, dist, cuda, mlp, iters, warmup)
        # the same MLP with the reduction done by the GEMM's epilogue, a fold kernel and two barrier
        # kernels over NVLink (no library collective)
        fused_ms, fused_err, fused_how = None, None, None
        if dist is not None and world > 1 and M % world == 0:
            # fp32 partial sums: the ranks' partials cancel in part, so rounding them to 16 bits first costs
            # up to 2^-9 of the LARGER magnitude (measured: 6 % of the outputs off by more than 2e-2 of
            # max(|ref|, 0.05) with bf16 partials at M = 8192, none with fp32)
            part = Dtype.F32
            rp = FusedRowParallelLinear(device, dist, M, p["d"], p["ffn"], w_down, Dtype.BF16, part_dtype=part)

            def mlp_fused():
                lin.local_forward(x)
                return rp.forward(lin.slab)

            _host_align(torch, dist)
            yf = mlp_fused().clone()
            fused_ms = _timed(torch, dist, cuda, mlp_fused, iters, warmup)
            fused_how = (f"reduce-scatter fused into the down GEMM's epilogue ({'bf16' if part == Dtype.BF16 else 'fp32'} partial sums "
                         "stored to the rows' owners over NVLink), fold kernel that stores the finished rows to every GPU, two barrier kernels")
        # float64 on sampled outputs: hidden = act(gate) * value in bf16 (as the column-split Linear stores it), then down
        lin.local_forward(x)
        y = down.forward(lin.slab).clone()
        err = None
        if rank == 0:
            rng = np.random.default_rng(5)
            rows = rng.integers(0, M, 8)
            wg = kept["w_host"].double().numpy()
            xs = x_host[rows].double().numpy()
            acc = xs @ wg.T
            hid = _act_f64(act, acc[:, :p["ffn"]]) * acc[:, p["ffn"]:]
            hid = torch.as_tensor(hid).to(torch.bfloat16).double().numpy()
            want = hid @ wd_host.double().numpy().T
            have = y[torch.as_tensor(rows)].double().cpu().numpy()
            err = float(np.max(np.abs(have - want) / np.maximum(np.abs(want), 0.05)))
            if fused_ms is not None:
                have = yf[torch.as_tensor(rows)].double().cpu().numpy()
                fused_err = float(np.max(np.abs(have - want) / np.maximum(np.abs(want), 0.05)))
        t1 = kept["t1_us"] + down_t1_us
        flops_all = 2.0 * M * (2 * p["ffn"]) * p["d"] + 2.0 * M * p["d"] * p["ffn"]
        bytes_all = (2 * p["ffn"] * p["d"] + p["d"] * p["ffn"]) * 2 + M * p["d"] * 2 * 2 + M * p["ffn"] * 2 * 2
        best_ms, how = total_ms, f"one NCCL all-reduce of the fp32 partial outputs [{M}, {p['d']}] ({M * p['d'] * 4} bytes)"
        if fused_ms is not None and fused_ms < total_ms:
            best_ms, how = fused_ms, fused_how
        e = figures("mlp: gate|value column split -> down split along K", flops_all, bytes_all, t1, best_ms * 1e3, local_ms * 1e3, how)
        e.update({"down_K_per_gpu": kc, "allreduce_bytes": M * p["d"] * 4, "gate_up_plus_down_local_us": round(local_ms * 1e3, 1),
                  "nccl_allreduce_us": round(total_ms * 1e3, 1),
                  "fused_reduce_scatter_us": None if fused_ms is None else round(fused_ms * 1e3, 1),
                  "max_rel_err_vs_float64": {"nccl": err, "fused": fused_err}})
        if fused_ms is not None:
            rp.close()
        out["layers"]["mlp_column_then_row_parallel"] = e
        down.close()
    lib.vaicu_linear_plan_destroy(lin.plan)
    torch.cuda.synchronize()
    _check_status(device, f"{preset} M={M}: a barrier between the ranks gave up waiting")
    return out


def sharded_report(device, dist, peaks):
    """What bench.py prints under roofline.sharded at N > 1: both sharded configurations, each layer
    with its one-GPU time, N-GPU time, speed-up, efficiency, fraction of N x roofline, the
    collective and its share, and the float64 check.  Raises if a check fails."""
    decode = bench_sharded(device, dist, "gemma-3-4b", 64, iters=10, warmup=3, peaks=peaks)
    prefill = bench_sharded(device, dist, "llama-3.2-3b", 8192, iters=5, warmup=2, peaks=peaks)
    keep = ("layer", "bound", "t1_us", "tN_us", "local_us", "speedup", "efficiency", "aggregate_TFLOPs", "aggregate_GBps",
            "frac_of_N_x_roofline", "collective", "collective_share", "nccl_allgather_us", "fused_gather_us",
            "nccl_allreduce_us", "fused_reduce_scatter_us",
            "fused_gather_matches_nccl", "greedy_head_matches_argmax_of_gathered_logits", "topk_head_us",
            "topk_head_matches_single_gpu_node", "max_rel_err_vs_float64")
    report = {"world": decode["world"], "bound_checked": "sampled outputs within 2e-2 of float64 (bf16 operands, fp32 accumulate)"}
    for key, res in (("gemma3_4b_decode_M64", decode), ("llama32_3b_prefill_M8192", prefill)):
        rows = []
        for layer in res["layers"].values():
            rows.append({k: layer[k] for k in keep if k in layer})
            errs = layer.get("max_rel_err_vs_float64")
            for v in (errs.values() if isinstance(errs, dict) else [errs]):
                if v is not None and not v <= 2e-2:
                    raise RuntimeError(f"{key} / {layer['layer']}: relative error {v} against float64 exceeds 2e-2")
            if (layer.get("fused_gather_matches_nccl") is False or layer.get("greedy_head_matches_argmax_of_gathered_logits") is False
                    or layer.get("topk_head_matches_single_gpu_node") is False):
                raise RuntimeError(f"{key} / {layer['layer']}: sharded result differs from the gathered reference")
        report[key] = rows
    # whole blocks (q, k, v, o replicated; the MLP tensor-parallel) as one replayed CUDA graph per rank
    report["blocks"] = [bench_blocks(device, dist, "gemma-3-4b", 64, 34, iters=10, warmup=3),
                        bench_blocks(device, dist, "llama-3.2-3b", 8192, 2, iters=5, warmup=2)]
    # the batched-decode step as the sum of its measured parts: 34 replayed blocks + the lm_head with greedy sampling
    try:
        head = next(r for r in report["gemma3_4b_decode_M64"] if r["layer"] == "lm_head + greedy sampling")
        blk = report["blocks"][0]
        report["gemma3_4b_decode_step_us"] = {
            "one_gpu": round(blk["blocks"] * blk["t1_us_per_block"] + head["t1_us"], 1),
            "n_gpus": round(blk["blocks"] * blk["tN_us_per_block"] + head["tN_us"], 1),
            "how": "34 blocks replayed as one graph per rank (per-block time x 34) + the lm_head (one GPU: its GEMM alone; "
                   "N GPUs: slab + argmax candidates + exchange + merge)"}
    except (StopIteration, KeyError):
        pass
    for b in report["blocks"]:
        diff = b.get("max_rel_diff_vs_one_gpu")
        if diff is not None and not diff <= 2e-2:
            raise RuntimeError(f"{b['preset']} blocks: tensor-parallel output differs from the one-GPU chain by {diff}")
    return report


def main():
    """torchrun --nproc-per-node N -m vai_b200.sharded [--preset gemma-3-4b] [--M 64]"""
    import argparse
    import json
    import os

    import torch
    import torch.distributed as dist

    from .engine import Device
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="gemma-3-4b")
    ap.add_argument("--M", type=int, default=64)
    ap.add_argument("--nodes-check", action="store_true",
                    help="run the tensor-parallel MLP built from engine nodes (RowParallelLinearNode) against float64 instead")
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    d = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        d = dist
    if a.nodes_check:
        if d is None:           # one rank: a process group of one, so that the same code path runs
            dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29549", rank=0, world_size=1)
            d = dist
        err, launches = tensor_parallel_mlp_check(Device(local), d, M=a.M)
        head_err, head_wrong = column_parallel_head_check(Device(local), d, M=a.M)
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"tp_nodes": {"world": world, "max_rel_err_vs_float64": err, "launches_recorded": launches,
                                           "head_max_rel_err_vs_float64": head_err, "head_token_mismatches": head_wrong}}))
        dist.destroy_process_group()
        return
    res = bench_sharded(Device(local), d, a.preset, a.M)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(res))
    if d is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
