"""LinearNode: the host side of vAi's `vai::node::Linear` (vai/nodes/linear.h:59-348),
with the same Config fields, slot names, shapes and formula, launching the sm_100a
kernels through the C ABI.  Python-facing signature as in the reference's binding
(python/bindings/nodes/linear.cpp:7-29).
"""
import ctypes

import numpy as np

from . import _lib
from .engine import (INPUT, OUTPUT, PERSISTENT, TEMPORARY, Dtype, Epilogue, GateNode, Node, ResidualOrder, Tensor)  # noqa: F401 (GateNode re-exported)

KERNEL_AUTO, KERNEL_GEMV, KERNEL_FMA_TILE, KERNEL_TC_GEMM, KERNEL_TC_SKINNY = 0, 1, 2, 3, 4


class LinearNode(Node):
    """out0 = scalar_scale * epilogue(in0 W^T + bias) + residual, or with the residual
    inside the epilogue per residual_order.  `bias` applies when it is set.
    accept_residual opens the `residual` input; bias and residual are each
    [..., out_dim] or rows that repeat over the output, such as [out_dim].
    split_size is the K length per split-K span (0 = the kernel's heuristic, otherwise
    >= 32) and only matters past 8 input rows.

    When the only reader of out0 is a GatedMulNode (the gateValue - gatedMul wiring of
    vAi's gated feed-forward, vai/groups/gated-feed-forward.h:38-46) and this node does
    nothing after the dot product but add a per-row bias, the net records the pair as one
    launch: `weight` [2H, K] holds the gate rows first, and the kernel writes
    [..., H] = activation(gate) * value straight from its accumulators.  Nothing in the
    node's signature asks for that; `gate_fuse` reports whether the current recording did it.
    """

    def __init__(self, in_dim, out_dim, accept_residual=False, residual_order=ResidualOrder.AFTER_EPILOGUE,
                 epilogue=Epilogue.NONE, scalar_scale=1.0, split_size=0, kernel=KERNEL_AUTO, tuning=None):
        super().__init__()
        if not (split_size == 0 or split_size >= 32):
            raise ValueError("split_size: must be 0 or >= 32")
        if in_dim <= 0 or out_dim <= 0:
            raise ValueError("in_dim and out_dim must be positive")
        self.in_dim, self.out_dim = int(in_dim), int(out_dim)
        self.accept_residual = bool(accept_residual)
        self.residual_order = ResidualOrder(residual_order)
        self.epilogue = Epilogue(epilogue)
        self.scalar_scale = float(scalar_scale)
        self.split_size = int(split_size)
        self.kernel = int(kernel)
        # Not in the reference's signature: `kernel` fixes the kernel family, `tuning` (a dict of
        # vaicu_linear_tuning fields) fixes tile and launch geometry; both default to the library's choice.
        self.tuning = dict(tuning) if tuning else None
        self._gate = None           # activation of the GatedMul recorded into this node's launch
        self._gate_o_dtype = None   # ... and that node's output dtype
        self._argmax_reader = None  # the ArgmaxNode that asked to share this node's launch, if any
        self._launch_taken = False  # that node issues the (fused) launch; this node's own is skipped
        # slot set of Linear::Linear (linear.h:2134-2144)
        self.add_slot("out0", OUTPUT)
        self.add_slot("in0", INPUT)
        self.add_slot("weight", PERSISTENT)
        self.add_slot("partial", TEMPORARY)
        self.add_slot("bias", PERSISTENT)
        if self.accept_residual:
            self.add_slot("residual", INPUT)
        self._plans = {}
        self._plan = None
        self.info = None

    def has_bias(self):
        return self["bias"].valid_shape()

    @property
    def gate_fuse(self):
        """True while a GatedMul is recorded into this node's launch."""
        return self._gate is not None

    def reset_fusion(self):
        self._gate = self._gate_o_dtype = None
        self._argmax_reader = None
        self._launch_taken = False

    def can_feed_argmax(self):
        """An Argmax that is this node's only reader may be folded into the launch when the node is
        not gated; whether the plan is on the weight-streaming kernel is known after prepare()."""
        return not self.gate_fuse

    def can_absorb_gate(self):
        """A GatedMul may ride in this node's epilogue when the node itself ends at
        `acc + bias[row]`: no epilogue, residual or scale of its own, an even out_dim,
        and a bias (if any) with one entry per weight row."""
        return (self.epilogue == Epilogue.NONE and not self.accept_residual and self.scalar_scale == 1.0
                and self.out_dim % 2 == 0 and (not self.has_bias() or self["bias"].num_elements() == self.out_dim))

    def absorb_gate(self, activation, o_dtype):
        self._gate, self._gate_o_dtype = Epilogue(activation), Dtype(o_dtype)

    def _device(self):
        from .engine import Device
        return self.net.device if self.net is not None else Device.default()

    def prepare(self):
        """Shape -> plan (Linear::prepare, linear.h:2291-2704): resolves dtypes, M, the
        bias / residual repeat lengths, asks the library for a plan, sizes `partial`
        and `out0`.  Touches no device memory."""
        x, w = self["in0"], self["weight"]
        if x.shape[-1] != self.in_dim:
            raise ValueError(f"in0 last axis {x.shape[-1]} != in_dim {self.in_dim}")
        if tuple(w.shape) != (self.out_dim, self.in_dim):
            raise ValueError(f"weight shape {w.shape} != {(self.out_dim, self.in_dim)}")
        o_dtype = self.o_dtype if self.o_dtype != Dtype.NONE else (self.net.o_default_dtype if self.net else Dtype.F32)
        if self.gate_fuse:
            o_dtype = self._gate_o_dtype          # the fused launch writes the GatedMul's output
        M = 1
        for s in x.shape[:-1]:
            M *= s
        N, K = self.out_dim, self.in_dim
        out_cols = N // 2 if self.gate_fuse else N

        def repeat_of(t, row_len, total):
            elems = t.num_elements()
            if t.shape[-1] != row_len or elems == 0 or total % elems:
                raise ValueError("operand does not tile the output")
            return 0 if elems == total else elems

        d = _lib.LinearDesc()
        d.M, d.N, d.K = M, N, K
        d.i_dtype, d.w_dtype, d.o_dtype = int(x.dtype), int(w.dtype), int(o_dtype)
        d.b_dtype = int(Dtype.NONE)
        if self.has_bias():
            b = self["bias"]
            d.has_bias, d.b_dtype = 1, int(b.dtype)
            d.bias_elems = N if self.gate_fuse else repeat_of(b, N, M * N)
        if self.accept_residual:
            r = self["residual"]
            if r.dtype != o_dtype:
                raise ValueError("residual dtype must equal the output dtype")
            d.has_residual = 1
            d.residual_elems = repeat_of(r, out_cols, M * out_cols)
        d.residual_order = int(self.residual_order)
        d.epilogue = int(self._gate if self.gate_fuse else self.epilogue)
        d.scalar_scale = self.scalar_scale
        d.split_size = self.split_size
        d.gate_fuse = 1 if self.gate_fuse else 0
        key = bytes(d)
        dev = self._device()
        plan = self._plans.get(key)
        if plan is None:
            h = ctypes.c_void_p()
            if self.tuning:
                t = _lib.LinearTuning(kernel=self.kernel, **self.tuning)
                rc = dev.lib.vaicu_linear_plan_create_tuned(dev.handle, ctypes.byref(d), ctypes.byref(t), ctypes.byref(h))
            elif self.kernel == KERNEL_AUTO:
                rc = dev.lib.vaicu_linear_plan_create(dev.handle, ctypes.byref(d), ctypes.byref(h))
            else:
                rc = dev.lib.vaicu_linear_plan_create_forced(dev.handle, ctypes.byref(d), self.kernel, ctypes.byref(h))
            _lib.check(rc, "vaicu_linear_plan_create")
            info = _lib.LinearInfo()
            _lib.check(dev.lib.vaicu_linear_plan_info(h, ctypes.byref(info)), "vaicu_linear_plan_info")
            plan = (h, info)
            self._plans[key] = plan
        self._plan, self.info = plan
        # `partial` carries the plan's whole workspace, as raw bytes
        ws = self.info.workspace_bytes
        self.slots["partial"] = Tensor((ws // 4,), Dtype.F32) if ws else Tensor()
        self.slots["out0"] = Tensor(tuple(x.shape[:-1]) + (out_cols,), o_dtype)

    def bind(self):
        """Linear::run (linear.h:2706-2798) with today's buffers: a callable(stream)
        that only enqueues work."""
        dev = self._device()
        plan = self._plan
        x, w, o = self["in0"].ptr, self["weight"].ptr, self["out0"].ptr
        b = self["bias"].ptr if self.has_bias() else None
        r = self["residual"].ptr if self.accept_residual else None
        ws = self["partial"].ptr if self["partial"].valid_shape() else None
        run = dev.lib.vaicu_linear_run

        node = self

        def launch(stream):
            if node._launch_taken:        # the Argmax behind this node launches the fused kernel
                return
            _lib.check(run(plan, stream, x, w, b, r, o, ws), "vaicu_linear_run")

        launch.kernel_launches = int(self.info.launches)
        self._launch = launch
        return launch

    def groupable(self):
        """Plain (nothing after the dot product) and on the weight-streaming kernel, or on a
        tensor-core kernel with a whole number of weight tiles: may share one launch with
        sibling Linears that read the same activations."""
        if self.info is None or self.has_bias() or self.accept_residual or self.epilogue != Epilogue.NONE:
            return False
        if self.gate_fuse or self.scalar_scale != 1.0 or self._argmax_reader is not None or self.split_size:
            return False
        if self.info.kernel == KERNEL_TC_GEMM:      # CTA pairs: whole 256-column tiles, 16-bit activations (no cast pass)
            return self.out_dim % 256 == 0 and self["in0"].dtype != Dtype.F32
        return self.info.kernel == KERNEL_GEMV or (self.info.kernel == KERNEL_TC_SKINNY and self.out_dim % 128 == 0)

    def group_key(self):
        """Nodes with equal keys (and the same in0 tensor) may form a group."""
        return (int(self.info.kernel), int(self["weight"].dtype), int(self["out0"].dtype))

    @staticmethod
    def bind_group(group, scratch):
        """One launch (plus one fold on the tensor-core kernel) for 2-3 groupable nodes with the
        same in0 (vaicu_linear_run_group).  `scratch(nbytes)` hands out device memory that lives
        as long as the recording.  Returns None when the library declines the group."""
        first = group[0]
        dev = first._device()
        n = len(group)
        plans = (ctypes.c_void_p * n)(*[g._plan for g in group])
        ws = (ctypes.c_void_p * n)(*[g["weight"].ptr for g in group])
        outs = (ctypes.c_void_p * n)(*[g["out0"].ptr for g in group])
        x = first["in0"].ptr
        if any(p % 16 for p in [x, *ws, *outs]):
            return None
        need = ctypes.c_size_t()
        if dev.lib.vaicu_linear_group_workspace_bytes(plans, n, ctypes.byref(need)) != 0:
            return None
        work = scratch(need.value).ptr if need.value else None
        run = dev.lib.vaicu_linear_run_group

        def launch(stream):
            _lib.check(run(plans, n, stream, x, ws, outs, work), "vaicu_linear_run_group")

        if first.info.kernel in (KERNEL_GEMV, KERNEL_TC_GEMM):
            launch.kernel_launches = 1
        else:
            # GEMM (+ the cast of fp32 activations) (+ the fold, unless the K splits fold inside clusters:
            # then the group needs no room for partial sums)
            cast = first["in0"].dtype == Dtype.F32
            cast_bytes = -(-first["in0"].num_elements() * 2 // 256) * 256 if cast else 0
            launch.kernel_launches = 1 + int(cast) + int(need.value > cast_bytes)
        return launch

    def __del__(self):
        try:
            lib = _lib.load()
            for h, _ in self._plans.values():
                lib.vaicu_linear_plan_destroy(h)
        except Exception:
            pass


class GatedMulNode(Node):
    """GLU gating (vAi vai/nodes/gated-mul.h:9-20): in0 [..., 2H] -> out0 [..., H] =
    activation(in0[..., j]) * in0[..., H + j]; the leading half is the activated one.
    activation names the variant (SILU: SwiGLU, GELU / GELU_TANH: GEGLU, RELU: ReGLU,
    NONE: bilinear).  Python-facing signature as in the reference's binding
    (python/bindings/nodes/gated-mul.cpp).

    Placed right after a gate|value LinearNode whose output nothing else reads, the node
    launches nothing: the net records it into that Linear's epilogue (see LinearNode) and
    out0 is the Linear's output.  Otherwise it is one streaming kernel."""

    fusion_kind = "gated_mul"       # NeuralNet(fuse_gated_mul=...) switches the merge

    def __init__(self, activation=Epilogue.SILU):
        super().__init__()
        self.activation = Epilogue(activation)
        self.add_slot("out0", OUTPUT)
        self.add_slot("in0", INPUT)
        self.fused = False

    def reset_fusion(self):
        self.fused = False

    def _resolved_o_dtype(self):
        return self.o_dtype if self.o_dtype != Dtype.NONE else (self.net.o_default_dtype if self.net else Dtype.F32)

    def absorb_into_producer(self, src, src_slot):
        """Called by the net while it records, when this node is the only reader of
        src's `src_slot`: merge into a Linear that can carry the gate in its epilogue."""
        if isinstance(src, LinearNode) and src_slot == "out0" and src.can_absorb_gate():
            src.absorb_gate(self.activation, self._resolved_o_dtype())
            self.fused = True
        return self.fused

    def prepare(self):
        x = self["in0"]
        if self.fused:
            self.slots["out0"] = x          # the Linear already wrote activation(gate) * value
            return
        if not x.valid_shape() or len(x.shape) < 1 or x.shape[-1] % 2:
            raise ValueError("in0 needs an even last axis")
        self.slots["out0"] = Tensor(tuple(x.shape[:-1]) + (x.shape[-1] // 2,), self._resolved_o_dtype())

    def bind(self):
        if self.fused:
            def nothing(stream):
                pass
            nothing.kernel_launches = 0
            return nothing
        from .engine import Device
        dev = self.net.device if self.net is not None else Device.default()
        x, o = self["in0"], self["out0"]
        h = o.shape[-1]
        rows = o.num_elements() // h
        args = (dev.handle, x.ptr, o.ptr, rows, h, int(x.dtype), int(o.dtype), int(self.activation))
        run = dev.lib.vaicu_gated_mul_run

        def launch(stream):
            _lib.check(run(args[0], stream, *args[1:]), "vaicu_gated_mul_run")

        launch.kernel_launches = 1
        return launch


class ArgmaxNode(Node):
    """Row-wise argmax (greedy decode) over logits: in0 [M, N] -> out0 [M] raw uint32
    indices in 4-byte slots (vAi vai/nodes/argmax.h:9-18; read them with
    Tensor.to_u32()).  Ties go to the lowest index.  Wide rows (a vocabulary) are scanned
    by many blocks in column segments and folded in a second launch; the candidates live
    in the `partial` temporary.

    Behind a LinearNode whose output nothing else reads (the lm_head of a greedy decoder) and
    whose plan is on the weight-streaming kernel, the node shares that Linear's launch: the
    kernel's blocks keep the best logit they produce and the last one folds the candidates
    (vaicu_linear_run_argmax), so the logits are not read a second time and the step is two
    launches shorter."""

    WIDE = 16384        # from this row length on, one block per row is the slower form
    fusion_kind = "argmax"          # NeuralNet(fuse_argmax=...) switches the merge

    def __init__(self):
        super().__init__()
        self.add_slot("out0", OUTPUT)
        self.add_slot("in0", INPUT)
        self.add_slot("partial", TEMPORARY)
        self._producer = None
        self.fused = False

    def reset_fusion(self):
        self._producer = None
        self.fused = False

    def absorb_into_producer(self, src, src_slot):
        """Called by the net while it records, when this node is the only reader of src's output:
        remember a Linear that may carry the argmax; prepare() decides once its plan is known."""
        if isinstance(src, LinearNode) and src_slot == "out0" and src.can_feed_argmax():
            self._producer = src
            src._argmax_reader = self
        return self._producer is not None

    def _fused_workspace_bytes(self, dev):
        lin = self._producer
        if lin is None or lin._plan is None or lin.gate_fuse:
            return 0
        ws = ctypes.c_size_t()
        _lib.check(dev.lib.vaicu_linear_argmax_workspace_bytes(lin._plan, ctypes.byref(ws)), "vaicu_linear_argmax_workspace_bytes")
        ptrs = (lin["in0"].ptr, lin["weight"].ptr)
        if any(p is None or p % 16 for p in ptrs):
            return 0                      # views the vector kernel cannot address: two nodes, two launches
        return ws.value

    def prepare(self):
        x = self["in0"]
        if not x.valid_shape() or len(x.shape) != 2:
            raise ValueError("in0 must be [M, N]")
        # a [M] tensor of raw uint32; the dtype enum has no integer kind, so fp32 is the
        # 4-byte container, as in the reference (argmax.h:75-78)
        self.slots["out0"] = Tensor((x.shape[0],), Dtype.F32)
        self.slots["partial"] = Tensor()
        self.fused = False
        if self._producer is not None:
            from .engine import Device
            dev = self.net.device if self.net is not None else Device.default()
            ws = self._fused_workspace_bytes(dev)
            if ws:
                self.fused = True
                self._producer._launch_taken = True
                self.slots["partial"] = Tensor((ws // 4,), Dtype.F32)
                return
        if x.shape[1] >= self.WIDE:
            from .engine import Device
            dev = self.net.device if self.net is not None else Device.default()
            ws = ctypes.c_size_t()
            _lib.check(dev.lib.vaicu_argmax_workspace_bytes(x.shape[0], x.shape[1], ctypes.byref(ws)), "vaicu_argmax_workspace_bytes")
            self.slots["partial"] = Tensor((ws.value // 4,), Dtype.F32)

    def bind(self):
        from .engine import Device
        dev = self.net.device if self.net is not None else Device.default()
        x, o = self["in0"], self["out0"]
        xp, op, dt, M, N = x.ptr, o.ptr, int(x.dtype), x.shape[0], x.shape[1]
        if self.fused:
            lin = self._producer
            plan, ws = lin._plan, self["partial"].ptr
            li, lw = lin["in0"].ptr, lin["weight"].ptr
            lb = lin["bias"].ptr if lin.has_bias() else None
            lr = lin["residual"].ptr if lin.accept_residual else None
            # the ticket counter at the head of the workspace starts at zero; the kernel leaves it at zero
            _lib.check(dev.lib.vaicu_memset(ws, 0, 256, self.net.stream if self.net is not None else None), "vaicu_memset")
            fused_run = dev.lib.vaicu_linear_run_argmax
            lin._launch.kernel_launches = 0

            def launch(stream):
                # nobody else reads the logits (that is why the nodes merged): they are not stored
                _lib.check(fused_run(plan, stream, li, lw, lb, lr, None, ws, 0, None, op), "vaicu_linear_run_argmax")

            launch.kernel_launches = 1
            return launch
        if self["partial"].valid_shape():
            ws = self["partial"].ptr
            pairs = dev.lib.vaicu_argmax_pairs_run

            def launch(stream):
                _lib.check(pairs(stream, xp, dt, M, N, N, 0, ws, None, op), "vaicu_argmax_pairs_run")

            launch.kernel_launches = 2
            return launch
        run = dev.lib.vaicu_argmax_run

        def launch(stream):
            _lib.check(run(stream, xp, dt, M, N, op), "vaicu_argmax_run")

        launch.kernel_launches = 1
        return launch


class TopKSamplingNode(Node):
    """Row-wise top-k sampling (vAi vai/nodes/topk-sampling.h:9-31): in0 [..., N] logits ->
    out0 [...] raw uint32 indices in 4-byte slots.  Keeps the k largest logits of each row,
    softmax over them at `temperature`, inverse-CDF sample with the uniform given by
    set_uniform(u) before each forward (the reference's setUniform).  The uniform lives in a
    4-byte device buffer that the recorded launch reads, so replays see the new value."""

    MAX_K = 128

    def __init__(self, k=40, temperature=1.0):
        super().__init__()
        if not 1 <= int(k) <= self.MAX_K:
            raise ValueError(f"k must be in 1..{self.MAX_K}")
        self.k, self.temperature = int(k), float(temperature)
        self.add_slot("out0", OUTPUT)
        self.add_slot("in0", INPUT)
        self.add_slot("partial", TEMPORARY)
        self._uniform = None          # DeviceBuffer of one float
        self._u_host = 0.0

    def _device(self):
        from .engine import Device
        return self.net.device if self.net is not None else Device.default()

    def set_uniform(self, u):
        """The uniform in [0, 1) used by the next forward."""
        self._u_host = float(u)
        if self._uniform is not None:
            self._uniform.upload(np.array([self._u_host], dtype=np.float32))

    def prepare(self):
        x = self["in0"]
        if not x.valid_shape() or len(x.shape) < 2:
            raise ValueError("in0 must have at least two axes")
        rows = x.num_elements() // x.shape[-1]
        self.slots["out0"] = Tensor(tuple(x.shape[:-1]), Dtype.F32)
        dev = self._device()
        ws = ctypes.c_size_t()
        _lib.check(dev.lib.vaicu_topk_workspace_bytes(rows, x.shape[-1], self.k, ctypes.byref(ws)), "vaicu_topk_workspace_bytes")
        self.slots["partial"] = Tensor((ws.value // 4,), Dtype.F32) if ws.value else Tensor()

    def bind(self):
        from .engine import DeviceBuffer
        dev = self._device()
        if self._uniform is None:
            self._uniform = DeviceBuffer(dev, 4)
        self._uniform.upload(np.array([self._u_host], dtype=np.float32))
        x, o = self["in0"], self["out0"]
        rows, n = x.num_elements() // x.shape[-1], x.shape[-1]
        xp, op, up, dt = x.ptr, o.ptr, self._uniform.ptr, int(x.dtype)
        ws = self["partial"].ptr if self["partial"].valid_shape() else None
        k, temp = self.k, self.temperature
        run = dev.lib.vaicu_topk_sample_run

        def launch(stream):
            _lib.check(run(stream, xp, dt, rows, n, k, temp, up, ws, op), "vaicu_topk_sample_run")

        launch.kernel_launches = 2 if ws else 1
        return launch


class RmsNormNode(Node):
    """RMS normalisation over the last axis (vAi vai/nodes/rms-norm.h:9-24):
    out0 = in0 * rsqrt(mean(in0^2) + eps) (* scale) (+ shift) (+ residual).
    `scale` / `shift` [D] apply when set (parameters, or inputs under coeffs_as_inputs);
    accept_residual opens the `residual` input (same shape and dtype as in0).  With
    set_o_dtype(F16 / BF16) the node hands 16-bit activations to the Linear after it."""

    _entry = "vaicu_rms_norm_run"

    def __init__(self, eps=1e-5, coeffs_as_inputs=False, accept_residual=False):
        super().__init__()
        self.eps = float(eps)
        self.coeffs_as_inputs = bool(coeffs_as_inputs)
        self.accept_residual = bool(accept_residual)
        self.add_slot("out0", OUTPUT)
        self.add_slot("in0", INPUT)
        kind = INPUT if self.coeffs_as_inputs else PERSISTENT
        self.add_slot("scale", kind)
        self.add_slot("shift", kind)
        if self.accept_residual:
            self.add_slot("residual", INPUT)

    def has_scale(self):
        return self["scale"].valid_shape()

    def has_shift(self):
        return self["shift"].valid_shape()

    def prepare(self):
        x = self["in0"]
        if not x.valid_shape() or len(x.shape) < 2:
            raise ValueError("in0 must have at least two axes")
        feat = x.shape[-1]
        w_dtype = Dtype.NONE
        for name in ("scale", "shift"):
            t = self[name]
            if t.valid_shape():
                if t.shape[-1] != feat or t.num_elements() != feat:
                    raise ValueError(f"{name} must hold {feat} elements")
                if w_dtype != Dtype.NONE and t.dtype != w_dtype:
                    raise ValueError("scale and shift must share a dtype")
                w_dtype = t.dtype
        if self.accept_residual:
            r = self["residual"]
            if tuple(r.shape) != tuple(x.shape) or r.dtype != x.dtype:
                raise ValueError("residual must match in0's shape and dtype")
        self._w_dtype = w_dtype
        o_dtype = self.o_dtype if self.o_dtype != Dtype.NONE else (self.net.o_default_dtype if self.net else Dtype.F32)
        self.slots["out0"] = Tensor(x.shape, o_dtype)

    def bind(self):
        from .engine import Device
        dev = self.net.device if self.net is not None else Device.default()
        x, o = self["in0"], self["out0"]
        rows = x.num_elements() // x.shape[-1]
        args = (dev.handle, x.ptr, self["scale"].ptr if self.has_scale() else None,
                self["shift"].ptr if self.has_shift() else None,
                self["residual"].ptr if self.accept_residual else None, o.ptr, rows, x.shape[-1],
                int(x.dtype), int(self._w_dtype), int(o.dtype), self.eps)
        entry = self._entry
        run = getattr(dev.lib, entry)

        def launch(stream):
            _lib.check(run(args[0], stream, *args[1:]), entry)

        launch.kernel_launches = 1
        return launch


class LayerNormNode(RmsNormNode):
    """Layer normalisation over the last axis (vAi vai/nodes/layer-norm.h:9-31):
    out0 = (in0 - mean) * rsqrt(var + eps) * scale (+ shift) (+ residual), biased variance,
    fp32 statistics.  Same slots and options as the reference node: `scale` is required,
    `shift` applies when set; both are parameters, or inputs under coeffs_as_inputs."""

    _entry = "vaicu_layer_norm_run"

    def prepare(self):
        if not self.has_scale():
            raise ValueError("LayerNorm needs a scale")
        super().prepare()
