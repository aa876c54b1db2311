"""Host side of the Linear path, mirroring the `pyvai` surface the reference's
node tests use (vAi python/bindings, python/tests/node_check.py): Dtype,
Epilogue, ResidualOrder, Tensor, Node, NeuralNet and the `input - node - output`
wiring.  Everything that touches the GPU goes through the C ABI (vai_b200._lib).

Scope: what a graph of Linear nodes needs.  A net records once per input-shape
set (prepare() + buffer binding + run(), vAi vai/engine/neural-net.cpp:406-518)
and afterwards replays the recording (neural-net.h:391-438) — here a CUDA graph.
"""
import ctypes
import enum
import threading

import numpy as np

from . import _lib


class Dtype(enum.IntEnum):
    """vai::Dtype (vai/engine/tensor.h:19); BF16 is the one added value."""
    F32 = 0
    F16 = 1
    NONE = 2
    BF16 = 3


class Epilogue(enum.IntEnum):
    """vai::Epilogue (vai/nodes/common.h:31-39)."""
    NONE = 0
    RELU = 1
    GELU = 2
    GELU_TANH = 3
    SILU = 4
    SIGMOID = 5


class ResidualOrder(enum.IntEnum):
    """vai::ResidualOrder (vai/nodes/common.h:42-45)."""
    AFTER_EPILOGUE = 0
    BEFORE_EPILOGUE = 1


def dtype_size(dt):
    return 4 if dt == Dtype.F32 else 2


# ---- host conversions (the loader's, vAi vai/engine/tensor.cpp:46-85) ---------

def f32_to_f16_bits(a):
    """fp32 -> fp16 bit patterns: round to nearest even, results below the smallest
    normal flush to zero, overflow saturates to inf."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    with np.errstate(over="ignore"):
        h = a.astype(np.float16)
    tiny = np.abs(a) < np.float32(2.0 ** -14)
    h = np.where(tiny, np.copysign(np.float16(0), a).astype(np.float16), h)
    return h.view(np.uint16)


def f32_to_bf16_bits(a):
    """fp32 -> bf16 bit patterns, round to nearest even, NaN quieted."""
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = ((b >> 23) & 0xFF == 0xFF) & ((b & 0x7FFFFF) != 0)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(nan, ((b >> 16) | 0x40).astype(np.uint16), r)


def bits_to_f32(bits, dt):
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    if dt == Dtype.F16:
        return bits.view(np.float16).astype(np.float32)
    return (bits.astype(np.uint32) << 16).view(np.float32)


def encode(a, dt):
    """fp32 values -> the array a device buffer of dtype `dt` holds."""
    if dt == Dtype.F32:
        return np.ascontiguousarray(a, dtype=np.float32)
    return f32_to_f16_bits(a) if dt == Dtype.F16 else f32_to_bf16_bits(a)


# ---- device objects ---------------------------------------------------------------

class Device:
    """One GPU (stands where eva::Device does, vAi vai/engine/neural-net.h:251-257)."""
    _default = None
    _lock = threading.Lock()

    def __init__(self, ordinal=0):
        self.lib = _lib.load()
        h = ctypes.c_void_p()
        _lib.check(self.lib.vaicu_device_open(ordinal, ctypes.byref(h)), "vaicu_device_open")
        self.handle = h
        self.ordinal = ordinal
        n = ctypes.c_int()
        _lib.check(self.lib.vaicu_device_sm_count(h, ctypes.byref(n)), "vaicu_device_sm_count")
        self.sm_count = n.value

    @classmethod
    def default(cls):
        with cls._lock:
            if cls._default is None:
                cls._default = Device(0)
            return cls._default

    def synchronize(self):
        _lib.check(self.lib.vaicu_device_synchronize(self.handle), "vaicu_device_synchronize")

    def check_status(self):
        """Raises if a kernel reported an expired bounded wait since the last check."""
        word = ctypes.c_int()
        _lib.check(self.lib.vaicu_device_status(self.handle, ctypes.byref(word)), "vaicu_device_status")

    def create_stream(self):
        s = ctypes.c_void_p()
        _lib.check(self.lib.vaicu_stream_create(self.handle, ctypes.byref(s)), "vaicu_stream_create")
        return s


class DeviceBuffer:
    """cudaMalloc'ed range owned through the C ABI (eva::Buffer's place)."""

    def __init__(self, device, nbytes):
        self.device = device
        h = ctypes.c_void_p()
        _lib.check(device.lib.vaicu_buffer_alloc(device.handle, nbytes, ctypes.byref(h)), "vaicu_buffer_alloc")
        self.handle = h
        self.ptr = device.lib.vaicu_buffer_ptr(h)
        self.nbytes = device.lib.vaicu_buffer_size(h)

    # Buffers whose last reference dies while a recording is being captured (the
    # garbage collector can run at any time) are freed after the capture ends.
    _capturing = 0
    _deferred = []

    def free(self):
        if self.handle:
            if DeviceBuffer._capturing:
                DeviceBuffer._deferred.append((self.device.lib, self.handle))
            else:
                self.device.lib.vaicu_buffer_free(self.handle)
            self.handle = None
            self.ptr = None

    @classmethod
    def end_capture(cls):
        cls._capturing -= 1
        if cls._capturing == 0:
            pending, cls._deferred = cls._deferred, []
            for lib, h in pending:
                lib.vaicu_buffer_free(h)

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def upload(self, array, stream=None):
        a = np.ascontiguousarray(array)
        assert a.nbytes <= self.nbytes
        _lib.check(self.device.lib.vaicu_memcpy_h2d(self.ptr, a.ctypes.data, a.nbytes, stream), "vaicu_memcpy_h2d")
        if stream is not None:
            _lib.check(self.device.lib.vaicu_stream_sync(stream), "vaicu_stream_sync")

    def download(self, array, stream=None):
        assert array.flags["C_CONTIGUOUS"] and array.nbytes <= self.nbytes
        _lib.check(self.device.lib.vaicu_memcpy_d2h(array.ctypes.data, self.ptr, array.nbytes, stream), "vaicu_memcpy_d2h")
        if stream is not None:
            _lib.check(self.device.lib.vaicu_stream_sync(stream), "vaicu_stream_sync")
        return array


class GuardedBuffer:
    """A pooled range with `guard` canary bytes on either side (debugging aid: with
    compute-sanitizer unavailable, this is how the tests see a kernel that writes outside
    its output or workspace).  Same surface as DeviceBuffer; `ptr` is the inner range."""
    CANARY = 0xA5

    def __init__(self, device, nbytes, guard):
        self.device, self.guard, self.nbytes = device, guard, nbytes
        self.outer = DeviceBuffer(device, nbytes + 2 * guard)
        _lib.check(device.lib.vaicu_memset(self.outer.ptr, self.CANARY, self.outer.nbytes, None), "vaicu_memset")
        device.synchronize()
        self.ptr = self.outer.ptr + guard

    def upload(self, array, stream=None):
        a = np.ascontiguousarray(array)
        assert a.nbytes <= self.nbytes
        _lib.check(self.device.lib.vaicu_memcpy_h2d(self.ptr, a.ctypes.data, a.nbytes, stream), "vaicu_memcpy_h2d")

    def download(self, array, stream=None):
        assert array.flags["C_CONTIGUOUS"] and array.nbytes <= self.nbytes
        _lib.check(self.device.lib.vaicu_memcpy_d2h(array.ctypes.data, self.ptr, array.nbytes, stream), "vaicu_memcpy_d2h")
        if stream is not None:
            _lib.check(self.device.lib.vaicu_stream_sync(stream), "vaicu_stream_sync")
        return array

    def intact(self):
        """True while both guard zones still hold the canary."""
        self.device.synchronize()
        lo = np.empty(self.guard, dtype=np.uint8)
        hi = np.empty(self.guard, dtype=np.uint8)
        lib = self.device.lib
        _lib.check(lib.vaicu_memcpy_d2h(lo.ctypes.data, self.outer.ptr, self.guard, None), "vaicu_memcpy_d2h")
        _lib.check(lib.vaicu_memcpy_d2h(hi.ctypes.data, self.ptr + self.nbytes, self.guard, None), "vaicu_memcpy_d2h")
        return bool((lo == self.CANARY).all() and (hi == self.CANARY).all())

    def free(self):
        self.outer.free()


class BufferPool:
    """Size-keyed reuse of device buffers (vAi vai/engine/buffer-pool.h:77-153).  With
    guard > 0 every range it hands out sits between canary zones of that many bytes
    (a multiple of 256, so the inner range keeps its alignment); check_guards() reports
    ranges whose zones were written."""

    def __init__(self, device, guard=0):
        self.device = device
        self.free = {}
        self.guard = (guard + 255) // 256 * 256 if guard else 0
        self.handed_out = []

    def request(self, nbytes):
        nbytes = max(256, (nbytes + 255) // 256 * 256)
        lst = self.free.get(nbytes)
        if lst:
            return lst.pop()
        if self.guard:
            buf = GuardedBuffer(self.device, nbytes, self.guard)
            self.handed_out.append(buf)
            return buf
        return DeviceBuffer(self.device, nbytes)

    def check_guards(self):
        bad = [b for b in self.handed_out if not b.intact()]
        if bad:
            raise AssertionError(f"{len(bad)} of {len(self.handed_out)} pooled ranges were written outside their bounds")
        return len(self.handed_out)

    def release(self, buf):
        self.free.setdefault(buf.nbytes, []).append(buf)


class HostMappedBuffer:
    """Page-locked host memory used as a kernel's output: with unified addressing the device
    stores to it directly, so a small result (a sampled token) reaches the host without a
    copy command of its own.  Same surface as DeviceBuffer where the engine needs it."""

    def __init__(self, net, nbytes):
        self.device = net.device
        self.view, p = net._pinned(nbytes, np.uint8, (max(nbytes, 4),))
        self.ptr = p.value
        self.nbytes = nbytes

    def download(self, array, stream=None):
        np.copyto(array.reshape(-1).view(np.uint8), self.view[:array.nbytes])
        return array

    def free(self):
        pass


class Tensor:
    """Shape + dtype + host array and/or device buffer (vAi vai/engine/tensor.h:111-332).
    Copies share storage, as the reference's handle does."""

    def __init__(self, shape=None, dtype=Dtype.F32):
        self.shape = tuple(int(s) for s in shape) if shape is not None else None
        self.dtype = Dtype(dtype)
        self.host = None        # np.float32, or np.uint16 bit patterns for F16 / BF16
        self.buffer = None      # DeviceBuffer
        self.byte_offset = 0

    @staticmethod
    def from_numpy(array, dtype=None):
        a = np.asarray(array)
        if dtype is None:
            dtype = Dtype.F16 if a.dtype == np.float16 else Dtype.F32
        t = Tensor(a.shape, dtype)
        if a.dtype == np.float16 and dtype == Dtype.F16:
            t.host = np.ascontiguousarray(a).view(np.uint16)
        elif a.dtype == np.uint16 and dtype != Dtype.F32:
            t.host = np.ascontiguousarray(a)
        else:
            t.host = encode(a.astype(np.float32), dtype)
        return t

    def valid_shape(self):
        return self.shape is not None

    def num_elements(self):
        return int(np.prod(self.shape)) if self.shape is not None else 0

    def nbytes(self):
        return self.num_elements() * dtype_size(self.dtype)

    def astype(self, dtype):
        """Host-side conversion (vAi Tensor dtype conversion, tensor.h:31-41)."""
        if Dtype(dtype) == self.dtype:
            return self
        assert self.host is not None
        vals = self.host if self.dtype == Dtype.F32 else bits_to_f32(self.host, self.dtype)
        t = Tensor(self.shape, dtype)
        t.host = encode(vals.reshape(self.shape), dtype)
        return t

    @property
    def ptr(self):
        return None if self.buffer is None else self.buffer.ptr + self.byte_offset

    def to_device(self, device, pool=None):
        if self.buffer is None:
            self.buffer = pool.request(self.nbytes()) if pool else DeviceBuffer(device, self.nbytes())
            if self.host is not None:
                self.buffer.upload(self.host)
        return self

    def download_bits(self):
        assert self.buffer is not None
        self.buffer.device.synchronize()
        out = np.empty(self.shape, dtype=np.float32 if self.dtype == Dtype.F32 else np.uint16)
        return self.buffer.download(out)

    def to_u32(self):
        """The 4-byte slots read as raw uint32 (index outputs such as Argmax's)."""
        raw = self.download_bits() if self.buffer is not None else self.host
        return np.array(raw, dtype=np.float32).view(np.uint32)

    def to_numpy(self):
        """float32 for F32 / BF16, float16 for F16."""
        raw = self.download_bits() if self.buffer is not None else self.host
        if self.dtype == Dtype.F32:
            return np.array(raw, dtype=np.float32)
        if self.dtype == Dtype.F16:
            return np.array(raw).view(np.float16)
        return bits_to_f32(raw, Dtype.BF16)


# ---- graph: slots, nodes, flows ----------------------------------------------------

INPUT, OUTPUT, TEMPORARY, PERSISTENT = "input", "output", "temporary", "persistent"


class Node:
    """Operator base (vAi vai/engine/neural-net.h:150-226): named slots, prepare(),
    run(stream).  A node attaches to the net being constructed on this thread."""

    def __init__(self):
        self.slots = {}
        self.slot_types = {}
        self.links = {}          # input slot -> (producer node, producer slot): the first producer wired
        self.producers = {}      # input slot -> every producer wired (two only where a gate's branches merge)
        self.o_dtype = Dtype.NONE
        self.net = NeuralNet._current()
        if self.net is not None:
            self.net._nodes.append(self)

    def add_slot(self, name, kind):
        self.slots[name] = Tensor()
        self.slot_types[name] = kind

    def __getitem__(self, name):
        return self.slots[name]

    def __setitem__(self, name, tensor):
        if name not in self.slots:
            raise KeyError(name)
        self.slots[name] = tensor
        if self.net is not None:
            self.net._dirty = True

    def set_o_dtype(self, dtype):
        self.o_dtype = Dtype(dtype)

    # `"slot" / node` picks the input slot, `node / "slot"` the output slot
    def __rtruediv__(self, slot):
        return Flow(self, in_slot=slot)

    def __truediv__(self, slot):
        return Flow(self, out_slot=slot)

    def __sub__(self, other):
        return Flow(self) - other

    def prepare(self):
        raise NotImplementedError

    def bind(self):
        """The launches of this node with the buffers bound right now, as a
        callable(stream); what run() would record into a command buffer."""
        raise NotImplementedError

    def run(self, stream):
        self.bind()(stream)


class Flow:
    """One hop of `a - b - c` (vAi vai/engine/graph-flow.h:26-63)."""

    def __init__(self, node, in_slot="in0", out_slot="out0"):
        self.node, self.in_slot, self.out_slot = node, in_slot, out_slot

    def __truediv__(self, slot):
        return Flow(self.node, self.in_slot, slot)

    def __sub__(self, other):
        nxt = other if isinstance(other, Flow) else Flow(other)
        if nxt.in_slot not in nxt.node.slots or self.out_slot not in self.node.slots:
            raise KeyError(f"no such slot: {self.out_slot} -> {nxt.in_slot}")
        srcs = nxt.node.producers.setdefault(nxt.in_slot, [])
        if (self.node, self.out_slot) not in srcs:
            srcs.append((self.node, self.out_slot))
        nxt.node.links[nxt.in_slot] = srcs[0]
        if nxt.node.net is not None:
            nxt.node.net._dirty = True
        return nxt


class InputNode(Node):
    def __init__(self, name):
        super().__init__()
        self.name = name
        self.add_slot("out0", OUTPUT)

    def prepare(self):
        pass

    def bind(self):
        return lambda stream: None


class OutputNode(Node):
    def __init__(self, name):
        super().__init__()
        self.name = name
        self.add_slot("in0", INPUT)

    def prepare(self):
        pass

    def bind(self):
        return lambda stream: None


class GateNode(Node):
    """Conditional branch without computation (vAi vai/nodes/gate.h:9-60): `then` and `else`
    both alias in0; one branch is recorded per recording, the engine leaves out every node that
    only the closed branch reaches, and a node both branches reach (the merge point, where two
    producers may share an input slot, and everything past it) is kept.  The condition is host
    state: the net keeps one recording per combination of gate states, so a decode loop that
    flips a gate back and forth records each state once and replays from then on."""

    def __init__(self):
        super().__init__()
        self.add_slot("in0", INPUT)
        self.add_slot("then", OUTPUT)
        self.add_slot("else", OUTPUT)
        self._open = True

    def is_open(self):
        return self._open

    def set_open(self, is_open):
        self._open = bool(is_open)

    def prepare(self):
        self.slots["then"] = self.slots["in0"]
        self.slots["else"] = self.slots["in0"]

    def bind(self):
        return lambda stream: None


class _Recording:
    def __init__(self):
        self.input_tensors = {}
        self.outputs = {}
        self.graph = None
        self.keep = []
        self.pinned = []        # page-locked host allocations made for this recording


class NeuralNet:
    """Graph owner (vAi vai/engine/neural-net.h:293-449) for graphs of the nodes in
    this package.  `net(x)` / `net(in0=x, residual=r)` returns the output Tensor (a
    dict when there are several outputs)."""
    _tls = threading.local()

    @classmethod
    def _current(cls):
        return getattr(cls._tls, "net", None)

    def __init__(self, w_default_dtype=Dtype.F16, o_default_dtype=Dtype.F32, device=None, use_graph=True,
                 parallel_branches=True, group_siblings=True, fuse_gated_mul=True, fuse_argmax=True, guard_bytes=0):
        if Dtype(w_default_dtype) == Dtype.NONE or Dtype(o_default_dtype) == Dtype.NONE:
            raise ValueError("default dtypes may not be NONE")
        self.w_default_dtype = Dtype(w_default_dtype)
        self.o_default_dtype = Dtype(o_default_dtype)
        self.device = device or Device.default()
        self.pool = BufferPool(self.device, guard_bytes)      # guard_bytes > 0: canary zones round every pooled range
        self.stream = self.device.create_stream()
        self._streams = [self.stream]
        self.parallel_branches = parallel_branches
        self.group_siblings = group_siblings
        # a GatedMul that is the only reader of a gate|value Linear is recorded into that
        # Linear's launch (False: always two launches and the [.., 2H] intermediate)
        self.fuse_gated_mul = fuse_gated_mul
        # an Argmax that is the only reader of a weight-streaming Linear shares that Linear's launch
        self.fuse_argmax = fuse_argmax
        self.max_side_streams = 3
        # outputs up to this size that nothing else reads are stored by their kernel directly into
        # page-locked host memory (0: always a device buffer and a device-to-host copy)
        self.direct_output_bytes = 4096
        self.use_graph = use_graph
        self._nodes = []
        self._inputs = {}
        self._outputs = {}
        self._recordings = {}
        self._dirty = False
        self._pinned_ptrs = []
        self._pin_sink = self._pinned_ptrs
        self._input_names = self._input_order = None
        self._gate_nodes = None
        self.h2d_bytes = self.d2h_bytes = 0
        NeuralNet._tls.net = self

    def input(self, name):
        if name not in self._inputs:
            self._inputs[name] = InputNode(name)
        return Flow(self._inputs[name])

    def output(self, name):
        if name not in self._outputs:
            self._outputs[name] = OutputNode(name)
        return Flow(self._outputs[name])

    def _sorted(self):
        # Kahn's algorithm over the links (vAi neural-net.cpp:282-354)
        indeg = {n: 0 for n in self._nodes}
        users = {n: [] for n in self._nodes}
        for n in self._nodes:
            for srcs in n.producers.values():
                for src, _ in srcs:
                    indeg[n] += 1
                    users[src].append(n)
        ready = [n for n in self._nodes if indeg[n] == 0]
        order = []
        while ready:
            n = ready.pop(0)
            order.append(n)
            for u in users[n]:
                indeg[u] -= 1
                if indeg[u] == 0:
                    ready.append(u)
        if len(order) != len(self._nodes):
            raise RuntimeError("the graph has a cycle")
        self._check_fan_in(order)
        return order

    def _check_fan_in(self, order):
        """Two producers may share an input slot only where one gate's two branches meet
        (vAi vai/engine/graph-controller.h:66-70): per node, which gate branches reach it."""
        gates = [n for n in order if isinstance(n, GateNode)]
        bit = {g: 1 << i for i, g in enumerate(gates)}
        then_bits, else_bits = {}, {}
        for n in order:
            t = e = 0
            for srcs in n.producers.values():
                for src, src_slot in srcs:
                    t |= then_bits[src]
                    e |= else_bits[src]
                    if isinstance(src, GateNode):
                        if src_slot == "then":
                            t |= bit[src]
                        elif src_slot == "else":
                            e |= bit[src]
            then_bits[n], else_bits[n] = t, e
        for n in order:
            for slot, srcs in n.producers.items():
                if len(srcs) == 1:
                    continue

                def side(src, src_slot):
                    t, e = then_bits[src], else_bits[src]
                    if isinstance(src, GateNode):
                        t |= bit[src] if src_slot == "then" else 0
                        e |= bit[src] if src_slot == "else" else 0
                    return t, e

                ok = False
                if len(srcs) == 2:
                    (t0, e0), (t1, e1) = side(*srcs[0]), side(*srcs[1])
                    ok = bool((t0 & ~e0) & (e1 & ~t1)) or bool((t1 & ~e1) & (e0 & ~t0))
                if not ok:
                    raise RuntimeError(f"slot {slot} has {len(srcs)} producers that are not the two branches of one gate")

    def _live(self, order, fed_names):
        """What this recording keeps (vAi graph-controller.h:13-32): an input node is live when
        it is fed, a gate's branch when the gate is live and set that way, any other node when
        every wired input slot has a live producer.  Returns {node: {slot: live producer}}."""
        chosen = {}

        def out_live(src, src_slot):
            if src not in chosen:
                return False
            if isinstance(src, GateNode):
                return (src_slot == "then") == src.is_open() if src_slot in ("then", "else") else True
            return True

        for n in order:
            if isinstance(n, InputNode):
                if n.name in fed_names:
                    chosen[n] = {}
                continue
            picks = {}
            alive = True
            for slot, srcs in n.producers.items():
                live = [p for p in srcs if out_live(*p)]
                if not live:
                    alive = False
                    break
                picks[slot] = live[0]
            if alive:
                chosen[n] = picks
        return chosen

    def _upload_params(self):
        # persistent slots -> device in the dtype their tensor carries; a slot the
        # loader left empty (Linear's "bias") stays off (vAi neural-net.cpp:356-404)
        for n in self._nodes:
            for name, kind in n.slot_types.items():
                t = n.slots[name]
                if kind == PERSISTENT and t.valid_shape() and t.buffer is None:
                    t.to_device(self.device)
                    t.host = None      # the device copy is the parameter from here on

    def _record(self, fed):
        rec = _Recording()
        self._pin_sink = rec.pinned
        try:
            return self._record_into(rec, fed)
        finally:
            self._pin_sink = self._pinned_ptrs

    def _record_into(self, rec, fed):
        lib = self.device.lib
        for name, t in fed.items():
            dev_t = Tensor(t.shape, t.dtype)
            dev_t.buffer = self.pool.request(dev_t.nbytes())
            rec.input_tensors[name] = dev_t
            self._inputs[name].slots["out0"] = dev_t
        live = self._live(self._sorted(), set(fed))
        order = [n for n in self._sorted() if n in live]
        # A small result that only the net's output reads (a sampled token) is written by its
        # kernel straight into page-locked host memory: no copy command after the launches.
        uses = {}
        for n in order:
            for src in (live[n].values() if n.producers else n.links.values()):
                uses[src] = uses.get(src, 0) + 1
        # Linear -> GatedMul becomes one launch when nothing else reads the Linear's output
        for n in self._nodes:
            if hasattr(n, "reset_fusion"):
                n.reset_fusion()
        for n in order:
            absorb = getattr(n, "absorb_into_producer", None)
            if absorb is not None and getattr(self, "fuse_" + n.fusion_kind):
                src = (live[n] if n.producers else n.links).get("in0")
                if src is not None and uses.get(src, 0) == 1:
                    absorb(*src)
        direct = set()
        for out in self._outputs.values():
            if out in live and "in0" in live[out] and uses.get(live[out]["in0"], 0) == 1:
                direct.add(live[out]["in0"])
        # prepare() fixes shapes and plans, then outputs / temporaries get buffers
        bound = {}
        level = {}
        for n in order:
            n.links = dict(live[n]) if n.producers else n.links      # this recording's producer of every slot
            for slot, (src, src_slot) in n.links.items():
                n.slots[slot] = src.slots[src_slot]
            n.prepare()
            for name, kind in n.slot_types.items():
                t = n.slots[name]
                if kind in (OUTPUT, TEMPORARY) and t.valid_shape() and t.buffer is None and t.nbytes() > 0:
                    if kind == OUTPUT and (n, name) in direct and t.nbytes() <= self.direct_output_bytes:
                        t.buffer = HostMappedBuffer(self, t.nbytes())
                    else:
                        t.buffer = self.pool.request(t.nbytes())
                    rec.keep.append(t)
            bound[n] = n.bind()
            level[n] = 1 + max((level[src] for src, _ in n.links.values()), default=-1)
        for name, out in self._outputs.items():
            if out not in live:
                continue            # nothing this recording keeps feeds it
            rec.outputs[name] = out.slots["in0"] if "in0" not in out.links else out.links["in0"][0].slots[out.links["in0"][1]]
        if not rec.outputs:
            raise RuntimeError("no output is reachable from the inputs given")
        # Nodes of one level do not depend on each other (q / k / v of a block): they go to
        # side streams between a fork and a join, so their launch latencies overlap.
        def scratch(nbytes):
            t = Tensor(((nbytes + 3) // 4,), Dtype.F32)
            t.buffer = self.pool.request(t.nbytes())
            rec.keep.append(t)
            return t

        by_level = {}
        for n in order:
            if not isinstance(n, (InputNode, OutputNode)):
                by_level.setdefault(level[n], []).append(n)
        ops = []
        for lv in sorted(by_level):
            group = by_level[lv]
            launches = []
            if self.group_siblings:
                # sibling Linears that read the same tensor and do nothing after the dot
                # product (q / k / v) share one launch
                rest, by_input = [], {}
                for n in group:
                    if getattr(n, "groupable", None) and n.groupable():
                        by_input.setdefault((id(n.slots["in0"]),) + n.group_key(), []).append(n)
                    else:
                        rest.append(n)
                for members in by_input.values():
                    while len(members) >= 2:
                        take, members = members[:3], members[3:]
                        fn = type(take[0]).bind_group(take, scratch)
                        if fn is None:
                            rest += take
                        else:
                            launches.append(fn)
                    rest += members
                launches += [bound[n] for n in rest]
            else:
                launches = [bound[n] for n in group]
            if len(launches) == 1 or not self.parallel_branches:
                ops += [("run", 0, fn) for fn in launches]
                continue
            width = min(len(launches), 1 + self.max_side_streams)
            sides = list(range(1, width))
            ops.append(("fork", sides, None))
            ops += [("run", i % width, fn) for i, fn in enumerate(launches)]
            ops.append(("join", sides, None))
        while len(self._streams) < 1 + self.max_side_streams and any(op[0] == "fork" for op in ops):
            self._streams.append(self.device.create_stream())
        rec.ops = ops
        rec.kernel_launches = sum(getattr(op[2], "kernel_launches", 0) for op in ops if op[0] == "run")
        if self.use_graph:
            _lib.check(lib.vaicu_graph_capture_begin(self.stream), "vaicu_graph_capture_begin")
            DeviceBuffer._capturing += 1
            try:
                self._play(ops)
            finally:
                g = ctypes.c_void_p()
                rc = lib.vaicu_graph_capture_end(self.stream, ctypes.byref(g))
                DeviceBuffer.end_capture()
            _lib.check(rc, "vaicu_graph_capture_end")
            rec.graph = g
        # page-locked staging for the net's inputs and outputs, and a second recording that
        # brackets the same launches with the host<->device copies: one submission per call
        rec.stage_in, rec.stage_out = {}, {}
        for name, t in rec.input_tensors.items():
            rec.stage_in[name] = self._pinned(t.nbytes(), np.float32 if t.dtype == Dtype.F32 else np.uint16, t.shape)
        for name, t in rec.outputs.items():
            np_dtype = np.float32 if t.dtype == Dtype.F32 else np.uint16
            if isinstance(t.buffer, HostMappedBuffer):
                rec.stage_out[name] = (t.buffer.view[:t.nbytes()].view(np_dtype).reshape(t.shape), None)
            else:
                rec.stage_out[name] = self._pinned(t.nbytes(), np_dtype, t.shape)
        rec.graph_io = None
        if self.use_graph:
            _lib.check(lib.vaicu_graph_capture_begin(self.stream), "vaicu_graph_capture_begin")
            DeviceBuffer._capturing += 1
            try:
                self._copies_in(rec)
                self._play(ops)
                self._copies_out(rec)
            finally:
                g = ctypes.c_void_p()
                rc = lib.vaicu_graph_capture_end(self.stream, ctypes.byref(g))
                DeviceBuffer.end_capture()
            _lib.check(rc, "vaicu_graph_capture_end")
            rec.graph_io = g
        return rec

    def _copies_in(self, rec):
        lib = self.device.lib
        for name, (view, hp) in rec.stage_in.items():
            _lib.check(lib.vaicu_memcpy_h2d(rec.input_tensors[name].ptr, hp, view.nbytes, self.stream), "vaicu_memcpy_h2d")

    def _copies_out(self, rec):
        lib = self.device.lib
        for name, t in rec.outputs.items():
            view, hp = rec.stage_out[name]
            if hp is not None:          # else the kernel wrote the host memory itself
                _lib.check(lib.vaicu_memcpy_d2h(hp, t.ptr, view.nbytes, self.stream), "vaicu_memcpy_d2h")

    def _play(self, ops):
        lib = self.device.lib
        st = self._streams
        for kind, where, fn in ops:
            if kind == "run":
                fn(st[where])
            elif kind == "fork":
                for i in where:
                    _lib.check(lib.vaicu_stream_wait_stream(st[i], st[0]), "vaicu_stream_wait_stream")
            else:
                for i in where:
                    _lib.check(lib.vaicu_stream_wait_stream(st[0], st[i]), "vaicu_stream_wait_stream")

    def _pinned(self, nbytes, np_dtype, shape):
        """Page-locked host staging viewed as a numpy array (vAi stages inputs the same
        way, vai/engine/neural-net.cpp:219-280)."""
        p = ctypes.c_void_p()
        _lib.check(self.device.lib.vaicu_host_alloc_pinned(max(nbytes, 4), ctypes.byref(p)), "vaicu_host_alloc_pinned")
        self._pin_sink.append(p)
        buf = (ctypes.c_uint8 * max(nbytes, 4)).from_address(p.value)
        return np.frombuffer(buf, dtype=np_dtype, count=int(np.prod(shape))).reshape(shape), p

    def __call__(self, *args, **kwargs):
        names = self._input_names
        if names is None or len(names) != len(self._inputs):
            names = self._input_names = sorted(self._inputs)
            self._input_order = list(self._inputs)
        fed = dict(zip(self._input_order, args))
        if kwargs:
            fed.update(kwargs)
        if not fed or any(k not in self._inputs for k in fed):
            raise ValueError(f"inputs {sorted(fed)} do not match the net's {names}")
        lib = self.device.lib
        # a recording is made for the inputs that came (and the gates as they stand): nodes
        # that need an input left out are not part of it
        key = tuple([(k, fed[k].shape, fed[k].dtype) for k in names if k in fed])
        # the gate nodes are looked up once per node count, not on every call (a step is a few hundred microseconds)
        if self._gate_nodes is None or self._gate_nodes[0] != len(self._nodes):
            self._gate_nodes = (len(self._nodes), [n for n in self._nodes if isinstance(n, GateNode)])
        if self._gate_nodes[1]:
            key += (("gates",) + tuple(n.is_open() for n in self._gate_nodes[1]),)
        if self._dirty:           # a parameter or a wire changed: every recording is stale
            self._drop_recordings()
            self._dirty = False
        rec = self._recordings.get(key)
        if rec is None:
            self._upload_params()
            rec = self._record(fed)
            rec.calls = 0
            rec.h2d_bytes = sum(v.nbytes for v, _ in rec.stage_in.values())
            rec.d2h_bytes = sum(v.nbytes for v, _ in rec.stage_out.values())
            self._recordings[key] = rec
        for name, t in fed.items():
            np.copyto(rec.stage_in[name][0], t.host.reshape(rec.stage_in[name][0].shape))
        if rec.graph_io is not None:
            _lib.check(lib.vaicu_graph_launch(rec.graph_io, self.stream), "vaicu_graph_launch")
        else:
            self._copies_in(rec)
            self._play(rec.ops)
            self._copies_out(rec)
        _lib.check(lib.vaicu_stream_sync(self.stream), "vaicu_stream_sync")
        # the kernels' bounded waits report through a device word: read it on the first
        # replay of a recording and then now and again, not on every step
        if rec.calls % 256 == 0:
            self.device.check_status()
        rec.calls += 1
        self.h2d_bytes, self.d2h_bytes = rec.h2d_bytes, rec.d2h_bytes
        outs = {}
        for name, t in rec.outputs.items():
            host = Tensor(t.shape, t.dtype)
            host.host = rec.stage_out[name][0].copy()
            outs[name] = host
        return outs[next(iter(outs))] if len(outs) == 1 else outs

    def _drop_recordings(self):
        """Recordings go with everything made for them: the graphs, the page-locked staging
        (freed) and the pooled device ranges (back to the pool)."""
        if not self._recordings:
            return
        lib = self.device.lib
        if lib is not None and self.stream is not None:
            lib.vaicu_stream_sync(self.stream)           # nothing recorded is still running
        for rec in self._recordings.values():
            for g in (rec.graph, getattr(rec, "graph_io", None)):
                if g is not None:
                    lib.vaicu_graph_destroy(g)
            rec.graph = rec.graph_io = None
            for p in rec.pinned:
                lib.vaicu_host_free_pinned(p)
            rec.pinned = []
            seen_buffers = set()
            for t in list(rec.input_tensors.values()) + rec.keep:
                b = t.buffer
                if isinstance(b, (DeviceBuffer, GuardedBuffer)) and id(b) not in seen_buffers and b.ptr is not None:
                    seen_buffers.add(id(b))
                    self.pool.release(b)
                t.buffer = None
        self._recordings.clear()

    def __del__(self):
        try:
            self._drop_recordings()
            for p in self._pinned_ptrs:
                self.device.lib.vaicu_host_free_pinned(p)
        except Exception:
            pass
