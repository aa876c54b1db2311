"""Linear shapes of the model presets that route through vAi's Linear node, and a
builder that wires one decode/prefill step's Linear nodes as a chain.

Shapes follow the reference's nets: Llama 3.2 (models/production/llama3/net.h:34-35,
50-62), GPT-2 small (models/production/gpt2/net.h:34,42-53), Gemma 3 4B
(models/production/gemma3/net.h:54).  Per block the reference has separate Linear
nodes for q, k, v, the attention output (+residual), one gate|value Linear, the GatedMul
behind it (vai/groups/gated-feed-forward.h:38-46) and the down projection (+residual); the
lm_head follows the last block.  Only those nodes are built here: attention, norms and
rope are other operators.  The stand-in wiring keeps every Linear's shape, dtype and
epilogue: `o` reads q's output in place of the attention result, the residual inputs
read the net input (unit variance) and the o / down projections carry a scalar_scale,
which together do the job of the missing norms: activations stay O(1) through any
number of blocks with N(0, 0.02) weights.
"""
import numpy as np

from .engine import Dtype, Epilogue, Tensor
from .nodes import GatedMulNode, LinearNode

PRESETS = {
    # name: layers, d_model, q_dim, kv_dim, ffn (H), vocab, gate activation, biases
    "llama-3.2-1b": dict(layers=16, d=2048, q=2048, kv=512, ffn=8192, vocab=128256, act="SILU", gated=True),
    "llama-3.2-3b": dict(layers=28, d=3072, q=3072, kv=1024, ffn=8192, vocab=128256, act="SILU", gated=True),
    "gemma-3-4b": dict(layers=34, d=2560, q=2048, kv=1024, ffn=10240, vocab=262144, act="GELU_TANH", gated=True),
    "gpt2-small": dict(layers=12, d=768, q=768, kv=768, ffn=3072, vocab=50257, act="GELU_TANH", gated=False),
}


def block_linears(p):
    """(name, K, N, extras) of one transformer block's Linear nodes."""
    if p["gated"]:
        return [("q", p["d"], p["q"], {}), ("k", p["d"], p["kv"], {}), ("v", p["d"], p["kv"], {}),
                ("o", p["q"], p["d"], {"residual": True}),
                ("gate_up", p["d"], 2 * p["ffn"], {"gate": True}),
                ("down", p["ffn"], p["d"], {"residual": True})]
    # GPT-2: fused qkv with bias, c_proj (+b +R), fc1 (+b, gelu-tanh), fc2 (+b +R)
    return [("qkv", p["d"], 3 * p["d"], {"bias": True}), ("o", p["d"], p["d"], {"bias": True, "residual": True}),
            ("fc1", p["d"], p["ffn"], {"bias": True, "act": True}), ("fc2", p["ffn"], p["d"], {"bias": True, "residual": True})]


def weight_elements(name):
    p = PRESETS[name]
    per_block = sum(k * n for _, k, n, _ in block_linears(p))
    return p["layers"] * per_block + p["d"] * p["vocab"]


def algorithmic_bytes(name, M, w_bytes=2, io_bytes=4):
    """Bytes one step must move (each operand once): weights, inputs, outputs,
    biases, residuals."""
    p = PRESETS[name]
    total = 0
    for _, k, n, ex in block_linears(p):
        out_n = n // 2 if ex.get("gate") else n
        total += n * k * w_bytes + M * k * io_bytes + M * out_n * io_bytes
        if ex.get("bias"):
            total += n * w_bytes
        if ex.get("residual"):
            total += M * out_n * io_bytes
    total *= p["layers"]
    total += p["vocab"] * p["d"] * w_bytes + M * p["d"] * io_bytes + M * p["vocab"] * io_bytes
    return total


def flops(name, M):
    p = PRESETS[name]
    per_block = sum(2 * M * k * n for _, k, n, _ in block_linears(p))
    return p["layers"] * per_block + 2 * M * p["d"] * p["vocab"]


class _BitsSource:
    """Seeded N(0, std) values in a 16-bit (or fp32) device representation.  One pool of
    random values is drawn once and sliced at rotating offsets, so that building a
    multi-GB model takes seconds; every weight still gets its own device buffer."""

    def __init__(self, dtype, std, seed, pool_elems=1 << 25):
        from .engine import encode
        rng = np.random.default_rng(seed)
        vals = (rng.standard_normal(pool_elems, dtype=np.float32) * np.float32(std))
        self.pool = encode(vals, dtype)
        self.dtype = dtype
        self.off = 0

    def take(self, shape):
        n = int(np.prod(shape))
        out = np.empty(n, dtype=self.pool.dtype)
        filled = 0
        while filled < n:
            m = min(n - filled, self.pool.size - self.off)
            out[filled:filled + m] = self.pool[self.off:self.off + m]
            filled += m
            self.off = (self.off + m + 977) % self.pool.size   # odd stride: slices do not line up
        t = Tensor(shape, self.dtype)
        t.host = out.reshape(shape)
        return t


def build_linear_chain(net, name, *, w_dtype=Dtype.BF16, fuse_gate=True, seed=0, layers=None, lm_head=True,
                       vocab_rows=None, argmax=False, share_weights=None):
    """Adds one step's Linear nodes to `net` and wires them; returns the list of Linear nodes.
    The gated MLP is wired as the reference's group does, gateValue - gatedMul - out;
    fuse_gate=False makes the net record the GatedMul as a launch of its own instead of
    folding it into the gate|value Linear.
    Input slot "x" [M, d]; output "logits" [M, vocab] (or the last hidden state when
    lm_head is False).  With argmax=True an Argmax node follows the lm_head and the
    output is "token" [M] (raw uint32), the greedy-decode step of the reference's nets.
    Weights ~ N(0, 0.02) in `w_dtype`; share_weights = the node list of another chain of
    the same preset makes this chain use those nodes' weight tensors (same storage)."""
    p = PRESETS[name]
    net.fuse_gated_mul = bool(fuse_gate)
    src = _BitsSource(w_dtype, 0.02, seed) if share_weights is None else None
    shared = iter(share_weights) if share_weights is not None else None

    def weight_for(node, shape):
        if shared is None:
            return src.take(shape)
        other = next(shared)
        assert tuple(other["weight"].shape) == tuple(shape)
        if other.has_bias():
            node["bias"] = other["bias"]
        return other["weight"]

    act = getattr(Epilogue, p["act"])
    nodes = []
    x = x0 = net.input("x")
    for _ in range(p["layers"] if layers is None else layers):
        specs = block_linears(p)
        made = {}
        for lname, k, n, ex in specs:
            node = LinearNode(in_dim=k, out_dim=n, accept_residual=bool(ex.get("residual")),
                              epilogue=act if ex.get("act") else Epilogue.NONE,
                              scalar_scale={"o": 0.5, "down": 0.25, "fc2": 0.25}.get(lname, 1.0))
            node["weight"] = weight_for(node, (n, k))
            if ex.get("bias") and shared is None:
                node["bias"] = src.take((n,))
            made[lname] = node
            nodes.append(node)
        if p["gated"]:
            x - made["q"]
            x - made["k"]
            x - made["v"]
            h = made["q"] - made["o"]
            x0 - "residual" / made["o"]
            h - made["gate_up"] - GatedMulNode(activation=act) - made["down"]
            x0 - "residual" / made["down"]
            x = Flow_of(made["down"])
        else:
            x - made["qkv"]
            # attention stand-in: o reads the block input (the reference feeds it the attention output)
            h = x - made["o"]
            x0 - "residual" / made["o"]
            h - made["fc1"] - made["fc2"]
            x0 - "residual" / made["fc2"]
            x = Flow_of(made["fc2"])
    if lm_head:
        v = p["vocab"] if vocab_rows is None else vocab_rows
        head = LinearNode(in_dim=p["d"], out_dim=v)
        head["weight"] = weight_for(head, (v, p["d"]))
        nodes.append(head)
        if argmax:
            from .nodes import ArgmaxNode
            x - head - ArgmaxNode() - net.output("token")
        else:
            x - head - net.output("logits")
    else:
        x - net.output("logits")
    return nodes


def Flow_of(node):
    from .engine import Flow
    return Flow(node)
