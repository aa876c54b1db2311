"""GPU: GPT-2-small-shaped model (12 blocks, d 768, 12 heads, ffn 3072, vocab 50257,
random fp16 weights ~N(0, 0.02), fp32 activations: the reference's deployed dtypes,
vAi models/production/gpt2/net.h:34,42-53) — 1024-token prefill of uniform random ids
(seed 1), then 128 greedy decode steps, batch 1.

Every Linear and the tied lm_head run on this library (tensor-core kernel in prefill,
weight-streaming kernel in decode); embeddings, LayerNorm and attention are PyTorch ops
standing in for the other vAi nodes.  The reference run shares everything except the
Linears, which it evaluates in float64 over the same stored operand values (fp16
weights; activations rounded to fp16 where the tensor-core path stages them so, as the
reference's cooperative-matrix kernel does).  Greedy tokens must be identical for all
128 steps; the smallest top-2 logit margin seen is printed next to the largest logit
difference.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

L, D, HEADS, FFN, VOCAB = 12, 768, 12, 3072, 50257
PROMPT, STEPS = 1024, 128


def _build(torch, dev):
    g = torch.Generator(device="cpu").manual_seed(0)

    def w(*shape):
        return (torch.randn(*shape, generator=g) * 0.02).to(torch.float16).to(dev)

    p = {"wte": w(VOCAB, D), "wpe": w(PROMPT + STEPS, D), "blocks": []}
    for _ in range(L):
        p["blocks"].append({"attn_w": w(3 * D, D), "attn_b": w(3 * D), "proj_w": w(D, D), "proj_b": w(D),
                            "fc1_w": w(FFN, D), "fc1_b": w(FFN), "fc2_w": w(D, FFN), "fc2_b": w(D)})
    return p


class _OurLinears:
    def __init__(self, params):
        from vai_b200 import Device, Epilogue
        from vai_b200.torch_linear import TorchLinear
        dev = Device.default()
        self.blocks = []
        for b in params["blocks"]:
            self.blocks.append({
                "attn": TorchLinear(b["attn_w"], b["attn_b"], device=dev),
                "proj": TorchLinear(b["proj_w"], b["proj_b"], device=dev),
                "fc1": TorchLinear(b["fc1_w"], b["fc1_b"], epilogue=Epilogue.GELU_TANH, device=dev),
                "fc2": TorchLinear(b["fc2_w"], b["fc2_b"], device=dev),
            })
        self.head = TorchLinear(params["wte"], device=dev)

    def __call__(self, layer, name, x, residual=None):
        lin = self.head if name == "head" else self.blocks[layer][name]
        return lin(x.contiguous(), residual=residual)


class _RefLinears:
    """float64 over the values the kernels read."""

    def __init__(self, torch, params):
        self.torch, self.p = torch, params

    def __call__(self, layer, name, x, residual=None):
        torch = self.torch
        F = torch.nn.functional
        if name == "head":
            wt, b = self.p["wte"], None
        else:
            blk = self.p["blocks"][layer]
            key = {"attn": "attn", "proj": "proj", "fc1": "fc1", "fc2": "fc2"}[name]
            wt, b = blk[key + "_w"], blk[key + "_b"]
        M = x.numel() // x.shape[-1]
        xs = x.to(torch.float16) if M > 8 else x      # tensor-core path stages fp32 activations as fp16
        acc = xs.double() @ wt.double().t()
        if b is not None:
            acc = acc + b.double()
        if name == "fc1":
            acc = F.gelu(acc, approximate="tanh")
        if residual is not None:
            acc = acc + residual.double()
        return acc.float()


def _forward(torch, params, linear, ids, cache, pos0):
    F = torch.nn.functional
    T = ids.numel()
    x = params["wte"][ids].float() + params["wpe"][pos0:pos0 + T].float()
    for i in range(L):
        h = F.layer_norm(x, (D,))
        qkv = linear(i, "attn", h)
        q, k, v = qkv.split(D, dim=-1)
        q, k, v = (t.view(T, HEADS, D // HEADS).transpose(0, 1) for t in (q, k, v))
        if cache[i] is not None:
            k = torch.cat([cache[i][0], k], dim=1)
            v = torch.cat([cache[i][1], v], dim=1)
        cache[i] = (k, v)
        att = F.scaled_dot_product_attention(q, k, v, is_causal=(T > 1))
        att = att.transpose(0, 1).reshape(T, D)
        x = linear(i, "proj", att, residual=x)
        h = F.layer_norm(x, (D,))
        x = linear(i, "fc2", linear(i, "fc1", h), residual=x)
    last = F.layer_norm(x[-1:], (D,))
    return linear(0, "head", last)      # lm_head on the last row only (vAi groups/transformer.h:69-71)


def _generate(torch, params, linear, prompt):
    cache = [None] * L
    logits = _forward(torch, params, linear, prompt, cache, 0)
    tokens, margins, all_logits = [], [], []
    for step in range(STEPS):
        top2 = torch.topk(logits[0], 2)
        tokens.append(int(top2.indices[0]))
        margins.append(float(top2.values[0] - top2.values[1]))
        all_logits.append(logits[0].clone())
        nxt = torch.tensor([tokens[-1]], device=prompt.device)
        logits = _forward(torch, params, linear, nxt, cache, PROMPT + step)
    return tokens, margins, all_logits


def test_gpt2_small_greedy_tokens_identical(device):
    import torch
    torch.backends.cuda.matmul.allow_tf32 = False
    dev = torch.device("cuda", 0)
    params = _build(torch, dev)
    prompt = torch.from_numpy(np.random.default_rng(1).integers(0, VOCAB, PROMPT)).to(dev)
    with torch.no_grad():
        ours, m_ours, lo = _generate(torch, params, _OurLinears(params), prompt)
        ref, m_ref, lr = _generate(torch, params, _RefLinears(torch, params), prompt)
    torch.cuda.synchronize()
    device.check_status()
    worst = max(float((a - b).abs().max()) for a, b in zip(lo, lr))
    print(f"\nmin top-2 margin: ours {min(m_ours):.3e}, reference {min(m_ref):.3e}; max |logit diff| {worst:.3e}; "
          f"distinct tokens generated: {len(set(ours))}")
    assert ours == ref, f"first mismatch at step {next(i for i, (a, b) in enumerate(zip(ours, ref)) if a != b)}"
    assert worst < 2e-2 * max(float(l.abs().max()) for l in lr)
