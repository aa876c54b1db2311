"""GPU: the Linear shapes of the benchmark configurations at FULL size (Llama-3.2-1B
decode, Llama-3.2-3B prefill at M = 8192, Gemma-3-4B batched decode at M = 64), bf16
weights ~N(0, 0.02).  A float64 oracle over the whole output would take minutes, so each
case checks (a) a few thousand sampled outputs against float64 dot products over the
stored operand values, and (b) a size-independent property: linearity in the activations
for the plain Linears, out(a*x1 + b*x2) = a*out(x1) + b*out(x2), evaluated on all outputs.
Tensors are drawn on the device with a seeded generator; the kernels run through the C ABI
on torch's stream (vai_b200.torch_linear)."""
import pytest

pytestmark = pytest.mark.gpu

CASES = [
    # name, M, K, N, gate activation or None, residual, activations dtype
    ("llama1b_lm_head", 1, 2048, 128256, None, False, "f32"),
    ("llama1b_gate_up", 1, 2048, 16384, "SILU", False, "f32"),
    ("llama1b_down", 1, 8192, 2048, None, True, "f32"),
    ("llama3b_gate_up_prefill", 8192, 3072, 16384, "SILU", False, "bf16"),
    ("llama3b_down_prefill", 8192, 8192, 3072, None, True, "bf16"),
    ("llama3b_q_prefill", 8192, 3072, 3072, None, False, "bf16"),
    ("gemma4b_lm_head_m64", 64, 2560, 262144, None, False, "bf16"),
    ("gemma4b_gate_up_m64", 64, 2560, 20480, "GELU_TANH", False, "bf16"),
    ("gemma4b_down_m64", 64, 10240, 2560, None, False, "bf16"),
]


@pytest.mark.parametrize("name,M,K,N,act,residual,xdt", CASES, ids=[c[0] for c in CASES])
def test_full_size_sampled_and_linear(name, M, K, N, act, residual, xdt, device):
    import torch
    import torch.nn.functional as F

    from vai_b200 import Epilogue
    from vai_b200.torch_linear import TorchLinear
    dev = torch.device("cuda", 0)
    import zlib
    g = torch.Generator(device=dev).manual_seed(zlib.crc32(name.encode()))
    x_dtype = torch.float32 if xdt == "f32" else torch.bfloat16
    w = (torch.randn(N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn(M, K, generator=g, device=dev).to(x_dtype)
    gate = act is not None
    n_out = N // 2 if gate else N
    res = torch.randn(M, n_out, generator=g, device=dev).to(x_dtype) if residual else None
    lin = TorchLinear(w, epilogue=getattr(Epilogue, act) if gate else Epilogue.NONE, gate_fuse=gate, device=device)
    out = lin(x, residual=res)
    torch.cuda.synchronize()
    device.check_status()
    assert out.shape == (M, n_out) and torch.isfinite(out.float()).all()

    # (a) sampled outputs against float64 over the values the kernel reads
    S = 4096
    ms = torch.randint(0, M, (S,), generator=g, device=dev)
    ns = torch.randint(0, n_out, (S,), generator=g, device=dev)
    xs = x[ms].double()
    if M > 4 and x_dtype == torch.float32:
        xs = x[ms].to(torch.bfloat16).double()      # tensor-core path stages fp32 activations as bf16
    acc = (xs * w[ns].double()).sum(-1)
    if gate:
        up = (xs * w[n_out + ns].double()).sum(-1)
        acc = (F.silu(acc) if act == "SILU" else F.gelu(acc, approximate="tanh")) * up
    if residual:
        acc = acc + res[ms, ns].double()
    got = out[ms, ns].double()
    tol = 2e-4 * acc.abs() + 5e-5
    if out.dtype == torch.bfloat16:
        tol = tol + 2.0 ** -8 * acc.abs() + 1e-6    # one rounding of the output
    bad = (got - acc).abs() > tol
    assert not bad.any(), f"{name}: {int(bad.sum())} of {S} sampled outputs off; worst {float((got - acc).abs().max()):.3e}"

    # (b) linearity over every output of the plain Linears, fp32 activations:
    #     L(a*x1 + b*x2) = a*L(x1) + b*L(x2).  Exact up to fp32 accumulation where the
    #     activations stay fp32 (M <= 4); where the tensor-core path stages them as bf16 the
    #     three roundings differ, so the bound is the bf16 rounding of the inputs.
    if not gate and not residual:
        lin32 = TorchLinear(w, device=device, out_dtype=torch.float32)
        x1 = torch.randn(M, K, generator=g, device=dev)
        x2 = torch.randn(M, K, generator=g, device=dev)
        a, b = 0.5, -2.0
        lhs = lin32((a * x1 + b * x2).contiguous())
        rhs = a * lin32(x1) + b * lin32(x2)
        again = lin32((a * x1 + b * x2).contiguous())
        torch.cuda.synchronize()
        assert torch.equal(lhs, again), f"{name}: two runs on the same input differ"
        err = (lhs - rhs).abs().max().item()
        scale = rhs.abs().max().item()
        bound = (1e-4 if M <= 4 else 2e-2) * scale + 1e-5
        assert err <= bound, f"{name}: linearity violated by {err:.3e} (scale {scale:.3e})"
