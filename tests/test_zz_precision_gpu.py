"""Double-benchmark accuracy check of hand-written kernels: the kernel's error against an fp64 result must be at most
a small multiple of the error that plain PyTorch makes at the same precision (``utils/precision.py``)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _skip_without_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")


def test_gemm_error_is_within_the_bf16_baseline():
    _skip_without_gpu()
    from mindformers_b200.ops import functional as Fn
    from mindformers_b200.utils.precision import DoubleBenchmarkComparator
    torch.manual_seed(0)
    x = torch.randn(512, 1024, device="cuda").to(torch.bfloat16)
    w = (torch.randn(768, 1024, device="cuda") * 0.05).to(torch.bfloat16)
    golden = x.double() @ w.double().t()
    baseline = torch.matmul(x, w.t())
    actual = Fn.gemm(x, w)
    ok, report = DoubleBenchmarkComparator(dtype=torch.bfloat16).check_pass_or_not(actual, baseline, golden)
    assert ok, report


def test_rmsnorm_error_is_within_the_bf16_baseline():
    _skip_without_gpu()
    from mindformers_b200.ops import functional as Fn
    from mindformers_b200.utils.precision import DoubleBenchmarkComparator
    torch.manual_seed(1)
    x = torch.randn(1024, 4096, device="cuda").to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(4096, device="cuda")).to(torch.bfloat16)
    eps = 1e-5
    xd = x.double()
    golden = xd * torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + eps) * w.double()
    baseline = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w          # every step rounded to bf16
    actual, _ = Fn.rmsnorm(x, w, eps)
    ok, report = DoubleBenchmarkComparator(dtype=torch.bfloat16).check_pass_or_not(actual, baseline, golden)
    assert ok, report


def _attention_fp64(q, k, v, causal=True):
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    kk = k.double().repeat_interleave(Hq // Hkv, dim=2)
    vv = v.double().repeat_interleave(Hq // Hkv, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.double(), kk) * D ** -0.5
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(S, S, device=q.device, dtype=torch.bool), 1), float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vv)


def test_flash_attention_forward_and_backward_errors_are_within_the_bf16_baseline():
    """Against fp64 attention, the kernel's output and input gradients must not be worse than PyTorch's own bf16
    attention (SDPA) by more than the criterion allows."""
    _skip_without_gpu()
    import torch.nn.functional as F
    from mindformers_b200.ops import functional as Fn
    from mindformers_b200.utils.precision import DoubleBenchmarkComparator
    torch.manual_seed(2)
    B, S, Hq, Hkv, D = 1, 1024, 8, 2, 128
    q, k, v = [(torch.randn(B, S, h, D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True) for h in (Hq, Hkv, Hkv)]
    dout = (torch.randn(B, S, Hq, D, device="cuda") * 0.1).to(torch.bfloat16)
    qd, kd, vd = [t.detach().double().requires_grad_(True) for t in (q, k, v)]
    gold = _attention_fp64(qd, kd, vd)
    gold.backward(dout.double())
    out = Fn.attention(q, k, v, causal=True)
    out.backward(dout)
    mine = [out.detach(), q.grad.clone(), k.grad.clone(), v.grad.clone()]
    q.grad = k.grad = v.grad = None
    base = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                          enable_gqa=True).transpose(1, 2)
    base.backward(dout)
    theirs = [base.detach(), q.grad, k.grad, v.grad]
    golden = [gold.detach(), qd.grad, kd.grad, vd.grad]
    cmp_ = DoubleBenchmarkComparator(dtype=torch.bfloat16)
    for name, a, b, g in zip(("out", "dq", "dk", "dv"), mine, theirs, golden):
        ok, report = cmp_.check_pass_or_not(a, b, g)
        assert ok, (name, report)


def test_cross_entropy_swiglu_and_decode_kernels_are_within_the_bf16_baseline():
    _skip_without_gpu()
    import torch.nn.functional as F
    from mindformers_b200.ops import functional as Fn
    from mindformers_b200.utils.precision import DoubleBenchmarkComparator
    cmp_ = DoubleBenchmarkComparator(dtype=torch.bfloat16)
    torch.manual_seed(3)
    # SwiGLU
    x = torch.randn(512, 2 * 1024, device="cuda").to(torch.bfloat16)
    g, u = x.double().chunk(2, -1)
    golden = F.silu(g) * u
    gb, ub = x.chunk(2, -1)
    ok, report = cmp_.check_pass_or_not(Fn.swiglu(x), F.silu(gb) * ub, golden)
    assert ok, ("swiglu", report)
    # cross-entropy (per-token losses from bf16 logits)
    logits = (torch.randn(256, 4096, device="cuda") * 2).to(torch.bfloat16)
    labels = torch.randint(0, 4096, (256,), device="cuda")
    golden = F.cross_entropy(logits.double(), labels, reduction="none")
    baseline = F.cross_entropy(logits, labels, reduction="none")
    ok, report = cmp_.check_pass_or_not(Fn.cross_entropy(logits, labels).to(torch.bfloat16), baseline, golden)
    assert ok, ("cross_entropy", report)
    # weight-on-rows decode GEMM
    xs = torch.randn(8, 4096, device="cuda").to(torch.bfloat16)
    w = (torch.randn(2048, 4096, device="cuda") * 0.05).to(torch.bfloat16)
    ok, report = cmp_.check_pass_or_not(Fn.gemm(xs, w), torch.matmul(xs, w.t()), xs.double() @ w.double().t())
    assert ok, ("decode gemm", report)
