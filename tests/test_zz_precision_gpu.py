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
