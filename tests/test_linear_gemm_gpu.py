"""The library's bf16 GEMM (CUDA-core kernel for small M, tcgen05/TMEM kernel above) against an fp32 torch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k,bias", [
    (1, 512, 1024, True), (4, 384, 3840, False), (16, 1000, 264, True),          # CUDA-core kernel
    (17, 128, 64, False), (128, 128, 128, True), (256, 384, 1024, True),         # tensor-core kernel
    (300, 1000, 264, True), (130, 136, 3840, False), (1024, 3840, 3840, True),
])
def test_matches_fp32_reference(m, n, k, bias):
    from entropack_b200.linear import linear_forward

    g = torch.Generator(device="cuda").manual_seed(m * 7 + n)
    x = torch.randn(m, k, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    b = torch.randn(n, generator=g, device="cuda").to(torch.bfloat16) if bias else None
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = linear_forward(x, w, b, error=error)
    torch.cuda.synchronize()
    assert int(error.item()) == 0
    expected = x.float() @ w.float().t() + (b.float() if bias else 0.0)
    # tolerance from the metric definition: max |y - y_ref| / max |y_ref| <= 1e-2 (bf16 output rounding is ~4e-3)
    assert float((out.float() - expected).abs().max() / expected.abs().max()) <= 1e-2
