"""fp8 block quantisation / dequantisation / GEMM kernels vs the PyTorch restatement."""
import pytest
import torch

from areal_b200.ops import _lib, fp8

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N", [(128, 128), (300, 520), (1024, 4096)])
@pytest.mark.parametrize("ue8m0", [False, True])
def test_quant_dequant_block128(M, N, ue8m0):
    torch.manual_seed(0)
    x = (torch.randn(M, N, device="cuda") * 3).bfloat16()
    q, s = fp8.quant_fp8_block128(x, ue8m0)
    _, sr = fp8.quant_block128_ref(x, ue8m0)
    torch.testing.assert_close(s, sr, rtol=1e-6, atol=0)
    # requantise with the kernel's own scales (a 1-ulp difference in a scale moves rounding ties)
    full = s.repeat_interleave(128, 0)[:M].repeat_interleave(128, 1)[:, :N]
    qr = (x.float() / full).clamp(-448, 448).to(fp8.FP8)
    assert torch.equal(q.float(), qr.float())
    d = fp8.dequant_fp8(q, s, 128)
    torch.testing.assert_close(d.float(), x.float(), rtol=0.07, atol=0.07 * float(s.max()) * 8)
    if ue8m0:
        assert torch.equal(torch.log2(s), torch.log2(s).round())


@pytest.mark.parametrize("M,K", [(1, 128), (77, 520), (512, 2048)])
def test_quant_1x128(M, K):
    torch.manual_seed(1)
    x = torch.randn(M, K, device="cuda").bfloat16()
    q, s = fp8.quant_fp8_1x128(x)
    _, sr = fp8.quant_1x128_ref(x)
    torch.testing.assert_close(s, sr, rtol=1e-6, atol=0)
    qr = (x.float() / s.repeat_interleave(128, 1)[:, :K]).clamp(-448, 448).to(fp8.FP8)
    assert torch.equal(q.float(), qr.float())
    d = fp8.dequant_fp8(q, s, 1)
    torch.testing.assert_close(d.float(), x.float(), rtol=0.07, atol=0.02)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 384, 512), (1024, 2048, 3584)])
def test_gemm_fp8_block(M, N, K):
    torch.manual_seed(2)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    a8, sa = fp8.quant_fp8_1x128(x)
    b8, sb = fp8.quant_fp8_block128(w)
    c = fp8.gemm_fp8_block(a8, sa, b8, sb)
    assert _lib.read_status() == 0
    ref = fp8.dequant_ref(a8, sa, 1).float() @ fp8.dequant_ref(b8, sb, 128).float().t()
    err = (c.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-2
    # and the whole fp8 path stays close to the bf16 product
    full = x.float() @ w.float().t()
    rel = (c.float() - full).norm() / full.norm()
    assert rel < 0.06


def test_fp8_linear_autograd():
    torch.manual_seed(3)
    x = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(384, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    y = fp8.fp8_linear(x, w)
    y.sum().backward()
    ref = x.detach().float() @ w.detach().float().t()
    assert ((y.float() - ref).norm() / ref.norm()).item() < 0.06
    assert x.grad is not None and w.grad is not None
    torch.testing.assert_close(w.grad.float(), x.detach().float().sum(0).expand(384, 256), atol=0.3, rtol=0.05)
