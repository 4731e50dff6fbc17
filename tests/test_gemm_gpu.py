"""tcgen05 GEMM vs a plain fp32 PyTorch matmul of the same bf16 inputs."""
import pytest
import torch

from areal_b200.ops import _lib
from areal_b200.ops.gemm import gemm, linear

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.t() if a_mn else a
    B = b.t() if b_mn else b
    return A.float() @ B.float().t()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K,bn", [(128, 256, 64, 256), (256, 512, 256, 256), (200, 328, 136, 256),
                                       (1000, 1000, 1000 // 8 * 8, 128), (4096, 2048, 2048, 0)])
def test_gemm_matches_fp32(M, N, K, bn, a_mn, b_mn):
    torch.manual_seed(0)
    dev = "cuda"
    a = torch.randn((K, M) if a_mn else (M, K), device=dev, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=dev, dtype=torch.bfloat16)
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("contiguous extent must be a multiple of 8")
    c = gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
    assert _lib.read_status() == 0
    ref = _ref(a, b, a_mn, b_mn)
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, f"max err {err} (scale {scale})"


def test_gemm_fp32_accumulate_and_bias():
    torch.manual_seed(1)
    a = torch.randn(300, 512, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(264, 512, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(264, device="cuda", dtype=torch.bfloat16)
    out = torch.ones(300, 264, device="cuda", dtype=torch.float32)
    gemm(a, b, bias=bias, out=out, accumulate=True)
    ref = 1.0 + a.float() @ b.float().t() + bias.float()
    assert _lib.read_status() == 0
    torch.testing.assert_close(out, ref, atol=2e-2, rtol=1e-3)


def test_linear_autograd():
    torch.manual_seed(2)
    x = torch.randn(3, 100, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(384, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    assert _lib.read_status() == 0
    torch.testing.assert_close(y.float(), yr, atol=0.25, rtol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, atol=0.5, rtol=2e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, atol=0.5, rtol=2e-2)


@pytest.mark.parametrize("M,N,K", [(64, 2048, 2048), (256, 2048, 6144), (300, 2048, 2048), (1, 2048, 2048)])
def test_skinny_gemm_takes_the_split_k_path(M, N, K):
    """Decode-step shapes: few output tiles, long K. The result must match fp32 and the launch count
    shows that the split-K kernel plus its reduction ran."""
    from areal_b200.ops import _lib

    torch.manual_seed(4)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * K ** -0.5).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    before = _lib.launch_count()
    y = gemm(x, w, bias=bias)
    assert _lib.launch_count() - before == 2
    assert _lib.read_status() == 0
    ref = x.float() @ w.float().t() + bias.float()
    torch.testing.assert_close(y.float(), ref, atol=3e-2, rtol=3e-2)
