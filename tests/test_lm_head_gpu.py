"""Fused LM-head logprob/entropy kernel vs log_softmax on materialised fp32 logits."""
import pytest
import torch

from areal_b200.ops import _lib
from areal_b200.ops.lm_head import lm_head_logprobs, lm_head_logprobs_ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,V,H,temp", [(1, 1000, 64, 1.0), (130, 5000, 256, 0.7), (300, 151936, 128, 1.0),
                                         (257, 4099 // 8 * 8, 512, 1.3)])
def test_lm_head_forward_backward(T, V, H, temp):
    torch.manual_seed(0)
    x = (torch.randn(T, H, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(V, H, device="cuda") * 0.1).bfloat16().requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    logp, ent = lm_head_logprobs(x, w, labels, temp)
    assert _lib.read_status() == 0
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    logp_r, ent_r = lm_head_logprobs_ref(xr, wr, labels, temp)
    torch.testing.assert_close(logp, logp_r, atol=2e-3, rtol=2e-3)
    torch.testing.assert_close(ent, ent_r, atol=2e-3, rtol=2e-3)
    g1 = torch.randn(T, device="cuda")
    g2 = torch.randn(T, device="cuda") * 0.1
    torch.autograd.backward([logp, ent], [g1, g2])
    torch.autograd.backward([logp_r, ent_r], [g1, g2])
    assert _lib.read_status() == 0
    def close(a, b, name):
        err = (a.float() - b).abs().max().item()
        scale = b.abs().max().item()
        assert err <= 2e-2 * scale + 1e-3, f"{name}: err {err} scale {scale}"
    close(x.grad, xr.grad, "dx")
    close(w.grad, wr.grad, "dw")
