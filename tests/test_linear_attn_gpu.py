"""Causal conv1d (forward + backward) and the linear-attention recurrences vs their fp32 restatements."""
import pytest
import torch

from areal_b200.ops import linear_attn as LA

pytestmark = pytest.mark.gpu


def test_causal_conv1d_forward_backward():
    torch.manual_seed(0)
    T, C, K = 300, 96, 4
    cu = torch.tensor([0, 7, 130, 131, 300], device="cuda")
    x = torch.randn(T, C, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(C, K, device="cuda") * 0.5).bfloat16().requires_grad_()
    b = torch.randn(C, device="cuda").bfloat16().requires_grad_()
    dy = torch.randn(T, C, device="cuda").bfloat16()
    y = LA.causal_conv1d(x, w, b, cu)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = LA.causal_conv1d_ref(xr, wr, br, cu)
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, atol=0.5, rtol=3e-2)
    torch.testing.assert_close(b.grad.float(), br.grad, atol=0.5, rtol=3e-2)
    # the first token of a sequence must not see the previous sequence
    x2 = x.detach().clone()
    x2[:7] += 5.0
    y2 = LA.causal_conv1d(x2, w.detach(), b.detach(), cu)
    assert torch.equal(y2[7:], y.detach()[7:])


@pytest.mark.parametrize("mode,DK,DV", [("gated_delta", 128, 128), ("simple_gla", 64, 128)])
def test_linear_attention_recurrence(mode, DK, DV):
    torch.manual_seed(1)
    T, H = 200, 3
    cu = torch.tensor([0, 1, 90, 200], device="cuda")
    q = (torch.randn(T, H, DK, device="cuda") * DK ** -0.5).bfloat16()
    k = torch.nn.functional.normalize(torch.randn(T, H, DK, device="cuda"), dim=-1).bfloat16()
    v = torch.randn(T, H, DV, device="cuda").bfloat16()
    a = torch.exp(-torch.rand(T, H, device="cuda") * 0.2)
    b = torch.rand(T, H, device="cuda")
    with torch.no_grad():
        o = LA.linear_attn(q, k, v, a, b, cu, mode=mode)
        ref = LA.linear_attn_ref(q, k, v, a, b, cu, DK ** -0.5, mode)
    torch.testing.assert_close(o.float(), ref.float(), atol=3e-2, rtol=3e-2)
    # under autograd the differentiable restatement runs and produces gradients
    qg = q.clone().requires_grad_()
    LA.linear_attn(qg, k, v, a, b, cu, mode=mode).float().sum().backward()
    assert qg.grad is not None and torch.isfinite(qg.grad.float()).all()
