"""RMSNorm / q-k-norm+RoPE / SwiGLU kernels vs their fp32 PyTorch references."""
import pytest
import torch

from areal_b200.ops import _lib, fused

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,H", [(1, 256), (37, 2048), (515, 4096), (64, 1000 // 8 * 8)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm_fwd_bwd(T, H, with_res):
    torch.manual_seed(0)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True) if with_res else None
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_()
    out = fused.rmsnorm(x, w, 1e-6, r)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    rr = r.detach().float().requires_grad_() if with_res else None
    if with_res:
        y, h = out
        hr = (xr + rr)
        yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
        g1, g2 = torch.randn_like(y), torch.randn_like(h)
        (y.float() * g1.float()).sum().backward(retain_graph=True) if False else torch.autograd.backward([y, h], [g1, g2])
        torch.autograd.backward([yr, hr], [g1.float(), g2.float()])
        torch.testing.assert_close(h.float(), hr, atol=3e-2, rtol=2e-2)
        torch.testing.assert_close(r.grad.float(), rr.grad, atol=6e-2, rtol=3e-2)
    else:
        y = out
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
        g1 = torch.randn_like(y)
        y.backward(g1)
        yr.backward(g1.float())
    torch.testing.assert_close(y.float(), yr, atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, atol=6e-2, rtol=3e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, atol=0.3 + 0.02 * T ** 0.5, rtol=5e-2)


@pytest.mark.parametrize("has_norm", [True, False])
def test_qknorm_rope_fwd_bwd(has_norm):
    torch.manual_seed(1)
    T, Hq, Hkv, D = 77, 4, 2, 128
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    qw = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16().requires_grad_() if has_norm else None
    kw = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16().requires_grad_() if has_norm else None
    cos, sin = fused.rope_tables(256, D, 1e6, "cuda")
    pos = torch.randint(0, 256, (T,), device="cuda", dtype=torch.int32)
    q, k, v = fused.qknorm_rope(qkv, qw, kw, cos, sin, pos, Hq, Hkv, D, 1e-6)
    gq, gk, gv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
    torch.autograd.backward([q, k, v], [gq, gk, gv])

    qkv_r = qkv.detach().float().requires_grad_()
    qw_r = qw.detach().float().requires_grad_() if has_norm else None
    kw_r = kw.detach().float().requires_grad_() if has_norm else None
    qr, kr, vr = fused.qknorm_rope_ref(qkv_r, qw_r, kw_r, cos, sin, pos, Hq, Hkv, D, 1e-6)
    torch.autograd.backward([qr, kr, vr], [gq.float(), gk.float(), gv.float()])
    torch.testing.assert_close(q.float(), qr, atol=4e-2, rtol=2e-2)
    torch.testing.assert_close(k.float(), kr, atol=4e-2, rtol=2e-2)
    torch.testing.assert_close(v.float(), vr, atol=0, rtol=0)
    torch.testing.assert_close(qkv.grad.float(), qkv_r.grad, atol=8e-2, rtol=3e-2)
    if has_norm:
        torch.testing.assert_close(qw.grad.float(), qw_r.grad, atol=0.5, rtol=5e-2)
        torch.testing.assert_close(kw.grad.float(), kw_r.grad, atol=0.5, rtol=5e-2)


def test_swiglu_fwd_bwd():
    torch.manual_seed(2)
    gu = torch.randn(100, 2 * 688, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = fused.swiglu(gu)
    g = torch.randn_like(y)
    y.backward(g)
    gr = gu.detach().float().requires_grad_()
    I = 688
    yr = torch.nn.functional.silu(gr[:, :I]) * gr[:, I:]
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(gu.grad.float(), gr.grad, atol=5e-2, rtol=2e-2)
    assert _lib.read_status() == 0


def test_embedding_gather_and_scatter_add():
    """Row gather and the fp32 scatter-add of its gradient (repeated ids, ids outside the table)."""
    torch.manual_seed(3)
    V, H, T = 1000, 256, 777
    w = torch.randn(V, H, device="cuda", dtype=torch.bfloat16).requires_grad_()
    w.main_grad = torch.zeros(V, H, device="cuda", dtype=torch.float32)
    ids = torch.randint(0, 40, (T,), device="cuda")  # many collisions
    ids[5], ids[9] = -1, V + 3
    y = fused.embedding(ids, w)
    ok = (ids >= 0) & (ids < V)
    ref = torch.where(ok[:, None], w.detach()[ids.clamp(0, V - 1)], torch.zeros((), device="cuda", dtype=w.dtype))
    assert torch.equal(y, ref)
    dy = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    y.backward(dy)
    want = torch.zeros(V, H, device="cuda", dtype=torch.float32)
    want.index_add_(0, ids[ok], dy[ok].float())
    torch.testing.assert_close(w.main_grad, want, atol=1e-4, rtol=1e-5)
    assert w.grad is None
