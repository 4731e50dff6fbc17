"""tcgen05 varlen attention forward/backward vs an fp32 masked-softmax reference."""
import pytest
import torch

from areal_b200.ops import _lib
from areal_b200.ops.attention import VarlenMeta, attention_ref, varlen_attention

pytestmark = pytest.mark.gpu


def _make(seqlens, Hq, Hkv, seed=0, fused_qkv=False):
    torch.manual_seed(seed)
    T, D = sum(seqlens), 128
    cu = [0]
    for s in seqlens:
        cu.append(cu[-1] + s)
    if fused_qkv:
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
        q = qkv[:, : Hq * D].reshape(T, Hq, D).contiguous()
        k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    else:
        q = torch.randn(T, Hq, D, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(T, Hkv, D, device="cuda", dtype=torch.bfloat16)
        v = torch.randn(T, Hkv, D, device="cuda", dtype=torch.bfloat16)
    return q, k, v, cu


@pytest.mark.parametrize("seqlens,Hq,Hkv,fused", [
    ([128], 1, 1, False), ([64], 2, 1, False), ([1], 2, 2, False), ([300], 2, 1, False),
    ([5, 129, 64, 257, 1000], 4, 2, True), ([2048, 77], 16, 8, False)])
def test_attn_forward(seqlens, Hq, Hkv, fused):
    q, k, v, cu = _make(seqlens, Hq, Hkv, fused_qkv=fused)
    meta = VarlenMeta(cu, "cuda")
    o = varlen_attention(q, k, v, meta)
    assert _lib.read_status() == 0
    ref = attention_ref(q.float(), k.float(), v.float(), cu)
    torch.testing.assert_close(o.float(), ref.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("seqlens,Hq,Hkv", [([128], 1, 1), ([64], 2, 1), ([300], 2, 1),
                                             ([5, 129, 64, 257, 700], 4, 2), ([1024, 77], 8, 4)])
def test_attn_backward(seqlens, Hq, Hkv):
    q, k, v, cu = _make(seqlens, Hq, Hkv, seed=3)
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    meta = VarlenMeta(cu, "cuda")
    o = varlen_attention(q, k, v, meta)
    g = torch.randn_like(o)
    o.backward(g)
    assert _lib.read_status() == 0
    qr = q.detach().float().requires_grad_()
    kr = k.detach().float().requires_grad_()
    vr = v.detach().float().requires_grad_()
    ref = attention_ref(qr, kr, vr, cu)
    ref.backward(g.float())
    for name, a, b in [("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)]:
        err = (a.float() - b).abs().max().item()
        scale = b.abs().max().item()
        assert err <= 3e-2 * scale + 2e-2, f"{name}: max err {err}, scale {scale}"
