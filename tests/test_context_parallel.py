"""Zig-zag context parallelism: one process plays every cp rank in turn (gathered K/V are formed by
hand); outputs and gradients, re-assembled, must equal ordinary causal attention."""
import pytest
import torch

from areal_b200.parallel import context_parallel as CP


def _run(device, dtype, D, seqlens, cp, atol):
    torch.manual_seed(0)
    Hq, Hkv = 4, 2
    T = sum(seqlens)
    q = torch.randn(T, Hq, D, device=device).to(dtype)
    k = torch.randn(T, Hkv, D, device=device).to(dtype)
    v = torch.randn(T, Hkv, D, device=device).to(dtype)
    do = torch.randn(T, Hq, D, device=device).to(dtype)
    qr, kr, vr = (x.detach().clone().float().requires_grad_() for x in (q, k, v))
    ref = CP.full_attention_reference(qr, kr, vr, seqlens)
    ref.backward(do.float())
    lays = [CP.CPLayout(seqlens, cp, r, device) for r in range(cp)]
    lay0 = lays[0]
    qp, kp, vp, dop = (lay0.pad_packed(x) for x in (q, k, v, do))
    out_full = torch.zeros_like(qp, dtype=torch.float32)
    dq_full = torch.zeros_like(qp, dtype=torch.float32)
    dk_full = torch.zeros_like(kp, dtype=torch.float32)
    dv_full = torch.zeros_like(vp, dtype=torch.float32)
    # the permutation tables are each other's inverse and cover every row once
    assert torch.equal(lay0.gather_to_seq[lay0.seq_to_gather].cpu(), torch.arange(lay0.T_full))
    gathered_k = torch.cat([lay.split(kp) for lay in lays])
    assert torch.equal(gathered_k.index_select(0, lay0.gather_to_seq), kp)
    for lay in lays:
        ql = lay.split(qp).clone().requires_grad_()
        kf, vf = kp.clone().requires_grad_(), vp.clone().requires_grad_()
        o = CP.cp_attention_local(ql, kf, vf, lay)
        o.backward(lay.split(dop))
        out_full[lay.local_index] = o.detach().float()
        dq_full[lay.local_index] = ql.grad.float()
        dk_full += kf.grad.float()
        dv_full += vf.grad.float()

    def unpad(x):
        return torch.cat([x[int(lay0.full_cu[s]):int(lay0.full_cu[s]) + L] for s, L in enumerate(seqlens)])

    for got, want in ((out_full, ref), (dq_full, qr.grad), (dk_full, kr.grad), (dv_full, vr.grad)):
        err = (unpad(got) - want.detach()).abs().max().item()
        assert err <= atol * (want.abs().max().item() + 1), err


def test_zigzag_cp_matches_full_attention_cpu():
    _run("cpu", torch.float32, 16, [300, 70, 513], 2, 1e-5)
    _run("cpu", torch.float32, 16, [1000], 4, 1e-5)


@pytest.mark.gpu
def test_zigzag_cp_kernels_match_full_attention():
    from areal_b200.ops import _lib

    _run("cuda", torch.bfloat16, 128, [700, 130, 1025], 2, 3e-2)
    _run("cuda", torch.bfloat16, 128, [2000], 4, 3e-2)
    assert _lib.read_status() == 0
