"""PPO-loss / group-norm / GAE kernels and the rollout kernels (KV write, paged
decode attention, sampler) against PyTorch restatements."""
import math

import pytest
import torch

from areal_b200.ops import _lib, rl_ops, rollout_ops

pytestmark = pytest.mark.gpu


def _ppo_ref(logp, prox, behav, adv, mask, eps, eps_hi, c_clip, cap, decoupled, weight=None):
    px = prox if decoupled else behav
    ratio = torch.exp(logp - px)
    clipped = torch.clamp(ratio, 1 - eps, 1 + (eps if eps_hi is None else eps_hi))
    l = torch.max(-adv * ratio, -adv * clipped)
    if c_clip is not None:
        l = torch.min(l, torch.sign(adv) * c_clip * adv)
    m = mask.bool()
    if cap is not None if weight is None else weight:
        w = torch.exp(px - behav).detach()
        if cap is not None:
            w = torch.where(w > cap, torch.zeros_like(w), w)
        l = l * w
    return torch.where(m, l, torch.zeros_like(l)).sum() / max(int(m.sum()), 1)


def _ppo_inputs(n=10007):
    torch.manual_seed(0)
    logp = (-torch.rand(n, device="cuda") * 3).requires_grad_()
    prox = logp.detach() + 0.3 * torch.randn(n, device="cuda")
    behav = prox + 0.8 * torch.randn(n, device="cuda")
    adv = torch.randn(n, device="cuda")
    mask = torch.rand(n, device="cuda") > 0.3
    return logp, prox, behav, adv, mask


@pytest.mark.parametrize("decoupled,c_clip,cap,eps_hi,weight", [
    (True, None, 5.0, None, None), (False, 3.0, None, 0.28, None), (True, 2.0, None, None, None),
    (True, None, None, None, True)])
def test_ppo_loss(decoupled, c_clip, cap, eps_hi, weight):
    logp, prox, behav, adv, mask = _ppo_inputs()
    loss, stats = rl_ops.ppo_loss_fused(logp, prox, behav, adv, mask, eps_clip=0.2, eps_clip_higher=eps_hi,
                                        c_clip=c_clip, behav_cap=cap, use_decoupled=decoupled,
                                        behav_weight=weight)
    loss.backward()
    lr = logp.detach().clone().requires_grad_()
    ref = _ppo_ref(lr, prox, behav, adv, mask, 0.2, eps_hi, c_clip, cap, decoupled, weight)
    ref.backward()
    torch.testing.assert_close(loss, ref, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(logp.grad, lr.grad, atol=1e-7, rtol=1e-3)


@pytest.mark.parametrize("with_rs", [False, True])
def test_ppo_loss_matches_the_functional_form(with_rs):
    """The fused kernel and ``functional.ppo_actor_loss_fn`` (the CPU path and the numerics specification)
    compute the same objective with and without rejection sampling: the behaviour importance weight is
    part of the loss only when rejection sampling is configured."""
    from areal_b200.api.cli_args import RejectionSamplingConfig
    from areal_b200.utils import functional as Fn

    logp, prox, behav, adv, mask = _ppo_inputs(4099)
    rs = RejectionSamplingConfig(level="token", action="mask", metric="ratio", upper=5.0) if with_rs else None
    loss, _ = rl_ops.ppo_loss_fused(logp, prox, behav, adv, mask, eps_clip=0.2, c_clip=None,
                                    behav_cap=rs.upper if rs else None, use_decoupled=True,
                                    behav_weight=rs is not None)
    loss.backward()
    lr = logp.detach().clone().requires_grad_()
    ref, _ = Fn.ppo_actor_loss_fn(lr, prox, behav, adv, 0.2, mask, rejection_sampling=rs)
    ref.backward()
    torch.testing.assert_close(loss, ref, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(logp.grad, lr.grad, atol=1e-7, rtol=1e-3)


def test_group_norm_and_gae():
    torch.manual_seed(1)
    r = torch.randn(12 * 8, device="cuda")
    out = rl_ops.group_norm(r, 8)
    g = r.view(12, 8)
    ref = (g - g.mean(1, keepdim=True)) / (g.std(1, unbiased=True, keepdim=True) + 1e-5)
    torch.testing.assert_close(out.view(12, 8), ref, atol=1e-5, rtol=1e-4)
    out = rl_ops.group_norm(r, 8, std_group=False, leave1out=True)
    ref = g - (g.sum(1, keepdim=True) - g) / 7
    torch.testing.assert_close(out.view(12, 8), ref, atol=1e-5, rtol=1e-4)
    # GAE vs the padded-batch loop formulation
    lens = [5, 9, 1, 12]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    T = sum(lens)
    rewards = torch.randn(T, device="cuda")
    values = torch.randn(T, device="cuda")
    mask = torch.rand(T, device="cuda") > 0.4
    no_eos = torch.tensor([0, 1, 0, 1], device="cuda", dtype=torch.uint8)
    gamma, lam = 0.99, 0.95
    adv, ret = rl_ops.gae_packed(rewards, values, mask, cu, no_eos, gamma, lam)
    for b, L in enumerate(lens):
        s = int(cu[b])
        rw, v, m = rewards[s:s + L].cpu(), values[s:s + L].cpu(), mask[s:s + L].cpu().float()
        last, nextv = 0.0, float(v[L - 1]) * float(no_eos[b])
        ref_adv = [0.0]
        for t in reversed(range(L - 1)):
            delta = float(rw[t]) + gamma * nextv - float(v[t])
            new = delta + gamma * lam * last
            nextv = nextv * (1 - float(m[t])) + float(v[t]) * float(m[t])
            last = last * (1 - float(m[t])) + new * float(m[t])
            ref_adv.append(last)
        ref_adv = torch.tensor(ref_adv[::-1])
        torch.testing.assert_close(adv[s:s + L].cpu(), ref_adv, atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(ret[s:s + L].cpu(), ref_adv + v, atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("Hq,Hkv", [(4, 2), (16, 8), (8, 1), (4, 4)])
def test_paged_decode_and_kv_write(Hq, Hkv):
    torch.manual_seed(2)
    D, bs, nb = 128, 16, 96
    lens = [1, 17, 250, 33, 400, 16]
    B = len(lens)
    k_cache = torch.zeros(nb, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    perm = torch.randperm(nb)
    max_blocks = 26
    bt = torch.zeros(B, max_blocks, dtype=torch.int32)
    used = 0
    slots, ks, vs = [], [], []
    for b, L in enumerate(lens):
        n = (L + bs - 1) // bs
        bt[b, :n] = perm[used:used + n].int()
        used += n
        for t in range(L):
            slots.append(int(bt[b, t // bs]) * bs + t % bs)
    T = sum(lens)
    # k/v as strided views of a fused buffer, like the model produces them
    fusedkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    k = fusedkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    v = fusedkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    rollout_ops.kv_cache_write(k, v, torch.tensor(slots, device="cuda"), k_cache, v_cache)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    bt_d = bt.cuda()
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    # the kernel's write lands where the reference layout expects it
    kc_ref, vc_ref = torch.zeros_like(k_cache), torch.zeros_like(v_cache)
    st = torch.tensor(slots, device="cuda")
    kc_ref[st // bs, :, st % bs] = k
    vc_ref[st // bs, :, st % bs] = v
    assert torch.equal(k_cache, kc_ref) and torch.equal(v_cache, vc_ref)
    from areal_b200.ops import _lib
    for nsplit in (1, 4):
        out = rollout_ops.paged_decode(q, k_cache, v_cache, bt_d, sl, nsplit=nsplit)
        ref = rollout_ops.paged_decode_ref(q, k_cache, v_cache, bt_d, sl)
        assert _lib.read_status() == 0
        torch.testing.assert_close(out.float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_sampler():
    torch.manual_seed(3)
    B, V = 6, 5003
    logits = torch.randn(B, V, device="cuda") * 3
    temp = torch.tensor([1.0, 0.7, 0.0, 1.0, 1.3, 1.0], device="cuda")
    top_k = torch.tensor([0, 0, 0, 50, 0, 20], device="cuda", dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 1.0, 1.0, 0.9, 0.8], device="cuda")
    u = torch.rand(B, device="cuda")
    tok, lp = rollout_ops.sample(logits, temp, top_k, top_p, u)
    tok_r, lp_r = rollout_ops.sample_ref(logits, temp, top_k, top_p, u)
    # the token must be the inverse-CDF pick up to rounding at interval boundaries:
    # check its CDF interval contains the target within a small tolerance
    for b in range(B):
        t = float(temp[b])
        if t <= 0:
            assert int(tok[b]) == int(logits[b].argmax())
            continue
        if int(tok[b]) != int(tok_r[b]):
            y = torch.log_softmax(logits[b] / t, -1).exp().double()
            cdf = y.cumsum(0)
            assert abs(int(tok[b]) - int(tok_r[b])) <= 3 or abs(float(cdf[int(tok[b])] - cdf[int(tok_r[b])])) < 1e-3
        expect = torch.log_softmax(logits[b] / t, -1)[int(tok[b])]
        assert abs(float(lp[b]) - float(expect)) < 1e-3
    # distribution check: many draws of one row follow softmax
    row = torch.randn(1, 64, device="cuda")
    n = 20000
    toks, _ = rollout_ops.sample(row.expand(n, 64).contiguous(), torch.ones(n, device="cuda"))
    freq = torch.bincount(toks.long(), minlength=64).float() / n
    p = torch.softmax(row[0], -1)
    assert (freq - p).abs().max().item() < 0.02


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N,with_res", [(64, 2048, 2048, True), (200, 6144, 2048, True), (7, 2048, 2048, False),
                                            (256, 1024, 1024, True), (300, 256, 2048, True)])
def test_linear_rmsnorm_matches_separate_kernels(M, K, N, with_res):
    """Residual add + RMSNorm inside the split-K reduction: bit-identical to projection, then norm
    (the last shape does not split and takes the separate kernels)."""
    from areal_b200.ops import fused
    from areal_b200.ops.gemm import linear, linear_rmsnorm

    torch.manual_seed(M + N)
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    nw = (1 + 0.1 * torch.randn(N, device="cuda")).bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16() if with_res else None
    y, h = linear_rmsnorm(x, w, nw, 1e-6, res)
    a = linear(x, w)
    if with_res:
        y_ref, h_ref = fused.rmsnorm(a, nw, 1e-6, residual=res)
    else:
        y_ref, h_ref = fused.rmsnorm(a, nw, 1e-6), a
    assert torch.equal(h, h_ref) and torch.equal(y, y_ref)
    hf = (x.float() @ w.float().t()) + (res.float() if with_res else 0)
    yf = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
    assert float((y.float() - yf).abs().max()) < 0.06 * float(yf.abs().max())


@pytest.mark.gpu
@pytest.mark.parametrize("has_norm", [True, False])
def test_qknorm_rope_kvwrite_matches_separate_kernels(has_norm):
    from areal_b200.ops import fused
    from areal_b200.ops.rollout_ops import kv_cache_write

    torch.manual_seed(3)
    T, Hq, Hkv, D, bs, nb = 37, 16, 8, 128, 16, 12
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    qw = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16() if has_norm else None
    kw = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16() if has_norm else None
    cos, sin = fused.rope_tables(512, D, 1e6, "cuda")
    pos = torch.randint(0, 512, (T,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(nb * bs, device="cuda")[:T].to(torch.int64)
    slots[5] = -1  # a padded row of a captured batch: no cache write
    kc1, vc1 = (torch.zeros(nb, Hkv, bs, D, device="cuda", dtype=torch.bfloat16) for _ in range(2))
    kc2, vc2 = torch.zeros_like(kc1), torch.zeros_like(vc1)
    q1 = fused.qknorm_rope_kvwrite(qkv, qw, kw, cos, sin, pos, Hq, Hkv, D, 1e-6, slots, kc1, vc1)
    q2, k2, v2 = fused.qknorm_rope(qkv, qw, kw, cos, sin, pos, Hq, Hkv, D, 1e-6)
    kv_cache_write(k2, v2, slots, kc2, vc2)
    assert torch.equal(q1, q2) and torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert float(kc1.abs().sum()) > 0
