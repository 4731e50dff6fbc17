"""Loss / normalisation numerics: hand-computed values and packed ≡ padded consistency."""
import math

import pytest
import torch

from areal_b200.api.cli_args import NormConfig, RejectionSamplingConfig
from areal_b200.utils import functional as Fn
from areal_b200.utils.data import KLEstimator, Normalization


def _rand(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    logp = -torch.rand(n, generator=g) * 2
    prox = logp + 0.2 * torch.randn(n, generator=g)
    old = prox + 0.5 * torch.randn(n, generator=g)
    adv = torch.randn(n, generator=g)
    mask = torch.rand(n, generator=g) > 0.3
    return logp, prox, old, adv, mask


def test_ppo_loss_hand_values():
    logp = torch.log(torch.tensor([1.5, 0.5, 1.0, 1.1]))
    prox = torch.zeros(4)
    adv = torch.tensor([1.0, 1.0, -1.0, 2.0])
    mask = torch.tensor([True, True, True, False])
    loss, st = Fn.ppo_actor_loss_fn(logp, prox, prox, adv, 0.2, mask)
    # token0: ratio 1.5 clipped to 1.2 → -1.2 ; token1: ratio .5 → max(-.5,-.8) = -.5 ; token2: A<0, ratio 1 → 1.0
    assert loss.item() == pytest.approx((-1.2 - 0.5 + 1.0) / 3, abs=1e-6)
    assert st["clip_mask"].tolist() == [True, False, False, False]


def test_dual_clip_and_asymmetric_clip():
    logp = torch.log(torch.tensor([5.0, 1.25]))
    z = torch.zeros(2)
    adv = torch.tensor([-1.0, 1.0])
    mask = torch.ones(2, dtype=torch.bool)
    loss, st = Fn.ppo_actor_loss_fn(logp, z, z, adv, 0.2, mask, eps_clip_higher=0.3, c_clip=3.0)
    # token0: -A*r = 5 vs clipped 1.3 → 5, dual-clipped to 3 ; token1: r=1.25 within [0.8, 1.3] → -1.25
    assert loss.item() == pytest.approx((3.0 - 1.25) / 2, abs=1e-6)
    assert st["dual_clip_mask"].tolist() == [True, False]


def test_denominator_fixed_before_rejection():
    logp, prox, old, adv, mask = _rand(400)
    rs = RejectionSamplingConfig(level="token", action="mask", metric="ratio", upper=1.5)
    loss, st = Fn.ppo_actor_loss_fn(logp, prox, old, adv, 0.2, mask, rejection_sampling=rs)
    w = torch.exp(prox - old)
    keep = mask & (w <= 1.5)
    ratio = torch.exp(logp - prox)
    l = torch.max(-adv * ratio, -adv * ratio.clamp(0.8, 1.2)) * w
    ref = l[keep].sum() / mask.sum()
    assert loss.item() == pytest.approx(ref.item(), rel=1e-5)
    assert st["filtered_fraction"] == pytest.approx(((mask & ~keep).sum() / mask.sum()).item())


@pytest.mark.parametrize("level,action,metric,agg", [
    ("token", "clamp", "ratio", "mean"), ("sequence", "mask", "ratio", "mean"), ("sequence", "mask", "kl_k2", "max"),
    ("sequence", "clamp", "ratio", "sum"), ("token", "mask", "kl_k3", "mean")])
def test_rejection_sampling_packed_equals_padded(level, action, metric, agg):
    lens = [5, 9, 3, 12]
    B, L = len(lens), max(lens)
    g = torch.Generator().manual_seed(1)
    prox2 = -torch.rand(B, L, generator=g)
    old2 = prox2 + 0.6 * torch.randn(B, L, generator=g)
    valid = torch.arange(L)[None, :] < torch.tensor(lens)[:, None]
    mask2 = valid & (torch.rand(B, L, generator=g) > 0.2)
    cfg = RejectionSamplingConfig(level=level, action=action, metric=metric, agg=agg, upper=1.3 if metric == "ratio" else 0.2,
                                  lower=0.5 if (metric == "ratio") else None)
    r2 = Fn.apply_rejection_sampling(prox2, old2, mask2, None, cfg)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    r1 = Fn.apply_rejection_sampling(prox2[valid], old2[valid], mask2[valid], cu, cfg)
    torch.testing.assert_close(r1.loss_mask, r2.loss_mask[valid])
    torch.testing.assert_close(r1.behave_imp_weight, r2.behave_imp_weight[valid])
    assert r1.filtered_fraction == pytest.approx(r2.filtered_fraction)


def test_gspo_sequence_level_ratio():
    lens = [3, 2]
    cu = torch.tensor([0, 3, 5], dtype=torch.int32)
    lr = torch.tensor([0.1, 0.2, 0.3, -0.4, 0.0])
    adv = torch.tensor([1.0, 2.0, 3.0, -1.0, -3.0])
    mask = torch.tensor([True, True, False, True, True])
    ratio, a = Fn.sequence_level_ratio_and_advantages(lr, adv, mask, cu)
    assert ratio[:2].tolist() == pytest.approx([math.exp(0.15)] * 2) and ratio[2] == 0
    assert ratio[3:].tolist() == pytest.approx([math.exp(-0.2)] * 2)
    assert a.tolist() == pytest.approx([1.5, 1.5, 0.0, -2.0, -2.0])


def test_sapo_gate():
    logp = torch.log(torch.tensor([1.0, 2.0]))
    z = torch.zeros(2)
    adv = torch.tensor([1.0, -1.0])
    loss, _ = Fn.sapo_loss_fn(logp, z, adv, 1.0, 1.05, torch.ones(2, dtype=torch.bool))
    g0 = torch.sigmoid(torch.tensor(0.0)) * 4
    g1 = torch.sigmoid(torch.tensor(1.05)) * 4 / 1.05
    assert loss.item() == pytest.approx(((-g0 * 1.0) + (g1 * 1.0)).item() / 2, rel=1e-6)


def test_prox_logp_approximations():
    old = torch.tensor([-1.0, -1.0, -1.0, -1.0])
    new = torch.tensor([-2.0, -2.0, -2.0, -2.0])
    versions = torch.tensor([-1, 3, 1, 0])  # prompt, fresh, two versions old, three old
    out = Fn.compute_prox_logp_approximations(old, new, versions, current_version=3)
    # v_prox = 2: alpha = (2 - v) / (3 - v) → prompt 0, v=3 → 0 (denominator 0), v=1 → .5, v=0 → 2/3
    assert out["loglinear"].tolist() == pytest.approx([-1.0, -1.0, -1.5, -1 - 2 / 3])
    lin = torch.log((1 - 0.5) * math.exp(-1) + 0.5 * math.exp(-2) + torch.tensor(1e-10))
    assert out["linear"][2].item() == pytest.approx(lin.item())
    assert out["rollout"].tolist() == old.tolist()


def test_m2po_masks_largest_gaps_only_until_threshold():
    old = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0])
    prox = torch.tensor([0.1, 2.0, 0.2, 1.0, 0.1])
    mask = torch.ones(5)
    out = Fn.apply_m2po_masking(old, prox, mask, m2_threshold=0.05)
    # squared gaps: .01, 4, .04, 1, .01 → drop 4 and 1: mean(.01,.04,.01) = .02 < .05
    assert out.tolist() == [1, 0, 1, 0, 1]
    out = Fn.apply_m2po_masking(old, prox * 100, mask, m2_threshold=1e-9)
    assert out.sum() == 1  # never masks everything


def test_critic_dpo_sft_rw_losses():
    v, vo, ret = torch.tensor([1.0, 3.0]), torch.tensor([0.0, 0.0]), torch.tensor([2.0, 2.0])
    loss, st = Fn.ppo_critic_loss_fn(v, vo, ret, 0.5, torch.ones(2, dtype=torch.bool))
    # unclipped: .5, .5 ; clipped values .5 → 1.125 each → max → 1.125
    assert loss.item() == pytest.approx(1.125)
    assert Fn.sft_loss(torch.tensor([-1.0, -3.0, -9.0]), torch.tensor([1, 1, 0])).item() == pytest.approx(2.0, abs=1e-4)
    l, st = Fn.rw_pairwise_loss(torch.tensor([2.0, 1.0, 0.0, 3.0]))
    assert l.item() == pytest.approx((-torch.nn.functional.logsigmoid(torch.tensor([1.0, -3.0]))).mean().item())
    cu = torch.tensor([0, 2, 4], dtype=torch.int32)
    logits, avg, _ = Fn.dpo_pair_logratios(torch.tensor([-1.0, -1.0, -2.0, -2.0]), torch.tensor([-1.5, -1.5, -1.5, -1.5]),
                                          torch.ones(4), cu)
    assert logits.tolist() == pytest.approx([2.0]) and avg.tolist() == pytest.approx([1.0])
    assert Fn.dpo_preference_loss(logits, avg, 0.1, "sigmoid").item() == pytest.approx(-math.log(1 / (1 + math.exp(-0.2))))
    assert Fn.dpo_preference_loss(logits, avg, 0.1, "ipo").item() == pytest.approx((1.0 - 5.0) ** 2)


def test_overlong_penalty():
    data = dict(rewards=torch.tensor([1.0, 1.0]), loss_mask=torch.cat([torch.ones(1, 90), torch.zeros(1, 10)], 1).repeat(2, 1))
    data["loss_mask"][1] = 1
    out = Fn.reward_overlong_penalty(data, overlong_tokens=20, overlong_penalty_factor=1.0, max_response_length=100)
    assert out["rewards"].tolist() == pytest.approx([1.0 - 0.5, 1.0 - 1.0])


@pytest.mark.parametrize("mean,std,loo", [("batch", "batch", False), ("group", "group", False), ("group", None, True),
                                          ("group", "batch", False), (None, "batch", False)])
def test_normalization_levels(mean, std, loo):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(12, generator=g) * 3 + 1
    n = Normalization(NormConfig(mean_level=mean, std_level=std, mean_leave1out=loo, group_size=4))
    y = n(x).double()
    xg = x.double().view(3, 4)
    if mean == "batch":
        m = x.double().mean().expand(12)
    elif mean == "group":
        m = ((xg.sum(1, keepdim=True) - xg) / 3 if loo else xg.mean(1, keepdim=True).expand(3, 4)).reshape(-1)
    else:
        m = torch.zeros(12, dtype=torch.float64)
    c = x.double() - m
    if std == "batch":
        s = (c.pow(2).sum() / 11).sqrt()
        ref = c / (s + 1e-5)
    elif std == "group":
        s = (c.view(3, 4).pow(2).sum(1, keepdim=True) / 3).sqrt()
        ref = (c.view(3, 4) / (s + 1e-5)).reshape(-1)
    else:
        ref = c
    torch.testing.assert_close(y, ref, atol=1e-6, rtol=1e-6)


def test_normalization_masked_and_degenerate():
    x = torch.tensor([[1.0, 2.0, 100.0], [3.0, 4.0, 100.0]])
    mask = torch.tensor([[1, 1, 0], [1, 1, 0]])
    y = Normalization(NormConfig("batch", False, "batch"))(x, mask)
    assert y[:, 2].abs().sum() == 0
    vals = torch.tensor([1.0, 2.0, 3.0, 4.0])
    ref = (vals - 2.5) / (vals.std(unbiased=True) + 1e-5)
    torch.testing.assert_close(y[:, :2].reshape(-1), ref)
    # group_size 1: leave-one-out mean is 0 and the unbiased std is defined as 1
    assert Normalization(NormConfig("group", True, "group", group_size=1))(torch.tensor([5.0, 7.0])).tolist() == \
        pytest.approx([5.0 / (1 + 1e-5), 7.0 / (1 + 1e-5)])
    z = Normalization(NormConfig())(x, torch.zeros_like(mask))
    torch.testing.assert_close(z, x)


def test_kl_estimators():
    a, b = torch.tensor([0.0, -1.0]), torch.tensor([-0.5, -0.5])
    d = a - b
    assert KLEstimator("k1")(a, b).tolist() == pytest.approx(d.tolist())
    assert KLEstimator("k2")(a, b).tolist() == pytest.approx((0.5 * d * d).tolist())
    assert KLEstimator("k3")(a, b).tolist() == pytest.approx((torch.exp(-d) - 1 + d).tolist())
    assert KLEstimator("k1")(torch.tensor([100.0]), torch.tensor([0.0])).item() == 10.0
