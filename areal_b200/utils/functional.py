"""RL / preference-learning numerics in plain PyTorch.

These functions define the semantics of every training objective of the
framework and are the CPU path and the oracle for the fused CUDA kernels
(``areal_b200.ops.rl_ops``). They accept packed 1-D tensors (with
``cu_seqlens``) or padded 2-D tensors. Semantics follow the reference
(areal/utils/functional/functional.py:16-804, areal/trainer/ppo/actor.py:604-851).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..api.cli_args import RejectionSamplingConfig

# --------------------------------------------------------------------------- helpers


def _seq_index(x: torch.Tensor, cu_seqlens: torch.Tensor | None) -> tuple[torch.Tensor, int]:
    """Sequence id of every element (flattened) and the number of sequences."""
    if x.dim() == 1:
        if cu_seqlens is None:
            raise ValueError("cu_seqlens is required for packed (1-D) tensors")
        lens = (cu_seqlens[1:] - cu_seqlens[:-1]).long()
        n = lens.numel()
        return torch.arange(n, device=x.device).repeat_interleave(lens), n
    B, L = x.shape
    return torch.arange(B, device=x.device).repeat_interleave(L), B


def _seg_sum(values: torch.Tensor, idx: torch.Tensor, n: int) -> torch.Tensor:
    return torch.zeros(n, dtype=values.dtype, device=values.device).index_add_(0, idx, values.reshape(-1))


def masked_normalization(x: torch.Tensor, mask: torch.Tensor | None = None, dim=None,
                         unbiased: bool = False, eps: float = 1e-5, high_precision: bool = True,
                         all_reduce: bool = True, reduce_group=None) -> torch.Tensor:
    """Whitening over the masked elements; sums are all-reduced when a process group exists."""
    dtype = torch.float64 if high_precision else torch.float32
    x = x.to(dtype)
    dim = tuple(range(x.dim())) if dim is None else dim
    if mask is None:
        factor = torch.tensor(float(x.numel()), dtype=dtype, device=x.device)
        xm = x
    else:
        mask = mask.to(dtype)
        xm = x * mask
        factor = mask.sum(dim, keepdim=True)
    s = xm.sum(dim, keepdim=True)
    ss = (xm * xm).sum(dim, keepdim=True)
    if all_reduce and dist.is_initialized():
        for t in (factor, s, ss):
            dist.all_reduce(t, group=reduce_group)
    mean = s / factor
    var = ss / factor - mean * mean
    if unbiased:
        var = var * factor / (factor - 1)
    out = (x - mean) / (var.sqrt() + eps)
    if mask is not None:
        out = out * mask
    return out.float()


def gather_logprobs(logits: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    lsm = torch.log_softmax(logits.float() / temperature, -1)
    return lsm.gather(-1, labels.long().unsqueeze(-1)).squeeze(-1)


def gather_logprobs_entropy(logits: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0):
    lsm = torch.log_softmax(logits.float() / temperature, -1)
    ent = -(lsm.exp() * lsm).sum(-1)
    return lsm.gather(-1, labels.long().unsqueeze(-1)).squeeze(-1), ent


# --------------------------------------------------------------------------- GSPO


def sequence_level_ratio_and_advantages(log_ratio, advantages, loss_mask, cu_seqlens=None):
    """GSPO: every token of a sequence uses exp(mean_t log-ratio) and the sequence's mean advantage."""
    m = loss_mask.bool()
    idx, n = _seq_index(log_ratio, cu_seqlens)
    cnt = _seg_sum(m.reshape(-1).to(log_ratio.dtype), idx, n).clamp(min=1)
    lr = _seg_sum(torch.where(m, log_ratio, 0.0).reshape(-1), idx, n) / cnt
    adv = _seg_sum(torch.where(m, advantages, 0.0).reshape(-1), idx, n) / cnt
    ratio = torch.exp(lr)[idx].view_as(log_ratio)
    adv = adv[idx].view_as(advantages)
    zero = torch.zeros((), dtype=ratio.dtype, device=ratio.device)
    return torch.where(m, ratio, zero), torch.where(m, adv, zero)


# --------------------------------------------------------------------------- rejection sampling


@dataclass
class RejectionSamplingResult:
    loss_mask: torch.Tensor
    behave_imp_weight: torch.Tensor
    filtered_fraction: float


def _kl_metric(logp, base, kind):
    d = logp.float() - base.float()
    if kind == "k1":
        return d
    if kind == "k2":
        return 0.5 * d * d
    return torch.exp(-d) - 1 + d


def _in_bounds(metric: torch.Tensor, cfg: RejectionSamplingConfig) -> torch.Tensor:
    ok = metric <= cfg.upper
    if cfg.lower is not None:
        ok = ok & (metric >= cfg.lower)
    return ok


def apply_rejection_sampling(proximal_logprobs, old_logprobs, loss_mask, cu_seqlens,
                             config: RejectionSamplingConfig) -> RejectionSamplingResult:
    """Filters (``mask``) or truncates (``clamp``) samples whose proximal/behaviour gap is
    out of bounds, per token or per sequence. Returns the updated mask, the behaviour
    importance weight ``π_prox/π_behave`` (zero outside the mask) and the affected fraction."""
    if proximal_logprobs.shape != old_logprobs.shape or proximal_logprobs.shape != loss_mask.shape:
        raise ValueError("proximal_logprobs, old_logprobs and loss_mask must have equal shapes")
    if proximal_logprobs.dim() not in (1, 2):
        raise ValueError(f"expected packed 1-D or padded 2-D tensors, got {proximal_logprobs.dim()}-D")
    m = loss_mask.bool()
    log_ratio = proximal_logprobs.detach().float() - old_logprobs.detach().float()
    log_ratio = torch.where(torch.isfinite(log_ratio), log_ratio, torch.zeros_like(log_ratio))
    is_ratio = config.metric == "ratio"
    metric = torch.exp(log_ratio) if is_ratio else _kl_metric(
        proximal_logprobs.detach(), old_logprobs.detach(), config.metric[3:])
    weight = torch.exp(log_ratio)
    original = weight
    in_bounds = None
    lo = config.lower if config.lower is not None else 0.0
    if config.level == "sequence":
        idx, n = _seq_index(log_ratio, cu_seqlens)
        vals = (log_ratio if is_ratio else metric)
        flat_m = m.reshape(-1)
        masked = torch.where(m, vals, torch.zeros_like(vals)).reshape(-1)
        raw_cnt = _seg_sum(flat_m.float(), idx, n)
        cnt = raw_cnt.clamp(min=1)
        if is_ratio:
            # the weight becomes the geometric mean of the per-token ratios
            weight = torch.exp(_seg_sum(masked, idx, n) / cnt)[idx].view_as(log_ratio)
            original = weight
        if config.agg == "sum":
            agg = _seg_sum(masked, idx, n)
        elif config.agg == "mean":
            agg = _seg_sum(masked, idx, n) / cnt
        elif config.agg == "max":
            neg = vals.masked_fill(~m, float("-inf")).reshape(-1)
            agg = torch.full((n,), float("-inf"), dtype=vals.dtype, device=vals.device)
            agg = agg.scatter_reduce(0, idx, neg, reduce="amax")
            agg = torch.where(raw_cnt == 0, torch.zeros_like(agg), agg)
        else:
            raise ValueError(f"unknown agg {config.agg}")
        seq_metric = torch.exp(agg) if is_ratio else agg
        ok_seq = _in_bounds(seq_metric, config)
        if config.action == "mask":
            in_bounds = ok_seq[idx].view_as(m)
        else:
            oob = (~ok_seq)[idx].view_as(m)
            weight = torch.where(oob, weight.clamp(min=lo, max=config.upper), weight)
    else:
        if config.action == "mask":
            in_bounds = _in_bounds(metric, config)
        else:
            weight = weight.clamp(min=lo, max=config.upper)
    if config.action == "mask":
        new_mask = (m & in_bounds).to(loss_mask.dtype)
        total = int(m.sum())
        frac = int((m & ~in_bounds).sum()) / max(total, 1)
    else:
        new_mask = loss_mask
        frac = int((m & (original != weight)).sum()) / max(int(m.sum()), 1)
    weight = torch.where(new_mask.bool(), weight, torch.zeros_like(weight))
    return RejectionSamplingResult(new_mask, weight, frac)


# --------------------------------------------------------------------------- PPO / GRPO actor loss


def ppo_actor_loss_fn(logprobs, proximal_logprobs, old_logprobs, advantages, eps_clip, loss_mask,
                      eps_clip_higher=None, c_clip=None, rejection_sampling=None,
                      importance_sampling_level="token", cu_seqlens=None):
    """Decoupled clipped policy loss.

    π_θ = ``logprobs``, π_prox = ``proximal_logprobs``, π_behave = ``old_logprobs``.
    ``loss = Σ_masked max(−A·r, −A·clip(r)) · w / N`` with ``r = π_θ/π_prox`` (token level, or
    the GSPO sequence-level geometric mean), optional dual clip, ``w = π_prox/π_behave``
    from rejection sampling, and ``N`` the mask count *before* any rejection.
    Returns ``(loss, stats dict of per-token tensors)``.
    """
    loss_mask = loss_mask.bool()
    denom = loss_mask.count_nonzero().clamp(min=1)
    filtered = 0.0
    weight = None
    if rejection_sampling is not None:
        rs = apply_rejection_sampling(proximal_logprobs, old_logprobs, loss_mask, cu_seqlens,
                                      rejection_sampling)
        loss_mask, weight, filtered = rs.loss_mask.bool(), rs.behave_imp_weight, rs.filtered_fraction
    if importance_sampling_level == "sequence":
        ratio, advantages = sequence_level_ratio_and_advantages(
            logprobs - proximal_logprobs, advantages, loss_mask, cu_seqlens)
    elif importance_sampling_level == "token":
        ratio = torch.where(loss_mask, torch.exp(logprobs - proximal_logprobs),
                            torch.zeros_like(logprobs))
    else:
        raise ValueError(f"importance_sampling_level must be token|sequence, got {importance_sampling_level}")
    hi = eps_clip if eps_clip_higher is None else eps_clip_higher
    clipped = torch.clamp(ratio, 1.0 - eps_clip, 1.0 + hi)
    l1, l2 = -advantages * ratio, -advantages * clipped
    clip_mask = l1.detach() < l2.detach()
    loss = torch.max(l1, l2)
    if c_clip is not None:
        assert c_clip > 1.0, c_clip
        l3 = torch.sign(advantages) * c_clip * advantages
        dual_mask = l3.detach() < loss.detach()
        loss = torch.min(loss, l3)
    else:
        dual_mask = torch.zeros_like(clip_mask)
    stat: dict[str, Any] = {}
    if weight is not None:
        kl = proximal_logprobs.detach() - old_logprobs.detach()
        bmask = (weight > 0) & loss_mask
        stat.update(behave_approx_kl=torch.where(bmask, kl, torch.zeros_like(kl)),
                    behave_imp_weight=weight.detach(), behave_mask=bmask, filtered_fraction=filtered)
        loss = loss * weight
    logging_loss = loss.detach()
    total = torch.where(loss_mask, loss, torch.zeros_like(loss)).sum() / denom
    stat.update(loss=logging_loss, importance_weight=ratio.detach(),
                approx_kl=(logprobs - proximal_logprobs).detach(),
                clip_mask=clip_mask & loss_mask, dual_clip_mask=dual_mask & loss_mask)
    return total, stat


def sapo_loss_fn(logprobs, old_logprobs, advantages, tau_pos, tau_neg, loss_mask,
                 importance_sampling_level="token", cu_seqlens=None):
    """SAPO: soft gate ``σ(τ(r−1))·4/τ`` (τ by the sign of A) instead of hard clipping."""
    loss_mask = loss_mask.bool()
    denom = loss_mask.count_nonzero().clamp(min=1)
    if importance_sampling_level == "sequence":
        ratio, advantages = sequence_level_ratio_and_advantages(
            logprobs - old_logprobs, advantages, loss_mask, cu_seqlens)
    else:
        ratio = torch.where(loss_mask, torch.exp(logprobs - old_logprobs), torch.zeros_like(logprobs))
    tau = torch.where(advantages >= 0, torch.full_like(ratio, tau_pos), torch.full_like(ratio, tau_neg))
    gate = torch.sigmoid(tau * (ratio - 1.0)) * (4.0 / tau)
    loss = -gate * advantages
    total = torch.where(loss_mask, loss, torch.zeros_like(loss)).sum() / denom
    stat = dict(loss=loss.detach(), importance_weight=ratio.detach(),
                approx_kl=(logprobs - old_logprobs).detach(),
                clip_mask=torch.zeros_like(loss_mask), dual_clip_mask=torch.zeros_like(loss_mask))
    return total, stat


# --------------------------------------------------------------------------- proximal-logp approximations


def compute_prox_logp_approximations(old_logp, logprobs, versions, current_version, method=None):
    """Approximates log π_prox (the policy one version back) from the behaviour
    logprob and the current logprob using per-token policy versions:
    ``α = clamp((v_prox − v_behave)/(v_θ − v_behave), 0, 1)`` with ``v_prox = v_θ − 1``;
    prompt tokens (version < 0) get α = 0. Returns a dict method → tensor."""
    v_theta = float(current_version)
    v_prox = v_theta - 1.0
    vb = versions.float()
    gen = versions >= 0
    denom = v_theta - vb
    alpha = torch.where((denom > 0) & gen, (v_prox - vb) / denom.clamp(min=1e-6), torch.zeros_like(vb))
    alpha = alpha.clamp(0.0, 1.0)
    out = {}
    want = (lambda m: method is None or method == m)
    if want("loglinear"):
        out["loglinear"] = old_logp + alpha * (logprobs - old_logp)
    if want("linear"):
        out["linear"] = torch.log((1 - alpha) * torch.exp(old_logp) + alpha * torch.exp(logprobs) + 1e-10)
    if want("rollout"):
        out["rollout"] = old_logp.clone()
    return out


def apply_m2po_masking(old_logp, prox_logp, loss_mask, m2_threshold):
    """M2PO: drop the tokens with the largest squared behaviour/proximal log-gap until the
    mean second moment of the remainder falls below ``m2_threshold`` (never all of them)."""
    m = loss_mask.bool()
    d2 = (old_logp.float() - prox_logp.float()) ** 2
    vals = d2[m]
    n = vals.numel()
    if n == 0:
        return loss_mask
    sorted_vals, order = torch.sort(vals, descending=True)
    # suffix means: mean of the elements kept after dropping the k largest
    suffix = sorted_vals.flip(0).cumsum(0).flip(0)
    counts = torch.arange(n, 0, -1, device=vals.device, dtype=vals.dtype)
    means = suffix / counts
    ok = (means < m2_threshold).nonzero()
    k = int(ok[0]) if ok.numel() else n - 1
    k = min(k, n - 1)
    keep = torch.ones(n, dtype=torch.bool, device=vals.device)
    keep[order[:k]] = False
    new_mask = torch.zeros_like(m)
    new_mask[m] = keep
    return new_mask.to(loss_mask.dtype)


# --------------------------------------------------------------------------- critic / SFT / RW / DPO


def ppo_critic_loss_fn(value, old_value, target_value, value_eps_clip, loss_mask, loss_fn_type="mse"):
    def base(x, y):
        if loss_fn_type == "huber":
            return F.huber_loss(x, y, reduction="none", delta=10.0)
        return 0.5 * (x - y) ** 2

    loss_mask = loss_mask.bool()
    l_orig = base(value, target_value)
    clipped_v = old_value + (value - old_value).clamp(-value_eps_clip, value_eps_clip)
    l_clip = base(clipped_v, target_value)
    loss = torch.max(l_orig, l_clip)
    clip_mask = (l_clip.detach() > l_orig.detach()) & loss_mask
    denom = loss_mask.count_nonzero().clamp(min=1)
    total = torch.where(loss_mask, loss, torch.zeros_like(loss)).sum() / denom
    return total, dict(clip_mask=clip_mask, loss=loss.detach())


def sft_loss(logprobs, loss_mask):
    """``−Σ_masked logp / (1e−5 + N)``."""
    m = loss_mask.bool()
    return -torch.where(m, logprobs, torch.zeros_like(logprobs)).sum() / (1e-5 + m.sum())


def rw_pairwise_loss(scores_last: torch.Tensor):
    """Bradley-Terry loss for interleaved (chosen, rejected) terminal scores ``[2P]``."""
    s = scores_last.view(-1, 2).float()
    margin = s[:, 0] - s[:, 1]
    return -F.logsigmoid(margin).mean(), dict(correct=(margin > 0).float(), margin=margin.detach())


def dpo_pair_logratios(logprobs, ref_logprobs, loss_mask, cu_seqlens):
    """Per-pair DPO logits from packed per-token logprobs with (chosen, rejected)
    sequences interleaved; sums are accumulated in fp64. Also returns per-pair token counts."""
    idx, n = _seq_index(logprobs, cu_seqlens)
    m = loss_mask.bool().reshape(-1)
    pi = _seg_sum(torch.where(m, logprobs.reshape(-1), 0.0).double(), idx, n)
    ref = _seg_sum(torch.where(m, ref_logprobs.reshape(-1), 0.0).double(), idx, n)
    cnt = _seg_sum(m.double(), idx, n).clamp(min=1)
    pi, ref, cnt = pi.view(-1, 2), ref.view(-1, 2), cnt.view(-1, 2)
    logits = (pi[:, 0] - pi[:, 1]) - (ref[:, 0] - ref[:, 1])
    logits_avg = (pi[:, 0] / cnt[:, 0] - pi[:, 1] / cnt[:, 1]) - (ref[:, 0] / cnt[:, 0] - ref[:, 1] / cnt[:, 1])
    return logits.float(), logits_avg.float(), (pi - ref).float()


def dpo_preference_loss(logits, logits_avg, beta: float, loss_type: str = "sigmoid"):
    if loss_type == "sigmoid":
        return -F.logsigmoid(beta * logits).mean()
    if loss_type == "ipo":
        return ((logits_avg - 1.0 / (2.0 * beta)) ** 2).mean()
    raise ValueError(f"unknown DPO loss type {loss_type}")


def reward_overlong_penalty(data: dict[str, Any], overlong_tokens: int, overlong_penalty_factor: float,
                            max_response_length: int) -> dict[str, Any]:
    """DAPO soft overlong punishment: ``r += min(−(len − (max − L_o)) / L_o · f, 0)``."""
    if "loss_mask" in data and data["loss_mask"].dim() == 2:
        resp_len = data["loss_mask"].sum(-1).float()
    else:
        cu = data["cu_seqlens"]
        idx, n = _seq_index(data["loss_mask"], cu)
        resp_len = _seg_sum(data["loss_mask"].float(), idx, n)
    expected = max_response_length - overlong_tokens
    penalty = torch.clamp(-(resp_len - expected) / overlong_tokens * overlong_penalty_factor, max=0.0)
    data["rewards"] = data["rewards"].float() + penalty.to(data["rewards"].device)
    return data
