"""PPO / GRPO actor: logprob recomputation, reward shaping, KL-regularised token
rewards, GAE, advantage normalisation and the mini-batched policy update with
the decoupled clipped objective (and its GSPO / SAPO / M2PO / distillation
variants, proximal-logprob approximations and staleness statistics).

Algorithm semantics follow the reference actor
(areal/trainer/ppo/actor.py:43-1109): rollout logprobs and the loss mask are
shifted to next-token form, the task reward lands on the last generated token,
GAE runs backwards through masked positions, and ``ppo_update`` performs
``ppo_n_minibatches`` sequential optimizer steps.
"""

from __future__ import annotations

import functools
from typing import Any

import torch

from ...api.cli_args import PROX_LOGP_METHOD_METRICS, PROX_LOGP_METHOD_RECOMPUTE, MicroBatchSpec, PPOActorConfig
from ...api.engine_api import TrainEngine
from ...utils import functional as Fn
from ...utils import stats_tracker
from ...utils.data import KLEstimator, Normalization, split_padded_tensor_dict_into_mb_list


class PPOActor:
    def __init__(self, config: PPOActorConfig, engine: TrainEngine):
        self.config = config
        self.engine = engine
        self.reward_bias = config.reward_bias
        self.reward_scaling = config.reward_scaling
        self.reward_clip = config.reward_clip
        self.reward_norm = Normalization(config.reward_norm) if config.reward_norm else None
        self.adv_norm = Normalization(config.adv_norm) if config.adv_norm else None
        self.kl_ctl = config.kl_ctl
        self.kl_estimator = KLEstimator(config.kl_estimator)
        self.discount = config.discount
        self.gae_lambda = config.gae_lambda
        self.mask_no_eos_with_zero = config.mask_no_eos_with_zero
        self.temperature = config.temperature
        self.m2_threshold = config.m2_threshold

    # ------------------------------------------------------------- logprobs
    @torch.no_grad()
    def compute_logp(self, data: dict[str, Any]) -> torch.Tensor:
        """Next-token logprobs of the sequences under the current weights, ``[B, L]``."""
        self.engine.eval()
        return self.engine.forward_batch(data)

    # ------------------------------------------------------------ advantages
    @torch.no_grad()
    def compute_advantages(self, data: dict[str, Any]) -> dict[str, Any]:
        cfg = self.config
        data = dict(data)
        ids = data["input_ids"]
        B, L = ids.shape
        rows = torch.arange(B)
        if cfg.overlong_reward_penalty:
            assert cfg.overlong_tokens is not None and cfg.overlong_penalty_factor is not None
            data = Fn.reward_overlong_penalty(data, cfg.overlong_tokens, cfg.overlong_penalty_factor,
                                              cfg.max_new_tokens)
        reward = (data["rewards"].float() + self.reward_bias) * self.reward_scaling
        reward = reward.clamp(-self.reward_clip, self.reward_clip)
        if self.reward_norm is not None:
            reward = self.reward_norm(reward, reduce_group=self.engine.data_parallel_group)
        loss_mask = torch.roll(data["loss_mask"].float(), shifts=-1, dims=-1)
        if not cfg.use_decoupled_loss and cfg.recompute_logprob:
            if data.get("prox_logp") is None:
                raise ValueError("recompute_logprob=True but prox_logp is missing (compute_logp was skipped)")
            old_logp = data["logprobs"] = data["prox_logp"]
        else:
            old_logp = torch.roll(data["logprobs"].float(), shifts=-1, dims=-1)
            if not cfg.use_decoupled_loss:
                data["prox_logp"] = old_logp
        ref_logp = data.get("ref_logp")
        ref_logp = torch.zeros_like(old_logp) if ref_logp is None else ref_logp.float().clone()
        ref_logp = ref_logp * loss_mask
        old_logp = old_logp * loss_mask
        attn = data["attention_mask"]
        seqlens = attn.sum(-1).long()
        no_eos = data.get("seq_no_eos_mask")
        no_eos = (seqlens == L) if no_eos is None else no_eos.bool()
        rewards = -self.kl_ctl * self.kl_estimator(old_logp, ref_logp)
        kl_rewards = rewards.clone()
        rewards[rows, seqlens - 1] = 0
        idx = (seqlens - 2).clamp(min=0)
        if self.mask_no_eos_with_zero:
            rewards[rows, idx] += torch.where(no_eos, torch.zeros_like(reward), reward)
        else:
            rewards[rows, idx] += reward
        values = data.get("values")
        values = torch.zeros_like(rewards) if values is None else values.float()
        adv = self._gae(rewards, values, loss_mask, seqlens, no_eos)
        data["returns"] = adv + values
        if self.adv_norm is not None:
            adv = self.adv_norm(adv, loss_mask, reduce_group=self.engine.data_parallel_group)
        data.update(advantages=adv, kl_rewards=kl_rewards, tot_rewards=rewards, loss_mask=loss_mask,
                    logprobs=old_logp)
        return data

    def _gae(self, rewards, values, loss_mask, seqlens, no_eos):
        """Reverse scan through masked positions; padded layout, vectorised over the batch."""
        B, L = rewards.shape
        gamma, lam = self.discount, self.gae_lambda
        if gamma == 1.0 and lam == 1.0 and not bool(values.any()):
            # GRPO case: reward-to-go over masked positions, via one cumulative sum
            masked = rewards * loss_mask
            togo = masked.flip(-1).cumsum(-1).flip(-1)
            # positions outside the mask carry the next masked position's value
            adv = torch.zeros_like(rewards)
            adv[:, : L - 1] = togo[:, : L - 1]
            adv[:, L - 1] = 0
            return adv
        adv_rev = [torch.zeros(B, dtype=torch.float32)]
        last = torch.zeros(B)
        nextv = values[:, L - 1] * no_eos.float()
        for t in reversed(range(L - 1)):
            delta = rewards[:, t] + gamma * nextv - values[:, t]
            new = delta + gamma * lam * last
            m = loss_mask[:, t]
            nextv = nextv * (1 - m) + values[:, t] * m
            last = last * (1 - m) + new * m
            adv_rev.append(last)
        return torch.stack(adv_rev[::-1], dim=1)

    # ---------------------------------------------------------------- update
    def ppo_update(self, data: dict[str, Any]) -> list[dict[str, float]]:
        cfg = self.config
        data = dict(data)
        B = data["input_ids"].shape[0]
        with stats_tracker.scope("ppo_actor"):
            self._log_batch_stats(data)
        for k in ("rewards", "tot_rewards", "kl_rewards", "versions_raw"):
            data.pop(k, None)
        if cfg.use_decoupled_loss and cfg.prox_logp_method != PROX_LOGP_METHOD_RECOMPUTE \
                and "versions" in data:
            data["versions_next"] = torch.roll(data["versions"], shifts=-1, dims=-1)
        if self.m2_threshold is not None and data.get("prox_logp") is not None:
            data["loss_mask"] = Fn.apply_m2po_masking(data["logprobs"], data["prox_logp"], data["loss_mask"],
                                                      self.m2_threshold).float()
        n_mb = min(cfg.ppo_n_minibatches, B)
        mbs = split_padded_tensor_dict_into_mb_list(
            data, MicroBatchSpec(n_mbs=n_mb, granularity=cfg.mb_spec.granularity))
        # re-pad each mini-batch (the engine splits it further into token-bounded micro-batches)
        from ...utils.data import unpack_to_padded

        loss_fn = functools.partial(grpo_loss_fn, config=cfg, current_version=self.engine.get_version(),
                                    distill=getattr(self, "distill_weights", None))
        all_stats = []
        self.engine.train()
        for mb in mbs.mbs:
            padded = unpack_to_padded(mb)
            st = self.engine.train_batch(padded, loss_fn=loss_fn,
                                         loss_weight_fn=lambda x: float(x["loss_mask"].count_nonzero()))
            stats_tracker.scalar(**{f"ppo_actor/{k}": v for k, v in st.items()})
            all_stats.append(st)
        return all_stats

    def _log_batch_stats(self, data):
        attn = data["attention_mask"].bool()
        lm = data["loss_mask"].bool()
        seqlens = attn.sum(-1).float()
        n_seqs = torch.ones(attn.shape[0], dtype=torch.bool)
        stats_tracker.denominator(n_seqs=n_seqs, n_tokens=attn, n_valid_tokens=lm)
        if "rewards" in data:
            stats_tracker.stat(task_reward=data["rewards"].float(), seq_len=seqlens,
                               prompt_len=seqlens - data["loss_mask"].sum(-1).float(), denominator="n_seqs")
        stats_tracker.stat(advantages=data["advantages"], kl_rewards=data.get("kl_rewards", torch.zeros_like(data["advantages"])),
                           denominator="n_valid_tokens")
        if "versions" in data:
            v = torch.roll(data["versions"], shifts=-1, dims=-1).float()
            cur = float(self.engine.get_version())
            stale = torch.where(lm, cur - v, torch.zeros_like(v))
            stats_tracker.stat(staleness=stale, denominator="n_valid_tokens")


def grpo_loss_fn(logprobs: torch.Tensor, entropy: torch.Tensor | None, input_data: dict[str, Any],
                 config: PPOActorConfig, current_version: int | None = None,
                 distill: tuple[float, float] | None = None) -> torch.Tensor:
    """Policy loss of one packed micro-batch. ``logprobs`` / ``entropy`` are the engine's
    next-token outputs ``[T]``; ``input_data`` holds the packed batch on the same device.
    ``distill = (rl_loss_weight, distill_loss_weight)`` mixes in the distillation term when the batch
    carries ``teacher_logp``."""
    cfg = config
    old_logp = input_data["logprobs"].float()
    adv = input_data["advantages"].float()
    loss_mask = input_data["loss_mask"].bool()
    cu = input_data.get("cu_seqlens")
    prox = input_data.get("prox_logp")
    if cfg.use_decoupled_loss and cfg.prox_logp_method != PROX_LOGP_METHOD_RECOMPUTE:
        versions = input_data.get("versions_next")
        if versions is None:
            raise ValueError("proximal-logp approximation needs per-token versions")
        approx = Fn.compute_prox_logp_approximations(old_logp, logprobs.detach().float(), versions,
                                                     current_version)
        if cfg.prox_logp_method == PROX_LOGP_METHOD_METRICS:
            if prox is None:
                raise ValueError("prox_logp_method=metrics needs the recomputed prox_logp")
            with stats_tracker.scope("prox_approx"):
                stats_tracker.denominator(n_valid_tokens=loss_mask)
                for name, val in approx.items():
                    stats_tracker.stat(**{f"{name}_abs_err": (val - prox.float()).abs()},
                                       denominator="n_valid_tokens")
        else:
            prox = approx[cfg.prox_logp_method]
    if prox is None:
        prox = old_logp
    prox = prox.float()
    teacher = input_data.get("teacher_logp")

    if cfg.use_sapo_loss:
        loss, stat = Fn.sapo_loss_fn(logprobs.float(), old_logp, adv, cfg.sapo_tau_pos, cfg.sapo_tau_neg,
                                     loss_mask, cfg.importance_sampling_level, cu)
    else:
        rs = cfg.rejection_sampling
        simple_rs = rs is None or (rs.level == "token" and rs.action == "mask" and rs.metric == "ratio"
                                   and rs.lower is None)
        fused_ok = (logprobs.is_cuda and cfg.importance_sampling_level == "token" and simple_rs
                    and teacher is None)
        if fused_ok:
            from ...ops.rl_ops import ppo_loss_fused

            decoupled = cfg.use_decoupled_loss or rs is not None
            loss, st = ppo_loss_fused(logprobs.float(), prox, old_logp, adv, loss_mask,
                                      eps_clip=cfg.eps_clip, eps_clip_higher=cfg.eps_clip_higher,
                                      c_clip=cfg.c_clip, behav_cap=(rs.upper if rs is not None else None),
                                      use_decoupled=decoupled, behav_weight=rs is not None)
            _record_fused_stats(st, loss_mask, entropy)
            return loss
        loss, stat = Fn.ppo_actor_loss_fn(logprobs.float(), prox, old_logp, adv, cfg.eps_clip, loss_mask,
                                          eps_clip_higher=cfg.eps_clip_higher, c_clip=cfg.c_clip,
                                          rejection_sampling=rs,
                                          importance_sampling_level=cfg.importance_sampling_level,
                                          cu_seqlens=cu)
    if teacher is not None:
        rl_w, kd_w = distill if distill is not None else (float(input_data.get("rl_loss_weight", 1.0)),
                                                         float(input_data.get("distill_loss_weight", 0.0)))
        denom = loss_mask.count_nonzero().clamp(min=1)
        lp = logprobs.float()
        if rl_w == 0.0:
            kd = -(torch.exp(lp - old_logp).detach() * (teacher.float() - lp.detach()) * lp)
            loss = kd_w * torch.where(loss_mask, kd, torch.zeros_like(kd)).sum() / denom
        else:
            kd = torch.where(loss_mask, lp - teacher.float(), torch.zeros_like(lp)).sum() / denom
            loss = rl_w * loss + kd_w * kd
    with stats_tracker.scope("ppo_actor"):
        stats_tracker.denominator(n_valid_tokens=loss_mask, clipped_tokens=stat["clip_mask"],
                                  dual_clipped_tokens=stat["dual_clip_mask"])
        stats_tracker.stat(importance_weight=stat["importance_weight"], approx_kl=stat["approx_kl"],
                           new_logp=logprobs.detach().float(), old_logp=old_logp,
                           actor_loss=stat["loss"], denominator="n_valid_tokens")
        if entropy is not None:
            stats_tracker.stat(entropy=entropy.detach().float(), denominator="n_valid_tokens")
        if "behave_imp_weight" in stat:
            stats_tracker.denominator(unclipped_behave_tokens=stat["behave_mask"])
            stats_tracker.stat(behave_imp_weight=stat["behave_imp_weight"],
                               behave_approx_kl=stat["behave_approx_kl"],
                               denominator="unclipped_behave_tokens")
    return loss


def _record_fused_stats(st: torch.Tensor, loss_mask: torch.Tensor, entropy):
    """Statistics of the fused kernel arrive as six sums; export them as scalars."""
    vals = st.detach().float().cpu().tolist()
    n = max(float(loss_mask.count_nonzero()), 1.0)
    stats_tracker.scalar(**{
        "ppo_actor/actor_loss": vals[0], "ppo_actor/clip_ratio": vals[1] / n,
        "ppo_actor/dual_clip_ratio": vals[2] / n, "ppo_actor/behave_imp_weight": vals[3] / n,
        "ppo_actor/ratio_abs_dev": vals[4] / n, "ppo_actor/behave_dropped_ratio": vals[5] / n})
    if entropy is not None:
        m = loss_mask
        stats_tracker.scalar(**{"ppo_actor/entropy": float((entropy.detach().float() * m).sum() / n)})


class PPOActorEngine:
    """A train engine with the actor's algorithm methods on it: the object a single-controller run creates in
    every worker process (``TrainController("...PPOActorEngine", config.actor, scheduler)``), so that
    ``compute_logp`` / ``compute_advantages`` / ``ppo_update`` run next to the model and only batches and
    statistics cross the process boundary. Every other attribute is the engine's.
    Reference: the ``FSDPPPOActor`` / ``as_controller`` pairing of areal/trainer/rl_trainer.py:876,933-1041."""

    def __init__(self, config: PPOActorConfig):
        from ...engine.train_engine import B200TrainEngine

        self.engine = B200TrainEngine(config)
        self.actor = PPOActor(config, self.engine)

    def compute_logp(self, data):
        return self.actor.compute_logp(data)

    def compute_advantages(self, data):
        return self.actor.compute_advantages(data)

    def ppo_update(self, data):
        return self.actor.ppo_update(data)

    def flat_checksum(self) -> float:
        """Sum of the weights (tests compare replicas with it)."""
        return float(self.engine.flat.flat.double().sum())

    def __getattr__(self, name):
        if name in ("engine", "actor"):
            raise AttributeError(name)
        return getattr(self.engine, name)


# controller-side handles of single-controller mode: a ``TrainController`` whose workers run the engine classes
# above; ``compute_logp`` / ``compute_advantages`` / ``ppo_update`` are forwarded to every data-parallel rank with
# the batch split by tokens (infra/controller/train_controller.py)
def _controller(engine_cls_name: str):
    from ...infra.controller.train_controller import TrainController

    class _Ctl(TrainController):
        def __init__(self, config, scheduler, engine: str | type | None = None):
            super().__init__(engine or f"{__name__}.{engine_cls_name}", config, scheduler)

    return _Ctl


PPOActorController = _controller("PPOActorEngine")
PPOActorController.__name__ = PPOActorController.__qualname__ = "PPOActorController"
PPOActorControllerV2 = PPOActorController
from ...utils.functional import compute_prox_logp_approximations  # noqa: E402,F401  (re-exported)
