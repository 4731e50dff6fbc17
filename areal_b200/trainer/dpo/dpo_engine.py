"""Direct preference optimisation (sigmoid and IPO) on packed interleaved
(chosen, rejected) pairs, with reference logprobs computed once per batch
(areal/trainer/dpo/dpo_engine.py, areal/utils/functional/functional.py:641-702)."""

from __future__ import annotations

import functools
from typing import Any

import torch

from ...api.cli_args import DPOEngineConfig
from ...api.engine_api import TrainEngine
from ...utils import functional as Fn
from ...utils import stats_tracker


def dpo_loss_fn(logprobs: torch.Tensor, entropy, input_data: dict[str, Any], beta: float, loss_type: str):
    cu = input_data["cu_seqlens"]
    loss_mask = torch.roll(input_data["loss_mask"].bool(), shifts=-1, dims=0)
    loss_mask[cu.long()[1:] - 1] = False
    ref = input_data["ref_logprobs"].float()
    logits, logits_avg, rewards = Fn.dpo_pair_logratios(logprobs.float(), ref, loss_mask, cu)
    loss = Fn.dpo_preference_loss(logits, logits_avg, beta, loss_type)
    with torch.no_grad():
        ok = torch.ones(logits.shape[0], dtype=torch.bool, device=logits.device)
        stats_tracker.denominator(n_pairs=ok)
        stats_tracker.stat(reward_accuracy=(logits > 0).float(), reward_margin=beta * logits.detach(),
                           chosen_reward=beta * rewards[:, 0].detach(), rejected_reward=beta * rewards[:, 1].detach(),
                           denominator="n_pairs")
    return loss


def dpo_loss_weight_fn(mb: dict[str, Any]) -> float:
    return float((mb["cu_seqlens"].numel() - 1) // 2)


class DPOEngine:
    """``engine`` is the policy, ``ref_engine`` a frozen copy used for the reference logprobs
    (micro-batches are split with granularity 2 so pairs stay together)."""

    def __init__(self, config: DPOEngineConfig, engine: TrainEngine, ref_engine: TrainEngine | None = None):
        self.config, self.engine, self.ref_engine = config, engine, ref_engine
        engine.config.mb_spec.granularity = 2
        if ref_engine is not None:
            ref_engine.config.mb_spec.granularity = 2

    @torch.no_grad()
    def compute_ref_logprobs(self, data: dict[str, Any]) -> torch.Tensor:
        eng = self.ref_engine or self.engine
        eng.eval()
        return eng.forward_batch(data)

    def train_dpo(self, data: dict[str, Any]) -> dict[str, float]:
        if "ref_logprobs" not in data:
            data = dict(data, ref_logprobs=self.compute_ref_logprobs(data))
        self.engine.train()
        fn = functools.partial(dpo_loss_fn, beta=self.config.beta, loss_type=self.config.loss_type)
        with stats_tracker.scope("dpo"):
            return self.engine.train_batch(data, loss_fn=fn, loss_weight_fn=dpo_loss_weight_fn)

    def evaluate_dpo(self, data: dict[str, Any]) -> float:
        if "ref_logprobs" not in data:
            data = dict(data, ref_logprobs=self.compute_ref_logprobs(data))
        self.engine.eval()
        fn = functools.partial(dpo_loss_fn, beta=self.config.beta, loss_type=self.config.loss_type)
        with stats_tracker.scope("dpo-eval"):
            return self.engine.eval_batch(data, loss_fn=fn, loss_weight_fn=dpo_loss_weight_fn)
