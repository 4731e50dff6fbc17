"""PPO critic: value prediction and the clipped value loss
(areal/trainer/ppo/critic.py:25-149 in the reference)."""

from __future__ import annotations

import functools
from typing import Any

import torch

from ...api.cli_args import MicroBatchSpec, PPOCriticConfig
from ...api.engine_api import TrainEngine
from ...utils import functional as Fn
from ...utils import stats_tracker
from ...utils.data import split_padded_tensor_dict_into_mb_list, unpack_to_padded


class PPOCritic:
    def __init__(self, config: PPOCriticConfig, engine: TrainEngine):
        self.config, self.engine = config, engine

    @torch.no_grad()
    def compute_values(self, data: dict[str, Any]) -> torch.Tensor:
        self.engine.eval()
        return self.engine.forward_batch(data)

    def ppo_update(self, data: dict[str, Any]) -> list[dict[str, float]]:
        cfg = self.config
        data = {k: v for k, v in data.items() if k in (
            "input_ids", "attention_mask", "loss_mask", "values", "returns", "seq_no_eos_mask")}
        B = data["input_ids"].shape[0]
        mbs = split_padded_tensor_dict_into_mb_list(data, MicroBatchSpec(n_mbs=min(cfg.ppo_n_minibatches, B)))
        loss_fn = functools.partial(critic_loss_fn, eps_clip=cfg.eps_clip)
        out = []
        self.engine.train()
        for mb in mbs.mbs:
            st = self.engine.train_batch(unpack_to_padded(mb), loss_fn=loss_fn,
                                         loss_weight_fn=lambda x: float(x["loss_mask"].count_nonzero()))
            stats_tracker.scalar(**{f"ppo_critic/{k}": v for k, v in st.items()})
            out.append(st)
        return out


def critic_loss_fn(values: torch.Tensor, input_data: dict[str, Any], eps_clip: float) -> torch.Tensor:
    loss_mask = input_data["loss_mask"].bool()
    loss, stat = Fn.ppo_critic_loss_fn(values.float(), input_data["values"].float(), input_data["returns"].float(),
                                       eps_clip, loss_mask)
    with stats_tracker.scope("ppo_critic"):
        stats_tracker.denominator(n_valid_tokens=loss_mask, clipped_tokens=stat["clip_mask"])
        stats_tracker.stat(value_loss=stat["loss"], new_values=values.detach().float(),
                           returns=input_data["returns"].float(), denominator="n_valid_tokens")
    return loss


ppo_loss_fn = critic_loss_fn  # the name of the reference's critic loss (areal/trainer/ppo/critic.py:105)


class PPOCriticEngine:
    """A train engine (``is_critic``) with the critic's algorithm methods on it: what a single-controller run creates
    in every worker process, so that ``compute_values`` / ``ppo_update`` run next to the model."""

    def __init__(self, config: PPOCriticConfig):
        from ...engine.train_engine import B200TrainEngine

        config.is_critic = True
        self.engine = B200TrainEngine(config)
        self.critic = PPOCritic(config, self.engine)

    def compute_values(self, data):
        return self.critic.compute_values(data)

    def ppo_update(self, data):
        return self.critic.ppo_update(data)

    def __getattr__(self, name):
        if name in ("engine", "critic"):
            raise AttributeError(name)
        return getattr(self.engine, name)


def _critic_controller():
    from ...infra.controller.train_controller import TrainController

    class PPOCriticController(TrainController):
        """Controller-side handle whose workers run :class:`PPOCriticEngine`."""

        def __init__(self, config, scheduler, engine: str | type | None = None):
            super().__init__(engine or f"{__name__}.PPOCriticEngine", config, scheduler)

    return PPOCriticController


PPOCriticController = _critic_controller()
PPOCriticControllerV2 = PPOCriticController
