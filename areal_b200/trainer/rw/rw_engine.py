"""Bradley-Terry reward-model training: the value head's score at the last token of
each sequence, (chosen, rejected) pairs interleaved, ``−logsigmoid(s_c − s_r)``
(areal/trainer/rw/rw_engine.py:115-146 in the reference)."""

from __future__ import annotations

from typing import Any

import torch

from ...api.engine_api import TrainEngine
from ...utils import functional as Fn
from ...utils import stats_tracker


def rw_loss_fn(values: torch.Tensor, input_data: dict[str, Any]) -> torch.Tensor:
    cu = input_data["cu_seqlens"].long()
    assert (cu.numel() - 1) % 2 == 0, "reward-model batches hold (chosen, rejected) pairs"
    last = values.float()[cu[1:] - 1]
    loss, st = Fn.rw_pairwise_loss(last)
    with torch.no_grad():
        ok = torch.ones_like(st["correct"], dtype=torch.bool)
        stats_tracker.denominator(n_pairs=ok)
        stats_tracker.stat(correct_ratio=st["correct"], pos_score=last.view(-1, 2)[:, 0].detach(),
                           neg_score=last.view(-1, 2)[:, 1].detach(), margin=st["margin"], denominator="n_pairs")
    return loss


def rw_loss_weight_fn(mb: dict[str, Any]) -> float:
    return float((mb["cu_seqlens"].numel() - 1) // 2)


class RWEngine:
    def __init__(self, engine: TrainEngine):
        self.engine = engine

    def train_rw(self, data: dict[str, Any]) -> dict[str, float]:
        self.engine.train()
        with stats_tracker.scope("rw"):
            return self.engine.train_batch(data, loss_fn=rw_loss_fn, loss_weight_fn=rw_loss_weight_fn)

    def evaluate_rw(self, data: dict[str, Any]) -> float:
        self.engine.eval()
        with stats_tracker.scope("rw-eval"):
            return self.engine.eval_batch(data, loss_fn=rw_loss_fn, loss_weight_fn=rw_loss_weight_fn)
