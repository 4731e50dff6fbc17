"""Supervised fine-tuning on packed sequences: ``−Σ_masked logp / (1e−5 + N)`` with
per-sequence perplexity logging (areal/trainer/sft/lm_engine.py:81-130 in the reference)."""

from __future__ import annotations

from typing import Any

import torch

from ...api.engine_api import TrainEngine
from ...utils import functional as Fn
from ...utils import stats_tracker


def sft_loss_fn(logprobs: torch.Tensor, entropy, input_data: dict[str, Any]) -> torch.Tensor:
    # the engine's logprobs are in next-token form: shift the mask the same way
    loss_mask = torch.roll(input_data["loss_mask"].bool(), shifts=-1, dims=0)
    cu = input_data["cu_seqlens"].long()
    loss_mask[cu[1:] - 1] = False  # the last position of a sequence predicts nothing of its own
    loss = Fn.sft_loss(logprobs.float(), loss_mask)
    with torch.no_grad():
        lp = torch.where(loss_mask, logprobs.detach().float(), torch.zeros_like(logprobs, dtype=torch.float32))
        seg = torch.arange(cu.numel() - 1, device=lp.device).repeat_interleave(cu[1:] - cu[:-1])
        s = torch.zeros(cu.numel() - 1, device=lp.device).index_add_(0, seg, lp)
        n = torch.zeros(cu.numel() - 1, device=lp.device).index_add_(0, seg, loss_mask.float())
        seq_ok = n > 0
        ppl = torch.exp(-s / n.clamp(min=1))
        stats_tracker.denominator(n_seqs=torch.ones_like(seq_ok), n_valid_seqs=seq_ok, n_tokens=torch.ones_like(loss_mask),
                                  n_valid_tokens=loss_mask)
        stats_tracker.stat(ppl=ppl, denominator="n_valid_seqs")
        stats_tracker.stat(loss=-lp, denominator="n_valid_tokens")
    return loss


def sft_loss_weight_fn(mb: dict[str, Any]) -> float:
    return float(mb["loss_mask"].count_nonzero())


class LMEngine:
    def __init__(self, engine: TrainEngine):
        self.engine = engine

    def train_lm(self, data: dict[str, Any]) -> dict[str, float]:
        self.engine.train()
        with stats_tracker.scope("sft"):
            return self.engine.train_batch(data, loss_fn=sft_loss_fn, loss_weight_fn=sft_loss_weight_fn)

    def evaluate_lm(self, data: dict[str, Any]) -> float:
        self.engine.eval()
        with stats_tracker.scope("sft-eval"):
            return self.engine.eval_batch(data, loss_fn=sft_loss_fn, loss_weight_fn=sft_loss_weight_fn)
