"""SFT / reward-model / DPO trainers on the tiny CPU model: losses decrease and match hand formulas."""
import math

import pytest
import torch

from areal_b200.api.cli_args import (DPOConfig, DPOEngineConfig, MicroBatchSpec, OptimizerConfig, RWConfig, SFTConfig,
                                     TrainEngineConfig, _propagate_names)
from areal_b200.trainer.sl_trainer import DPOTrainer, RWTrainer, SFTTrainer, collate_pairs, collate_sft


def _engine_cfg(cls=TrainEngineConfig, **kw):
    return cls(backend="fsdp:d1", model_preset="tiny-qwen2", init_from_scratch=True,
               optimizer=OptimizerConfig(lr=2e-3, warmup_steps_proportion=0.0, weight_decay=0.0),
               mb_spec=MicroBatchSpec(max_tokens_per_mb=512), **kw)


def _base(cfg, tmp_path, bs=8):
    cfg.experiment_name, cfg.trial_name = "t", "t"
    cfg.cluster.fileroot = str(tmp_path)
    cfg.train_dataset.batch_size = bs
    cfg.train_dataset.shuffle = False
    cfg.total_train_epochs = 6
    _propagate_names(cfg)
    return cfg


def test_sft_loss_decreases_and_eval(tmp_path):
    g = torch.Generator().manual_seed(0)
    data = []
    for _ in range(8):
        n = int(torch.randint(12, 24, (1,), generator=g))
        ids = torch.randint(0, 1024, (n,), generator=g).tolist()
        data.append(dict(input_ids=ids, loss_mask=[0] * 4 + [1] * (n - 4)))
    cfg = _base(SFTConfig(actor=_engine_cfg()), tmp_path)
    losses = []
    with SFTTrainer(cfg, data, data) as tr:
        first = tr.wrapper.evaluate_lm(collate_sft(data))
        assert first == pytest.approx(math.log(1024), rel=0.05)  # random init ≈ uniform over the vocabulary
        tr.train(max_steps=6, step_callback=lambda s, st: losses.append(st["step/loss"]))
        last = tr.wrapper.evaluate_lm(collate_sft(data))
    assert len(losses) == 6 and losses[-1] < losses[0] and last < first


def _pairs(n=8, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        p = torch.randint(0, 1024, (6,), generator=g).tolist()
        out.append(dict(chosen_ids=p + torch.randint(0, 512, (8,), generator=g).tolist(),
                        rejected_ids=p + torch.randint(512, 1024, (5,), generator=g).tolist(),
                        chosen_loss_mask=[0] * 6 + [1] * 8, rejected_loss_mask=[0] * 6 + [1] * 5))
    return out


def test_reward_model_learns_pairs(tmp_path):
    cfg = _base(RWConfig(actor=_engine_cfg()), tmp_path)
    data = _pairs()
    losses = []
    with RWTrainer(cfg, data) as tr:
        tr.train(max_steps=6, step_callback=lambda s, st: losses.append(st["step/loss"]))
    assert losses[0] == pytest.approx(math.log(2), abs=0.2) and losses[-1] < losses[0]


@pytest.mark.parametrize("loss_type", ["sigmoid", "ipo"])
def test_dpo_trainer(tmp_path, loss_type):
    ref = _engine_cfg(DPOEngineConfig)
    ref.optimizer = None  # frozen reference policy with the same initial weights
    cfg = _base(DPOConfig(actor=_engine_cfg(DPOEngineConfig, beta=0.1, loss_type=loss_type), ref=ref), tmp_path)
    data = _pairs(seed=1)
    losses = []
    with DPOTrainer(cfg, data) as tr:
        b = collate_pairs(data)
        assert b["input_ids"].shape[0] == 16
        tr.train(max_steps=4, step_callback=lambda s, st: losses.append(st["step/loss"]))
    # policy == reference at step 0: sigmoid loss is log 2, IPO loss is (0 - 1/(2β))²
    expect = math.log(2) if loss_type == "sigmoid" else 25.0
    assert losses[0] == pytest.approx(expect, rel=1e-3) and losses[-1] < losses[0]


def test_gradient_checkpointing_gives_identical_gradients():
    """Recomputing block activations in backward must not change a single gradient."""
    import torch

    from areal_b200.models.config import PRESETS
    from areal_b200.models.qwen import build_model
    from areal_b200.ops.attention import VarlenMeta

    torch.manual_seed(0)
    ids = torch.randint(0, 1000, (40,))
    pos = torch.cat([torch.arange(25), torch.arange(15)])
    meta = VarlenMeta([0, 25, 40], "cpu")
    grads = []
    for every in (0, 1):
        m = build_model(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=3)
        m.checkpoint_every = every
        m(ids, pos, meta).square().mean().backward()
        grads.append({n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None})
    assert set(grads[0]) == set(grads[1]) and len(grads[0]) > 10
    for n in grads[0]:
        assert torch.allclose(grads[0][n], grads[1][n], atol=1e-7), n
