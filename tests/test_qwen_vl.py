"""Vision-language model (Qwen2.5-VL): parity with transformers, position triples, engine path."""

import dataclasses

import pytest
import torch

from areal_b200.models.config import PRESETS, ModelConfig
from areal_b200.models.qwen import build_model
from areal_b200.models.qwen_vl import QwenVLModel, mrope_position_ids, mrope_tables
from areal_b200.ops.attention import VarlenMeta
from areal_b200.utils.hf_io import load_hf_weights, save_hf_checkpoint

CFG = PRESETS["tiny-qwen2_5-vl"]
IMG = CFG.image_token_id


def _model(seed=0):
    m = build_model(CFG, dtype=torch.float32, seed=seed)
    g = torch.Generator().manual_seed(seed + 100)
    with torch.no_grad():  # biases and norm weights start at 0 / 1: perturb them so that parity exercises them
        for n, p in m.named_parameters():
            if n.endswith("bias") or n.endswith("norm"):
                p.add_(torch.randn(p.shape, generator=g) * 0.05)
    return m


def _sample(grids, texts, seed=0):
    """One sequence: text run, image, text run, image, ... → ids, pixel rows."""
    g = torch.Generator().manual_seed(seed)
    ids = []
    for i, n in enumerate(texts):
        ids += torch.randint(0, 900, (n,), generator=g).tolist()
        if i < len(grids):
            t, h, w = grids[i]
            ids += [CFG.vision_start_token_id] + [IMG] * (t * h * w // 4) + [CFG.vision_end_token_id]
    n_patch = sum(t * h * w for t, h, w in grids)
    pix = torch.randn(n_patch, 3 * 2 * 14 * 14, generator=g)
    return ids, pix


def test_position_triples():
    ids, _ = _sample([(1, 4, 6)], [3, 2])
    pos, deltas = mrope_position_ids(ids, [0, len(ids)], [(1, 4, 6)], CFG)
    # 3 text + start marker → 0..3; image 2×3 merged grid at offset 4; end marker + 2 text after max+1 = 7
    assert pos[:, :4].tolist() == [[0, 1, 2, 3]] * 3
    assert pos[0, 4:10].tolist() == [4] * 6
    assert pos[1, 4:10].tolist() == [4, 4, 4, 5, 5, 5]
    assert pos[2, 4:10].tolist() == [4, 5, 6, 4, 5, 6]
    assert pos[:, 10:].tolist() == [[7, 8, 9]] * 3
    assert deltas == [10 - len(ids)]
    with pytest.raises(ValueError):
        mrope_position_ids(ids, [0, len(ids)], [(1, 4, 8)], CFG)
    with pytest.raises(ValueError):
        mrope_position_ids(ids, [0, len(ids)], [], CFG)
    # text-only tables equal the ordinary rotary tables
    from areal_b200.ops.fused import rope_tables
    p = torch.arange(7)[None].expand(3, -1)
    cos, sin = mrope_tables(p, 64, 1e4, [8, 12, 12])
    c0, s0 = rope_tables(7, 64, 1e4, "cpu")
    assert torch.allclose(cos, c0) and torch.allclose(sin, s0)


def test_matches_transformers(tmp_path):
    transformers = pytest.importorskip("transformers")
    m = _model()
    assert isinstance(m, QwenVLModel)
    save_hf_checkpoint(m, CFG, str(tmp_path))
    hf = transformers.Qwen2_5_VLForConditionalGeneration.from_pretrained(str(tmp_path), torch_dtype=torch.float32)
    hf.eval()
    grids = [(1, 6, 8), (1, 4, 4)]  # 3×4 merged units (ragged 2×2 windows) and 2×2
    ids, pix = _sample(grids, [5, 4, 6], seed=3)
    ids_t = torch.tensor(ids)
    meta = VarlenMeta(torch.tensor([0, len(ids)], dtype=torch.int32), "cpu")
    grid_t = torch.tensor(grids)
    with torch.no_grad():
        feats = m.visual(pix, grid_t)
        theirs_feats = hf.model.visual(pix, grid_thw=grid_t).pooler_output
        assert float((feats - theirs_feats).abs().max()) < 1e-4
        mine = m.logits(m(ids_t, torch.arange(len(ids)), meta, pixel_values=pix, image_grid_thw=grid_t))
        pos, _ = m.positions(ids_t, meta, grid_t)
        theirs = hf(input_ids=ids_t[None], pixel_values=pix, image_grid_thw=grid_t,
                    position_ids=pos[:, None, :]).logits[0]
    assert float((mine - theirs).abs().max()) < 5e-4
    # text-only input: same as the text path of transformers with ordinary positions
    txt = torch.randint(0, 900, (17,), generator=torch.Generator().manual_seed(9))
    meta2 = VarlenMeta(torch.tensor([0, 17], dtype=torch.int32), "cpu")
    with torch.no_grad():
        a = m.logits(m(txt, torch.arange(17), meta2))
        b = hf(input_ids=txt[None]).logits[0]
    assert float((a - b).abs().max()) < 5e-4
    # round trip through the checkpoint (and the older `visual.*` / `model.*` naming)
    m2 = build_model(ModelConfig.from_hf_config(str(tmp_path)), dtype=torch.float32, seed=7)
    load_hf_weights(m2, str(tmp_path))
    for (n1, p1), (n2, p2) in zip(m.named_parameters(), m2.named_parameters()):
        assert n1 == n2 and torch.equal(p1, p2), n1
    old = [((n[len("model."):] if n.startswith("model.visual.") else n.replace("model.language_model.", "model.")), t)
           for n, t in m.to_hf()]
    m3 = build_model(CFG, dtype=torch.float32, seed=8).load_hf(old)
    assert all(torch.equal(p1, p3) for p1, p3 in zip(m.parameters(), m3.parameters()))


def _vl_items(n=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    items = []
    for i in range(n):
        if i % 3 == 2:  # a text-only sample in the mix
            ids = torch.randint(0, 900, (14,), generator=g).tolist()
            items.append(dict(input_ids=ids, loss_mask=[0] * 8 + [1] * 6))
            continue
        grid = [(1, 4, 4), (1, 4, 6)][i % 2]
        ids, pix = _sample([grid], [4, 6], seed=seed * 100 + i)
        items.append(dict(input_ids=ids, loss_mask=[0] * (len(ids) - 6) + [1] * 6,
                          multi_modal_input=[dict(pixel_values=pix, image_grid_thw=torch.tensor([grid]))]))
    return items


def test_engine_trains_on_images(tmp_path):
    """SFT through the trainer: micro-batches keep each sequence's images, the loss falls, the tower gets
    gradients, and the engine's logprobs equal a direct model call."""
    from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, SFTConfig, TrainEngineConfig, _propagate_names
    from areal_b200.trainer.sl_trainer import SFTTrainer, collate_sft

    data = _vl_items()
    cfg = SFTConfig(actor=TrainEngineConfig(
        backend="fsdp:d1", model_preset="tiny-qwen2_5-vl", init_from_scratch=True, dtype="float32",
        optimizer=OptimizerConfig(lr=2e-3, warmup_steps_proportion=0.0, weight_decay=0.0),
        mb_spec=MicroBatchSpec(max_tokens_per_mb=40)))  # several micro-batches per step
    cfg.experiment_name, cfg.trial_name = "t", "t"
    cfg.cluster.fileroot = str(tmp_path)
    cfg.train_dataset.batch_size = 6
    cfg.train_dataset.shuffle = False
    cfg.total_train_epochs = 6
    _propagate_names(cfg)
    losses = []
    with SFTTrainer(cfg, data, data) as tr:
        eng = tr.engine
        assert isinstance(eng.model, QwenVLModel)
        batch = collate_sft(data)
        assert len(batch["multi_modal_input"]) == 6 and batch["multi_modal_input"][2] == {}
        w0 = eng.model.visual.patch_embed.detach().clone()
        logp = eng.forward(batch)  # [B, L] padded next-token logprobs
        ids, pix = data[1]["input_ids"], data[1]["multi_modal_input"][0]
        meta = VarlenMeta(torch.tensor([0, len(ids)], dtype=torch.int32), "cpu")
        with torch.no_grad():
            h = eng.model(torch.tensor(ids), torch.arange(len(ids)), meta, pixel_values=pix["pixel_values"],
                          image_grid_thw=pix["image_grid_thw"])
            ref = torch.log_softmax(eng.model.logits(h), -1)[:-1].gather(1, torch.tensor(ids)[1:, None])[:, 0]
        assert torch.allclose(logp[1, :len(ids) - 1], ref, atol=1e-4)
        tr.train(max_steps=6, step_callback=lambda s, st: losses.append(st["step/loss"]))
        assert losses[-1] < losses[0]
        assert not torch.equal(eng.model.visual.patch_embed, w0), "the vision tower must train"
