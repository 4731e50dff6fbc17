"""Parity with the Hugging Face implementations: a randomly initialised tiny model of every family is
exported with ``save_hf_checkpoint``, loaded by ``transformers`` from that directory, and both must give
the same logits. This checks the exported config, the tensor naming / fusion layout and the numerics
of the model code at once."""
import dataclasses

import pytest
import torch

from areal_b200.models.config import PRESETS, ModelConfig
from areal_b200.models.qwen import build_model
from areal_b200.ops.attention import VarlenMeta
from areal_b200.utils.hf_io import load_hf_weights, save_hf_checkpoint

transformers = pytest.importorskip("transformers")


def _logits(model, ids):
    L = ids.numel()
    meta = VarlenMeta(torch.tensor([0, L], dtype=torch.int32), "cpu")
    with torch.no_grad():
        return model.logits(model(ids, torch.arange(L), meta))


def _roundtrip(cfg: ModelConfig, tmp_path, atol=2e-4):
    torch.manual_seed(0)
    m = build_model(cfg, dtype=torch.float32, seed=1)
    with torch.no_grad():  # non-trivial norm weights and biases
        for n, p in m.named_parameters():
            if n.endswith("norm") or "_norm" in n or n.endswith("bias"):
                p.add_(torch.randn_like(p) * 0.1)
    save_hf_checkpoint(m, cfg, str(tmp_path))
    hf = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path), torch_dtype=torch.float32)
    hf.eval()
    ids = torch.randint(0, cfg.vocab_size, (37,), generator=torch.Generator().manual_seed(2))
    mine = _logits(m, ids)
    with torch.no_grad():
        theirs = hf(input_ids=ids[None]).logits[0]
    err = float((mine - theirs).abs().max())
    assert err < atol, f"max logit difference {err}"
    # and back: a model built from the exported config loads the same weights
    m2 = build_model(ModelConfig.from_hf_config(str(tmp_path)), dtype=torch.float32, seed=None)
    load_hf_weights(m2, str(tmp_path))
    assert torch.allclose(_logits(m2, ids), mine, atol=1e-5)
    return hf


def test_qwen2_matches_transformers(tmp_path):
    _roundtrip(PRESETS["tiny-qwen2"], tmp_path)


def test_qwen3_matches_transformers(tmp_path):
    cfg = dataclasses.replace(PRESETS["tiny-qwen2"], model_type="qwen3", attention_bias=False, qk_norm=True,
                              tie_word_embeddings=True, head_dim=32)
    _roundtrip(cfg, tmp_path)


def test_qwen3_moe_matches_transformers(tmp_path):
    _roundtrip(PRESETS["tiny-qwen3-moe"], tmp_path)


def test_qwen3_5_hybrid_matches_transformers(tmp_path):
    """GatedDeltaNet + gated attention, partial rotary embedding, 1-centred norms against transformers'
    Qwen3.5 text model (its PyTorch fallback of the gated delta rule)."""
    pytest.importorskip("transformers.models.qwen3_5")
    _roundtrip(PRESETS["tiny-qwen3_5"], tmp_path, atol=5e-4)


def test_qwen3_5_moe_matches_transformers(tmp_path):
    """Hybrid layers + routed experts + sigmoid-gated shared expert against transformers' Qwen3.5-MoE."""
    pytest.importorskip("transformers.models.qwen3_5_moe")
    cfg = dataclasses.replace(PRESETS["tiny-qwen3_5"], num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64,
                              shared_expert_intermediate_size=96, norm_topk_prob=True)
    _roundtrip(cfg, tmp_path, atol=5e-4)


def test_critic_matches_transformers_token_classification(tmp_path):
    """A critic / reward model (scalar head) exports to what `AutoModelForTokenClassification(num_labels=1)` reads."""
    cfg = dataclasses.replace(PRESETS["tiny-qwen2"], is_critic=True, tie_word_embeddings=False)
    m = build_model(cfg, dtype=torch.float32, seed=4)
    save_hf_checkpoint(m, cfg, str(tmp_path))
    hf = transformers.AutoModelForTokenClassification.from_pretrained(str(tmp_path), num_labels=1, torch_dtype=torch.float32)
    hf.eval()
    ids = torch.randint(0, cfg.vocab_size, (29,), generator=torch.Generator().manual_seed(5))
    meta = VarlenMeta(torch.tensor([0, 29], dtype=torch.int32), "cpu")
    with torch.no_grad():
        mine = m.values(m(ids, torch.arange(29), meta))
        theirs = hf(input_ids=ids[None]).logits[0, :, 0]
    assert float((mine - theirs).abs().max()) < 2e-4


def test_block_quantised_fp8_checkpoint_is_dequantised_on_load(tmp_path):
    """A checkpoint whose linear weights are float8_e4m3 with one fp32 ``weight_scale_inv`` per 128 x 128 tile
    (split over two files) loads as bf16 within the quantisation error."""
    import json

    import torch
    from safetensors.torch import save_file

    from areal_b200.utils.hf_io import dequant_fp8_blockwise, iter_hf_tensors

    torch.manual_seed(0)
    w = torch.randn(300, 260) * 0.05
    nb0, nb1 = 3, 3
    pad = torch.zeros(nb0 * 128, nb1 * 128)
    pad[:300, :260] = w
    amax = pad.view(nb0, 128, nb1, 128).abs().amax(dim=(1, 3)).clamp(min=1e-8)
    scale_inv = amax / 448.0
    q = (pad / scale_inv.repeat_interleave(128, 0).repeat_interleave(128, 1))[:300, :260].to(torch.float8_e4m3fn)
    norm = torch.ones(260, dtype=torch.bfloat16)
    save_file({"model.layers.0.mlp.down_proj.weight": q, "model.norm.weight": norm}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({"model.layers.0.mlp.down_proj.weight_scale_inv": scale_inv}, str(tmp_path / "model-00002-of-00002.safetensors"))
    json.dump({"quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128]}}, open(tmp_path / "config.json", "w"))
    got = dict(iter_hf_tensors(str(tmp_path)))
    assert set(got) == {"model.layers.0.mlp.down_proj.weight", "model.norm.weight"}
    d = got["model.layers.0.mlp.down_proj.weight"]
    assert d.dtype == torch.bfloat16 and d.shape == (300, 260)
    assert (d.float() - w).abs().max() < 0.07 * w.abs().max()
    assert torch.equal(d, dequant_fp8_blockwise(q, scale_inv))


def test_llama_matches_transformers(tmp_path):
    cfg = dataclasses.replace(PRESETS["tiny-qwen2"], model_type="llama", attention_bias=False, qk_norm=False,
                              tie_word_embeddings=False)
    hf = _roundtrip(cfg, tmp_path)
    assert type(hf).__name__ == "LlamaForCausalLM"


def test_mistral_matches_transformers(tmp_path):
    cfg = dataclasses.replace(PRESETS["tiny-qwen2"], model_type="mistral", attention_bias=False, qk_norm=False,
                              tie_word_embeddings=False)
    hf = _roundtrip(cfg, tmp_path)
    assert type(hf).__name__ == "MistralForCausalLM"


@pytest.mark.parametrize("scaling", [
    {"rope_type": "linear", "factor": 4.0},
    {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
     "original_max_position_embeddings": 16},
    {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 16},
])
def test_rope_scaling_matches_transformers(tmp_path, scaling):
    cfg = dataclasses.replace(PRESETS["tiny-qwen2"], model_type="llama", attention_bias=False, qk_norm=False,
                              tie_word_embeddings=False, rope_scaling=scaling, max_position_embeddings=64)
    _roundtrip(cfg, tmp_path)
    assert ModelConfig.from_hf_config(str(tmp_path)).rope_scaling["rope_type"] == scaling["rope_type"]


def test_unknown_model_type_and_scaling_are_rejected():
    base = PRESETS["tiny-qwen2"].to_hf_config()
    with pytest.raises(NotImplementedError):
        ModelConfig.from_hf_config(dict(base, model_type="gpt2"))
    with pytest.raises(NotImplementedError):
        ModelConfig.from_hf_config(dict(base, rope_scaling={"rope_type": "longrope", "factor": 2.0}))


def test_qwen2_moe_matches_transformers(tmp_path):
    """Shared expert behind a sigmoid gate, top-k probabilities not renormalised, bias on q/k/v."""
    cfg = dataclasses.replace(PRESETS["tiny-qwen3-moe"], model_type="qwen2_moe", qk_norm=False, attention_bias=True,
                              norm_topk_prob=False, shared_expert_intermediate_size=96)
    hf = _roundtrip(cfg, tmp_path)
    assert type(hf).__name__ == "Qwen2MoeForCausalLM"
    back = ModelConfig.from_hf_config(str(tmp_path))
    assert (back.shared_expert_intermediate_size, back.norm_topk_prob, back.attention_bias) == (96, False, True)


def test_mixtral_matches_transformers_and_uses_its_checkpoint_names(tmp_path):
    cfg = dataclasses.replace(PRESETS["tiny-qwen3-moe"], model_type="mixtral", qk_norm=False, attention_bias=False,
                              norm_topk_prob=True, intermediate_size=128, moe_intermediate_size=128)
    hf = _roundtrip(cfg, tmp_path)
    assert type(hf).__name__ == "MixtralForCausalLM"
    from safetensors import safe_open

    import glob as _glob

    names = set()
    for f in _glob.glob(str(tmp_path / "*.safetensors")):
        with safe_open(f, "pt") as sf:
            names |= set(sf.keys())
    assert "model.layers.0.block_sparse_moe.gate.weight" in names
    assert "model.layers.1.block_sparse_moe.experts.7.w3.weight" in names
    assert not any(".mlp." in n for n in names)
    back = ModelConfig.from_hf_config(str(tmp_path))
    assert back.num_experts == 8 and back.moe_intermediate_size == 128 and back.is_moe


def test_deepseek_v3_matches_transformers(tmp_path):
    """Latent attention (low-rank query and key / value paths, a rotary part beside a position-free part, rotary
    pairs interleaved in the checkpoint), a dense first layer, then mixtures with sigmoid scores, group-limited
    routing, the checkpoint's selection bias, a scale on the routing weights and an ungated shared expert."""
    cfg = PRESETS["tiny-deepseek-v3"]
    torch.manual_seed(0)
    m = build_model(cfg, dtype=torch.float32, seed=1)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("norm") or "_norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
        for layer in m.layers:   # a bias large enough to change which experts win
            if getattr(layer.mlp, "expert_bias", None) is not None:
                layer.mlp.expert_bias.copy_(torch.randn(cfg.num_experts) * 0.2)
    save_hf_checkpoint(m, cfg, str(tmp_path))
    hf = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path), torch_dtype=torch.float32).eval()
    assert type(hf).__name__ == "DeepseekV3ForCausalLM"
    ids = torch.randint(0, cfg.vocab_size, (41,), generator=torch.Generator().manual_seed(2))
    mine = _logits(m, ids)
    with torch.no_grad():
        theirs = hf(input_ids=ids[None]).logits[0]
    assert float((mine - theirs).abs().max()) < 2e-4
    back = ModelConfig.from_hf_config(str(tmp_path))
    assert back.is_mla and (back.q_lora_rank, back.kv_lora_rank, back.qk_nope_head_dim, back.qk_rope_head_dim,
                            back.v_head_dim) == (96, 64, 32, 16, 32)
    assert (back.moe_n_group, back.moe_topk_group, back.moe_route_scale, back.mlp_only_layers,
            back.shared_expert_gated, back.moe_expert_bias) == (4, 2, 2.5, [0], False, True)
    m2 = build_model(back, dtype=torch.float32, seed=None)
    load_hf_weights(m2, str(tmp_path))
    assert torch.allclose(_logits(m2, ids), mine, atol=1e-5)
    assert torch.equal(m2.layers[1].mlp.expert_bias, m.layers[1].mlp.expert_bias)


def test_deepseek_v3_without_query_bottleneck_and_with_yarn(tmp_path):
    """``q_lora_rank`` absent (the Lite models' plain query projection), rotary pairs not interleaved, and a YaRN
    table whose magnitude factor enters the softmax scale."""
    cfg = dataclasses.replace(PRESETS["tiny-deepseek-v3"], q_lora_rank=0, rope_interleave=False,
                              max_position_embeddings=256,
                              rope_scaling={"rope_type": "yarn", "factor": 4.0, "beta_fast": 32, "beta_slow": 1,
                                            "mscale": 1.0, "mscale_all_dim": 0.7,
                                            "original_max_position_embeddings": 64})
    hf = _roundtrip(cfg, tmp_path)
    assert type(hf).__name__ == "DeepseekV3ForCausalLM" and not hasattr(hf.model.layers[0].self_attn, "q_a_proj")


def test_deepseek_v2_matches_transformers(tmp_path):
    """The V2 generation of the family: softmax scores that are scaled but not renormalised, no selection bias;
    V2-Lite's plain query projection."""
    cfg = dataclasses.replace(PRESETS["tiny-deepseek-v3"], model_type="deepseek_v2", moe_score_func="softmax",
                              moe_expert_bias=False, moe_group_score_top=1, norm_topk_prob=False, q_lora_rank=0,
                              moe_n_group=1, moe_topk_group=1)
    hf = _roundtrip(cfg, tmp_path)
    assert type(hf).__name__ == "DeepseekV2ForCausalLM"
    back = ModelConfig.from_hf_config(str(tmp_path))
    assert dataclasses.asdict(back) == dataclasses.asdict(cfg)
    assert PRESETS["deepseek-v2-lite"].num_params() / 1e9 == pytest.approx(15.7, abs=0.2)


def test_deepseek_v2_group_limited_routing_rule():
    """``group_limited_greedy`` (the larger V2 models): a group is scored by its best expert, tokens pick among the
    experts of their best groups, weights are the plain softmax scores times the scale. (Checked against the rule
    itself: the ``transformers`` class cannot run this branch, it reads an attribute it never sets.)"""
    from areal_b200.models.qwen import MoEMLP

    cfg = dataclasses.replace(PRESETS["tiny-deepseek-v3"], model_type="deepseek_v2", moe_score_func="softmax",
                              moe_expert_bias=False, moe_group_score_top=1, norm_topk_prob=False, moe_n_group=4,
                              moe_topk_group=2)
    back = ModelConfig.from_hf_config(cfg.to_hf_config())
    assert (back.moe_n_group, back.moe_topk_group, back.moe_group_score_top, back.moe_score_func) == (4, 2, 1, "softmax")
    torch.manual_seed(0)
    mlp = MoEMLP(cfg, torch.float32, "cpu").eval()
    torch.nn.init.normal_(mlp.router, std=0.5)
    x = torch.randn(50, cfg.hidden_size)
    with torch.no_grad():
        idx, w = mlp.route(x)
    p = torch.softmax(x @ mlp.router.T, -1)
    best_groups = p.view(50, 4, 2).max(-1).values.topk(2, -1).indices           # [50, 2]
    assert bool(((idx.long() // 2)[:, :, None] == best_groups[:, None, :]).any(-1).all())
    masked = p.view(50, 4, 2).masked_fill(~torch.zeros(50, 4, dtype=torch.bool).scatter_(1, best_groups, True)[..., None], 0.0)
    want = masked.view(50, 8).topk(cfg.num_experts_per_tok, -1)
    assert torch.equal(idx.long().sort(-1).values, want.indices.sort(-1).values)
    assert torch.allclose(w.sort(-1).values, (want.values * cfg.moe_route_scale).sort(-1).values, atol=1e-6)
