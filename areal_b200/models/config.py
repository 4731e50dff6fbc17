"""Architecture description shared by the train and rollout engines.

Covers the dense Qwen2 / Qwen2.5 / Qwen3 families and Qwen3-MoE, i.e. the model
registry of the reference's torch-native engine
(areal/experimental/models/archon/{qwen2,qwen3}/spec.py). The field names of
``from_hf_config`` follow the HF ``config.json`` of those checkpoints.
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path


@dataclass
class ModelConfig:
    model_type: str = "qwen3"  # qwen2 | qwen3 | qwen3_moe | qwen3_5 | llama | mistral | the vision-language types
    vocab_size: int = 151936
    hidden_size: int = 2048
    intermediate_size: int = 6144
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    # frequency scaling of the rotary table (HF `rope_scaling` / `rope_parameters`): rope_type default | linear |
    # llama3 | yarn with their parameters; empty = unscaled
    rope_scaling: dict = field(default_factory=dict)
    max_position_embeddings: int = 40960
    tie_word_embeddings: bool = True
    attention_bias: bool = False  # Qwen2: bias on q/k/v
    qk_norm: bool = True  # Qwen3: per-head RMSNorm on q and k
    # block-scaled fp8 forward GEMMs of the dense projections (bf16 master weights)
    fp8: bool = False
    fp8_ue8m0: bool = True
    # low-rank adapters on the dense projections (0 = off); targets are HF module names
    lora_rank: int = 0
    lora_alpha: float = 16.0
    lora_targets: list[str] = field(default_factory=list)
    # hybrid models (qwen3_5): per-layer "full_attention" | "linear_attention"; empty = all full attention
    layer_types: list[str] = field(default_factory=list)
    partial_rotary_factor: float = 1.0   # fraction of head_dim that carries rotary embedding
    attn_output_gate: bool = False       # q_proj emits query + sigmoid output gate per head
    norm_one_plus: bool = False          # checkpoints store RMSNorm weights 1-centred: (1 + w) * norm(x)
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    # MoE (qwen3_moe)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    # router variants (defaults = Qwen3-MoE): score function, scale on the routing weights, and aux-loss-free load
    # balancing (a per-expert bias that only affects WHICH experts are picked, nudged by `moe_load_balance_coeff`
    # towards the mean load after every training forward; 0 = off)
    moe_score_func: str = "softmax"  # softmax | sigmoid
    moe_route_scale: float = 1.0
    moe_load_balance_coeff: float = 0.0
    # shared expert that every token passes through, scaled by a sigmoid gate (Qwen2-MoE / Qwen3.5-MoE); 0 = none
    shared_expert_intermediate_size: int = 0
    shared_expert_gated: bool = True  # DeepSeek-V3: the shared experts' output is added as it is
    # group-limited routing (DeepSeek-V3): experts form `moe_n_group` groups, a token may only pick from its
    # `moe_topk_group` best groups (a group's score: the sum of its two best experts); `moe_expert_bias`: the
    # checkpoint carries the selection bias (`e_score_correction_bias`)
    moe_n_group: int = 1
    moe_topk_group: int = 1
    moe_expert_bias: bool = False
    # multi-head latent attention (DeepSeek-V3): queries and keys / values go through low-rank bottlenecks; a head's
    # query / key is a `qk_nope_head_dim` part without position plus a `qk_rope_head_dim` rotary part (the key's
    # rotary part is shared by all heads); `kv_lora_rank > 0` selects it, `q_lora_rank = 0` keeps a plain q projection
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    rope_interleave: bool = False  # rotary pairs are neighbours (2i, 2i + 1) in the checkpoint's q / k layout
    # Bailing hybrid: layers come in groups of `lightning_group_size`; all but the last of a group use lightning
    # (linear) attention with heads of `lightning_head_dim` and a gate norm over `lightning_norm_groups` groups of
    # heads, the last uses latent attention. 0 / 1 = no lightning layers
    lightning_group_size: int = 0
    lightning_head_dim: int = 128
    lightning_norm_groups: int = 1
    moe_group_score_top: int = 2  # a group's score: the sum of its this many best experts
    decoder_sparse_step: int = 1
    mlp_only_layers: list[int] = field(default_factory=list)
    # critic / reward model: scalar head instead of the LM head
    is_critic: bool = False
    # vision-language models (qwen2_5_vl): the vision tower's config (HF `vision_config` keys; empty = text-only),
    # the split of the rotary frequencies over the (temporal, height, width) position axes, and the placeholder ids
    vision: dict = field(default_factory=dict)
    mrope_section: list[int] = field(default_factory=list)
    mrope_interleaved: bool = False  # Qwen3-VL: the three axes alternate over the rotary frequencies
    image_token_id: int = -1
    video_token_id: int = -1
    vision_start_token_id: int = -1
    vision_end_token_id: int = -1

    @property
    def is_vl(self) -> bool:
        return bool(self.vision)

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def layer_is_moe(self, i: int) -> bool:
        return (self.is_moe and i not in self.mlp_only_layers
                and (i + 1) % max(self.decoder_sparse_step, 1) == 0)

    def layer_is_lightning(self, i: int) -> bool:
        g = self.lightning_group_size
        return g > 1 and (i + 1) % g != 0

    @property
    def has_recurrent_state(self) -> bool:
        """Some layers carry a per-sequence recurrent state through generation (linear-attention layers)."""
        return self.is_hybrid or self.lightning_group_size > 1

    def layer_type(self, i: int) -> str:
        if self.layer_is_lightning(i):
            return "lightning_attention"
        return self.layer_types[i] if self.layer_types else "full_attention"

    @property
    def is_hybrid(self) -> bool:
        return self.attn_output_gate or any(t == "linear_attention" for t in self.layer_types)

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    @property
    def rotary_dim(self) -> int:
        if self.is_mla:
            return self.qk_rope_head_dim
        return int(self.head_dim * self.partial_rotary_factor) // 2 * 2

    def attn_params(self, layer: int | None = None) -> int:
        h, nh = self.hidden_size, self.num_attention_heads
        if layer is not None and self.layer_is_lightning(layer):
            d = nh * self.lightning_head_dim
            return 5 * d * h + d + 2 * self.lightning_head_dim
        if self.is_mla:
            qk = self.qk_nope_head_dim + self.qk_rope_head_dim
            q = (h * self.q_lora_rank + self.q_lora_rank + self.q_lora_rank * nh * qk) if self.q_lora_rank \
                else h * nh * qk
            kv = h * (self.kv_lora_rank + self.qk_rope_head_dim) + self.kv_lora_rank \
                + self.kv_lora_rank * nh * (self.qk_nope_head_dim + self.v_head_dim)
            return q + kv + nh * self.v_head_dim * h
        return h * (self.q_size + 2 * self.kv_size) + self.q_size * h

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def num_params(self) -> int:
        h, L = self.hidden_size, self.num_hidden_layers
        attn = self.attn_params()
        if self.attention_bias:
            attn += self.q_size + 2 * self.kv_size
        if self.qk_norm:
            attn += 2 * self.head_dim
        dense_mlp = 3 * h * self.intermediate_size
        moe_mlp = self.num_experts * 3 * h * self.moe_intermediate_size + h * self.num_experts
        if self.shared_expert_intermediate_size:
            moe_mlp += 3 * h * self.shared_expert_intermediate_size + (h if self.shared_expert_gated else 0)
        n = 0
        for i in range(L):
            a = self.attn_params(i) if self.layer_is_lightning(i) else attn
            n += a + 2 * h + (moe_mlp if self.layer_is_moe(i) else dense_mlp)
        n += self.vocab_size * h + h
        if not self.tie_word_embeddings and not self.is_critic:
            n += self.vocab_size * h
        if self.is_critic:
            n += h
        return n + self.vision_params()

    def vision_params(self) -> int:
        """Parameters of the vision tower (0 for text models)."""
        v = self.vision
        if not v:
            return 0
        d, inter, unit = v["hidden_size"], v["intermediate_size"], v.get("spatial_merge_size", 2) ** 2
        kind = v.get("variant", "qwen2_5_vl")
        gated, ln = kind == "qwen2_5_vl", kind != "qwen2_5_vl"
        patch = v.get("in_channels", 3) * v.get("temporal_patch_size", 2) * v["patch_size"] ** 2
        block = 3 * d * d + 3 * d + d * d + d + (3 if gated else 2) * d * inter + (2 if gated else 1) * inter + d \
            + 2 * d * (2 if ln else 1)
        merger = d * (2 if ln else 1) + (d * unit) ** 2 + d * unit + d * unit * v["out_hidden_size"] + v["out_hidden_size"]
        n = d * patch + v["depth"] * block + merger
        if kind == "qwen3_vl":
            deep = 2 * d * unit + (d * unit) ** 2 + d * unit + d * unit * v["out_hidden_size"] + v["out_hidden_size"]
            n += d + v["num_position_embeddings"] * d + len(v.get("deepstack_visual_indexes", [])) * deep
        return n

    def flops_per_token(self, seq_len: int, backward: bool = True) -> float:
        """Model FLOPs per token for a sequence of ``seq_len`` (causal attention)."""
        h, L = self.hidden_size, self.num_hidden_layers
        lin = self.attn_params()
        act_mlp = (3 * h * self.moe_intermediate_size * self.num_experts_per_tok
                   if self.is_moe else 3 * h * self.intermediate_size)
        qk_v = (self.num_attention_heads * (self.qk_nope_head_dim + self.qk_rope_head_dim + self.v_head_dim) / 2
                if self.is_mla else self.q_size)
        per_layer = 2 * (lin + act_mlp) + 4 * qk_v * (seq_len / 2)
        total = L * per_layer + 2 * h * self.vocab_size
        return total * (3 if backward else 1)

    @classmethod
    def from_hf_config(cls, cfg: dict | str | Path, **overrides) -> "ModelConfig":
        if not isinstance(cfg, dict):
            p = Path(cfg)
            p = p / "config.json" if p.is_dir() else p
            cfg = json.loads(p.read_text())
        top = cfg
        if "text_config" in cfg:  # composite (vision-language) checkpoints nest the decoder's config
            cfg = cfg["text_config"]
        mt = cfg.get("model_type", "qwen3")
        if mt in ("bailing_moe_linear", "bailing_hybrid"):
            mt = "bailing_hybrid"
        if top.get("model_type") in _VL_TYPES:
            mt = top["model_type"]
        if mt.startswith("qwen3_5"):
            mt = "qwen3_5"
        heads = cfg["num_attention_heads"]
        rope_params = cfg.get("rope_parameters") or {}
        if mt not in _TEXT_TYPES and mt not in _VL_TYPES:
            raise NotImplementedError(f"model_type {mt!r}: supported are {sorted(_TEXT_TYPES | set(_VL_TYPES))}")
        if cfg.get("mlp_bias"):
            raise NotImplementedError("bias on the MLP projections is not supported")
        window = cfg.get("sliding_window") if cfg.get("use_sliding_window", mt == "mistral") else None
        if window and window < cfg.get("max_position_embeddings", 0):
            import warnings

            warnings.warn(f"sliding-window attention is not implemented: sequences longer than the window "
                          f"({window} tokens) attend to their whole prefix", stacklevel=2)
        scaling = dict(cfg.get("rope_scaling") or {})
        if not scaling and rope_params.get("rope_type", "default") != "default":
            scaling = {k: v for k, v in rope_params.items() if k not in ("rope_theta", "partial_rotary_factor",
                                                                         "mrope_section", "mrope_interleaved")}
        if "type" in scaling and "rope_type" not in scaling:
            scaling["rope_type"] = scaling.pop("type")
        if scaling.get("rope_type") in (None, "default", "mrope"):
            scaling = {}
        elif scaling["rope_type"] not in ("linear", "llama3", "yarn"):
            raise NotImplementedError(f"rope scaling {scaling['rope_type']!r} is not supported")
        out = cls(
            model_type=mt,
            vocab_size=cfg["vocab_size"],
            hidden_size=cfg["hidden_size"],
            intermediate_size=cfg.get("intermediate_size", 0),
            num_hidden_layers=cfg["num_hidden_layers"],
            num_attention_heads=heads,
            num_key_value_heads=cfg.get("num_key_value_heads", heads),
            head_dim=cfg.get("head_dim") or cfg["hidden_size"] // heads,
            rms_norm_eps=cfg.get("rms_norm_eps", 1e-6),
            rope_theta=cfg.get("rope_theta") or rope_params.get("rope_theta", 1e4),
            rope_scaling=scaling,
            max_position_embeddings=cfg.get("max_position_embeddings", 32768),
            tie_word_embeddings=cfg.get("tie_word_embeddings", False),
            attention_bias=cfg.get("attention_bias", mt in ("qwen2", "qwen2_moe", "qwen2_5_vl", "qwen2_vl")),
            qk_norm=mt.startswith("qwen3"),
            num_experts=cfg.get("num_experts", 0) or cfg.get("num_local_experts", 0)
            or cfg.get("n_routed_experts", 0) or 0,
            num_experts_per_tok=cfg.get("num_experts_per_tok", 0) or 0,
            moe_intermediate_size=cfg.get("moe_intermediate_size", 0) or 0,
            norm_topk_prob=cfg.get("norm_topk_prob", mt != "qwen2_moe"),
            shared_expert_intermediate_size=cfg.get("shared_expert_intermediate_size", 0) or 0,
            decoder_sparse_step=cfg.get("decoder_sparse_step", 1) or 1,
            mlp_only_layers=list(cfg.get("mlp_only_layers", []) or []),
        )
        if mt == "mixtral":  # every MLP is a mixture whose experts have the dense MLP's width
            out.moe_intermediate_size = out.intermediate_size
        if mt == "bailing_hybrid":
            if cfg.get("use_qkv_bias") or cfg.get("use_bias"):
                raise NotImplementedError("bias on the Bailing projections is not supported")
            out.qk_norm = False
            out.moe_score_func = cfg.get("scoring_func") or cfg.get("score_function") or "sigmoid"
            out.moe_expert_bias, out.shared_expert_gated = True, False
            out.moe_route_scale = float(cfg.get("routed_scaling_factor") or 1.0)
            out.moe_n_group, out.moe_topk_group = int(cfg.get("n_group") or 1), int(cfg.get("topk_group") or 1)
            out.moe_group_score_top = max(out.num_experts_per_tok // max(out.moe_topk_group, 1), 1)
            shared = cfg.get("moe_shared_expert_intermediate_size")
            out.shared_expert_intermediate_size = int(shared) if shared else \
                int(cfg.get("num_shared_experts") or 0) * (out.moe_intermediate_size or out.intermediate_size)
            out.mlp_only_layers = list(range(int(cfg.get("first_k_dense_replace") or 0)))
            out.q_lora_rank = int(cfg.get("q_lora_rank") or 0)
            out.kv_lora_rank = int(cfg.get("kv_lora_rank") or 512)
            out.qk_nope_head_dim = int(cfg.get("qk_nope_head_dim") or 128)
            out.qk_rope_head_dim = int(cfg.get("qk_rope_head_dim") or 64)
            out.v_head_dim = int(cfg.get("v_head_dim") or 128)
            out.rope_interleave = True
            out.lightning_group_size = int(cfg.get("layer_group_size") or 1)
            out.lightning_head_dim = int(cfg.get("attn_head_dim") or cfg.get("head_dim") or 256)
            out.head_dim = out.qk_nope_head_dim + out.qk_rope_head_dim
            out.partial_rotary_factor = float(cfg.get("partial_rotary_factor") or 0.5)
            out.lightning_norm_groups = int(cfg.get("linear_attn_norm_group_size") or cfg.get("group_norm_size") or 1)
        if mt in ("deepseek_v2", "deepseek_v3"):
            if cfg.get("attention_bias"):
                raise NotImplementedError("bias on the latent-attention projections is not supported")
            out.qk_norm = False
            out.shared_expert_gated = False
            if mt == "deepseek_v3":  # sigmoid scores, a selection bias, groups scored by their two best experts
                out.moe_score_func, out.moe_expert_bias = "sigmoid", True
                out.moe_n_group, out.moe_topk_group = int(cfg.get("n_group") or 1), int(cfg.get("topk_group") or 1)
            else:  # V2: softmax scores, never renormalised unless asked; groups (if any) scored by their best expert
                out.norm_topk_prob = bool(cfg.get("norm_topk_prob", False))
                out.moe_group_score_top = 1
                if cfg.get("topk_method", "greedy") == "group_limited_greedy":
                    out.moe_n_group, out.moe_topk_group = int(cfg.get("n_group") or 1), int(cfg.get("topk_group") or 1)
            out.moe_route_scale = float(cfg.get("routed_scaling_factor", 1.0))
            out.shared_expert_intermediate_size = int(cfg.get("n_shared_experts") or 0) * out.moe_intermediate_size
            out.mlp_only_layers = list(range(int(cfg.get("first_k_dense_replace") or 0)))
            out.q_lora_rank = int(cfg.get("q_lora_rank") or 0)
            for key in ("kv_lora_rank", "qk_nope_head_dim", "qk_rope_head_dim", "v_head_dim"):
                setattr(out, key, int(cfg[key]))
            out.head_dim = out.qk_nope_head_dim + out.qk_rope_head_dim
            out.rope_interleave = bool(cfg.get("rope_interleave", True))
        if mt == "qwen3_5":
            out.layer_types = list(cfg.get("layer_types") or [])
            out.partial_rotary_factor = (cfg.get("partial_rotary_factor")
                                         or rope_params.get("partial_rotary_factor", 0.25))
            out.attn_output_gate = out.norm_one_plus = True
            for key in ("linear_conv_kernel_dim", "linear_key_head_dim", "linear_value_head_dim",
                        "linear_num_key_heads", "linear_num_value_heads"):
                if key in cfg:
                    setattr(out, key, cfg[key])
        if mt in _VL_TYPES:
            vc = dict(top.get("vision_config") or {})
            if mt.startswith("qwen3_vl"):
                vc["variant"] = "qwen3_vl"
                out.mrope_interleaved = bool(rope_params.get("mrope_interleaved", True))
            if mt == "qwen2_vl":
                # Qwen2-VL names the tower width `embed_dim`, the merger's output `hidden_size` and the MLP by ratio
                vc = dict(vc, hidden_size=vc["embed_dim"], out_hidden_size=vc["hidden_size"],
                          intermediate_size=int(vc["embed_dim"] * vc.get("mlp_ratio", 4)), variant="qwen2_vl")
            out.vision = {k: v for k, v in vc.items() if k in _VISION_KEYS}
            rope_scaling = cfg.get("rope_scaling") or top.get("rope_scaling") or {}
            out.mrope_section = list(rope_params.get("mrope_section") or rope_scaling.get("mrope_section")
                                     or [out.head_dim // 8, 3 * out.head_dim // 16, 3 * out.head_dim // 16])
            out.tie_word_embeddings = top.get("tie_word_embeddings", out.tie_word_embeddings)
            for key in ("image_token_id", "video_token_id", "vision_start_token_id", "vision_end_token_id"):
                setattr(out, key, top.get(key, cfg.get(key, -1)))
        for k, v in overrides.items():
            setattr(out, k, v)
        return out

    def to_hf_config(self) -> dict:
        if self.is_vl:
            return self._to_hf_config_vl()
        arch = {"qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM",
                "qwen3_moe": "Qwen3MoeForCausalLM", "qwen3_5": "Qwen3_5ForCausalLM",
                "llama": "LlamaForCausalLM", "mistral": "MistralForCausalLM",
                "qwen2_moe": "Qwen2MoeForCausalLM", "mixtral": "MixtralForCausalLM",
                "deepseek_v3": "DeepseekV3ForCausalLM", "deepseek_v2": "DeepseekV2ForCausalLM", "bailing_hybrid": "BailingMoeV2_5ForCausalLM"}[self.model_type]
        if self.model_type == "qwen3_5" and self.is_moe:
            arch = "Qwen3_5MoeForCausalLM"
        d = {
            "architectures": [arch], "model_type": self.model_type,
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias, "hidden_act": "silu",
            "torch_dtype": "bfloat16",
        }
        if self.model_type in ("llama", "mistral", "mixtral"):
            d.update(mlp_bias=False, sliding_window=None)
        if self.model_type == "qwen2_moe":
            d.update(use_sliding_window=False, qkv_bias=self.attention_bias)
        if self.rope_scaling:
            d["rope_scaling"] = dict(self.rope_scaling)
            d["rope_parameters"] = dict(self.rope_scaling, rope_theta=self.rope_theta)
        if self.model_type == "qwen3_5":
            # transformers reads the text decoder as `qwen3_5_text` (`qwen3_5_moe_text` with experts), with the
            # rotary settings inside `rope_parameters`
            d["model_type"] = "qwen3_5_moe_text" if self.is_moe else "qwen3_5_text"
            d["rope_parameters"] = {"rope_type": "default", "rope_theta": self.rope_theta,
                                    "partial_rotary_factor": self.partial_rotary_factor}
            d.update(layer_types=self.layer_types, partial_rotary_factor=self.partial_rotary_factor,
                     linear_conv_kernel_dim=self.linear_conv_kernel_dim,
                     linear_key_head_dim=self.linear_key_head_dim, linear_value_head_dim=self.linear_value_head_dim,
                     linear_num_key_heads=self.linear_num_key_heads,
                     linear_num_value_heads=self.linear_num_value_heads)
        if self.is_moe:
            d.update(num_experts=self.num_experts, num_experts_per_tok=self.num_experts_per_tok,
                     moe_intermediate_size=self.moe_intermediate_size,
                     norm_topk_prob=self.norm_topk_prob,
                     shared_expert_intermediate_size=self.shared_expert_intermediate_size,
                     decoder_sparse_step=self.decoder_sparse_step,
                     mlp_only_layers=self.mlp_only_layers)
        if self.model_type in ("deepseek_v2", "deepseek_v3"):
            if self.model_type == "deepseek_v2":
                d["topk_method"] = "group_limited_greedy" if self.moe_n_group > 1 else "greedy"
            for key in ("num_experts", "shared_expert_intermediate_size", "decoder_sparse_step", "mlp_only_layers"):
                d.pop(key, None)
            d.update(n_routed_experts=self.num_experts, routed_scaling_factor=self.moe_route_scale,
                     n_shared_experts=self.shared_expert_intermediate_size // max(self.moe_intermediate_size, 1),
                     n_group=self.moe_n_group, topk_group=self.moe_topk_group,
                     first_k_dense_replace=len(self.mlp_only_layers), q_lora_rank=self.q_lora_rank or None,
                     kv_lora_rank=self.kv_lora_rank, qk_nope_head_dim=self.qk_nope_head_dim,
                     qk_rope_head_dim=self.qk_rope_head_dim, v_head_dim=self.v_head_dim,
                     head_dim=self.qk_rope_head_dim, rope_interleave=self.rope_interleave)
            if not self.rope_scaling:
                d["rope_parameters"] = {"rope_type": "default", "rope_theta": self.rope_theta}
        if self.model_type == "bailing_hybrid":
            for key in ("shared_expert_intermediate_size", "decoder_sparse_step", "mlp_only_layers", "head_dim"):
                d.pop(key, None)
            d.update(model_type="bailing_hybrid", scoring_func=self.moe_score_func,
                     routed_scaling_factor=self.moe_route_scale, n_group=self.moe_n_group,
                     topk_group=self.moe_topk_group,
                     moe_shared_expert_intermediate_size=self.shared_expert_intermediate_size,
                     first_k_dense_replace=len(self.mlp_only_layers), q_lora_rank=self.q_lora_rank or None,
                     kv_lora_rank=self.kv_lora_rank, qk_nope_head_dim=self.qk_nope_head_dim,
                     qk_rope_head_dim=self.qk_rope_head_dim, v_head_dim=self.v_head_dim,
                     layer_group_size=self.lightning_group_size, attn_head_dim=self.lightning_head_dim,
                     partial_rotary_factor=self.partial_rotary_factor,
                     linear_attn_norm_group_size=self.lightning_norm_groups)
        if self.model_type == "mixtral":
            d.update(num_local_experts=self.num_experts, intermediate_size=self.moe_intermediate_size,
                     router_jitter_noise=0.0)
        return d

    def _to_hf_config_vl(self) -> dict:
        v2 = self.model_type == "qwen2_vl"
        vision = dict(self.vision, model_type=self.model_type)
        vision.pop("variant", None)
        if v2:
            vision = {k: v for k, v in vision.items() if k not in ("intermediate_size", "out_hidden_size")}
            vision.update(embed_dim=self.vision["hidden_size"], hidden_size=self.vision["out_hidden_size"],
                          mlp_ratio=self.vision["intermediate_size"] // self.vision["hidden_size"],
                          hidden_act="quick_gelu")
        text = {
            "model_type": self.model_type + "_text", "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
            "rms_norm_eps": self.rms_norm_eps, "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings, "hidden_act": "silu", "rope_theta": self.rope_theta,
            "rope_parameters": {"rope_type": "default", "rope_theta": self.rope_theta,
                                "mrope_section": list(self.mrope_section)},
        }
        if self.model_type.startswith("qwen3_vl"):
            text.update(head_dim=self.head_dim, attention_bias=self.attention_bias)
            text["rope_parameters"]["mrope_interleaved"] = self.mrope_interleaved
        if self.is_moe:
            text.update(num_experts=self.num_experts, num_experts_per_tok=self.num_experts_per_tok,
                        moe_intermediate_size=self.moe_intermediate_size, norm_topk_prob=self.norm_topk_prob,
                        decoder_sparse_step=self.decoder_sparse_step, mlp_only_layers=self.mlp_only_layers)
        arch = {"qwen2_vl": "Qwen2VLForConditionalGeneration", "qwen3_vl": "Qwen3VLForConditionalGeneration",
                "qwen3_vl_moe": "Qwen3VLMoeForConditionalGeneration"}.get(
            self.model_type, "Qwen2_5_VLForConditionalGeneration")
        return {"architectures": [arch], "model_type": self.model_type,
                "text_config": text, "vision_config": vision,
                "image_token_id": self.image_token_id, "video_token_id": self.video_token_id,
                "vision_start_token_id": self.vision_start_token_id,
                "vision_end_token_id": self.vision_end_token_id,
                "tie_word_embeddings": self.tie_word_embeddings, "torch_dtype": "bfloat16"}

    def asdict(self) -> dict:
        return asdict(self)


_VISION_KEYS = ("depth", "hidden_size", "intermediate_size", "num_heads", "in_channels", "patch_size",
                "spatial_merge_size", "temporal_patch_size", "tokens_per_second", "window_size", "out_hidden_size",
                "fullatt_block_indexes", "hidden_act", "variant", "num_position_embeddings",
                "deepstack_visual_indexes")
_VL_TYPES = ("qwen2_5_vl", "qwen2_vl", "qwen3_vl", "qwen3_vl_moe")
_TEXT_TYPES = {"qwen2", "qwen3", "qwen3_moe", "qwen3_5", "llama", "mistral", "qwen2_moe", "mixtral", "deepseek_v2", "deepseek_v3", "bailing_hybrid"}

# Named shapes used by the benchmark configurations (random-init, synthetic data).
PRESETS: dict[str, ModelConfig] = {
    "tiny-qwen2": ModelConfig(model_type="qwen2", vocab_size=1024, hidden_size=256,
                              intermediate_size=688, num_hidden_layers=2, num_attention_heads=4,
                              num_key_value_heads=2, head_dim=64, rope_theta=1e4,
                              tie_word_embeddings=False, attention_bias=True, qk_norm=False),
    "tiny-qwen2-4l": ModelConfig(model_type="qwen2", vocab_size=1024, hidden_size=256,
                                 intermediate_size=688, num_hidden_layers=6, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=64, rope_theta=1e4,
                                 tie_word_embeddings=True, attention_bias=True, qk_norm=False),
    "tiny-qwen2_5-vl": ModelConfig(model_type="qwen2_5_vl", vocab_size=1024, hidden_size=256, intermediate_size=688,
                                   num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                                   rope_theta=1e4, tie_word_embeddings=False, attention_bias=True, qk_norm=False,
                                   mrope_section=[8, 12, 12], image_token_id=1000, video_token_id=1001,
                                   vision_start_token_id=1002, vision_end_token_id=1003,
                                   vision=dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=2,
                                               in_channels=3, patch_size=14, spatial_merge_size=2,
                                               temporal_patch_size=2, tokens_per_second=1, window_size=56,
                                               out_hidden_size=256, fullatt_block_indexes=[1], hidden_act="silu")),
    "tiny-qwen2-vl": ModelConfig(model_type="qwen2_vl", vocab_size=1024, hidden_size=256, intermediate_size=688,
                                 num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                                 rope_theta=1e4, tie_word_embeddings=False, attention_bias=True, qk_norm=False,
                                 mrope_section=[8, 12, 12], image_token_id=1000, video_token_id=1001,
                                 vision_start_token_id=1002, vision_end_token_id=1003,
                                 vision=dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=2,
                                             in_channels=3, patch_size=14, spatial_merge_size=2,
                                             temporal_patch_size=2, out_hidden_size=256, variant="qwen2_vl")),
    "tiny-qwen3-vl": ModelConfig(model_type="qwen3_vl", vocab_size=1024, hidden_size=256, intermediate_size=512,
                                 num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                                 rope_theta=1e4, tie_word_embeddings=False, attention_bias=False, qk_norm=True,
                                 mrope_section=[12, 10, 10], mrope_interleaved=True, image_token_id=1000,
                                 video_token_id=1001, vision_start_token_id=1002, vision_end_token_id=1003,
                                 vision=dict(depth=3, hidden_size=64, intermediate_size=128, num_heads=2,
                                             in_channels=3, patch_size=14, spatial_merge_size=2,
                                             temporal_patch_size=2, out_hidden_size=256, variant="qwen3_vl",
                                             num_position_embeddings=64, deepstack_visual_indexes=[0, 1],
                                             hidden_act="gelu_pytorch_tanh")),
    "tiny-qwen3-vl-moe": ModelConfig(model_type="qwen3_vl_moe", vocab_size=1024, hidden_size=256, intermediate_size=512,
                                     num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                                     rope_theta=1e4, tie_word_embeddings=False, attention_bias=False, qk_norm=True,
                                     num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64,
                                     mrope_section=[12, 10, 10], mrope_interleaved=True, image_token_id=1000,
                                     video_token_id=1001, vision_start_token_id=1002, vision_end_token_id=1003,
                                     vision=dict(depth=2, hidden_size=64, intermediate_size=128, num_heads=2,
                                                 in_channels=3, patch_size=14, spatial_merge_size=2,
                                                 temporal_patch_size=2, out_hidden_size=256, variant="qwen3_vl",
                                                 num_position_embeddings=64, deepstack_visual_indexes=[0],
                                                 hidden_act="gelu_pytorch_tanh")),
    "tiny-qwen3_5": ModelConfig(model_type="qwen3_5", vocab_size=1024, hidden_size=256, intermediate_size=512,
                                num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                                rope_theta=1e4, tie_word_embeddings=False, partial_rotary_factor=0.25,
                                attn_output_gate=True, norm_one_plus=True,
                                layer_types=["linear_attention", "linear_attention", "linear_attention",
                                             "full_attention"],
                                linear_key_head_dim=32, linear_value_head_dim=32, linear_num_key_heads=2,
                                linear_num_value_heads=4),
    "tiny-qwen3-moe": ModelConfig(model_type="qwen3_moe", vocab_size=1024, hidden_size=256, intermediate_size=512,
                                  num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                                  rope_theta=1e4, tie_word_embeddings=False, num_experts=8, num_experts_per_tok=2,
                                  moe_intermediate_size=128),
    "qwen3-1.7b": ModelConfig(model_type="qwen3", hidden_size=2048, intermediate_size=6144,
                              num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                              tie_word_embeddings=True),
    "qwen3-8b": ModelConfig(model_type="qwen3", hidden_size=4096, intermediate_size=12288,
                            num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                            tie_word_embeddings=False),
    "qwen2.5-7b": ModelConfig(model_type="qwen2", vocab_size=152064, hidden_size=3584,
                              intermediate_size=18944, num_hidden_layers=28,
                              num_attention_heads=28, num_key_value_heads=4, head_dim=128,
                              rope_theta=1e6, tie_word_embeddings=False, attention_bias=True,
                              qk_norm=False),
    "qwen3-30b-a3b": ModelConfig(model_type="qwen3_moe", hidden_size=2048, intermediate_size=6144,
                                 num_hidden_layers=48, num_attention_heads=32,
                                 num_key_value_heads=4, tie_word_embeddings=False,
                                 num_experts=128, num_experts_per_tok=8,
                                 moe_intermediate_size=768),
    "llama3.1-8b": ModelConfig(model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                               num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                               rms_norm_eps=1e-5, rope_theta=5e5, max_position_embeddings=131072,
                               tie_word_embeddings=False, qk_norm=False,
                               rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                             "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}),
    "mixtral-8x7b": ModelConfig(model_type="mixtral", vocab_size=32000, hidden_size=4096, intermediate_size=14336,
                                num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                                rms_norm_eps=1e-5, rope_theta=1e6, max_position_embeddings=32768,
                                tie_word_embeddings=False, qk_norm=False, num_experts=8, num_experts_per_tok=2,
                                moe_intermediate_size=14336),
    # DeepSeek-V3 architecture at test size: latent attention, one dense
    # layer, then mixtures with grouped sigmoid routing and an ungated shared expert
    "tiny-deepseek-v3": ModelConfig(model_type="deepseek_v3", vocab_size=1024, hidden_size=256, intermediate_size=512,
                                    num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4, head_dim=48,
                                    rope_theta=1e4, tie_word_embeddings=False, qk_norm=False, num_experts=8,
                                    num_experts_per_tok=2, moe_intermediate_size=64, moe_score_func="sigmoid",
                                    moe_route_scale=2.5, moe_n_group=4, moe_topk_group=2, moe_expert_bias=True,
                                    shared_expert_intermediate_size=64, shared_expert_gated=False,
                                    mlp_only_layers=[0], q_lora_rank=96, kv_lora_rank=64, qk_nope_head_dim=32,
                                    qk_rope_head_dim=16, v_head_dim=32, rope_interleave=True),
    # Bailing hybrid architecture at test size: groups of two layers (lightning attention, then latent attention)
    "tiny-bailing-hybrid": ModelConfig(model_type="bailing_hybrid", vocab_size=1024, hidden_size=256,
                                       intermediate_size=512, num_hidden_layers=4, num_attention_heads=4,
                                       num_key_value_heads=4, head_dim=48, rope_theta=1e4, tie_word_embeddings=False,
                                       qk_norm=False, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                                       moe_score_func="sigmoid", moe_route_scale=2.5, moe_n_group=4, moe_topk_group=2,
                                       moe_group_score_top=1, moe_expert_bias=True, shared_expert_intermediate_size=64,
                                       shared_expert_gated=False, mlp_only_layers=[0], q_lora_rank=96, kv_lora_rank=64,
                                       qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, rope_interleave=True,
                                       lightning_group_size=2, lightning_head_dim=32, lightning_norm_groups=2,
                                       partial_rotary_factor=0.5, max_position_embeddings=32768),
    # DeepSeek-V2-Lite: latent attention without the query bottleneck, softmax routing, two shared experts
    "deepseek-v2-lite": ModelConfig(model_type="deepseek_v2", vocab_size=102400, hidden_size=2048,
                                    intermediate_size=10944, num_hidden_layers=27, num_attention_heads=16,
                                    num_key_value_heads=16, head_dim=192, rope_theta=1e4,
                                    max_position_embeddings=163840, tie_word_embeddings=False, qk_norm=False,
                                    num_experts=64, num_experts_per_tok=6, moe_intermediate_size=1408,
                                    norm_topk_prob=False, moe_group_score_top=1, shared_expert_intermediate_size=2816,
                                    shared_expert_gated=False, mlp_only_layers=[0], kv_lora_rank=512,
                                    qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, rope_interleave=True,
                                    rope_scaling={"rope_type": "yarn", "factor": 40.0, "beta_fast": 32, "beta_slow": 1,
                                                  "mscale": 0.707, "mscale_all_dim": 0.707,
                                                  "original_max_position_embeddings": 4096}),
    "deepseek-v3": ModelConfig(model_type="deepseek_v3", vocab_size=129280, hidden_size=7168, intermediate_size=18432,
                               num_hidden_layers=61, num_attention_heads=128, num_key_value_heads=128, head_dim=192,
                               rope_theta=1e4, max_position_embeddings=163840, tie_word_embeddings=False,
                               qk_norm=False, num_experts=256, num_experts_per_tok=8, moe_intermediate_size=2048,
                               moe_score_func="sigmoid", moe_route_scale=2.5, moe_n_group=8, moe_topk_group=4,
                               moe_expert_bias=True, shared_expert_intermediate_size=2048, shared_expert_gated=False,
                               mlp_only_layers=[0, 1, 2], q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
                               qk_rope_head_dim=64, v_head_dim=128, rope_interleave=True,
                               rope_scaling={"rope_type": "yarn", "factor": 40.0, "beta_fast": 32, "beta_slow": 1,
                                             "mscale": 1.0, "mscale_all_dim": 1.0,
                                             "original_max_position_embeddings": 4096}),
    "mistral-7b": ModelConfig(model_type="mistral", vocab_size=32768, hidden_size=4096, intermediate_size=14336,
                              num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                              rms_norm_eps=1e-5, rope_theta=1e6, max_position_embeddings=32768,
                              tie_word_embeddings=False, qk_norm=False),
}
