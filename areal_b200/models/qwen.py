"""Qwen2 / Qwen2.5 / Qwen3 (dense and MoE) decoder on this library's kernels.

The module owns no HF modeling code. Projections are stored fused (``qkv``,
``gate_up``) so each transformer block is four GEMMs, and every other op is one
of the fused kernels in ``areal_b200.ops`` (RMSNorm+residual, q/k-norm+RoPE,
varlen attention, SwiGLU). On CPU the same ops run their PyTorch reference, so
this file is also the oracle model of the tests.

Inputs are packed: ``input_ids [T]``, ``position_ids [T]`` and a ``VarlenMeta``
built from ``cu_seqlens``. Architecture facts follow the reference's model code
(areal/experimental/models/archon/qwen2/model/model.py:72-83,208;
qwen3/model/model.py:75-101,103-274): pre-norm blocks, GQA, bias on q/k/v only
for Qwen2, per-head q/k RMSNorm before RoPE for Qwen3, ``w2(silu(w1 x) * w3 x)``.
HF checkpoint names are the interchange format (``to_hf`` / ``from_hf``).
"""

from __future__ import annotations

import math
from typing import Iterable, Iterator

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import fused
from ..ops.attention import VarlenMeta, varlen_attention
from ..ops.gemm import gemm, linear
from ..ops.rollout_ops import kv_cache_write, paged_decode
from .config import ModelConfig


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        h = cfg.hidden_size
        self.qkv = nn.Parameter(torch.empty(cfg.q_size + 2 * cfg.kv_size, h, dtype=dtype, device=device))
        self.qkv_bias = (nn.Parameter(torch.zeros(cfg.q_size + 2 * cfg.kv_size, dtype=dtype, device=device))
                         if cfg.attention_bias else None)
        self.o = nn.Parameter(torch.empty(h, cfg.q_size, dtype=dtype, device=device))
        if cfg.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(cfg.head_dim, dtype=dtype, device=device))
            self.k_norm = nn.Parameter(torch.ones(cfg.head_dim, dtype=dtype, device=device))
        else:
            self.q_norm = self.k_norm = None

    def project_qkv(self, x, cos, sin, pos):
        cfg = self.cfg
        qkv = linear(x, self.qkv, self.qkv_bias)
        return fused.qknorm_rope(qkv, self.q_norm, self.k_norm, cos, sin, pos,
                                 cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                                 cfg.rms_norm_eps)

    def forward(self, x, cos, sin, pos, meta: VarlenMeta, attn_fn=None):
        q, k, v = self.project_qkv(x, cos, sin, pos)
        a = (attn_fn or varlen_attention)(q, k, v, meta)
        return linear(a.reshape(a.shape[0], -1), self.o)


class DenseMLP(nn.Module):
    def __init__(self, hidden, inter, dtype, device):
        super().__init__()
        self.gate_up = nn.Parameter(torch.empty(2 * inter, hidden, dtype=dtype, device=device))
        self.down = nn.Parameter(torch.empty(hidden, inter, dtype=dtype, device=device))

    def forward(self, x):
        return linear(fused.swiglu(linear(x, self.gate_up)), self.down)


class MoEMLP(nn.Module):
    """Top-k routed experts (softmax router in fp32, optional top-k prob
    renormalisation), as in Qwen3-MoE. Expert weights are 3-D parameters
    ``gate_up [E, 2I, H]`` and ``down [E, H, I]``."""

    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        E, I, H = cfg.num_experts, cfg.moe_intermediate_size, cfg.hidden_size
        self.router = nn.Parameter(torch.empty(E, H, dtype=dtype, device=device))
        self.gate_up = nn.Parameter(torch.empty(E, 2 * I, H, dtype=dtype, device=device))
        self.down = nn.Parameter(torch.empty(E, H, I, dtype=dtype, device=device))
        self.last_routing = None  # (topk_idx, topk_w) of the last forward, for stats / replay

    def route(self, x):
        cfg = self.cfg
        logits = F.linear(x.float(), self.router.float())
        probs = logits.softmax(-1)
        w, idx = probs.topk(cfg.num_experts_per_tok, dim=-1)
        if cfg.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        return idx, w

    def forward(self, x):
        from ..ops.moe import moe_experts_forward

        idx, w = self.route(x)
        self.last_routing = (idx.detach(), w.detach())
        return moe_experts_forward(x, idx, w, self.gate_up, self.down)


class Block(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device):
        super().__init__()
        h = cfg.hidden_size
        self.input_norm = nn.Parameter(torch.ones(h, dtype=dtype, device=device))
        self.attn = Attention(cfg, dtype, device)
        self.post_norm = nn.Parameter(torch.ones(h, dtype=dtype, device=device))
        self.mlp = (MoEMLP(cfg, dtype, device) if cfg.layer_is_moe(layer_idx)
                    else DenseMLP(h, cfg.intermediate_size, dtype, device))
        self.eps = cfg.rms_norm_eps

    def forward(self, x, res, cos, sin, pos, meta, attn_fn=None):
        if res is None:
            y, res = fused.rmsnorm(x, self.input_norm, self.eps), x
        else:
            y, res = fused.rmsnorm(x, self.input_norm, self.eps, residual=res)
        a = self.attn(y, cos, sin, pos, meta, attn_fn)
        y, res = fused.rmsnorm(a, self.post_norm, self.eps, residual=res)
        return self.mlp(y), res


class QwenModel(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device))
        self.layers = nn.ModuleList(Block(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers))
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
        if cfg.is_critic:
            self.score = nn.Parameter(torch.empty(1, cfg.hidden_size, dtype=dtype, device=device))
            self.lm_head = None
        else:
            self.score = None
            self.lm_head = (None if cfg.tie_word_embeddings else
                            nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)))
        self._rope = None

    # ------------------------------------------------------------------ init
    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator(device="cpu").manual_seed(seed)
        dev_gen = None
        for name, p in self.named_parameters():
            if name.endswith("norm") or "_norm" in name:
                p.fill_(1.0)
            elif name.endswith("bias"):
                p.zero_()
            elif p.is_cuda:
                # large models: draw on the device (same seed ⇒ same values on every rank)
                if dev_gen is None:
                    dev_gen = torch.Generator(device=p.device).manual_seed(seed)
                p.normal_(0.0, std, generator=dev_gen)
            else:
                # generated on the host in fp32 so that every dtype sees the same values
                chunk = 1 << 24
                flat = p.view(-1)
                for s in range(0, flat.numel(), chunk):
                    n = min(chunk, flat.numel() - s)
                    flat[s:s + n].copy_(torch.empty(n, dtype=torch.float32).normal_(0.0, std, generator=g))
        return self

    def output_weight(self) -> torch.Tensor:
        return self.embed if self.lm_head is None else self.lm_head

    def rope(self, device, max_pos=None):
        max_pos = max_pos or self.cfg.max_position_embeddings
        if self._rope is None or self._rope[0].device != torch.device(device) or self._rope[0].shape[0] < max_pos:
            self._rope = fused.rope_tables(max_pos, self.cfg.head_dim, self.cfg.rope_theta, device)
        return self._rope

    # --------------------------------------------------------------- forward
    def forward(self, input_ids, position_ids, meta: VarlenMeta, attn_fn=None):
        """Packed forward; returns the final-normed hidden states ``[T, H]``."""
        cos, sin = self.rope(input_ids.device)
        pos = position_ids.to(torch.int32)
        x = fused.embedding(input_ids, self.embed)
        res = None
        for layer in self.layers:
            x, res = layer(x, res, cos, sin, pos, meta, attn_fn)
        y, _ = fused.rmsnorm(x, self.norm, self.cfg.rms_norm_eps, residual=res)
        return y

    def logits(self, hidden, out_dtype=torch.float32):
        w = self.output_weight()
        if hidden.is_cuda and hidden.dtype == torch.bfloat16:
            return gemm(hidden, w, out_dtype=out_dtype)
        return F.linear(hidden, w).to(out_dtype)

    def values(self, hidden):
        return F.linear(hidden.float(), self.score.float()).squeeze(-1)

    # -------------------------------------------------- rollout (paged cache)
    @torch.no_grad()
    def prefill(self, input_ids, position_ids, meta: VarlenMeta, kv_caches, slot_mapping):
        """Packed prompt forward that also writes K/V of every layer into the
        paged caches; returns hidden states of all tokens."""
        cos, sin = self.rope(input_ids.device)
        pos = position_ids.to(torch.int32)
        x = F.embedding(input_ids.long(), self.embed)
        res = None
        for i, layer in enumerate(self.layers):
            if res is None:
                y, res = fused.rmsnorm(x, layer.input_norm, layer.eps), x
            else:
                y, res = fused.rmsnorm(x, layer.input_norm, layer.eps, residual=res)
            q, k, v = layer.attn.project_qkv(y, cos, sin, pos)
            kv_cache_write(k, v, slot_mapping, kv_caches[i][0], kv_caches[i][1])
            a = varlen_attention(q, k, v, meta)
            a = linear(a.reshape(a.shape[0], -1), layer.attn.o)
            y, res = fused.rmsnorm(a, layer.post_norm, layer.eps, residual=res)
            x = layer.mlp(y)
        y, _ = fused.rmsnorm(x, self.norm, self.cfg.rms_norm_eps, residual=res)
        return y

    @torch.no_grad()
    def decode(self, input_ids, position_ids, kv_caches, block_table, seq_lens, slot_mapping,
               max_seq_len=None):
        """One new token per sequence: ``input_ids [B]`` at ``position_ids [B]``;
        ``seq_lens`` already counts the new token."""
        cos, sin = self.rope(input_ids.device)
        pos = position_ids.to(torch.int32)
        x = F.embedding(input_ids.long(), self.embed)
        res = None
        for i, layer in enumerate(self.layers):
            if res is None:
                y, res = fused.rmsnorm(x, layer.input_norm, layer.eps), x
            else:
                y, res = fused.rmsnorm(x, layer.input_norm, layer.eps, residual=res)
            q, k, v = layer.attn.project_qkv(y, cos, sin, pos)
            kv_cache_write(k, v, slot_mapping, kv_caches[i][0], kv_caches[i][1])
            a = paged_decode(q, kv_caches[i][0], kv_caches[i][1], block_table, seq_lens,
                             max_seq_len=max_seq_len)
            a = linear(a.reshape(a.shape[0], -1), layer.attn.o)
            y, res = fused.rmsnorm(a, layer.post_norm, layer.eps, residual=res)
            x = layer.mlp(y)
        y, _ = fused.rmsnorm(x, self.norm, self.cfg.rms_norm_eps, residual=res)
        return y

    # ------------------------------------------------------ HF name mapping
    def to_hf(self) -> Iterator[tuple[str, torch.Tensor]]:
        """Yields ``(hf_name, tensor)`` views/slices in HF checkpoint naming."""
        cfg = self.cfg
        yield "model.embed_tokens.weight", self.embed
        qs, ks = cfg.q_size, cfg.kv_size
        I = cfg.intermediate_size
        for i, layer in enumerate(self.layers):
            p = f"model.layers.{i}."
            yield p + "input_layernorm.weight", layer.input_norm
            a = layer.attn
            yield p + "self_attn.q_proj.weight", a.qkv[:qs]
            yield p + "self_attn.k_proj.weight", a.qkv[qs:qs + ks]
            yield p + "self_attn.v_proj.weight", a.qkv[qs + ks:]
            if a.qkv_bias is not None:
                yield p + "self_attn.q_proj.bias", a.qkv_bias[:qs]
                yield p + "self_attn.k_proj.bias", a.qkv_bias[qs:qs + ks]
                yield p + "self_attn.v_proj.bias", a.qkv_bias[qs + ks:]
            if a.q_norm is not None:
                yield p + "self_attn.q_norm.weight", a.q_norm
                yield p + "self_attn.k_norm.weight", a.k_norm
            yield p + "self_attn.o_proj.weight", a.o
            yield p + "post_attention_layernorm.weight", layer.post_norm
            m = layer.mlp
            if isinstance(m, DenseMLP):
                yield p + "mlp.gate_proj.weight", m.gate_up[:I]
                yield p + "mlp.up_proj.weight", m.gate_up[I:]
                yield p + "mlp.down_proj.weight", m.down
            else:
                Im = cfg.moe_intermediate_size
                yield p + "mlp.gate.weight", m.router
                for e in range(cfg.num_experts):
                    q = p + f"mlp.experts.{e}."
                    yield q + "gate_proj.weight", m.gate_up[e, :Im]
                    yield q + "up_proj.weight", m.gate_up[e, Im:]
                    yield q + "down_proj.weight", m.down[e]
        yield "model.norm.weight", self.norm
        if self.score is not None:
            yield "score.weight", self.score
        elif self.lm_head is not None:
            yield "lm_head.weight", self.lm_head

    def hf_name_map(self) -> dict[str, torch.Tensor]:
        return dict(self.to_hf())

    @torch.no_grad()
    def load_hf(self, tensors: Iterable[tuple[str, torch.Tensor]], strict: bool = True):
        """Copies HF-named tensors into the fused parameters."""
        dst = self.hf_name_map()
        seen = set()
        for name, t in tensors:
            if name == "lm_head.weight" and self.lm_head is None and self.score is None:
                seen.add(name)
                continue  # tied
            if name not in dst:
                if strict:
                    raise KeyError(f"unexpected tensor {name}")
                continue
            d = dst[name]
            if d.shape != t.shape:
                raise ValueError(f"{name}: shape {tuple(t.shape)} != {tuple(d.shape)}")
            d.copy_(t.to(device=d.device, dtype=d.dtype))
            seen.add(name)
        missing = set(dst) - seen
        if strict and missing:
            raise KeyError(f"missing tensors: {sorted(missing)[:8]} ...")
        return self


def build_model(cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", seed: int | None = 0) -> QwenModel:
    m = QwenModel(cfg, dtype=dtype, device=device)
    if seed is not None:
        m.init_weights(seed)
    return m
