"""Multi-head latent attention (DeepSeek-V2 / V3): queries and keys / values pass through low-rank bottlenecks with
an RMSNorm inside, every head's query and key is a part without position (``qk_nope_head_dim``) next to a rotary
part (``qk_rope_head_dim``; the key's rotary part is computed once and shared by all heads), and values are
``v_head_dim`` wide.

    q   = W_qb · norm(W_qa · x)                      (or W_q · x when ``q_lora_rank`` is 0)
    c,r = split(W_kva · x)                           latent [kv_lora_rank], shared rotary key [rope]
    k,v = split(W_kvb · norm(c))                     per head: [nope], [v]
    attention over q = [q_nope | rope(q_rope)], k = [k_nope | rope(r)], scale 1/sqrt(nope + rope) (times the
    square of the YaRN magnitude factor when the rotary table is scaled that way)

The attention itself is the packed causal attention op with ``v`` zero-padded to the query width (the op wants one
head width; the padded columns of the output are dropped), so every attention variant that plugs into a block
(Ulysses exchange, tree attention) also takes this layer. Head widths other than 128 take the op's general path.
Runs under data, sequence (Ulysses), pipeline, expert and tensor parallelism. Under tensor parallelism
(sequence-parallel activations: every rank holds a slice of the tokens between blocks) the projections INTO the
bottlenecks and their norms are replicated and run on the rank's own tokens; the projections out of them are split
by head and gather the tokens (column-parallel); the shared rotary key is gathered to all tokens with a backward
that sums the ranks' partial gradients; the output projection is row-parallel. The rollout engine serves it with
the EXPANDED keys and values in its paged cache (per head: the full-width key, the value padded to that width),
not with the compressed latent: simple and exact, at ``heads * 2 * (nope + rope)`` cache elements per token
instead of ``kv_lora_rank + rope``; decode steps run eagerly on the paged-attention op's general path.

Checkpoint names follow Hugging Face's DeepseekV3 (``self_attn.{q_a_proj,q_a_layernorm,q_b_proj,
kv_a_proj_with_mqa,kv_a_layernorm,kv_b_proj,o_proj}``).
Reference: the DeepSeek-V3 converter of the Megatron engine, areal/engine/megatron_utils/megatron.py
(``convert_deepseekv3_to_hf``), which maps Megatron's MLA projections to the same names.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import fused
from ..ops.attention import VarlenMeta, varlen_attention
from ..ops.gemm import linear
from .config import ModelConfig


def rope_rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleave: bool) -> torch.Tensor:
    """``x [T, H, R]``, ``cos`` / ``sin`` ``[T, R/2]`` (already gathered at the tokens' positions). With
    ``interleave`` the pairs are neighbours ``(2i, 2i+1)`` on input; the output is always in the half-split
    layout ``[first components | second components]``, for queries and keys alike, so their products agree."""
    xf = x.float()
    if interleave:
        a, b = xf[..., 0::2], xf[..., 1::2]
    else:
        a, b = xf.chunk(2, dim=-1)
    c, s = cos[:, None, :].float(), sin[:, None, :].float()
    return torch.cat((a * c - b * s, b * c + a * s), dim=-1).to(x.dtype)


class MLAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, pctx=None, layer_idx: int = 0):
        super().__init__()
        tp = pctx.tp_size if pctx is not None else 1
        assert cfg.num_attention_heads % tp == 0, "tensor parallelism needs the head count to divide by its size"
        if cfg.lora_rank > 0 and any(t in ("q_proj", "k_proj", "v_proj", "o_proj") for t in (cfg.lora_targets or [])):
            raise NotImplementedError("latent attention takes no LoRA adapters: target the MLP projections")
        self.cfg, self.pctx = cfg, pctx
        h, nh = cfg.hidden_size, cfg.num_attention_heads // tp   # nh: this rank's heads
        self.nh, self.dn, self.dr, self.dv = nh, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        assert self.dr % 2 == 0 and self.dv <= self.dn + self.dr
        mk = lambda *shape: nn.Parameter(torch.empty(*shape, dtype=dtype, device=device))
        ones = lambda n: nn.Parameter(torch.ones(n, dtype=dtype, device=device))
        qk = self.dn + self.dr
        if cfg.q_lora_rank:
            self.q_a, self.q_a_norm, self.q_b = mk(cfg.q_lora_rank, h), ones(cfg.q_lora_rank), mk(nh * qk, cfg.q_lora_rank)
            self.q = None
        else:
            self.q_a = self.q_a_norm = self.q_b = None
            self.q = mk(nh * qk, h)
        self.kv_a = mk(cfg.kv_lora_rank + self.dr, h)
        self.kv_a_norm = ones(cfg.kv_lora_rank)
        self.kv_b = mk(nh * (self.dn + self.dv), cfg.kv_lora_rank)
        self.o = mk(h, nh * self.dv)
        self.lora_o = None  # (the decode loop asks)
        # softmax scale relative to the attention op's default 1/sqrt(width): the YaRN magnitude correction
        self.q_scale = 1.0
        sc = cfg.rope_scaling or {}
        if sc.get("rope_type") == "yarn" and sc.get("mscale_all_dim"):
            f = float(sc["factor"])
            m = 1.0 if f <= 1 else 0.1 * float(sc["mscale_all_dim"]) * math.log(f) + 1.0
            self.q_scale = m * m

    def _tp(self):
        p = self.pctx
        return p.tp_fused if (p is not None and p.tp_size > 1) else None

    def project(self, x, cos, sin, pos):
        """``q, k [T, heads, nope + rope]`` and ``v [T, heads, v]``: this rank's heads of ALL tokens of the
        sequence-parallel shard (``x`` holds this rank's tokens only under tensor parallelism; ``pos`` always the
        positions of all of them)."""
        cfg = self.cfg
        tp = self._tp()
        if tp is not None:
            from ..parallel.tensor_parallel import column_parallel_linear, gather_seq

            up = lambda t, w: column_parallel_linear(t, w, tp)   # gathers the tokens, multiplies by this rank's rows
        else:
            up = linear
        if self.q is None:
            q = up(fused.rmsnorm(linear(x, self.q_a), self.q_a_norm, cfg.rms_norm_eps), self.q_b)
        else:
            q = up(x, self.q)
        T = q.shape[0]
        q = q.view(T, self.nh, self.dn + self.dr)
        ckv = linear(x, self.kv_a)
        c, k_rot = ckv[:, :cfg.kv_lora_rank], ckv[:, cfg.kv_lora_rank:]
        kv = up(fused.rmsnorm(c.contiguous(), self.kv_a_norm, cfg.rms_norm_eps), self.kv_b)
        kv = kv.view(T, self.nh, self.dn + self.dv)
        if tp is not None:
            k_rot = gather_seq(k_rot.contiguous(), tp)   # shared by every head on every rank: gradients are summed
        cs, sn = cos[pos.long()], sin[pos.long()]
        q_rot = rope_rotate(q[..., self.dn:], cs, sn, cfg.rope_interleave)
        k_rot = rope_rotate(k_rot[:, None, :], cs, sn, cfg.rope_interleave)
        q_nope = q[..., :self.dn]
        if self.q_scale != 1.0:
            q_nope, q_rot = q_nope * self.q_scale, q_rot * self.q_scale
        q = torch.cat((q_nope, q_rot), dim=-1)
        k = torch.cat((kv[..., :self.dn], k_rot.expand(T, self.nh, self.dr)), dim=-1)
        return q, k, kv[..., self.dn:]

    def project_qkv(self, x, cos, sin, pos):
        """``q, k, v`` of one width (``v`` zero-padded): what the attention ops and the paged cache take."""
        q, k, v = self.project(x, cos, sin, pos)
        pad = q.shape[-1] - self.dv
        if pad:
            v = F.pad(v, (0, pad))
        return q.contiguous(), k.contiguous(), v.contiguous()

    def project_q_write_kv(self, x, cos, sin, pos, slot_mapping, k_cache, v_cache):
        """Decode step: returns ``q``; the new tokens' keys and (padded) values go into the paged caches."""
        from ..ops.rollout_ops import kv_cache_write

        q, k, v = self.project_qkv(x, cos, sin, pos)
        kv_cache_write(k, v, slot_mapping, k_cache, v_cache)
        return q

    def out_proj(self, a):
        """Output projection of an attention result ``[T, heads, nope + rope]``: the padding columns are dropped."""
        a = a[..., :self.dv].reshape(a.shape[0], self.nh * self.dv)
        tp = self._tp()
        if tp is not None:
            from ..parallel.tensor_parallel import row_parallel_linear

            return row_parallel_linear(a, self.o, tp)
        return linear(a, self.o)

    def forward(self, x, cos, sin, pos, meta: VarlenMeta, attn_fn=None):
        q, k, v = self.project_qkv(x, cos, sin, pos)
        return self.out_proj((attn_fn or varlen_attention)(q, k, v, meta))

    def hf_tensors(self, p: str):
        """``(checkpoint name, tensor)`` of this layer, ``p`` = ``model.layers.<i>.``. Bailing checkpoints call the
        module ``attention`` and its output projection ``dense``."""
        bailing = self.cfg.model_type == "bailing_hybrid"
        p = p + ("attention." if bailing else "self_attn.")
        if self.q is None:
            yield p + "q_a_proj.weight", self.q_a
            yield p + "q_a_layernorm.weight", self.q_a_norm
            yield p + "q_b_proj.weight", self.q_b
        else:
            yield p + "q_proj.weight", self.q
        yield p + "kv_a_proj_with_mqa.weight", self.kv_a
        yield p + "kv_a_layernorm.weight", self.kv_a_norm
        yield p + "kv_b_proj.weight", self.kv_b
        yield p + ("dense.weight" if bailing else "o_proj.weight"), self.o
