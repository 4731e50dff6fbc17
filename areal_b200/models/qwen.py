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

import re

from typing import Any, Iterable, Iterator

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import _lib, fused
from ..ops.attention import VarlenMeta, varlen_attention
from ..ops.gemm import gemm, linear, linear_rmsnorm
from ..ops.rollout_ops import kv_cache_write, paged_decode
from .config import ModelConfig


def _dense(x, w, bias, cfg: ModelConfig):
    """Projection of a dense layer: block-scaled fp8 forward when the model is configured for it."""
    if cfg.fp8 and bias is None and x.is_cuda and x.dtype == torch.bfloat16:
        from ..ops.fp8 import fp8_linear

        return fp8_linear(x, w, cfg.fp8_ue8m0)
    return linear(x, w, bias)


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, pctx=None, layer_idx: int = 0):
        super().__init__()
        self.cfg = cfg
        self.pctx = pctx
        tp = pctx.tp_size if pctx is not None else 1
        assert cfg.num_attention_heads % tp == 0 and cfg.num_key_value_heads % tp == 0, \
            "tensor parallelism needs the head counts to divide by the tp size"
        self.n_q, self.n_kv = cfg.num_attention_heads // tp, cfg.num_key_value_heads // tp
        h = cfg.hidden_size
        qs, ks = cfg.q_size // tp, cfg.kv_size // tp
        self.qkv = nn.Parameter(torch.empty(qs + 2 * ks, h, dtype=dtype, device=device))
        self.qkv_bias = (nn.Parameter(torch.zeros(qs + 2 * ks, dtype=dtype, device=device))
                         if cfg.attention_bias else None)
        self.o = nn.Parameter(torch.empty(h, qs, dtype=dtype, device=device))
        if cfg.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(cfg.head_dim, dtype=dtype, device=device))
            self.k_norm = nn.Parameter(torch.ones(cfg.head_dim, dtype=dtype, device=device))
        else:
            self.q_norm = self.k_norm = None
        from .lora import make_adapter

        self.lora_qkv = make_adapter(cfg, h, [("q_proj", qs), ("k_proj", ks), ("v_proj", ks)], dtype, device,
                                     seed=2 * layer_idx + 1000, tp_mode="column", pctx=pctx)
        self.lora_o = make_adapter(cfg, qs, [("o_proj", h)], dtype, device, seed=2 * layer_idx + 1001,
                                   tp_mode="row", pctx=pctx)

    def _tp(self):
        p = self.pctx
        return p.tp_fused if (p is not None and p.tp_size > 1) else None

    def project_qkv(self, x, cos, sin, pos):
        cfg = self.cfg
        tp = self._tp()
        if tp is not None:
            from ..parallel.tensor_parallel import column_parallel_linear

            qkv = column_parallel_linear(x, self.qkv, tp, self.qkv_bias)
        else:
            qkv = _dense(x, self.qkv, self.qkv_bias, cfg)
        if self.lora_qkv is not None:
            qkv = qkv + self.lora_qkv(x)
        return fused.qknorm_rope(qkv, self.q_norm, self.k_norm, cos, sin, pos,
                                 self.n_q, self.n_kv, cfg.head_dim, cfg.rms_norm_eps)

    def project_q_write_kv(self, x, cos, sin, pos, slot_mapping, k_cache, v_cache):
        """Decode-step form of :meth:`project_qkv`: returns ``q`` only; the normalised, rotated ``k`` and
        ``v`` go into the paged caches inside the same kernel (no separate cache-write launch)."""
        cfg = self.cfg
        if self._tp() is not None:
            q, k, v = self.project_qkv(x, cos, sin, pos)
            kv_cache_write(k, v, slot_mapping, k_cache, v_cache)
            return q
        qkv = _dense(x, self.qkv, self.qkv_bias, cfg)
        if self.lora_qkv is not None:
            qkv = qkv + self.lora_qkv(x)
        return fused.qknorm_rope_kvwrite(qkv, self.q_norm, self.k_norm, cos, sin, pos, self.n_q, self.n_kv,
                                         cfg.head_dim, cfg.rms_norm_eps, slot_mapping, k_cache, v_cache)

    def _fused_ulysses(self, x, cos, sin, pos, meta, attn_fn=None):
        """Ulysses with the projection and the sequence→head exchange fused into one kernel: the
        q/k norms and RoPE then run after the exchange, on this rank's heads of ALL tokens."""
        p = self.pctx
        external = attn_fn is not None and not getattr(attn_fn, "is_ulysses", False)  # tree / zig-zag attention
        if (external or p is None or p.sp_size == 1 or p.tp_size > 1 or self.qkv_bias is not None
                or p.sp_fused is None or p.extras.get("cp_mode") == "zigzag"
                or "full_positions" not in p.extras or self.lora_qkv is not None):
            return None
        from ..parallel.ulysses import fused_qkv_seq_to_head, head_to_seq

        cfg = self.cfg
        qkv = fused_qkv_seq_to_head(x, self.qkv, p, self.n_q, self.n_kv, cfg.head_dim)
        if qkv is None:
            return None
        S = p.sp_size
        q, k, v = fused.qknorm_rope(qkv, self.q_norm, self.k_norm, cos, sin, p.extras["full_positions"],
                                    self.n_q // S, self.n_kv // S, cfg.head_dim, cfg.rms_norm_eps)
        a = varlen_attention(q, k, v, meta)
        if not cfg.fp8 and self.lora_o is None:
            from ..parallel.ulysses import fused_head_to_seq_proj

            # the head→sequence exchange fused into the output projection (K loop split by source rank)
            y = fused_head_to_seq_proj(a.reshape(a.shape[0], -1), self.o, p)
            if y is not None:
                return y, True
        return head_to_seq(a, p), False

    def forward(self, x, cos, sin, pos, meta: VarlenMeta, attn_fn=None):
        """``pos`` are the positions of the tokens that reach the q/k projection output: all
        tokens of this sequence-parallel shard (tensor parallelism gathers its token shards
        inside the projection)."""
        fused_out = self._fused_ulysses(x, cos, sin, pos, meta, attn_fn)
        if fused_out is not None and fused_out[1]:
            return fused_out[0]  # the output projection ran inside the fused exchange
        if fused_out is None:
            q, k, v = self.project_qkv(x, cos, sin, pos)
            a = (attn_fn or varlen_attention)(q, k, v, meta)
        else:
            a = fused_out[0]
        a = a.reshape(a.shape[0], -1)
        tp = self._tp()
        if tp is not None:
            from ..parallel.tensor_parallel import row_parallel_linear

            y = row_parallel_linear(a, self.o, tp)
            return y if self.lora_o is None else y + self.lora_o(a)
        y = _dense(a, self.o, None, self.cfg)
        return y if self.lora_o is None else y + self.lora_o(a)


class DenseMLP(nn.Module):
    def __init__(self, hidden, inter, dtype, device, pctx=None, cfg: ModelConfig | None = None, layer_idx: int = 0):
        super().__init__()
        self.pctx = pctx
        self.cfg = cfg
        tp = pctx.tp_size if pctx is not None else 1
        assert inter % tp == 0
        self.gate_up = nn.Parameter(torch.empty(2 * inter // tp, hidden, dtype=dtype, device=device))
        self.down = nn.Parameter(torch.empty(hidden, inter // tp, dtype=dtype, device=device))
        from .lora import make_adapter

        self.lora_gate_up = make_adapter(cfg, hidden, [("gate_proj", inter // tp), ("up_proj", inter // tp)],
                                         dtype, device, seed=2 * layer_idx + 2000, tp_mode="column", pctx=pctx)
        self.lora_down = make_adapter(cfg, inter // tp, [("down_proj", hidden)], dtype, device,
                                      seed=2 * layer_idx + 2001, tp_mode="row", pctx=pctx)

    def forward(self, x):
        p = self.pctx
        if p is not None and p.tp_size > 1:
            from ..parallel.tensor_parallel import column_parallel_linear, row_parallel_linear

            gu = column_parallel_linear(x, self.gate_up, p.tp_fused)
            if self.lora_gate_up is not None:
                gu = gu + self.lora_gate_up(x)
            a = fused.swiglu(gu)
            y = row_parallel_linear(a, self.down, p.tp_fused)
            return y if self.lora_down is None else y + self.lora_down(a)
        dense = (lambda t, w: _dense(t, w, None, self.cfg)) if (self.cfg is not None and self.cfg.fp8) else linear
        gu = dense(x, self.gate_up)
        if self.lora_gate_up is not None:
            gu = gu + self.lora_gate_up(x)
        a = fused.swiglu(gu)
        y = dense(a, self.down)
        return y if self.lora_down is None else y + self.lora_down(a)


class MoEMLP(nn.Module):
    """Top-k routed experts (softmax router in fp32, optional top-k prob
    renormalisation), as in Qwen3-MoE. Expert weights are 3-D parameters
    ``gate_up [E, 2I, H]`` and ``down [E, H, I]``."""

    def __init__(self, cfg: ModelConfig, dtype, device, pctx=None):
        super().__init__()
        self.cfg = cfg
        self.pctx = pctx
        E, I, H = cfg.num_experts, cfg.moe_intermediate_size, cfg.hidden_size
        ep = pctx.ep_size if pctx is not None else 1
        etp = pctx.etp_size if pctx is not None else 1
        assert E % ep == 0, "the expert count must divide by the expert-parallel size"
        assert I % etp == 0, "the expert width must divide by the expert-tensor-parallel size"
        self.router = nn.Parameter(torch.empty(E, H, dtype=dtype, device=device))
        # under expert parallelism this rank owns experts [ep_rank * E/ep, (ep_rank + 1) * E/ep); under expert
        # tensor parallelism it holds rows [etp_rank * I/etp, (etp_rank + 1) * I/etp) of their gate and up
        # projections and the matching columns of their down projection
        self.gate_up = nn.Parameter(torch.empty(E // ep, 2 * I // etp, H, dtype=dtype, device=device))
        self.down = nn.Parameter(torch.empty(E // ep, H, I // etp, dtype=dtype, device=device))
        self.last_routing = None  # (topk_idx, topk_w) of the last forward, for stats / replay
        # aux-loss-free balancing: a selection-only bias, a buffer (not trained by the optimizer, replicated)
        if cfg.moe_load_balance_coeff > 0 or cfg.moe_expert_bias:
            self.register_buffer("expert_bias", torch.zeros(E, dtype=torch.float32, device=device))
        else:
            self.expert_bias = None
        # tokens routed to every expert since the last bias update. A stand-alone module updates the bias after
        # every training forward; a train engine sets `defer_bias_update` and updates once per optimizer step from
        # the counts of ALL ranks that hold this layer (`update_expert_bias`), so the replicas' biases stay equal
        if cfg.moe_load_balance_coeff > 0:
            self.register_buffer("load_acc", torch.zeros(E, dtype=torch.float32, device=device), persistent=False)
        else:
            self.load_acc = None
        self.defer_bias_update = False
        # shared expert: a dense SwiGLU MLP applied to every token, scaled by sigmoid(x . w_gate); replicated
        # over the expert-parallel group (every rank applies it to its own tokens)
        Is = cfg.shared_expert_intermediate_size
        if Is:
            self.shared_gate_up = nn.Parameter(torch.empty(2 * Is, H, dtype=dtype, device=device))
            self.shared_down = nn.Parameter(torch.empty(H, Is, dtype=dtype, device=device))
            self.shared_gate = (nn.Parameter(torch.empty(1, H, dtype=dtype, device=device))
                                if cfg.shared_expert_gated else None)
        else:
            self.shared_gate_up = self.shared_down = self.shared_gate = None

    def _shared(self, x):
        y = linear(fused.swiglu(linear(x, self.shared_gate_up)), self.shared_down)
        if self.shared_gate is None:
            return y
        if x.is_cuda:
            _lib.count_fallback("moe.shared_expert_gate[F.linear]")
        g = torch.sigmoid(F.linear(x.float(), self.shared_gate.float()))
        return (y.float() * g).to(x.dtype)

    def route(self, x):
        cfg = self.cfg
        if x.is_cuda:
            _lib.count_fallback("moe.router[F.linear fp32]")
        logits = F.linear(x.float(), self.router.float())
        plain = (cfg.moe_score_func == "softmax" and cfg.moe_route_scale == 1.0 and self.expert_bias is None
                 and cfg.moe_n_group <= 1)
        if not plain:
            return self._route_general(logits)
        if not (torch.is_grad_enabled() and (x.requires_grad or self.router.requires_grad)):
            from ..ops.moe import route as route_kernel

            return route_kernel(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob)
        probs = logits.softmax(-1)
        w, idx = probs.topk(cfg.num_experts_per_tok, dim=-1)
        if cfg.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        return idx, w

    def _route_general(self, logits):
        """Sigmoid or softmax scores; experts are PICKED by ``score + expert_bias`` but weighted by the plain
        score (so the bias steers load without entering the gradient); optional renormalisation and scale.
        After a training forward the bias moves by ``coeff * sign(mean_load - load)`` per expert. The bias
        is a buffer of the trainer's model: it is saved with ``state_dict`` but is not part of the flat
        weight buffer, so rollout engines route by the plain scores and the decoupled loss's
        behaviour-policy weights absorb the difference."""
        cfg = self.cfg
        scores = torch.sigmoid(logits) if cfg.moe_score_func == "sigmoid" else logits.softmax(-1)
        pick = scores if self.expert_bias is None else scores + self.expert_bias
        if cfg.moe_n_group > 1:
            # group-limited routing: a group scores the sum of its two best experts; experts outside the token's
            # best `moe_topk_group` groups cannot be picked
            G = cfg.moe_n_group
            grouped = pick.view(-1, G, cfg.num_experts // G)
            best = grouped.topk(min(cfg.moe_group_score_top, grouped.shape[-1]), dim=-1).values.sum(-1).topk(cfg.moe_topk_group, dim=-1).indices
            allowed = torch.zeros(grouped.shape[:2], dtype=torch.bool, device=pick.device).scatter_(1, best, True)
            pick = grouped.masked_fill(~allowed[..., None], 0.0).view_as(pick)
        idx = pick.topk(cfg.num_experts_per_tok, dim=-1).indices
        w = scores.gather(-1, idx)
        if cfg.norm_topk_prob:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        w = w * cfg.moe_route_scale
        if self.load_acc is not None and self.training and torch.is_grad_enabled():
            with torch.no_grad():
                self.load_acc.add_(torch.bincount(idx.reshape(-1), minlength=cfg.num_experts).float())
            if not self.defer_bias_update:
                self.update_expert_bias()
        return idx.to(torch.int32), w

    @torch.no_grad()
    def update_expert_bias(self, groups=()):
        """``bias += coeff * sign(mean load - load)`` from the tokens counted since the last call, summed over
        ``groups`` (the process groups whose ranks hold replicas of this layer and routed other tokens)."""
        if self.load_acc is None:
            return
        import torch.distributed as dist

        load = self.load_acc
        for g in groups:
            dist.all_reduce(load, group=g)
        if float(load.sum()) > 0:
            self.expert_bias.add_(self.cfg.moe_load_balance_coeff * torch.sign(load.mean() - load))
        load.zero_()

    def forward(self, x):
        from ..ops.moe import moe_experts_forward

        idx, w = self.route(x)
        self.last_routing = (idx.detach(), w.detach())
        p = self.pctx

        def experts(x_, idx_, w_):
            if p is not None and p.ep_size > 1:
                from ..parallel.expert_parallel import ep_moe_forward

                return ep_moe_forward(x_, idx_, w_, self.gate_up, self.down, p.extras.get("ep_state", p.ep_group))
            return moe_experts_forward(x_, idx_, w_, self.gate_up, self.down)

        if p is not None and p.etp_size > 1:
            # expert tensor parallelism: the ranks of the group hold slices of the same experts, so they pool their
            # tokens (each routed its own), every rank applies its slice to all of them and the partial outputs are
            # summed back to the rank each token came from
            from ..parallel.expert_parallel import etp_moe_forward

            y = etp_moe_forward(x, idx, w, p.etp_group, experts)
        else:
            y = experts(x, idx, w)
        return y if self.shared_gate_up is None else y + self._shared(x)


class Block(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype, device, pctx=None):
        super().__init__()
        h = cfg.hidden_size
        self.input_norm = nn.Parameter(torch.ones(h, dtype=dtype, device=device))
        if cfg.is_hybrid:
            from .qwen3_5 import GatedAttention, GatedDeltaNet

            kind = GatedDeltaNet if cfg.layer_type(layer_idx) == "linear_attention" else GatedAttention
            self.attn = kind(cfg, dtype, device, pctx, layer_idx)
        elif cfg.layer_is_lightning(layer_idx):
            from .lightning import LightningAttention

            self.attn = LightningAttention(cfg, dtype, device, pctx, layer_idx)
        elif cfg.is_mla:
            from .mla import MLAttention

            self.attn = MLAttention(cfg, dtype, device, pctx, layer_idx)
        else:
            self.attn = Attention(cfg, dtype, device, pctx, layer_idx)
        self.post_norm = nn.Parameter(torch.ones(h, dtype=dtype, device=device))
        if cfg.layer_is_moe(layer_idx):
            if pctx is not None and pctx.tp_size > 1 and pctx.ep_size * pctx.etp_size == 1:
                # under tensor parallelism every rank holds a different slice of the tokens at this point, so the
                # experts are spread over those ranks (expert parallelism over the tensor-parallel group, e = t)
                raise NotImplementedError("mixture layers under tensor parallelism need expert parallelism over the "
                                          "same ranks: give e = t (or a multiple), e.g. megatron:(attn:d1t4|ffn:d1e4)")
            self.mlp = MoEMLP(cfg, dtype, device, pctx)
        else:
            self.mlp = DenseMLP(h, cfg.intermediate_size, dtype, device, pctx, cfg, layer_idx)
        self.eps = cfg.rms_norm_eps

    def forward(self, x, res, cos, sin, pos, meta, attn_fn=None, recompute_mlp: bool = False):
        if res is None:
            y, res = fused.rmsnorm(x, self.input_norm, self.eps), x
        else:
            y, res = fused.rmsnorm(x, self.input_norm, self.eps, residual=res)
        a = self.attn(y, cos, sin, pos, meta, attn_fn)
        y, res = fused.rmsnorm(a, self.post_norm, self.eps, residual=res)
        if recompute_mlp and torch.is_grad_enabled():
            # op-selective activation checkpointing: the MLP half keeps only its input
            from torch.utils.checkpoint import checkpoint

            return checkpoint(self.mlp, y, use_reentrant=False), res
        return self.mlp(y), res


class QwenModel(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", pctx=None):
        """``pctx`` (``parallel.context.ParallelContext``) turns on tensor parallelism (vocab-parallel
        embedding / LM head, head- and column-sharded projections, token-sharded activations
        between blocks) and Ulysses sequence parallelism; parameters then have their LOCAL shapes."""
        super().__init__()
        self.cfg = cfg
        self.pctx = pctx
        tp = pctx.tp_size if pctx is not None else 1
        assert cfg.vocab_size % tp == 0
        vloc = cfg.vocab_size // tp
        # pipeline parallelism: this stage owns a contiguous range of blocks; the embedding lives on
        # the first stage, the final norm and the head on the last (a tied head keeps its own copy of
        # the embedding there; the two copies' gradients are summed before the optimizer step)
        pp = pctx.pp_size if pctx is not None else 1
        self.first_stage = pctx.is_first_stage if pp > 1 else True
        self.last_stage = pctx.is_last_stage if pp > 1 else True
        # virtual stages: every rank holds `vpp` chunks of blocks; chunk v of rank p is virtual stage v * pp + p,
        # so the embedding still sits on the first rank (its chunk 0) and the head on the last rank (its last chunk);
        # with the V-shaped placement (chunk 1 of rank p = stage 2 pp - 1 - p) the first rank holds both
        self.vpp = int(pctx.extras.get("vpp", 1)) if pp > 1 else 1
        if pp > 1:
            from ..parallel.context import partition_layers

            # the last virtual stage also runs the LM head (or value head) and the loss: weigh it in units of one block
            per_layer = max((cfg.num_params() - cfg.vocab_size * cfg.hidden_size *
                             (1 if (cfg.tie_word_embeddings or cfg.is_critic) else 2)) / cfg.num_hidden_layers, 1.0)
            head = 0.0 if cfg.is_critic else cfg.vocab_size * cfg.hidden_size / per_layer
            if self.vpp == 1:
                self.chunk_ranges = [pctx.layer_range(cfg.num_hidden_layers, last_extra=head)]
            else:
                from ..parallel.pipeline import stage_of

                ranges = partition_layers([1.0] * cfg.num_hidden_layers, pp * self.vpp, 0.0, head)
                placement = pctx.extras.get("pp_placement", "interleaved")
                self.chunk_ranges = [ranges[stage_of(pctx.pp_rank, v, pp, placement)] for v in range(self.vpp)]
        else:
            self.chunk_ranges = [(0, cfg.num_hidden_layers)]
        self.layer_ids = [i for a, b in self.chunk_ranges for i in range(a, b)]  # global index of every local block
        self.chunk_slices, o = [], 0
        for a, b in self.chunk_ranges:
            self.chunk_slices.append((o, o + b - a))
            o += b - a
        self.layer_start, self.layer_end = self.chunk_ranges[0][0], self.chunk_ranges[-1][1]
        mk = lambda *shape: nn.Parameter(torch.empty(*shape, dtype=dtype, device=device))
        need_embed = self.first_stage or (self.last_stage and cfg.tie_word_embeddings and not cfg.is_critic)
        self.embed = mk(vloc, cfg.hidden_size) if need_embed else None
        self.layers = nn.ModuleList(Block(cfg, i, dtype, device, pctx) for i in self.layer_ids)
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device)) if self.last_stage else None
        self.score = self.lm_head = None
        if self.last_stage:
            if cfg.is_critic:
                self.score = mk(1, cfg.hidden_size)
            elif not cfg.tie_word_embeddings:
                self.lm_head = mk(vloc, cfg.hidden_size)
        self._rope = None
        self.checkpoint_every = 0  # k > 0: recompute every k-th block's activations in backward

    # ------------------------------------------------------------------ init
    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator(device="cpu").manual_seed(seed)
        dev_gen = None
        tp = self.pctx.tp_size if self.pctx is not None else 1
        tp_rank = self.pctx.tp_rank if self.pctx is not None else 0
        if len(self.layer_ids) != self.cfg.num_hidden_layers:
            return self._init_weights_pipeline(seed, std)
        for name, p in self.named_parameters():
            if ".lora_" in name:
                continue  # adapters initialise themselves and do not consume the base model's stream
            if name.endswith("norm") or "_norm" in name:
                p.fill_(1.0)
                continue
            if name.endswith(("attn.conv_w", "attn.A_log", "attn.dt_bias")):
                continue  # set by GatedDeltaNet.init_special below
            if name.endswith("bias"):
                p.zero_()
                continue
            dst = p
            ep = self.pctx.ep_size if self.pctx is not None else 1
            etp = self.pctx.etp_size if self.pctx is not None else 1
            is_expert = ep * etp > 1 and name.endswith(("mlp.gate_up", "mlp.down")) and p.dim() == 3
            if is_expert:
                # the full stack of experts at full width: values do not depend on the layout
                full = [p.shape[0] * ep, p.shape[1], p.shape[2]]
                full[1 if name.endswith("gate_up") else 2] *= etp
                dst = torch.empty(tuple(full), dtype=p.dtype, device=p.device)
            if tp > 1:
                # draw the FULL tensor (so values do not depend on the tp size), keep this rank's shard
                from ..parallel.tensor_parallel import is_tp_replicated, tp_slice

                if not is_tp_replicated(name) and not is_expert:  # experts are split by expert, not by tp
                    dst = torch.empty(self._full_shape(name, p), dtype=p.dtype, device=p.device)
            if dst.is_cuda:
                # large models: draw on the device (same seed ⇒ same values on every rank)
                if dev_gen is None:
                    dev_gen = torch.Generator(device=p.device).manual_seed(seed)
                dst.normal_(0.0, std, generator=dev_gen)
            else:
                # generated on the host in fp32 so that every dtype sees the same values
                chunk = 1 << 24
                flat = dst.view(-1)
                for s in range(0, flat.numel(), chunk):
                    n = min(chunk, flat.numel() - s)
                    flat[s:s + n].copy_(torch.empty(n, dtype=torch.float32).normal_(0.0, std, generator=g))
            if is_expert:
                n = p.shape[0]
                mine = dst[self.pctx.ep_rank * n:(self.pctx.ep_rank + 1) * n]
                if etp > 1:
                    from ..parallel.tensor_parallel import expert_slice

                    mine = expert_slice(name, mine, self.pctx.etp_rank, etp)
                p.copy_(mine)
            elif dst is not p:
                p.copy_(tp_slice(name, dst, self.cfg, tp_rank, tp))
        for li, layer in enumerate(self.layers):
            if hasattr(layer.attn, "init_special"):
                layer.attn.init_special(torch.Generator(device="cpu").manual_seed(seed * 1000 + li))
        return self

    @torch.no_grad()
    def _init_weights_pipeline(self, seed: int, std: float):
        """A pipeline stage draws the whole model's random stream (stage-independent values) on a
        meta-free throwaway copy and keeps what it owns. Meant for small / test models; real runs
        load checkpoints."""
        import copy

        from ..parallel.context import ParallelContext

        p = self.pctx
        flat_ctx = ParallelContext(tp_group=p.tp_group, tp_rank=p.tp_rank, tp_size=p.tp_size,
                                   ep_group=p.ep_group, ep_rank=p.ep_rank, ep_size=p.ep_size,
                                   etp_group=p.etp_group, etp_rank=p.etp_rank, etp_size=p.etp_size)
        full = type(self)(self.cfg, dtype=next(self.parameters()).dtype, device=next(self.parameters()).device,
                          pctx=flat_ctx if (p.tp_size > 1 or p.ep_size > 1 or p.etp_size > 1) else None)
        full.init_weights(seed, std)
        src = dict(full.named_parameters())
        for name, prm in self.named_parameters():
            if name.startswith("layers."):
                _, idx, rest = name.split(".", 2)
                key = f"layers.{self.layer_ids[int(idx)]}.{rest}"
            else:
                key = name
            prm.copy_(src[key])
        return self

    def _full_shape(self, name: str, p: torch.Tensor) -> tuple[int, ...]:
        tp = self.pctx.tp_size
        if name.endswith(("attn.o", "mlp.down")):
            return (p.shape[0], p.shape[1] * tp)
        return (p.shape[0] * tp,) + tuple(p.shape[1:])

    def output_weight(self) -> torch.Tensor:
        return self.embed if self.lm_head is None else self.lm_head

    def rope(self, device, max_pos=None):
        max_pos = max_pos or self.cfg.max_position_embeddings
        if self._rope is None or self._rope[0].device != torch.device(device) or self._rope[0].shape[0] < max_pos:
            self._rope = fused.rope_tables(max_pos, self.cfg.rotary_dim, self.cfg.rope_theta, device,
                                            self.cfg.rope_scaling or None)
        return self._rope

    # --------------------------------------------------------------- forward
    def forward(self, input_ids, position_ids, meta: VarlenMeta, attn_fn=None, stage_input=None,
                embeds=None, rope=None, layer_adds=None, chunk=None):
        """Packed forward; returns the final-normed hidden states ``[T, H]``. On a pipeline stage
        other than the first, ``stage_input = (x, res)`` are the activations received from the
        previous stage; a stage other than the last returns ``(x, res)`` for the next one.
        ``embeds`` replaces the embedding lookup and ``rope = (cos, sin)`` the rotary tables that
        ``position_ids`` index (a vision-language model passes image features merged into the token
        embeddings and one table row per token). ``layer_adds = (rows, [f_0, f_1, …])`` adds ``f_l`` to the
        hidden states of ``rows`` after block ``l`` (deep-stack vision features). ``chunk`` runs one of this rank's
        chunks of blocks only (virtual pipeline stages): the embedding belongs to chunk 0 of the first rank, the
        final norm to the last chunk of the last rank."""
        cos, sin = rope if rope is not None else self.rope(input_ids.device)
        pos = position_ids.to(torch.int32)
        p = self.pctx
        if p is not None and p.sp_size > 1 and attn_fn is None:
            from ..parallel.ulysses import ulysses_attention

            attn_fn = ulysses_attention(p)
        if stage_input is not None:
            x, res = stage_input
        elif embeds is not None:
            x, res = embeds, None  # under tensor parallelism: this rank's token rows, like the lookup below
        elif p is not None and p.tp_size > 1:
            # input_ids / position_ids hold every token of this sequence-parallel shard; the
            # vocab-parallel lookup leaves each tp rank with its T/tp rows
            from ..parallel.tensor_parallel import vocab_parallel_embedding

            x, res = vocab_parallel_embedding(input_ids, self.embed, p.tp_fused), None
        else:
            x, res = fused.embedding(input_ids, self.embed), None
        ckpt_every = getattr(self, "checkpoint_every", 0)
        policy = getattr(self, "ac_policy", None)
        lo, hi = (0, len(self.layers)) if chunk is None else self.chunk_slices[chunk]
        for li in range(lo, hi):
            layer = self.layers[li]
            whole = (ckpt_every and li % ckpt_every == 0) or (policy is not None and li in policy.full_layers)
            if whole and torch.is_grad_enabled():
                # activation checkpointing: keep only the block's inputs, recompute the rest in backward
                from torch.utils.checkpoint import checkpoint

                x, res = checkpoint(layer, x, res, cos, sin, pos, meta, attn_fn, use_reentrant=False)
            elif policy is not None and policy.mlp_only:
                x, res = layer(x, res, cos, sin, pos, meta, attn_fn, recompute_mlp=True)
            else:
                x, res = layer(x, res, cos, sin, pos, meta, attn_fn)
            if layer_adds is not None and li < len(layer_adds[1]):
                x = x.index_add(0, layer_adds[0], layer_adds[1][li].to(x.dtype))  # hidden = x + res: add to x
        if not self.last_stage or (chunk is not None and chunk != self.vpp - 1):
            return x, res
        y, _ = fused.rmsnorm(x, self.norm, self.cfg.rms_norm_eps, residual=res)
        if p is not None and p.tp_size > 1:
            from ..parallel.tensor_parallel import gather_seq, gather_seq_replicated

            # the vocab-parallel head needs every token and returns PARTIAL input gradients (summed
            # in the backward); a critic's value head is replicated work, so its backward only slices
            y = gather_seq_replicated(y, p.tp_fused) if self.cfg.is_critic else gather_seq(y, p.tp_fused)
        return y

    def logits(self, hidden, out_dtype=torch.float32):
        w = self.output_weight()
        if hidden.is_cuda and hidden.dtype == torch.bfloat16:
            return gemm(hidden, w, out_dtype=out_dtype)
        return F.linear(hidden, w).to(out_dtype)

    def values(self, hidden):
        if hidden.is_cuda:
            _lib.count_fallback("critic.value_head[F.linear fp32]")
        return F.linear(hidden.float(), self.score.float()).squeeze(-1)

    # -------------------------------------------------- rollout (paged cache)
    @torch.no_grad()
    def prefill(self, input_ids, position_ids, meta: VarlenMeta, kv_caches, slot_mapping, hybrid_state=None,
                state_slots=None, embeds=None, rope=None, layer_adds=None):
        """Packed prompt forward that also writes K/V of every layer into the
        paged caches; returns hidden states of all tokens. Hybrid models also take the per-sequence
        state of their linear-attention layers and the slot of every sequence in it. ``embeds`` /
        ``rope`` as in :meth:`forward` (image features merged into the embeddings, one rotary row per token)."""
        if self.cfg.is_hybrid:
            from .qwen3_5 import hybrid_prefill

            return hybrid_prefill(self, input_ids, position_ids, meta, kv_caches, slot_mapping, hybrid_state, state_slots)
        cos, sin = rope if rope is not None else self.rope(input_ids.device)
        pos = position_ids.to(torch.int32)
        x = embeds if embeds is not None else fused.embedding(input_ids, self.embed)
        res = None
        for i, layer in enumerate(self.layers):
            if res is None:
                y, res = fused.rmsnorm(x, layer.input_norm, layer.eps), x
            else:
                y, res = fused.rmsnorm(x, layer.input_norm, layer.eps, residual=res)
            if hasattr(layer.attn, "prefill"):  # a layer with recurrent state (lightning attention)
                a = layer.attn.prefill(y, pos, meta, hybrid_state.rec[i], state_slots)
            else:
                q, k, v = layer.attn.project_qkv(y, cos, sin, pos)
                kv_cache_write(k, v, slot_mapping, kv_caches[i][0], kv_caches[i][1])
                a = varlen_attention(q, k, v, meta)
                a = layer.attn.out_proj(a) if hasattr(layer.attn, "out_proj") else \
                    linear(a.reshape(a.shape[0], -1), layer.attn.o)
            y, res = fused.rmsnorm(a, layer.post_norm, layer.eps, residual=res)
            x = layer.mlp(y)
            if layer_adds is not None and i < len(layer_adds[1]):
                x = x.index_add(0, layer_adds[0], layer_adds[1][i].to(x.dtype))
        y, _ = fused.rmsnorm(x, self.norm, self.cfg.rms_norm_eps, residual=res)
        return y

    @torch.no_grad()
    def decode(self, input_ids, position_ids, kv_caches, block_table, seq_lens, slot_mapping,
               max_seq_len=None, hybrid_state=None, state_slots=None):
        """One new token per sequence: ``input_ids [B]`` at ``position_ids [B]``;
        ``seq_lens`` already counts the new token."""
        if self.cfg.is_hybrid:
            from .qwen3_5 import hybrid_decode

            return hybrid_decode(self, input_ids, position_ids, kv_caches, block_table, seq_lens, slot_mapping,
                                 hybrid_state, state_slots, max_seq_len)
        cos, sin = self.rope(input_ids.device)
        pos = position_ids.to(torch.int32)
        x = fused.embedding(input_ids, self.embed)
        res = None
        y = None  # normalised input of the next block, when the previous projection already produced it
        # A block of a plain dense model runs 9 kernels here instead of 13: k/v go into the cache from the
        # q/k-norm + RoPE kernel, and each residual add + RMSNorm runs inside the split-K reduction of the
        # projection in front of it (o-proj → post-norm, down-proj → the next block's input norm).
        tp1 = self.pctx is None or self.pctx.tp_size == 1
        plain = tp1 and not self.cfg.fp8 and not self.cfg.is_hybrid and not self.cfg.is_mla
        n_layers = len(self.layers)
        for i, layer in enumerate(self.layers):
            if y is None:
                if res is None:
                    y, res = fused.rmsnorm(x, layer.input_norm, layer.eps), x
                else:
                    y, res = fused.rmsnorm(x, layer.input_norm, layer.eps, residual=res)
            if hasattr(layer.attn, "step"):  # lightning attention: advances the sequence's recurrent state
                a = layer.attn.step(y, pos, hybrid_state.rec[i], state_slots)
                y, res = fused.rmsnorm(a, layer.post_norm, layer.eps, residual=res)
                x = layer.mlp(y)
                y = None
                continue
            q = layer.attn.project_q_write_kv(y, cos, sin, pos, slot_mapping, kv_caches[i][0], kv_caches[i][1])
            a = paged_decode(q, kv_caches[i][0], kv_caches[i][1], block_table, seq_lens,
                             max_seq_len=max_seq_len)
            if hasattr(layer.attn, "out_proj"):  # latent attention: drops the value padding itself
                y, res = fused.rmsnorm(layer.attn.out_proj(a), layer.post_norm, layer.eps, residual=res)
            elif plain and layer.attn.lora_o is None:
                y, res = linear_rmsnorm(a.reshape(a.shape[0], -1), layer.attn.o, layer.post_norm, layer.eps, res)
            else:
                y, res = fused.rmsnorm(linear(a.reshape(a.shape[0], -1), layer.attn.o), layer.post_norm, layer.eps,
                                       residual=res)
            m = layer.mlp
            if plain and isinstance(m, DenseMLP) and m.lora_gate_up is None and m.lora_down is None:
                nxt_w, nxt_eps = ((self.layers[i + 1].input_norm, self.layers[i + 1].eps) if i + 1 < n_layers
                                  else (self.norm, self.cfg.rms_norm_eps))
                h = fused.swiglu(linear(y, m.gate_up))
                y, res = linear_rmsnorm(h, m.down, nxt_w, nxt_eps, res)
                x = None
            else:
                x = m(y)
                y = None
        if y is None:
            y, _ = fused.rmsnorm(x, self.norm, self.cfg.rms_norm_eps, residual=res)
        return y

    # ------------------------------------------------------ HF name mapping
    _TP_DIM0 = ("embed_tokens.weight", "lm_head.weight", "q_proj.weight", "k_proj.weight", "v_proj.weight",
                "q_proj.bias", "k_proj.bias", "v_proj.bias", "gate_proj.weight", "up_proj.weight",
                "q_b_proj.weight", "kv_b_proj.weight")
    _TP_DIM1 = ("o_proj.weight", "down_proj.weight")

    def _tp_dim(self, hf_name: str) -> int | None:
        """Dimension along which an HF tensor is split over the tp group (None: replicated)."""
        if self.pctx is None or self.pctx.tp_size == 1 or ".experts." in hf_name or "shared_expert" in hf_name:
            return None  # (experts are split by expert; a shared expert is replicated over the group)
        if hf_name.endswith(self._TP_DIM0):
            return 0
        if hf_name.endswith(self._TP_DIM1):
            return 1
        return None

    def shard_spec(self, hf_name: str) -> tuple[int, int, int, Any] | None:
        """``(dimension, rank, size, group)`` of the split of an HF tensor over a model-parallel group, ``None``
        for a tensor this rank holds whole: dense projections over the tensor-parallel group, the projections of
        one expert over the expert-tensor-parallel group."""
        p = self.pctx
        if p is None:
            return None
        if ".experts." in hf_name:
            if p.etp_size == 1:
                return None
            dim = 1 if hf_name.endswith("down_proj.weight") else 0
            return dim, p.etp_rank, p.etp_size, p.etp_group
        dim = self._tp_dim(hf_name)
        return None if dim is None else (dim, p.tp_rank, p.tp_size, p.tp_group)

    def to_hf(self) -> Iterator[tuple[str, torch.Tensor]]:
        """Yields ``(hf_name, tensor)`` in HF checkpoint naming: views of the fused parameters, or,
        under tensor parallelism, full tensors gathered over the tp group (a collective: every tp
        rank must iterate)."""
        import torch.distributed as dist

        for name, t in self.to_hf_local(export=True):
            spec = self.shard_spec(name)
            if spec is None:
                yield self.checkpoint_name(name), t
            else:
                d, _, size, group = spec
                parts = [torch.empty_like(t) for _ in range(size)]
                dist.all_gather(parts, t.contiguous(), group=group)
                yield self.checkpoint_name(name), torch.cat(parts, d)
        for name, t in self._selection_biases():
            yield self.checkpoint_name(name), t

    def _selection_biases(self, always: bool = False):
        """The routers' selection biases of a family whose checkpoints carry them: buffers, not parameters (no
        gradient, not in the flat weight buffer), so they travel beside ``to_hf_local``'s tensors. ``always``: also
        those of a model that only balances with them during training (recover checkpoints keep them)."""
        if not (self.cfg.moe_expert_bias or always):
            return
        for i, layer in zip(self.layer_ids, self.layers):
            if getattr(layer.mlp, "expert_bias", None) is not None:
                yield f"model.layers.{i}.mlp.gate.e_score_correction_bias", layer.mlp.expert_bias

    # Families whose checkpoint files name the same tensors differently (Mixtral: ``block_sparse_moe`` with
    # experts ``w1`` / ``w3`` / ``w2``). Inside the package every tensor goes by the canonical (Qwen-style)
    # name; the translation happens where tensors enter (``load_hf``) or leave (``to_hf``).
    _MIXTRAL_PROJ = {"gate_proj": "w1", "up_proj": "w3", "down_proj": "w2"}

    _BAILING_NAMES = (("model.embed_tokens.weight", "model.word_embeddings.weight"),
                      (".mlp.gate.e_score_correction_bias", ".mlp.gate.expert_bias"))

    def checkpoint_name(self, name: str) -> str:
        if self.cfg.model_type == "bailing_hybrid":
            for ours, theirs in self._BAILING_NAMES:
                if name.endswith(ours):
                    return name[: len(name) - len(ours)] + theirs
            return name
        if self.cfg.model_type != "mixtral" or ".mlp." not in name:
            return name
        head, _, tail = name.partition(".mlp.")
        if tail == "gate.weight":
            return head + ".block_sparse_moe.gate.weight"
        m = re.match(r"experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$", tail)
        if m is not None:
            return f"{head}.block_sparse_moe.experts.{m.group(1)}.{self._MIXTRAL_PROJ[m.group(2)]}.weight"
        return name

    def canonical_name(self, name: str) -> str:
        if self.cfg.model_type == "bailing_hybrid":
            for ours, theirs in self._BAILING_NAMES:
                if name.endswith(theirs):
                    return name[: len(name) - len(theirs)] + ours
            return name
        if self.cfg.model_type != "mixtral" or ".block_sparse_moe." not in name:
            return name
        head, _, tail = name.partition(".block_sparse_moe.")
        if tail == "gate.weight":
            return head + ".mlp.gate.weight"
        m = re.match(r"experts\.(\d+)\.(w1|w2|w3)\.weight$", tail)
        if m is not None:
            proj = {v: k for k, v in self._MIXTRAL_PROJ.items()}[m.group(2)]
            return f"{head}.mlp.experts.{m.group(1)}.{proj}.weight"
        return name

    def to_hf_local(self, export: bool = False) -> Iterator[tuple[str, torch.Tensor]]:
        """``(hf_name, view)`` of this rank's (tp-local) parameters. Families whose checkpoints store
        RMSNorm weights 1-centred get ``w - 1`` copies instead of views when ``export`` is set."""
        cfg = self.cfg
        if cfg.is_hybrid:
            yield from self._to_hf_hybrid(export)
            return
        tp = self.pctx.tp_size if self.pctx is not None else 1
        if self.embed is not None and self.first_stage:
            yield "model.embed_tokens.weight", self.embed
        qs, ks = cfg.q_size // tp, cfg.kv_size // tp
        I = cfg.intermediate_size // tp
        for i, layer in zip(self.layer_ids, self.layers):
            p = f"model.layers.{i}."
            yield p + "input_layernorm.weight", layer.input_norm
            a = layer.attn
            if hasattr(a, "hf_tensors"):  # latent attention names its own projections
                yield from a.hf_tensors(p)
            else:
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
                Im = m.gate_up.shape[1] // 2  # the local width under expert tensor parallelism
                yield p + "mlp.gate.weight", m.router
                # under expert parallelism this rank holds (and names) experts [ep_rank * n, (ep_rank + 1) * n)
                n_loc = m.gate_up.shape[0]
                e0 = self.pctx.ep_rank * n_loc if (self.pctx is not None and self.pctx.ep_size > 1) else 0
                for e in range(n_loc):
                    q = p + f"mlp.experts.{e0 + e}."
                    yield q + "gate_proj.weight", m.gate_up[e, :Im]
                    yield q + "up_proj.weight", m.gate_up[e, Im:]
                    yield q + "down_proj.weight", m.down[e]
                yield from self._shared_expert_hf(p, m)
        if self.norm is not None:
            yield "model.norm.weight", self.norm
        if self.score is not None:
            yield "score.weight", self.score
        elif self.lm_head is not None:
            yield "lm_head.weight", self.lm_head

    def _shared_expert_hf(self, p: str, m):
        if getattr(m, "shared_gate_up", None) is None:
            return
        Is = self.cfg.shared_expert_intermediate_size
        q = p + ("mlp.shared_expert." if m.shared_gate is not None else "mlp.shared_experts.")
        yield q + "gate_proj.weight", m.shared_gate_up[:Is]
        yield q + "up_proj.weight", m.shared_gate_up[Is:]
        yield q + "down_proj.weight", m.shared_down
        if m.shared_gate is not None:
            yield p + "mlp.shared_expert_gate.weight", m.shared_gate

    def _to_hf_hybrid(self, export: bool):
        from .qwen3_5 import hf_tensors

        cfg = self.cfg
        nw = (lambda t: t - 1) if (export and cfg.norm_one_plus) else (lambda t: t)
        if self.embed is not None and self.first_stage:
            yield "model.embed_tokens.weight", self.embed
        I = cfg.intermediate_size
        for i, layer in zip(self.layer_ids, self.layers):
            p = f"model.layers.{i}."
            yield p + "input_layernorm.weight", nw(layer.input_norm)
            yield from hf_tensors(layer.attn, p, cfg, nw)
            yield p + "post_attention_layernorm.weight", nw(layer.post_norm)
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
                yield from self._shared_expert_hf(p, m)
        if self.norm is not None:
            yield "model.norm.weight", nw(self.norm)
        if self.score is not None:
            yield "score.weight", self.score
        elif self.lm_head is not None:
            yield "lm_head.weight", self.lm_head

    _ONE_PLUS = ("input_layernorm.weight", "post_attention_layernorm.weight", "model.norm.weight",
                 "self_attn.q_norm.weight", "self_attn.k_norm.weight")

    def hf_name_map(self) -> dict[str, torch.Tensor]:
        return dict(self.to_hf_local())

    def owned_by_other_stage(self, name: str) -> bool:
        """True for a checkpoint tensor that belongs to another pipeline stage: a block outside this
        stage's range, the embedding when this stage has none, the final norm / head off the last stage."""
        if len(self.layer_ids) == self.cfg.num_hidden_layers:
            return False
        m = re.match(r"model\.layers\.(\d+)\.", name)
        if m is not None:
            return int(m.group(1)) not in self.layer_ids
        if name == "model.embed_tokens.weight":
            return self.embed is None
        if name in ("model.norm.weight", "lm_head.weight", "score.weight"):
            return not self.last_stage
        return False

    @torch.no_grad()
    def load_hf(self, tensors: Iterable[tuple[str, torch.Tensor]], strict: bool = True):
        """Copies HF-named tensors into the fused parameters."""
        dst = self.hf_name_map()
        if self.embed is not None and not self.first_stage:
            dst["model.embed_tokens.weight"] = self.embed  # the last stage's copy of a tied embedding
        dst.update(self._selection_biases())
        seen = set()
        for name, t in tensors:
            if name.startswith("model.language_model."):  # decoder of a composite checkpoint
                name = "model." + name[len("model.language_model."):]
            name = self.canonical_name(name)
            if self.cfg.norm_one_plus and name.endswith(self._ONE_PLUS):
                t = t.float() + 1.0
            if name == "lm_head.weight" and self.lm_head is None and self.score is None:
                seen.add(name)
                continue  # tied
            if name not in dst:
                if ".mlp.experts." in name and self.pctx is not None and self.pctx.ep_size > 1:
                    continue  # an expert that lives on another expert-parallel rank
                if self.owned_by_other_stage(name):
                    continue
                if strict:
                    raise KeyError(f"unexpected tensor {name}")
                continue
            d = dst[name]
            spec = self.shard_spec(name)
            if spec is not None:
                dim, rank, size, _ = spec
                n = t.shape[dim] // size
                t = t.narrow(dim, rank * n, n)
            if d.shape != t.shape:
                raise ValueError(f"{name}: shape {tuple(t.shape)} != {tuple(d.shape)}")
            d.copy_(t.to(device=d.device, dtype=d.dtype))
            seen.add(name)
        missing = set(dst) - seen
        if strict and missing:
            raise KeyError(f"missing tensors: {sorted(missing)[:8]} ...")
        return self


def build_model(cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", seed: int | None = 0, pctx=None) -> QwenModel:
    if cfg.is_vl:
        from .qwen_vl import QwenVLModel

        m = QwenVLModel(cfg, dtype=dtype, device=device, pctx=pctx)
    else:
        m = QwenModel(cfg, dtype=dtype, device=device, pctx=pctx)
    if seed is not None:
        m.init_weights(seed)
    return m
