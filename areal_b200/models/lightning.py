"""Lightning attention: the linear-attention layer of the Bailing hybrid models (groups of layers in which all but
the last use it and the last uses latent softmax attention).

    q, k, v = split(W_qkv x)                       checkpoint layout [Q | K | V], heads of ``head_dim``
    q, k    = rmsnorm_head(q), rmsnorm_head(k)     one weight vector per projection, shared by the heads
    q, k    = rope(q, k) on the first ``rotary_dim`` columns of every head (half-split pairs)
    S_t     = exp(g_h) S_{t-1} + k_t v_t^T ;  o_t = S_t^T q_t / sqrt(head_dim)        per head h
    y       = W_o ( group_rmsnorm(o) * sigmoid(W_g x) )

The decay is not learned: ``g_h = -slope_h * (1 - layer / (layers - 1) + 1e-5)`` with the ALiBi slopes of the head
count (geometric sequence from ``2^(-8/n)``; head counts that are not powers of two interleave the next power's
slopes), so early layers forget fastest. The recurrence is ``ops/linear_attn.py``'s ``simple_gla`` mode with a
constant decay per head (chunk-parallel under autograd, the CUDA recurrence kernel without gradients).

Sequence parallelism (Ulysses): the recurrence needs every token of a sequence, in order, for the heads it runs;
q / k / v are rotated on the rank that holds the tokens, exchanged tokens → heads (each rank then runs ``heads /
sp`` heads over the whole packed stream with their slice of the decays), and the outputs are exchanged back.

Generation: the rollout engine keeps the state ``S [heads, head_dim, head_dim]`` (fp32) of every running sequence
per lightning layer (:class:`LightningState`); a prefill leaves the state after the prompt's last token there, a decode
step reads, advances and writes it back.

Checkpoint names: ``attention.{query_key_value,query_layernorm,key_layernorm,g_proj,g_norm,dense}``.
Reference: areal/models/mcore/lightning_attention.py:100-125 (slopes), :241-342 (core, decay per layer),
:345-385 (group norm), :387-672 (layer, head <-> sequence exchange under context parallelism).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import fused
from ..ops.attention import VarlenMeta
from ..ops.gemm import linear
from ..ops.linear_attn import linear_attn
from .config import ModelConfig


def alibi_slopes(n_heads: int) -> torch.Tensor:
    def power_of_two(n):
        start = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [start ** (i + 1) for i in range(n)]

    if math.log2(n_heads).is_integer():
        return torch.tensor(power_of_two(n_heads), dtype=torch.float32)
    below = 2 ** math.floor(math.log2(n_heads))
    extra = power_of_two(2 * below)[0::2][: n_heads - below]
    return torch.tensor(power_of_two(below) + extra, dtype=torch.float32)


def layer_log_decay(n_heads: int, layer_idx: int, n_layers: int) -> torch.Tensor:
    """``g [heads]`` (negative): the per-step log decay of every head in layer ``layer_idx`` (0-based)."""
    return -alibi_slopes(n_heads) * (1.0 - layer_idx / max(n_layers - 1, 1) + 1e-5)


def group_rmsnorm(x: torch.Tensor, w: torch.Tensor, n_groups: int, eps: float) -> torch.Tensor:
    """``x [T, H, D]``: RMS over each group of ``H / n_groups`` whole heads, then an element-wise weight ``[H * D]``."""
    T, H, D = x.shape
    xf = x.float().view(T, n_groups, (H // n_groups) * D)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y.view(T, H, D).to(x.dtype)) * w.view(H, D)


def _rope_partial(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rot: int) -> torch.Tensor:
    """Rotates the first ``rot`` columns of every head of ``x [T, H, D]`` (pairs ``(i, i + rot/2)``)."""
    if rot == 0:
        return x
    xr = x[..., :rot].float()
    a, b = xr.chunk(2, dim=-1)
    c, s = cos[:, None, :].float(), sin[:, None, :].float()
    out = torch.cat((a * c - b * s, b * c + a * s), dim=-1).to(x.dtype)
    return torch.cat((out, x[..., rot:]), dim=-1) if rot < x.shape[-1] else out


class LightningState:
    """``rec[i] [slots, heads, head_dim, head_dim]`` fp32 for lightning layer ``i``, ``None`` for the others."""

    def __init__(self, cfg: ModelConfig, max_slots: int, dtype, device):
        D = cfg.lightning_head_dim
        self.rec = [torch.zeros(max_slots, cfg.num_attention_heads, D, D, dtype=torch.float32, device=device)
                    if cfg.layer_is_lightning(i) else None for i in range(cfg.num_hidden_layers)]


class LightningAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, pctx=None, layer_idx: int = 0):
        super().__init__()
        if pctx is not None and pctx.tp_size > 1:
            raise NotImplementedError("the Bailing hybrid family does not run under tensor parallelism: use data, "
                                      "sequence, pipeline and expert parallelism")
        self.cfg, self.pctx = cfg, pctx
        h, nh, D = cfg.hidden_size, cfg.num_attention_heads, cfg.lightning_head_dim
        self.nh, self.D = nh, D
        self.rot = int(D * cfg.partial_rotary_factor) // 2 * 2
        self.n_groups = max(int(cfg.lightning_norm_groups), 1)
        sp = pctx.sp_size if pctx is not None else 1
        assert nh % self.n_groups == 0, "the gate norm's groups must hold whole heads"
        assert nh % sp == 0, "sequence parallelism needs the head count to divide by its size"
        mk = lambda *shape: nn.Parameter(torch.empty(*shape, dtype=dtype, device=device))
        ones = lambda n: nn.Parameter(torch.ones(n, dtype=dtype, device=device))
        self.qkv = mk(3 * nh * D, h)
        self.q_norm, self.k_norm = ones(D), ones(D)
        self.gate = mk(nh * D, h)
        self.g_norm = ones(nh * D)
        self.o = mk(h, nh * D)
        self.register_buffer("log_decay", layer_log_decay(nh, layer_idx, cfg.num_hidden_layers).to(device),
                             persistent=False)
        self._tables = None

    def _rope_tables(self, device, n: int):
        # the layer's own table: ``rot`` columns at the model's base, no long-context scaling
        t = self._tables
        if t is None or t[0].device != torch.device(device) or t[0].shape[0] < n:
            self._tables = fused.rope_tables(max(n, self.cfg.max_position_embeddings), self.rot, self.cfg.rope_theta,
                                             device)
        return self._tables

    def _qkv(self, x, pos):
        cfg, T, nh, D = self.cfg, x.shape[0], self.nh, self.D
        qkv = linear(x, self.qkv).view(T, 3, nh, D)
        q = fused.rmsnorm(qkv[:, 0].contiguous(), self.q_norm, cfg.rms_norm_eps)
        k = fused.rmsnorm(qkv[:, 1].contiguous(), self.k_norm, cfg.rms_norm_eps)
        v = qkv[:, 2]
        if self.rot:
            p = pos.long()
            c, s = self._rope_tables(x.device, int(p.max()) + 1 if p.numel() else 1)
            q, k = _rope_partial(q, c[p], s[p], self.rot), _rope_partial(k, c[p], s[p], self.rot)
        return q, k, v

    def _gate_out(self, o, x):
        T, nh, D = x.shape[0], self.nh, self.D
        o = group_rmsnorm(o, self.g_norm, self.n_groups, self.cfg.rms_norm_eps)
        o = o * torch.sigmoid(linear(x, self.gate).view(T, nh, D).float()).to(o.dtype)
        return linear(o.reshape(T, nh * D), self.o)

    @torch.no_grad()
    def prefill(self, x, pos, meta: VarlenMeta, rec: torch.Tensor, slots: torch.Tensor):
        """Prompt forward of a rollout engine: also leaves every sequence's final state in ``rec[slots]``."""
        from ..ops.linear_attn import linear_attn_prefill

        q, k, v = self._qkv(x, pos)
        a = self.log_decay.exp()[None, :].expand(q.shape[0], -1)
        o, final = linear_attn_prefill(q.contiguous(), k.contiguous(), v.contiguous(), a, None, meta.cu_seqlens,
                                       self.D ** -0.5, mode="simple_gla")
        rec[slots] = final
        return self._gate_out(o, x)

    @torch.no_grad()
    def step(self, x, pos, rec: torch.Tensor, slots: torch.Tensor):
        """One new token per sequence: advances ``rec[slots]``."""
        from ..ops.linear_attn import linear_attn_step

        q, k, v = self._qkv(x, pos)
        a = self.log_decay.exp()[None, :].expand(q.shape[0], -1)
        o, new = linear_attn_step(q, k, v, a, None, rec[slots], self.D ** -0.5, mode="simple_gla")
        rec[slots] = new
        return self._gate_out(o, x)

    def forward(self, x, cos, sin, pos, meta: VarlenMeta, attn_fn=None):
        T, nh, D = x.shape[0], self.nh, self.D
        q, k, v = self._qkv(x, pos)
        g = self.log_decay
        pc = self.pctx
        sharded = pc is not None and pc.sp_size > 1
        if sharded:
            from ..parallel.ulysses import head_to_seq, seq_to_head

            q, k, v = seq_to_head(q.contiguous(), pc), seq_to_head(k.contiguous(), pc), seq_to_head(v.contiguous(), pc)
            hs = nh // pc.sp_size
            g = g[pc.sp_rank * hs:(pc.sp_rank + 1) * hs]
        a = g.exp()[None, :].expand(q.shape[0], -1)
        o = linear_attn(q.contiguous(), k.contiguous(), v.contiguous(), a, None, meta.cu_seqlens, D ** -0.5,
                        mode="simple_gla")
        if sharded:
            o = head_to_seq(o.contiguous(), pc)
        return self._gate_out(o, x)

    def hf_tensors(self, p: str):
        yield p + "attention.query_key_value.weight", self.qkv
        yield p + "attention.query_layernorm.weight", self.q_norm
        yield p + "attention.key_layernorm.weight", self.k_norm
        yield p + "attention.g_proj.weight", self.gate
        yield p + "attention.g_norm.weight", self.g_norm
        yield p + "attention.dense.weight", self.o
