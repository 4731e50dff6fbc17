"""Qwen3.5 hybrid layers: gated full attention and GatedDeltaNet linear attention.

A Qwen3.5 decoder alternates ``linear_attention`` layers (GatedDeltaNet: fused input projection →
causal depthwise conv1d + SiLU → L2-normalised q/k → gated delta rule → per-head gated RMSNorm →
output projection) with ``full_attention`` layers whose query projection is twice as wide (query
and an output gate per head), with q/k RMSNorm, rotary embedding on the first
``partial_rotary_factor`` of the head dimensions only, and ``sigmoid(gate)`` on the attention
output. RMSNorm weights are "1-centred" in checkpoints (``(1 + w) * norm(x)``); this model stores
the effective multiplier ``1 + w`` so the same fused RMSNorm kernels serve every family, and the
checkpoint reader / writer adds and subtracts the one.

The fused input projection holds, in row order, ``in_proj_qkv`` (q, k, v of the conv channels),
``in_proj_z``, ``in_proj_a``, ``in_proj_b``; the attention projection holds ``q_proj`` (per head:
query then gate, the checkpoint's own layout), ``k_proj``, ``v_proj``.

Kernels: the projections run on the tcgen05 GEMM, the convolution on ``csrc/linear_attn.cu``
(forward and backward), the recurrence on its forward kernel when no gradient is needed and on the
chunk-parallel form (``ops.linear_attn.linear_attn_chunked``) under autograd; attention with head
dimension 128 runs the tcgen05 attention kernels, other head dimensions (Qwen3.5 ships 256) fall
back to PyTorch scaled-dot-product attention per sequence.

Rollout: full-attention layers use the paged KV cache like every other family; a linear-attention
layer keeps, per running sequence, its recurrent state ``S [heads, dk, dv]`` (fp32) and the last
``K - 1`` inputs of its convolution (:class:`HybridState`). Prefill computes both from the prompt
(the recurrence kernel returns its final state), a decode step advances them by one token with
batched tensor ops (:func:`hybrid_prefill`, :func:`hybrid_decode`).

Reference: areal/experimental/models/archon/qwen3_5/model/model.py (GatedDeltaNet :141-336,
GatedAttention :344-470, norms :31-92), rope.py :90-126, state_dict_adapter.py :45-88.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import fused
from ..ops.attention import VarlenMeta, attention_ref, varlen_attention
from ..ops.gemm import linear
from ..ops.linear_attn import causal_conv1d, linear_attn, linear_attn_prefill, linear_attn_step
from ..ops.rollout_ops import kv_cache_write, paged_decode
from .config import ModelConfig


def _partial_rope(x, cos, sin, pos, rotary_dim: int):
    """Rotates the first ``rotary_dim`` dimensions (rotate-half pairing inside them)."""
    c = cos[pos.long()][:, None, :].float()
    s = sin[pos.long()][:, None, :].float()
    c, s = torch.cat((c, c), -1), torch.cat((s, s), -1)
    xr, xp = x[..., :rotary_dim].float(), x[..., rotary_dim:]
    h = rotary_dim // 2
    rot = torch.cat((-xr[..., h:], xr[..., :h]), -1)
    return torch.cat(((xr * c + rot * s).to(x.dtype), xp), -1)


def _sdpa_varlen(q, k, v, meta: VarlenMeta, scale: float):
    """Causal attention per packed sequence through PyTorch SDPA (head dimensions the tcgen05
    kernels do not cover)."""
    if not q.is_cuda:
        return attention_ref(q, k, v, meta.cu_cpu, scale)
    cu = [int(c) for c in meta.cu_cpu]
    outs = []
    for s, e in zip(cu[:-1], cu[1:]):
        if e > s:
            o = F.scaled_dot_product_attention(q[s:e].transpose(0, 1)[None], k[s:e].transpose(0, 1)[None],
                                               v[s:e].transpose(0, 1)[None], is_causal=True, scale=scale,
                                               enable_gqa=True)
            outs.append(o[0].transpose(0, 1))
    return torch.cat(outs, 0) if outs else torch.zeros_like(q)


class GatedAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, pctx=None, layer_idx: int = 0):
        super().__init__()
        assert pctx is None or pctx.tp_size == 1, "hybrid models run under data / sequence parallelism"
        self.cfg, self.pctx = cfg, pctx
        self.n_q, self.n_kv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        h = cfg.hidden_size
        self.qkv = nn.Parameter(torch.empty(2 * self.n_q * D + 2 * self.n_kv * D, h, dtype=dtype, device=device))
        self.qkv_bias = None
        self.o = nn.Parameter(torch.empty(h, self.n_q * D, dtype=dtype, device=device))
        self.q_norm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
        self.k_norm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))

    def forward(self, x, cos, sin, pos, meta: VarlenMeta, attn_fn=None):
        cfg = self.cfg
        T, D, nq, nkv = x.shape[0], cfg.head_dim, self.n_q, self.n_kv
        qkv = linear(x, self.qkv)
        qg = qkv[:, :2 * nq * D].view(T, nq, 2 * D)
        q, gate = qg[..., :D], qg[..., D:]
        k = qkv[:, 2 * nq * D: (2 * nq + nkv) * D].view(T, nkv, D)
        v = qkv[:, (2 * nq + nkv) * D:].view(T, nkv, D)
        q = fused.rmsnorm_ref(q, self.q_norm, cfg.rms_norm_eps)
        k = fused.rmsnorm_ref(k, self.k_norm, cfg.rms_norm_eps)
        R = cfg.rotary_dim
        q = _partial_rope(q, cos, sin, pos, R).contiguous()
        k = _partial_rope(k, cos, sin, pos, R).contiguous()
        scale = 1.0 / math.sqrt(D)
        if attn_fn is not None:
            a = attn_fn(q, k, v, meta)
        elif D == 128:
            a = varlen_attention(q, k, v.contiguous(), meta, scale)
        else:
            a = _sdpa_varlen(q, k, v, meta, scale)
        a = (a.float() * torch.sigmoid(gate.float())).to(x.dtype)
        return linear(a.reshape(T, nq * D), self.o)


    # -- rollout ------------------------------------------------------------------------------
    def _qkv_gate(self, x, cos, sin, pos):
        cfg = self.cfg
        T, D, nq, nkv = x.shape[0], cfg.head_dim, self.n_q, self.n_kv
        qkv = linear(x, self.qkv)
        qg = qkv[:, :2 * nq * D].view(T, nq, 2 * D)
        q, gate = qg[..., :D], qg[..., D:]
        k = qkv[:, 2 * nq * D: (2 * nq + nkv) * D].view(T, nkv, D)
        v = qkv[:, (2 * nq + nkv) * D:].view(T, nkv, D)
        q = fused.rmsnorm_ref(q, self.q_norm, cfg.rms_norm_eps)
        k = fused.rmsnorm_ref(k, self.k_norm, cfg.rms_norm_eps)
        q = _partial_rope(q, cos, sin, pos, cfg.rotary_dim).contiguous()
        k = _partial_rope(k, cos, sin, pos, cfg.rotary_dim).contiguous()
        return q, k, v.contiguous(), gate

    def _finish(self, a, gate, dtype):
        a = (a.float() * torch.sigmoid(gate.float())).to(dtype)
        return linear(a.reshape(a.shape[0], -1), self.o)

    @torch.no_grad()
    def prefill(self, x, cos, sin, pos, meta, slot_mapping, k_cache, v_cache):
        q, k, v, gate = self._qkv_gate(x, cos, sin, pos)
        kv_cache_write(k, v, slot_mapping, k_cache, v_cache)
        D = self.cfg.head_dim
        scale = 1.0 / math.sqrt(D)
        a = varlen_attention(q, k, v, meta, scale) if D == 128 else _sdpa_varlen(q, k, v, meta, scale)
        return self._finish(a, gate, x.dtype)

    @torch.no_grad()
    def decode(self, x, cos, sin, pos, k_cache, v_cache, block_table, seq_lens, slot_mapping, max_seq_len=None):
        q, k, v, gate = self._qkv_gate(x, cos, sin, pos)
        kv_cache_write(k, v, slot_mapping, k_cache, v_cache)
        a = paged_decode(q, k_cache, v_cache, block_table, seq_lens, max_seq_len=max_seq_len)
        return self._finish(a, gate, x.dtype)


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, pctx=None, layer_idx: int = 0):
        super().__init__()
        assert pctx is None or (pctx.tp_size == 1 and pctx.sp_size == 1), \
            "GatedDeltaNet layers run under data parallelism"
        self.cfg = cfg
        self.nk, self.nv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        self.dk, self.dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        assert self.nv % self.nk == 0
        self.key_dim, self.value_dim = self.nk * self.dk, self.nv * self.dv
        self.conv_dim = 2 * self.key_dim + self.value_dim
        h = cfg.hidden_size
        self.in_proj = nn.Parameter(torch.empty(self.conv_dim + self.value_dim + 2 * self.nv, h,
                                                dtype=dtype, device=device))
        self.conv_w = nn.Parameter(torch.empty(self.conv_dim, cfg.linear_conv_kernel_dim, dtype=dtype, device=device))
        # the decay parameters live in the model dtype with everything else (one flat buffer); the
        # forward lifts them to fp32 before exp / softplus
        self.dt_bias = nn.Parameter(torch.ones(self.nv, dtype=dtype, device=device))
        self.A_log = nn.Parameter(torch.zeros(self.nv, dtype=dtype, device=device))
        self.gate_norm = nn.Parameter(torch.ones(self.dv, dtype=dtype, device=device))
        self.out_proj = nn.Parameter(torch.empty(h, self.value_dim, dtype=dtype, device=device))

    @torch.no_grad()
    def init_special(self, gen: torch.Generator):
        """``A`` uniform in (0, 16) (log-space parameter), ``dt_bias`` ones, conv taps ~ U(±1/sqrt(K))."""
        a = torch.empty(self.nv).uniform_(1e-3, 16.0, generator=gen)
        self.A_log.copy_(a.log().to(self.A_log.dtype))
        self.dt_bias.fill_(1.0)
        self.gate_norm.fill_(1.0)
        K = self.conv_w.shape[1]
        w = (torch.rand(self.conv_dim, K, generator=gen) * 2 - 1) / math.sqrt(K)
        self.conv_w.copy_(w.to(self.conv_w.dtype))

    def forward(self, x, cos, sin, pos, meta: VarlenMeta, attn_fn=None):
        assert attn_fn is None, "linear-attention layers take no external attention function"
        T = x.shape[0]
        nk, nv, dk, dv = self.nk, self.nv, self.dk, self.dv
        y = linear(x, self.in_proj)
        mixed = y[:, :self.conv_dim]
        z = y[:, self.conv_dim: self.conv_dim + self.value_dim]
        a = y[:, self.conv_dim + self.value_dim: self.conv_dim + self.value_dim + nv]
        b = y[:, self.conv_dim + self.value_dim + nv:]
        cu = meta.cu_seqlens
        mixed = causal_conv1d(mixed.contiguous(), self.conv_w, None, cu, activation=True)
        q = mixed[:, :self.key_dim].reshape(T, nk, dk).float()
        k = mixed[:, self.key_dim: 2 * self.key_dim].reshape(T, nk, dk).float()
        v = mixed[:, 2 * self.key_dim:].reshape(T, nv, dv)
        q = (q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6)).to(x.dtype)
        k = (k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)).to(x.dtype)
        if nv > nk:
            q = q.repeat_interleave(nv // nk, dim=1)
            k = k.repeat_interleave(nv // nk, dim=1)
        beta = torch.sigmoid(b.float())
        g = -torch.exp(self.A_log.float()) * F.softplus(a.float() + self.dt_bias.float())
        o = linear_attn(q, k, v, torch.exp(g), beta, cu, scale=dk ** -0.5, mode="gated_delta")
        # per-head gated RMSNorm: weight * norm(o) * silu(z)
        of = o.float()
        of = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + self.cfg.rms_norm_eps)
        of = (self.gate_norm.float() * of.to(x.dtype).float()) * F.silu(z.reshape(T, nv, dv).float())
        return linear(of.to(x.dtype).reshape(T, self.value_dim), self.out_proj)


def _gdn_project(m: "GatedDeltaNet", x):
    y = linear(x, m.in_proj)
    c, vd, nv = m.conv_dim, m.value_dim, m.nv
    return y[:, :c], y[:, c:c + vd], y[:, c + vd:c + vd + nv], y[:, c + vd + nv:]


def _gdn_heads(m: "GatedDeltaNet", mixed, a, b, dtype):
    """Conv output → L2-normalised q/k, v, decay and write strength, all per value head."""
    T = mixed.shape[0]
    q = mixed[:, :m.key_dim].reshape(T, m.nk, m.dk).float()
    k = mixed[:, m.key_dim: 2 * m.key_dim].reshape(T, m.nk, m.dk).float()
    v = mixed[:, 2 * m.key_dim:].reshape(T, m.nv, m.dv)
    q = (q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6)).to(dtype)
    k = (k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)).to(dtype)
    if m.nv > m.nk:
        q = q.repeat_interleave(m.nv // m.nk, dim=1)
        k = k.repeat_interleave(m.nv // m.nk, dim=1)
    beta = torch.sigmoid(b.float())
    decay = torch.exp(-torch.exp(m.A_log.float()) * F.softplus(a.float() + m.dt_bias.float()))
    return q, k, v, decay, beta


def _gdn_out(m: "GatedDeltaNet", o, z, dtype):
    T = o.shape[0]
    of = o.float()
    of = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + m.cfg.rms_norm_eps)
    of = (m.gate_norm.float() * of.to(dtype).float()) * F.silu(z.reshape(T, m.nv, m.dv).float())
    return linear(of.to(dtype).reshape(T, m.value_dim), m.out_proj)


@torch.no_grad()
def gdn_prefill(m: "GatedDeltaNet", x, meta: VarlenMeta, conv_state, rec_state, state_slots):
    """Prompt forward of a linear-attention layer that also leaves, for every sequence, the last ``K - 1``
    convolution inputs and the final recurrent state in ``conv_state`` / ``rec_state`` at ``state_slots``."""
    mixed_in, z, a, b = _gdn_project(m, x)
    mixed_in = mixed_in.contiguous()
    cu = meta.cu_seqlens
    mixed = causal_conv1d(mixed_in, m.conv_w, None, cu, activation=True)
    q, k, v, decay, beta = _gdn_heads(m, mixed, a, b, x.dtype)
    o, final = linear_attn_prefill(q, k, v, decay, beta, cu, scale=m.dk ** -0.5, mode="gated_delta")
    K1 = m.conv_w.shape[1] - 1
    cu_l = [int(c) for c in meta.cu_cpu]
    for i, (s0, s1) in enumerate(zip(cu_l[:-1], cu_l[1:])):
        tail = mixed_in[max(s0, s1 - K1):s1]                    # [<=K-1, C]
        st = conv_state[state_slots[i]]
        st.zero_()
        if tail.shape[0]:
            st[:, K1 - tail.shape[0]:] = tail.t()
    rec_state.index_copy_(0, state_slots, final)
    return _gdn_out(m, o, z, x.dtype)


@torch.no_grad()
def gdn_decode(m: "GatedDeltaNet", x, conv_state, rec_state, state_slots):
    """One token per sequence: advances the convolution window and the recurrent state in place."""
    mixed_in, z, a, b = _gdn_project(m, x)
    win = torch.cat([conv_state.index_select(0, state_slots), mixed_in.unsqueeze(-1).to(conv_state.dtype)], -1)  # [B, C, K]
    conv_state.index_copy_(0, state_slots, win[..., 1:].contiguous())
    mixed = F.silu((win.float() * m.conv_w.float()).sum(-1)).to(x.dtype)
    q, k, v, decay, beta = _gdn_heads(m, mixed, a, b, x.dtype)
    S = rec_state.index_select(0, state_slots)
    o, S = linear_attn_step(q, k, v, decay, beta, S, scale=m.dk ** -0.5, mode="gated_delta")
    rec_state.index_copy_(0, state_slots, S)
    return _gdn_out(m, o, z, x.dtype)


class HybridState:
    """Per-sequence state of the linear-attention layers of a rollout engine: for layer ``i`` (None for
    full-attention layers) ``conv[i] [slots, conv_dim, K - 1]`` and ``rec[i] [slots, heads, dk, dv]`` (fp32)."""

    def __init__(self, cfg: ModelConfig, max_slots: int, dtype, device):
        self.conv, self.rec = [], []
        nk, nv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        conv_dim = 2 * nk * cfg.linear_key_head_dim + nv * cfg.linear_value_head_dim
        for i in range(cfg.num_hidden_layers):
            if cfg.layer_type(i) == "linear_attention":
                self.conv.append(torch.zeros(max_slots, conv_dim, cfg.linear_conv_kernel_dim - 1, dtype=dtype, device=device))
                self.rec.append(torch.zeros(max_slots, nv, cfg.linear_key_head_dim, cfg.linear_value_head_dim,
                                            dtype=torch.float32, device=device))
            else:
                self.conv.append(None)
                self.rec.append(None)


def _run_blocks(model, x, attn_step):
    """The residual / norm / MLP skeleton shared by prefill and decode; ``attn_step(i, layer, y)`` runs the
    token mixer of block ``i``."""
    res = None
    for i, layer in enumerate(model.layers):
        if res is None:
            y, res = fused.rmsnorm(x, layer.input_norm, layer.eps), x
        else:
            y, res = fused.rmsnorm(x, layer.input_norm, layer.eps, residual=res)
        a = attn_step(i, layer, y)
        y, res = fused.rmsnorm(a, layer.post_norm, layer.eps, residual=res)
        x = layer.mlp(y)
    y, _ = fused.rmsnorm(x, model.norm, model.cfg.rms_norm_eps, residual=res)
    return y


@torch.no_grad()
def hybrid_prefill(model, input_ids, position_ids, meta, kv_caches, slot_mapping, state: HybridState, state_slots):
    cos, sin = model.rope(input_ids.device)
    pos = position_ids.to(torch.int32)
    x = fused.embedding(input_ids, model.embed)

    def step(i, layer, y):
        if isinstance(layer.attn, GatedDeltaNet):
            return gdn_prefill(layer.attn, y, meta, state.conv[i], state.rec[i], state_slots)
        return layer.attn.prefill(y, cos, sin, pos, meta, slot_mapping, kv_caches[i][0], kv_caches[i][1])

    return _run_blocks(model, x, step)


@torch.no_grad()
def hybrid_decode(model, input_ids, position_ids, kv_caches, block_table, seq_lens, slot_mapping, state: HybridState,
                  state_slots, max_seq_len=None):
    cos, sin = model.rope(input_ids.device)
    pos = position_ids.to(torch.int32)
    x = fused.embedding(input_ids, model.embed)

    def step(i, layer, y):
        if isinstance(layer.attn, GatedDeltaNet):
            return gdn_decode(layer.attn, y, state.conv[i], state.rec[i], state_slots)
        return layer.attn.decode(y, cos, sin, pos, kv_caches[i][0], kv_caches[i][1], block_table, seq_lens,
                                 slot_mapping, max_seq_len)

    return _run_blocks(model, x, step)


def hf_tensors(layer_attn, prefix: str, cfg: ModelConfig, norm_out):
    """``(hf_name, tensor)`` of one hybrid attention module; ``norm_out`` maps an effective norm
    weight to its checkpoint form (identity for loading views, ``w - 1`` for export)."""
    if isinstance(layer_attn, GatedDeltaNet):
        m, p = layer_attn, prefix + "linear_attn."
        c, vd, nv = m.conv_dim, m.value_dim, m.nv
        yield p + "in_proj_qkv.weight", m.in_proj[:c]
        yield p + "in_proj_z.weight", m.in_proj[c:c + vd]
        yield p + "in_proj_a.weight", m.in_proj[c + vd:c + vd + nv]
        yield p + "in_proj_b.weight", m.in_proj[c + vd + nv:]
        yield p + "conv1d.weight", m.conv_w.unsqueeze(1)  # [C, 1, K] as nn.Conv1d stores it
        yield p + "A_log", m.A_log
        yield p + "dt_bias", m.dt_bias
        yield p + "norm.weight", m.gate_norm
        yield p + "out_proj.weight", m.out_proj
    else:
        m, p = layer_attn, prefix + "self_attn."
        D = cfg.head_dim
        nq, nkv = m.n_q, m.n_kv
        yield p + "q_proj.weight", m.qkv[:2 * nq * D]
        yield p + "k_proj.weight", m.qkv[2 * nq * D:(2 * nq + nkv) * D]
        yield p + "v_proj.weight", m.qkv[(2 * nq + nkv) * D:]
        yield p + "q_norm.weight", norm_out(m.q_norm)
        yield p + "k_norm.weight", norm_out(m.k_norm)
        yield p + "o_proj.weight", m.o
