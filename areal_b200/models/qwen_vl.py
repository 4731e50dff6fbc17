"""Qwen2.5-VL, Qwen2-VL, Qwen3-VL and Qwen3-VL-MoE: a vision transformer in front of the Qwen2 decoder with multimodal rotary positions.

The decoder is the package's ``QwenModel`` unchanged (fused projections, own kernels); this module adds

* ``VisionTower``: patch embedding (the 3-D convolution with stride = kernel is one GEMM over flattened
  patches), blocks of RMSNorm → attention with 2-D rotary embedding → SwiGLU MLP, where most blocks attend inside
  windows of ``window_size`` pixels and the ``fullatt_block_indexes`` blocks inside a whole image, and the
  merger that turns each ``spatial_merge_size²`` group of patches into one decoder token. The Qwen2-VL tower is
  the same skeleton with LayerNorm, a fc1 → quick-GELU → fc2 MLP and no windows; the Qwen3-VL tower adds a learned
  position table (interpolated to each image's grid) and "deep-stack" mergers whose outputs are added to the
  decoder's hidden states at the image rows after its first blocks;
* ``mrope_position_ids`` / ``mrope_tables``: every token gets a (temporal, height, width) position triple (text
  tokens: three equal values; image tokens: their grid coordinates offset by the running position) and the rotary
  frequencies are split over the three axes by ``mrope_section``. The decoder's rotary kernels read a table row per
  token, so the multimodal table is built per packed batch and indexed by the token's row number;
* ``QwenVLModel``: embeds tokens, overwrites the rows of image placeholders with the tower's output and runs the
  decoder. Without pixel inputs it is exactly the text model.

The tower runs on PyTorch library operators (its head size of 80 and non-causal windowed attention are outside the
shapes the package's attention kernels take); segments of equal length are batched into one attention call.

Reference behaviour: the vision-language path of areal/engine/fsdp_engine.py (``multi_modal_input`` carrying
``pixel_values`` / ``image_grid_thw``, positions from the HF model's ``get_rope_index``) and
areal/models/transformers/{qwen2_vl,qwen3_vl}.py.
"""

from __future__ import annotations

from typing import Iterable, Iterator, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import fused
from ..ops.attention import VarlenMeta
from .config import ModelConfig
from .qwen import QwenModel


# ------------------------------------------------------------------------------------------ positions


def mrope_position_ids(input_ids: Sequence[int], cu_seqlens: Sequence[int], grids: Sequence[Sequence[int]],
                       cfg: ModelConfig, second_per_grid: Sequence[float] | None = None):
    """Position triples of a packed batch.

    ``grids``: ``(t, h, w)`` patch counts of every image / video in the order their placeholder runs appear.
    Returns ``(pos [3, T] int64, deltas)``; ``deltas[i]`` = (next position after sequence ``i``) − (its length): a
    generation step ``k`` tokens past the prompt sits at position ``len + k + delta`` on all three axes."""
    merge = int(cfg.vision.get("spatial_merge_size", 2))
    tps = float(cfg.vision.get("tokens_per_second", 1))
    vis = (cfg.image_token_id, cfg.video_token_id)
    ids = list(input_ids)
    out = torch.empty(3, len(ids), dtype=torch.long)
    deltas, gi = [], 0
    for a, b in zip(cu_seqlens[:-1], cu_seqlens[1:]):
        cur, i = 0, a
        while i < b:
            if ids[i] not in vis:
                j = i
                while j < b and ids[j] not in vis:
                    j += 1
                out[:, i:j] = torch.arange(cur, cur + j - i)
                cur += j - i
                i = j
                continue
            if gi >= len(grids):
                raise ValueError("more image placeholder runs than image grids")
            t, h, w = (int(x) for x in grids[gi])
            hh, ww = h // merge, w // merge
            n = t * hh * ww
            if i + n > b or any(ids[k] != ids[i] for k in range(i, i + n)):
                raise ValueError(f"image {gi} needs {n} placeholder tokens in a row at offset {i - a}")
            if ids[i] == cfg.video_token_id:
                sec = float(second_per_grid[gi]) if second_per_grid is not None else 1.0
                tt = (torch.arange(t).float() * sec * tps).long()
            else:
                tt = torch.zeros(t, dtype=torch.long)
            out[0, i:i + n] = cur + tt.repeat_interleave(hh * ww)
            out[1, i:i + n] = cur + torch.arange(hh).repeat_interleave(ww).repeat(t)
            out[2, i:i + n] = cur + torch.arange(ww).repeat(t * hh)
            cur = int(out[:, i:i + n].max()) + 1
            gi += 1
            i += n
        deltas.append(cur - (b - a))
    if gi != len(grids):
        raise ValueError(f"{len(grids)} image grids but only {gi} placeholder runs")
    return out, deltas


def mrope_tables(pos3: torch.Tensor, rotary_dim: int, theta: float, sections: Sequence[int],
                 interleaved: bool = False):
    """``cos, sin [T, rotary_dim / 2]``: frequency ``j`` rotates by the position on the axis that owns it.
    Chunked layout (Qwen2-VL / 2.5-VL): the first ``sections[0]`` frequencies follow the temporal axis, the next
    the height, the rest the width. Interleaved (Qwen3-VL): axes alternate t, h, w, t, h, w, … while the height
    and width sections last, the remaining frequencies are temporal."""
    assert sum(sections) == rotary_dim // 2, f"mrope_section {list(sections)} must sum to {rotary_dim // 2}"
    dev = pos3.device
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32, device=dev) / rotary_dim))
    if interleaved:
        j = torch.arange(rotary_dim // 2, device=dev)
        axis = torch.zeros_like(j)
        for a in (1, 2):
            axis[(j % 3 == a) & (j < 3 * sections[a])] = a
    else:
        axis = torch.repeat_interleave(torch.arange(3, device=dev), torch.tensor(list(sections), device=dev))
    fr = pos3[axis].t().float() * inv
    return fr.cos().contiguous(), fr.sin().contiguous()


# ------------------------------------------------------------------------------------------ vision tower


def _rot_half(x):
    d = x.shape[-1] // 2
    return torch.cat((-x[..., d:], x[..., :d]), -1)


def _segment_attention(q, k, v, cu: list[int]):
    """Bidirectional attention inside each ``[cu[i], cu[i+1])`` segment. ``q, k, v``: ``[N, heads, d]``.
    Segments of one length share a batched call (windows of a block all have the same few sizes)."""
    out = torch.empty_like(q)
    by_len: dict[int, list[int]] = {}
    for a, b in zip(cu[:-1], cu[1:]):
        if b > a:
            by_len.setdefault(b - a, []).append(a)
    for n, starts in by_len.items():
        idx = (torch.tensor(starts, device=q.device)[:, None] + torch.arange(n, device=q.device)[None, :]).reshape(-1)
        qs, ks, vs = (x.index_select(0, idx).view(len(starts), n, x.shape[1], x.shape[2]).transpose(1, 2)
                      for x in (q, k, v))
        o = F.scaled_dot_product_attention(qs, ks, vs)
        out.index_copy_(0, idx, o.transpose(1, 2).reshape(-1, q.shape[1], q.shape[2]))
    return out


def _norm(x, w, shift, eps: float = 1e-6):
    """RMSNorm (Qwen2.5-VL, ``shift`` None) or LayerNorm with bias (Qwen2-VL)."""
    if shift is None:
        return fused.rmsnorm_ref(x, w, eps)
    return F.layer_norm(x, (x.shape[-1],), w, shift, eps)


class VisionBlock(nn.Module):
    """``gated``: RMSNorm + SwiGLU MLP (Qwen2.5-VL); otherwise LayerNorm + fc1 → quick-GELU → fc2 (Qwen2-VL)."""

    def __init__(self, dim: int, inter: int, heads: int, dtype, device, gated: bool = True, act: str = "quick_gelu"):
        super().__init__()
        mk = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype, device=device))
        self.heads, self.gated, self.act = heads, gated, act
        self.attn_norm, self.mlp_norm = mk(dim), mk(dim)
        self.attn_shift, self.mlp_shift = (None, None) if gated else (mk(dim), mk(dim))
        self.qkv, self.qkv_bias = mk(3 * dim, dim), mk(3 * dim)
        self.proj, self.proj_bias = mk(dim, dim), mk(dim)
        # SwiGLU keeps gate and up fused; the plain MLP's fc1 has the same role with half the rows
        self.gate_up, self.gate_up_bias = mk((2 if gated else 1) * inter, dim), mk((2 if gated else 1) * inter)
        self.down, self.down_bias = mk(dim, inter), mk(dim)

    def forward(self, x, cos, sin, cu: list[int]):
        n, dim = x.shape
        h = _norm(x, self.attn_norm, self.attn_shift)
        q, k, v = F.linear(h, self.qkv, self.qkv_bias).view(n, 3, self.heads, dim // self.heads).unbind(1)
        qf, kf = q.float(), k.float()
        q = (qf * cos + _rot_half(qf) * sin).to(x.dtype)
        k = (kf * cos + _rot_half(kf) * sin).to(x.dtype)
        x = x + F.linear(_segment_attention(q, k, v, cu).reshape(n, dim), self.proj, self.proj_bias)
        h = F.linear(_norm(x, self.mlp_norm, self.mlp_shift), self.gate_up, self.gate_up_bias)
        if self.gated:
            g, u = h.chunk(2, -1)
            h = F.silu(g) * u
        elif self.act == "quick_gelu":
            h = h * torch.sigmoid(1.702 * h)
        else:
            h = F.gelu(h, approximate="tanh")
        return x + F.linear(h, self.down, self.down_bias)


class DeepStackMerger(nn.Module):
    """Qwen3-VL: an extra merger on an intermediate block's output (LayerNorm over the merged group)."""

    def __init__(self, dim: int, unit: int, out: int, dtype, device):
        super().__init__()
        mk = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype, device=device))
        self.norm, self.shift = mk(dim * unit), mk(dim * unit)
        self.fc1, self.fc1_bias = mk(dim * unit, dim * unit), mk(dim * unit)
        self.fc2, self.fc2_bias = mk(out, dim * unit), mk(out)

    def forward(self, x):
        x = _norm(x.view(-1, self.norm.shape[0]), self.norm, self.shift)
        return F.linear(F.gelu(F.linear(x, self.fc1, self.fc1_bias)), self.fc2, self.fc2_bias)


class VisionTower(nn.Module):
    """``forward(pixel_values [N, C·tp·p·p], grid_thw [n_img, 3]) → [N / merge², out_hidden_size]``, one row per
    image placeholder token, images in input order and rows in raster order of the merged grid."""

    def __init__(self, vc: dict, dtype, device):
        super().__init__()
        self.vc = vc
        self.variant = vc.get("variant", "qwen2_5_vl")
        self.gated = self.variant == "qwen2_5_vl"
        v3 = self.variant == "qwen3_vl"
        dim, self.heads = vc["hidden_size"], vc["num_heads"]
        self.merge = vc.get("spatial_merge_size", 2)
        self.unit = self.merge * self.merge
        self.patch_dim = vc.get("in_channels", 3) * vc.get("temporal_patch_size", 2) * vc["patch_size"] ** 2
        mk = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype, device=device))
        self.patch_proj = mk(dim, self.patch_dim)
        # Qwen3-VL: bias on the patch projection, a learned position table (a square grid, interpolated to each
        # image's patch grid) and extra mergers on the outputs of the `deepstack_visual_indexes` blocks
        self.patch_proj_bias = mk(dim) if v3 else None
        self.pos_table = mk(vc["num_position_embeddings"], dim) if v3 else None
        self.deepstack_at = list(vc.get("deepstack_visual_indexes", [])) if v3 else []
        self.deepstack = nn.ModuleList(DeepStackMerger(dim, self.unit, vc["out_hidden_size"], dtype, device)
                                       for _ in self.deepstack_at)
        act = "gelu_tanh" if v3 else "quick_gelu"
        self.blocks = nn.ModuleList(VisionBlock(dim, vc["intermediate_size"], self.heads, dtype, device, self.gated, act)
                                    for _ in range(vc["depth"]))
        self.merger_norm = mk(dim)
        self.merger_shift = None if self.gated else mk(dim)
        self.merger_fc1, self.merger_fc1_bias = mk(dim * self.unit, dim * self.unit), mk(dim * self.unit)
        self.merger_fc2, self.merger_fc2_bias = mk(vc["out_hidden_size"], dim * self.unit), mk(vc["out_hidden_size"])

    # patch order: the image processor emits patches grouped by merge unit (each 2×2 block contiguous), images
    # one after another; `_grid_coords` reproduces the (row, column) of every patch in that order
    def _grid_coords(self, grids: list[list[int]]) -> torch.Tensor:
        m, out = self.merge, []
        for t, h, w in grids:
            r = torch.arange(h)[:, None].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            c = torch.arange(w)[None, :].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            out.append(torch.stack((r, c), -1).repeat(t, 1))
        return torch.cat(out, 0)

    def _windows(self, grids: list[list[int]]):
        """Permutation of merge units that makes every attention window contiguous, and the windows' bounds in
        patches. A window covers ``window_size`` pixels per side = ``window_size / patch / merge`` units."""
        m = self.merge
        ws = self.vc.get("window_size", 112) // m // self.vc["patch_size"]
        order, cu, base = [], [0], 0
        for t, h, w in grids:
            gh, gw = h // m, w // m
            idx = torch.arange(t * gh * gw).view(t, gh, gw)
            ph, pw = ws - gh % ws, ws - gw % ws  # a full extra window of padding when already a multiple
            idx = F.pad(idx, (0, pw, 0, ph), value=-1)
            nh, nw = (gh + ph) // ws, (gw + pw) // ws
            idx = idx.view(t, nh, ws, nw, ws).permute(0, 1, 3, 2, 4).reshape(t * nh * nw, ws * ws)
            for row in idx:
                keep = row[row >= 0]
                if keep.numel():
                    order.append(keep + base)
                    cu.append(cu[-1] + keep.numel() * self.unit)
            base += t * gh * gw
        return torch.cat(order), cu

    def _pos_embed(self, grids: list[list[int]]) -> torch.Tensor:
        """Bilinear interpolation of the square position table onto each image's ``h × w`` patch grid, rows in
        the processor's patch order (merge groups contiguous)."""
        side = int(self.pos_table.shape[0] ** 0.5)
        m, out = self.merge, []
        for t, h, w in grids:
            hi, wi = torch.linspace(0, side - 1, h), torch.linspace(0, side - 1, w)
            h0, w0 = hi.int(), wi.int()
            h1, w1 = (h0 + 1).clip(max=side - 1), (w0 + 1).clip(max=side - 1)
            dh, dw = (hi - h0)[:, None], (wi - w0)[None, :]
            e = 0
            for hh, ww, wt in ((h0, w0, (1 - dh) * (1 - dw)), (h0, w1, (1 - dh) * dw), (h1, w0, dh * (1 - dw)),
                               (h1, w1, dh * dw)):
                idx = (hh[:, None] * side + ww[None, :]).reshape(-1).long().to(self.pos_table.device)
                e = e + self.pos_table.index_select(0, idx) * wt.reshape(-1, 1).to(self.pos_table)
            e = e.view(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
            out.append(e.repeat(t, 1))
        return torch.cat(out, 0)

    def forward(self, pixel_values: torch.Tensor, grid_thw, return_deepstack: bool = False):
        grids = [[int(v) for v in g] for g in (grid_thw.tolist() if torch.is_tensor(grid_thw) else grid_thw)]
        dev, dt = self.patch_proj.device, self.patch_proj.dtype
        x = F.linear(pixel_values.to(device=dev, dtype=dt).view(-1, self.patch_dim), self.patch_proj,
                     self.patch_proj_bias)
        n, dim = x.shape
        assert n == sum(t * h * w for t, h, w in grids), "pixel_values rows do not match image_grid_thw"
        if self.pos_table is not None:
            x = x + self._pos_embed(grids)
        hd = dim // self.heads
        # 2-D rotary: the first half of the rotated pairs turns with the patch's row, the second with its column
        inv = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float32) / (hd // 2)))
        rc = self._grid_coords(grids).float()
        fr = torch.cat((rc[:, :1] * inv, rc[:, 1:] * inv), -1)  # [N, hd / 2]
        if self.gated:
            order, cu_win = self._windows(grids)
        else:  # Qwen2-VL: every block attends inside a whole frame, patches stay in input order
            order, cu_win = torch.arange(n // self.unit), None
        pidx = (order[:, None] * self.unit + torch.arange(self.unit)[None, :]).reshape(-1)
        x = x.index_select(0, pidx.to(dev))
        fr = fr.index_select(0, pidx).to(dev)
        emb = torch.cat((fr, fr), -1)
        cos, sin = emb.cos()[:, None, :], emb.sin()[:, None, :]
        cu_img = [0]
        for t, h, w in grids:
            for _ in range(t):
                cu_img.append(cu_img[-1] + h * w)
        full = set(self.vc.get("fullatt_block_indexes", []))
        deep = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, cu_img if (cu_win is None or i in full) else cu_win)
            if i in self.deepstack_at:
                deep.append(self.deepstack[self.deepstack_at.index(i)](x))
        x = _norm(x, self.merger_norm, self.merger_shift).view(-1, dim * self.unit)
        x = F.linear(F.gelu(F.linear(x, self.merger_fc1, self.merger_fc1_bias)), self.merger_fc2, self.merger_fc2_bias)
        x = x.index_select(0, torch.argsort(order).to(dev)) if cu_win is not None else x
        return (x, deep) if return_deepstack else x

    # HF names (without the tower's prefix) ↔ parameters; fused gate/up are two HF tensors
    def hf_tensors(self) -> Iterator[tuple[str, torch.Tensor]]:
        vc = self.vc
        yield "patch_embed.proj.weight", self.patch_proj.view(
            -1, vc.get("in_channels", 3), vc.get("temporal_patch_size", 2), vc["patch_size"], vc["patch_size"])
        inter = vc["intermediate_size"]
        v3 = self.variant == "qwen3_vl"
        fc1, fc2 = ("mlp.linear_fc1", "mlp.linear_fc2") if v3 else ("mlp.fc1", "mlp.fc2")
        if v3:
            yield "patch_embed.proj.bias", self.patch_proj_bias
            yield "pos_embed.weight", self.pos_table
            for i, d in enumerate(self.deepstack):
                q = f"deepstack_merger_list.{i}."
                yield q + "norm.weight", d.norm
                yield q + "norm.bias", d.shift
                yield q + "linear_fc1.weight", d.fc1
                yield q + "linear_fc1.bias", d.fc1_bias
                yield q + "linear_fc2.weight", d.fc2
                yield q + "linear_fc2.bias", d.fc2_bias
        for i, b in enumerate(self.blocks):
            p = f"blocks.{i}."
            yield p + "norm1.weight", b.attn_norm
            yield p + "norm2.weight", b.mlp_norm
            yield p + "attn.qkv.weight", b.qkv
            yield p + "attn.qkv.bias", b.qkv_bias
            yield p + "attn.proj.weight", b.proj
            yield p + "attn.proj.bias", b.proj_bias
            if self.gated:
                yield p + "mlp.gate_proj.weight", b.gate_up[:inter]
                yield p + "mlp.gate_proj.bias", b.gate_up_bias[:inter]
                yield p + "mlp.up_proj.weight", b.gate_up[inter:]
                yield p + "mlp.up_proj.bias", b.gate_up_bias[inter:]
                yield p + "mlp.down_proj.weight", b.down
                yield p + "mlp.down_proj.bias", b.down_bias
            else:
                yield p + "norm1.bias", b.attn_shift
                yield p + "norm2.bias", b.mlp_shift
                yield p + fc1 + ".weight", b.gate_up
                yield p + fc1 + ".bias", b.gate_up_bias
                yield p + fc2 + ".weight", b.down
                yield p + fc2 + ".bias", b.down_bias
        ln, m1, m2 = ("norm", "linear_fc1", "linear_fc2") if v3 else ("ln_q", "mlp.0", "mlp.2")
        if not self.gated:
            yield f"merger.{ln}.bias", self.merger_shift
        yield f"merger.{ln}.weight", self.merger_norm
        yield f"merger.{m1}.weight", self.merger_fc1
        yield f"merger.{m1}.bias", self.merger_fc1_bias
        yield f"merger.{m2}.weight", self.merger_fc2
        yield f"merger.{m2}.bias", self.merger_fc2_bias


# ------------------------------------------------------------------------------------------ full model


class _GatherSumGrad(torch.autograd.Function):
    """All-gather of equally shaped tensors; the backward sums every rank's gradient of the gathered result and
    hands each rank the part it contributed."""

    @staticmethod
    def forward(ctx, x, group, rank):
        import torch.distributed as dist

        ctx.group, ctx.rank = group, rank
        parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.stack(parts, 0)

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist

        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g[ctx.rank], None, None


class QwenVLModel(QwenModel):
    """The decoder plus ``self.visual``. ``forward`` takes the packed token ids as usual and, optionally,
    ``pixel_values`` / ``image_grid_thw`` of all images of the packed batch in order of appearance."""

    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", pctx=None):
        if pctx is not None and getattr(pctx, "ep_size", 1) > 1:
            raise NotImplementedError("the vision-language model runs under data, tensor, pipeline and Ulysses "
                                      "sequence parallelism (no expert parallelism)")
        super().__init__(cfg, dtype=dtype, device=device, pctx=pctx)
        assert cfg.vision["out_hidden_size"] == cfg.hidden_size
        # the tower feeds the embeddings: it lives on the first pipeline stage only
        self.visual = VisionTower(cfg.vision, dtype, device) if self.first_stage else None
        n_deep = len(cfg.vision.get("deepstack_visual_indexes", [])) if cfg.vision.get("variant") == "qwen3_vl" else 0
        if self.first_stage and len(self.layers) < n_deep:
            raise ValueError(f"the first pipeline stage needs at least {n_deep} decoder blocks (deep-stack features)")
        # set by the engine (`shard_vision_across_sp`): the images of a micro-batch are divided over the
        # sequence-parallel ranks instead of every rank running the tower on all of them
        self.shard_vision = False

    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02):
        super().init_weights(seed, std)  # draws every matrix, zeroes every bias
        for name, p in (self.visual.named_parameters() if self.visual is not None else ()):
            if name.endswith("norm"):
                p.fill_(1.0)
            elif name.endswith("shift"):
                p.zero_()
        return self

    def positions(self, input_ids, meta: VarlenMeta, image_grid_thw=None, video_second_per_grid=None):
        grids = [] if image_grid_thw is None else (
            image_grid_thw.tolist() if torch.is_tensor(image_grid_thw) else list(image_grid_thw))
        return mrope_position_ids(input_ids.tolist(), meta.cu_cpu.tolist(), grids, self.cfg, video_second_per_grid)

    def embed_inputs(self, input_ids, pixel_values=None, image_grid_thw=None, features=None,
                     seq_slice: slice | None = None):
        """``(x, layer_adds)``: token embeddings with the image placeholder rows replaced by the tower's output,
        and (Qwen3-VL) ``(rows, [features…])`` to add to those rows after the first decoder layers.
        ``features = (feats, deep)`` skips the tower (a caller that cached its output). ``input_ids`` are all
        tokens of the micro-batch; the result covers ``seq_slice`` of them (this Ulysses rank's rows), and under
        tensor parallelism this rank's share of those rows (activations between blocks are token-sharded)."""
        p = self.pctx
        lo, hi = (seq_slice.start, seq_slice.stop) if seq_slice is not None else (0, input_ids.shape[0])
        if p is not None and p.tp_size > 1:
            from ..parallel.tensor_parallel import vocab_parallel_embedding

            x = vocab_parallel_embedding(input_ids[lo:hi], self.embed, p.tp_fused)
            n = (hi - lo) // p.tp_size
            lo, hi = lo + p.tp_rank * n, lo + (p.tp_rank + 1) * n
        else:
            x = fused.embedding(input_ids[lo:hi], self.embed)
        if features is None and (pixel_values is None or pixel_values.numel() == 0):
            return x, None
        if features is not None:
            feats, deep = features
        elif self.shard_vision and p is not None and p.sp_size > 1:
            feats, deep = self._sharded_visual(pixel_values, image_grid_thw)
        else:
            feats, deep = self.visual(pixel_values, image_grid_thw, return_deepstack=True)
        mask = (input_ids == self.cfg.image_token_id) | (input_ids == self.cfg.video_token_id)
        rows = mask.nonzero().squeeze(-1)
        if rows.numel() != feats.shape[0]:
            raise ValueError(f"{rows.numel()} image placeholder tokens but {feats.shape[0]} image features")
        if lo != 0 or hi != input_ids.shape[0]:
            keep = ((rows >= lo) & (rows < hi)).nonzero().squeeze(-1)
            rows = rows.index_select(0, keep) - lo
            feats, deep = feats.index_select(0, keep), [d.index_select(0, keep) for d in deep]
        adds = (rows, [d.to(x.dtype) for d in deep]) if deep else None
        return x.index_copy(0, rows, feats.to(x.dtype)), adds

    def _sharded_visual(self, pixel_values, image_grid_thw):
        """Tower work divided over the sequence-parallel group: image ``i`` runs on rank ``i mod S``, the
        features (and deep-stack features) are all-gathered; in the backward every rank's gradient of the
        gathered features is summed onto the owner. Reference: areal/models/transformers/vision_sp_shard.py."""
        p = self.pctx
        S, r = p.sp_size, p.sp_rank
        grids = [[int(v) for v in g] for g in (image_grid_thw.tolist() if torch.is_tensor(image_grid_thw)
                                               else image_grid_thw)]
        unit = self.visual.unit
        n_patch = [t * h * w for t, h, w in grids]
        starts = [0]
        for n in n_patch:
            starts.append(starts[-1] + n)
        mine = [i for i in range(len(grids)) if i % S == r]
        n_deep = len(self.visual.deepstack_at)
        H = self.cfg.hidden_size
        dev, dt = self.embed.device, self.embed.dtype
        if mine:
            pix = torch.cat([pixel_values[starts[i]:starts[i + 1]] for i in mine], 0)
            f, deep = self.visual(pix, [grids[i] for i in mine], return_deepstack=True)
            local = torch.cat([f] + list(deep), -1)
        else:
            # a rank without images still takes part in the gather and (so that its backward runs) in the
            # gradient sum
            local = torch.zeros(0, (1 + n_deep) * H, dtype=dt, device=dev, requires_grad=torch.is_grad_enabled())
        per_rank = [sum(n_patch[i] // unit for i in range(len(grids)) if i % S == k) for k in range(S)]
        width = max(per_rank)
        local = F.pad(local, (0, 0, 0, width - local.shape[0]))
        allf = _GatherSumGrad.apply(local, p.sp_group, r)  # [S, width, C]
        rows, offs = [], [0] * S
        for i, n in enumerate(n_patch):
            k, m = i % S, n // unit
            rows.append(allf[k, offs[k]:offs[k] + m])
            offs[k] += m
        full = torch.cat(rows, 0)
        return full[:, :H], [full[:, (j + 1) * H:(j + 2) * H] for j in range(n_deep)]

    def forward(self, input_ids, position_ids, meta: VarlenMeta, attn_fn=None, stage_input=None,
                pixel_values=None, image_grid_thw=None, mrope_pos=None, seq_slice: slice | None = None):
        """``mrope_pos [3, T]`` overrides the position triples derived from the token ids (a caller that
        already holds them, e.g. from a processor). ``position_ids`` is ignored when there are images: the
        rotary table is built per token. Under Ulysses sequence parallelism the caller passes ALL tokens of the
        (padded) micro-batch and ``seq_slice``, this rank's rows: embeddings, image features and the rotary
        table are built for the whole batch, the decoder runs on the slice."""
        if mrope_pos is None:
            if pixel_values is None or pixel_values.numel() == 0:
                mrope_pos = position_ids.to(torch.long)[None, :].expand(3, -1)
            else:
                mrope_pos, _ = self.positions(input_ids, meta, image_grid_thw)
        mrope_pos = mrope_pos.to(input_ids.device)
        cos, sin = mrope_tables(mrope_pos, self.cfg.rotary_dim, self.cfg.rope_theta, self.cfg.mrope_section,
                                self.cfg.mrope_interleaved)
        rows = torch.arange(input_ids.shape[0], dtype=torch.int32, device=input_ids.device)
        if stage_input is not None:
            x = adds = None  # a later pipeline stage: activations arrive, only the rotary table is built here
        else:
            x, adds = self.embed_inputs(input_ids, pixel_values, image_grid_thw, seq_slice=seq_slice)
        if seq_slice is not None:
            # the rotary table stays whole: local rows index it before the sequence→head exchange, all rows after
            self.pctx.extras["full_positions"] = rows
            input_ids, rows = input_ids[seq_slice], rows[seq_slice]
        return super().forward(input_ids, rows, meta, attn_fn=attn_fn, stage_input=stage_input, embeds=x,
                               rope=(cos, sin), layer_adds=adds)

    # ------------------------------------------------------------------ HF layout
    _LM = "model.language_model."
    _VIS = "model.visual."

    def to_hf_local(self, export: bool = False) -> Iterator[tuple[str, torch.Tensor]]:
        for name, t in super().to_hf_local(export):
            if ".mlp.experts." in name:
                continue  # written fused below
            yield (self._LM + name[len("model."):] if name.startswith("model.") else name), t
        if self.cfg.is_moe:
            # Qwen3-VL-MoE checkpoints hold all experts of a layer in two tensors, input dimension first:
            # gate_up_proj [E, H, 2I], down_proj [E, I, H] (transposed views of the fused parameters)
            for i, layer in zip(self.layer_ids, self.layers):
                if hasattr(layer.mlp, "router"):
                    p = f"{self._LM}layers.{i}.mlp.experts."
                    yield p + "gate_up_proj", layer.mlp.gate_up.transpose(1, 2)
                    yield p + "down_proj", layer.mlp.down.transpose(1, 2)
        for name, t in (self.visual.hf_tensors() if self.visual is not None else ()):
            yield self._VIS + name, t

    def _tp_dim(self, hf_name: str) -> int | None:
        # the tower is replicated over tensor-parallel ranks; decoder names keep their rule under the prefix
        return None if hf_name.startswith(self._VIS) else super()._tp_dim(hf_name)

    def _other_stage(self, name: str) -> bool:
        """A checkpoint tensor of another pipeline stage: decoder tensors by the text model's rule, the vision
        tower when this stage has none (it lives on the first stage)."""
        if name.startswith(self._VIS):
            return self.visual is None
        if name.startswith(self._LM):
            return self.owned_by_other_stage("model." + name[len(self._LM):])
        return self.owned_by_other_stage(name)

    @torch.no_grad()
    def load_hf(self, tensors: Iterable[tuple[str, torch.Tensor]], strict: bool = True):
        """Accepts the current layout (``model.language_model.*`` / ``model.visual.*``) and the older one
        (``model.*`` / ``visual.*``)."""
        def rename():
            for name, t in tensors:
                if name.startswith("visual."):
                    name = "model." + name
                elif name.startswith("model.") and not name.startswith((self._LM, self._VIS)):
                    name = self._LM + name[len("model."):]
                yield name, t

        dst = dict(self.to_hf_local())
        if self.embed is not None and not self.first_stage:
            dst[self._LM + "embed_tokens.weight"] = self.embed  # the last stage's copy of a tied embedding
        seen = set()
        for name, t in rename():
            if name == "lm_head.weight" and self.lm_head is None and self.score is None:
                seen.add(name)
                continue
            if name not in dst:
                if ".mlp.experts." in name and self.pctx is not None and self.pctx.ep_size > 1:
                    continue  # an expert that lives on another expert-parallel rank
                if self._other_stage(name):
                    continue
                if strict:
                    raise KeyError(f"unexpected tensor {name}")
                continue
            d = dst[name]
            dim = self._tp_dim(name)
            if dim is not None:
                n = t.shape[dim] // self.pctx.tp_size
                t = t.narrow(dim, self.pctx.tp_rank * n, n)
            if d.shape != t.shape and name.endswith(("experts.gate_up_proj", "experts.down_proj")) \
                    and t.dim() == 3 and d.shape == t.transpose(1, 2).shape:
                t = t.transpose(1, 2)  # written output dimension first (what transformers holds in memory)
            if d.shape != t.shape:
                raise ValueError(f"{name}: shape {tuple(t.shape)} != {tuple(d.shape)}")
            d.copy_(t.to(device=d.device, dtype=d.dtype))
            seen.add(name)
        missing = set(dst) - seen
        if strict and missing:
            raise KeyError(f"missing tensors: {sorted(missing)[:8]} ...")
        return self
