"""Low-rank adapters (LoRA) on the fused projections.

The model keeps q/k/v and gate/up as one fused weight each, while adapter
checkpoints name one ``lora_A`` / ``lora_B`` pair per original projection
(``q_proj``, ``k_proj`` …). One ``LoRAAdapter`` therefore serves one fused
weight: the down-projections ``A_i`` of its targeted sub-blocks are stacked
into one matrix (one GEMM over the input), the up-projections ``B_i`` stay
per sub-block, and the result is laid out like the fused output.

The rank is padded to a multiple of 64 internally so that both products run on
the tcgen05 GEMM with whole K blocks; the padding rows of ``A`` and columns of
``B`` are zero and stay zero under AdamW (their gradients are products with the
other factor's zero padding). Exports slice the padding off.

Base weights are frozen while adapters train. The rollout engine receives
merged weights ``W + (alpha / r) * B @ A`` (``merged`` below), so generation
runs the unmodified dense kernels.

Reference behaviour: ``use_lora`` / ``lora_rank`` / ``lora_alpha`` /
``target_modules`` of the train-engine config (areal/api/cli_args.py), applied
with PEFT in areal/engine/fsdp_engine.py.
"""

from __future__ import annotations

import json
import math
import os
from contextlib import contextmanager
from typing import Iterator, Sequence

import torch
import torch.nn as nn

from ..ops.gemm import linear

ALL_LINEAR = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def normalize_targets(targets: Sequence[str] | None) -> tuple[str, ...]:
    """``[]`` and ``["all-linear"]`` select every dense projection."""
    if not targets or "all-linear" in targets:
        return ALL_LINEAR
    bad = [t for t in targets if t not in ALL_LINEAR]
    if bad:
        raise ValueError(f"unknown LoRA target modules {bad}; choose from {ALL_LINEAR}")
    return tuple(targets)


def padded_rank(rank: int) -> int:
    return (rank + 63) // 64 * 64


class LoRAAdapter(nn.Module):
    """Adapter of one fused weight ``[sum(outs), in_features]``.

    ``blocks``: ``(hf_module_name, out_features)`` per sub-block in the fused row order;
    ``targeted``: the module names that get an adapter (the others contribute zeros)."""

    def __init__(self, in_features: int, blocks: Sequence[tuple[str, int]], targeted: Sequence[str],
                 rank: int, alpha: float, dtype, device, seed: int = 0, tp_mode: str | None = None, pctx=None):
        """``tp_mode`` (tensor parallelism; ``in_features`` and the block sizes are then the LOCAL ones):
        ``"column"``: the fused weight is split by output rows, the input arrives as this rank's token slice.
        ``A`` is replicated, every ``B`` holds this rank's rows; the tokens are gathered first.
        ``"row"``: the fused weight is split along its input, the output leaves as this rank's token slice.
        ``A`` holds this rank's input columns, ``B`` is replicated; the rank-sized partial products are summed
        and scattered by token before ``B`` is applied."""
        super().__init__()
        self.tp_mode, self.pctx = tp_mode, pctx
        self.in_features = in_features
        self.blocks = list(blocks)
        self.names = [n for n, _ in self.blocks if n in targeted]
        assert self.names, "adapter without a targeted sub-block"
        self.rank, self.rp = rank, padded_rank(rank)
        self.scale = float(alpha) / float(rank)
        k = len(self.names)
        self.lora_A = nn.Parameter(torch.zeros(k * self.rp, in_features, dtype=dtype, device=device))
        self.lora_B = nn.ParameterDict({
            n: nn.Parameter(torch.zeros(o, self.rp, dtype=dtype, device=device))
            for n, o in self.blocks if n in self.names})
        # A: uniform(-1/sqrt(in), 1/sqrt(in)) (kaiming with a=sqrt(5), the PEFT default); B: zeros, so
        # the adapted model starts equal to the base model
        g = torch.Generator(device="cpu").manual_seed(seed)
        tp = pctx.tp_size if (pctx is not None and tp_mode == "row") else 1
        full_in = in_features * tp  # a row-parallel adapter draws the whole A and keeps its columns
        bound = 1.0 / math.sqrt(full_in)
        with torch.no_grad():
            for i in range(k):
                a = (torch.rand(rank, full_in, generator=g) * 2 - 1) * bound
                if tp > 1:
                    a = a[:, pctx.tp_rank * in_features:(pctx.tp_rank + 1) * in_features]
                self.lora_A[i * self.rp: i * self.rp + rank].copy_(a.to(dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Delta of the fused projection's output, ``[T, sum(outs)]``."""
        if self.tp_mode == "column":
            from ..parallel.tensor_parallel import gather_seq

            x = gather_seq(x, self.pctx.tp_fused)
        u = linear(x, self.lora_A)
        if self.tp_mode == "row":
            from ..parallel.tensor_parallel import scatter_seq_sum

            u = scatter_seq_sum(u, self.pctx.tp_fused)
        parts, i = [], 0
        for n, o in self.blocks:
            if n in self.lora_B:
                parts.append(linear(u[:, i * self.rp:(i + 1) * self.rp], self.lora_B[n]))
                i += 1
            else:
                parts.append(u.new_zeros(u.shape[0], o))
        d = parts[0] if len(parts) == 1 else torch.cat(parts, dim=-1)
        return d * self.scale

    @torch.no_grad()
    def merged_delta(self) -> torch.Tensor:
        """``scale * B @ A`` laid out like the fused weight (fp32)."""
        rows, i = [], 0
        for n, o in self.blocks:
            if n in self.lora_B:
                a = self.lora_A[i * self.rp:(i + 1) * self.rp].float()
                rows.append(self.lora_B[n].float() @ a * self.scale)
                i += 1
            else:
                rows.append(torch.zeros(o, self.in_features, dtype=torch.float32, device=self.lora_A.device))
        return rows[0] if len(rows) == 1 else torch.cat(rows, 0)

    def _tp(self) -> tuple[int, int, object]:
        p = self.pctx
        return (p.tp_size, p.tp_rank, p.tp_group) if (p is not None and self.tp_mode and p.tp_size > 1) else (1, 0, None)

    def peft_tensors(self, prefix: str) -> Iterator[tuple[str, torch.Tensor]]:
        """``(name, tensor)`` in the adapter-checkpoint naming, padding removed; under tensor parallelism the
        full factors (a collective over the tensor-parallel group: every rank of it must iterate)."""
        tp, _, group = self._tp()

        def full(t, dim):
            if tp == 1:
                return t
            import torch.distributed as dist

            parts = [torch.empty_like(t) for _ in range(tp)]
            dist.all_gather(parts, t.contiguous(), group=group)
            return torch.cat(parts, dim)

        for i, n in enumerate(self.names):
            a, b = self.lora_A[i * self.rp: i * self.rp + self.rank], self.lora_B[n][:, :self.rank]
            yield f"{prefix}{n}.lora_A.weight", (full(a, 1) if self.tp_mode == "row" else a)
            yield f"{prefix}{n}.lora_B.weight", (full(b, 0) if self.tp_mode == "column" else b)

    @torch.no_grad()
    def load_peft(self, tensors: dict[str, torch.Tensor], prefix: str):
        tp, r, _ = self._tp()
        for i, n in enumerate(self.names):
            a, b = tensors[f"{prefix}{n}.lora_A.weight"], tensors[f"{prefix}{n}.lora_B.weight"]
            if tp > 1 and self.tp_mode == "row":
                a = a[:, r * self.in_features:(r + 1) * self.in_features]
            if tp > 1 and self.tp_mode == "column":
                rows = self.lora_B[n].shape[0]
                b = b[r * rows:(r + 1) * rows]
            assert a.shape == (self.rank, self.in_features) and b.shape[1] == self.rank
            self.lora_A[i * self.rp: i * self.rp + self.rank].copy_(a)
            self.lora_B[n][:, :self.rank].copy_(b)


def make_adapter(cfg, in_features, blocks, dtype, device, seed, tp_mode: str | None = None,
                 pctx=None) -> LoRAAdapter | None:
    """Adapter for a fused weight, or ``None`` when LoRA is off or no sub-block is targeted."""
    if not getattr(cfg, "lora_rank", 0):
        return None
    targets = normalize_targets(cfg.lora_targets)
    if not any(n in targets for n, _ in blocks):
        return None
    if pctx is None or pctx.tp_size == 1:
        tp_mode = None
    return LoRAAdapter(in_features, blocks, targets, cfg.lora_rank, cfg.lora_alpha, dtype, device, seed,
                       tp_mode=tp_mode, pctx=pctx if tp_mode else None)


def is_lora_param(name: str) -> bool:
    return ".lora_A" in name or ".lora_B." in name


def iter_adapters(model) -> Iterator[tuple[str, torch.Tensor, LoRAAdapter]]:
    """``(hf_prefix, fused_weight, adapter)`` for every adapter of a ``QwenModel``."""
    # a vision-language checkpoint nests its decoder under `language_model`
    lm = "language_model." if getattr(model.cfg, "is_vl", False) else ""
    for i, layer in zip(model.layer_ids, model.layers):
        p = f"base_model.model.model.{lm}layers.{i}."
        a, m = layer.attn, layer.mlp
        if getattr(a, "lora_qkv", None) is not None:
            yield p + "self_attn.", a.qkv, a.lora_qkv
        if getattr(a, "lora_o", None) is not None:
            yield p + "self_attn.", a.o, a.lora_o
        if getattr(m, "lora_gate_up", None) is not None:
            yield p + "mlp.", m.gate_up, m.lora_gate_up
        if getattr(m, "lora_down", None) is not None:
            yield p + "mlp.", m.down, m.lora_down


@contextmanager
def merged(model):
    """Inside the block the base weights hold ``W + scale * B @ A``; the exact original bits are
    restored on exit (from a copy: subtracting the delta again would round in bf16)."""
    saved = []
    with torch.no_grad():
        for _, w, ad in iter_adapters(model):
            saved.append((w, w.detach().clone()))
            w.add_(ad.merged_delta().to(w.dtype))
    try:
        yield model
    finally:
        with torch.no_grad():
            for w, old in saved:
                w.copy_(old)


def save_adapter(model, cfg, path: str, base_model_path: str = "", gather_group=None, write: bool = True):
    """Writes ``adapter_model.safetensors`` + ``adapter_config.json`` (the layout PEFT reads). Under pipeline
    parallelism the stages hold different layers' adapters: ``gather_group`` (the pipeline group; collective) brings
    them to its first rank, which writes the one file."""
    from safetensors.torch import save_file

    tensors = {}
    for prefix, _, ad in iter_adapters(model):
        for n, t in ad.peft_tensors(prefix):
            tensors[n] = t.detach().to("cpu").contiguous().clone()
    if not write:
        return  # a tensor-parallel peer: it only took part in the gathers above
    if gather_group is not None:
        import torch.distributed as dist

        parts = [None] * dist.get_world_size(gather_group)
        dist.all_gather_object(parts, tensors, group=gather_group)
        if dist.get_rank(gather_group) != 0:
            return
        tensors = {k: v for part in parts for k, v in part.items()}
    os.makedirs(path, exist_ok=True)
    save_file(tensors, os.path.join(path, "adapter_model.safetensors"), metadata={"format": "pt"})
    conf = {"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": cfg.lora_rank, "lora_alpha": cfg.lora_alpha,
            "target_modules": list(normalize_targets(cfg.lora_targets)), "lora_dropout": 0.0, "bias": "none",
            "base_model_name_or_path": base_model_path, "inference_mode": True, "fan_in_fan_out": False}
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump(conf, f, indent=2)


def load_adapter(model, path: str):
    from safetensors.torch import load_file

    tensors = load_file(os.path.join(path, "adapter_model.safetensors"))
    for prefix, _, ad in iter_adapters(model):
        ad.load_peft(tensors, prefix)
