"""Batch containers: padded ↔ packed conversion, micro-batch splitting,
normalisation, KL estimators and tensor-dict collectives.

Trajectories arrive as padded dicts (``input_ids [B, L]``, ``attention_mask``,
``loss_mask``, ``logprobs``, ``versions``, ``rewards [B]`` …). Engines work on the
packed form: every ``[B, L]`` tensor flattened to ``[T]`` over valid tokens plus
``cu_seqlens`` / ``max_seqlen``. Behaviour follows the reference
(areal/utils/data.py:492-1656).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Sequence

import numpy as np
import torch
import torch.distributed as dist

from ..api.cli_args import MicroBatchSpec, NormConfig
from . import seqpack

N_TOKENS_PER_PAGE = 256


# --------------------------------------------------------------------------- basics


def get_batch_size(data: dict[str, Any]) -> int:
    if "attention_mask" in data:
        return data["attention_mask"].shape[0]
    if "cu_seqlens" in data:
        return data["cu_seqlens"].shape[0] - 1
    for v in data.values():
        if torch.is_tensor(v):
            return v.shape[0]
    raise ValueError("cannot infer the batch size")


def pad_sequences_to_tensors(seqs: list[dict[str, Any]], pad_value: float = 0.0) -> dict[str, Any]:
    """List of per-sequence dicts of 1-D tensors/lists → padded batch with ``attention_mask``."""
    if not seqs:
        return {}
    skip = {"rewards"}
    skip_len = lambda k: k in skip or k.startswith("multi_modal_input")
    max_len = max(len(s[k]) for s in seqs for k in s if not skip_len(k) and hasattr(s[k], "__len__")
                  and not isinstance(s[k], str))
    out: dict[str, Any] = {}
    for k in seqs[0]:
        vals = [s[k] for s in seqs]
        if k.startswith("multi_modal_input"):
            # per-sequence image tensors: one dict per row of the batch (a trajectory stores a one-element list)
            out[k] = [(v[0] if isinstance(v, (list, tuple)) and v else (v or {})) for v in vals]
            continue
        if k in skip or not hasattr(vals[0], "__len__"):
            out[k] = torch.as_tensor(vals)
            continue
        rows = []
        for v in vals:
            t = torch.as_tensor(v)
            rows.append(torch.nn.functional.pad(t, (0, max_len - t.shape[0]), value=pad_value))
        out[k] = torch.stack(rows)
    lens = [len(next(v for kk, v in s.items() if not skip_len(kk) and hasattr(v, "__len__"))) for s in seqs]
    out["attention_mask"] = torch.arange(max_len)[None, :] < torch.tensor(lens)[:, None]
    return out


def concat_padded_tensors(dicts: Sequence[dict[str, Any]], pad_value: float = 0.0) -> dict[str, Any]:
    """Concatenates padded batches along the batch dimension, right-padding to the longest."""
    dicts = [d for d in dicts if d]
    if not dicts:
        return {}
    max_len = max(d["attention_mask"].shape[1] for d in dicts)
    out: dict[str, Any] = {}
    # text-only trajectories carry no image entry: give them one empty dict per row when others have images
    mm_keys = {k for d in dicts for k in d if k.startswith("multi_modal_input")}
    keys = list(dicts[0]) + [k for k in sorted(mm_keys) if k not in dicts[0]]
    for k in keys:
        parts = []
        for d in dicts:
            v = d[k] if k in d else [{} for _ in range(d["attention_mask"].shape[0])]
            if torch.is_tensor(v) and v.dim() >= 2 and v.shape[1] == d["attention_mask"].shape[1]:
                pad = max_len - v.shape[1]
                if pad:
                    fill = False if v.dtype == torch.bool else (pad_value if k != "versions" else -1)
                    shape = list(v.shape)
                    shape[1] = pad
                    v = torch.cat([v, torch.full(shape, fill, dtype=v.dtype, device=v.device)], 1)
            parts.append(v)
        if torch.is_tensor(parts[0]):
            out[k] = torch.cat(parts, 0)
        elif isinstance(parts[0], list):
            out[k] = [x for p in parts for x in p]
        else:
            out[k] = parts
    return out


def to_device(data: dict[str, Any], device) -> dict[str, Any]:
    return {k: (v.to(device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in data.items()}


# --------------------------------------------------------------------------- packing


def pack_tensor_dict(data: dict[str, Any]) -> dict[str, Any]:
    """Padded → packed. ``[B, L, ...]`` tensors keep only attended positions."""
    if "cu_seqlens" in data:
        return data
    mask = data["attention_mask"].bool()
    B, L = mask.shape
    lens = mask.sum(1).to(torch.int32)
    cu = torch.zeros(B + 1, dtype=torch.int32, device=mask.device)
    cu[1:] = lens.cumsum(0)
    out: dict[str, Any] = {}
    for k, v in data.items():
        if k == "attention_mask":
            continue
        if torch.is_tensor(v) and v.dim() >= 2 and v.shape[0] == B and v.shape[1] == L:
            out[k] = v[mask]
        else:
            out[k] = v
    out["cu_seqlens"] = cu
    out["max_seqlen"] = int(lens.max()) if B else 0
    return out


def unpack_to_padded(packed: dict[str, Any], pad_value: float = 0.0) -> dict[str, Any]:
    cu = packed["cu_seqlens"].tolist()
    B = len(cu) - 1
    L = max((cu[i + 1] - cu[i] for i in range(B)), default=0)
    T = cu[-1]
    mask = torch.zeros(B, L, dtype=torch.bool)
    for i in range(B):
        mask[i, : cu[i + 1] - cu[i]] = True
    out: dict[str, Any] = {"attention_mask": mask}
    for k, v in packed.items():
        if k in ("cu_seqlens", "max_seqlen"):
            continue
        if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == T and T != B:
            buf = torch.full((B, L) + tuple(v.shape[1:]), pad_value, dtype=v.dtype)
            buf[mask] = v.cpu()
            out[k] = buf
        else:
            out[k] = v
    return out


def amend_position_ids(data: dict[str, Any]) -> dict[str, Any]:
    if "position_ids" in data:
        return data
    if "cu_seqlens" in data:
        cu = data["cu_seqlens"]
        T = int(cu[-1])
        idx = torch.arange(T, device=cu.device)
        seq = torch.searchsorted(cu[1:].long(), idx, right=True)
        data["position_ids"] = (idx - cu[seq].long()).to(torch.int32)
    else:
        m = data["attention_mask"].long()
        data["position_ids"] = ((m.cumsum(1) - 1) * m).to(torch.int32)
    return data


@dataclass
class MicroBatchList:
    """Micro-batches of one batch plus the permutation that restores sample order."""

    data: dict[str, Any]
    mb_spec: MicroBatchSpec
    mbs: list[dict[str, Any]]
    forward_indices: list[int]
    backward_indices: list[int]
    group_lens: list[int]
    padded_mbs: list[dict[str, Any]] | None = None
    padding_lengths: list[int] | None = None
    old_cu_seqlens_list: list[torch.Tensor] | None = None

    def __len__(self):
        return len(self.mbs)


def _select_rows(data: dict[str, Any], idx: list[int], B: int) -> dict[str, Any]:
    it = torch.as_tensor(idx, dtype=torch.long)
    out = {}
    for k, v in data.items():
        if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == B:
            out[k] = v[it.to(v.device)]
        elif isinstance(v, list) and len(v) == B:
            out[k] = [v[i] for i in idx]
        else:
            out[k] = v
    return out


def split_padded_tensor_dict_into_mb_list(data: dict[str, Any], mb_spec: MicroBatchSpec,
                                          group: dist.ProcessGroup | None = None) -> MicroBatchList:
    """Splits a padded batch into packed micro-batches of at most
    ``max_tokens_per_mb`` tokens (at least ``n_mbs`` of them), keeping
    ``granularity`` consecutive samples together. With ``group`` all ranks use
    the same number of micro-batches (the maximum over ranks)."""
    mask = data["attention_mask"].bool()
    B = mask.shape[0]
    lens = mask.sum(1).tolist()
    g = max(mb_spec.granularity, 1)
    assert B % g == 0, f"batch size {B} not divisible by granularity {g}"
    unit_lens = [sum(lens[i:i + g]) for i in range(0, B, g)]
    min_groups = mb_spec.n_mbs or 1
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        groups = seqpack.allocate(unit_lens, mb_spec.max_tokens_per_mb, min_groups,
                                  mb_spec.packing_algorithm, mb_spec.n_mbs_divisor)
        n = torch.tensor([len(groups)], dtype=torch.int64,
                         device=data["attention_mask"].device if dist.get_backend(group) == "nccl" else "cpu")
        dist.all_reduce(n, op=dist.ReduceOp.MAX, group=group)
        if int(n) != len(groups):
            groups = seqpack.allocate(unit_lens, mb_spec.max_tokens_per_mb, int(n),
                                      mb_spec.packing_algorithm, mb_spec.n_mbs_divisor)
            while len(groups) < int(n):  # fewer samples than micro-batches: split the largest
                big = max(groups, key=len)
                if len(big) < 2:
                    break
                groups.remove(big)
                groups += [big[: len(big) // 2], big[len(big) // 2:]]
    else:
        groups = seqpack.allocate(unit_lens, mb_spec.max_tokens_per_mb, min_groups,
                                  mb_spec.packing_algorithm, mb_spec.n_mbs_divisor)
    groups = [sorted(gr) for gr in groups if gr]
    forward: list[int] = []
    mbs, group_lens = [], []
    for gr in groups:
        rows = [u * g + j for u in gr for j in range(g)]
        forward += rows
        sub = _select_rows(data, rows, B)
        L = int(sub["attention_mask"].sum(1).max()) if rows else 0
        sub = {k: (v[:, :L] if torch.is_tensor(v) and v.dim() >= 2 and v.shape[1] == mask.shape[1] else v)
               for k, v in sub.items()}
        mbs.append(pack_tensor_dict(sub))
        group_lens.append(len(rows))
    backward = [0] * len(forward)
    for pos, src in enumerate(forward):
        backward[src] = pos
    return MicroBatchList(data=data, mb_spec=mb_spec, mbs=mbs, forward_indices=forward,
                          backward_indices=backward, group_lens=group_lens)


def pad_packed_tensor_dict(mb: dict[str, Any], pad_to: int, pad_value: float = 0.0):
    """Appends one dummy sequence so that the packed length becomes ``pad_to``."""
    T = int(mb["cu_seqlens"][-1])
    pad = pad_to - T
    if pad <= 0:
        return mb, 0
    out = {}
    for k, v in mb.items():
        if k == "cu_seqlens":
            out[k] = torch.cat([v, torch.tensor([pad_to], dtype=v.dtype, device=v.device)])
        elif k == "max_seqlen":
            out[k] = max(v, pad)
        elif torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == T:
            fill = torch.full((pad,) + tuple(v.shape[1:]), 0 if v.dtype != torch.bool else False,
                              dtype=v.dtype, device=v.device)
            if k == "position_ids":
                fill = torch.arange(pad, dtype=v.dtype, device=v.device)
            out[k] = torch.cat([v, fill])
        else:
            out[k] = v
    return out, pad


def pad_mb_list(mb_list: MicroBatchList, pad_value: float = 0.0, align_to: int = N_TOKENS_PER_PAGE,
                pad_to_maximum: bool = False) -> MicroBatchList:
    """Pads every packed micro-batch to a multiple of ``align_to`` tokens (or to
    ``max_tokens_per_mb``), recording the added length so outputs can be trimmed."""
    padded, pads, old = [], [], []
    for mb in mb_list.mbs:
        T = int(mb["cu_seqlens"][-1])
        if pad_to_maximum and mb_list.mb_spec.max_tokens_per_mb:
            target = mb_list.mb_spec.max_tokens_per_mb
        else:
            target = -(-max(T, 1) // align_to) * align_to
        old.append(mb["cu_seqlens"])
        p, n = pad_packed_tensor_dict(mb, target, pad_value)
        padded.append(p)
        pads.append(n)
    mb_list.padded_mbs, mb_list.padding_lengths, mb_list.old_cu_seqlens_list = padded, pads, old
    return mb_list


def unpad_logits(x: torch.Tensor, padding_length: int) -> torch.Tensor:
    return x[: x.shape[0] - padding_length] if padding_length else x


def reorder_list(xs: list, indices: list[int]) -> list:
    return [xs[i] for i in indices]


def split_packed_by_cu(x: torch.Tensor, cu: Sequence[int]) -> list[torch.Tensor]:
    return [x[cu[i]:cu[i + 1]] for i in range(len(cu) - 1)]


# --------------------------------------------------------------------------- normalisation


class Normalization:
    """Mean / std normalisation at batch or group level with fp64 accumulation.

    The mean (optionally leave-one-out) is computed at ``mean_level``; the std is
    the root mean square deviation *from that mean* taken at ``std_level``.
    Batch-level sums are all-reduced over ``reduce_group`` (the data-parallel
    group). Masked-out positions come out as zero.
    """

    def __init__(self, config: NormConfig):
        self.cfg = config

    @torch.no_grad()
    def __call__(self, x: torch.Tensor, loss_mask: torch.Tensor | None = None,
                 reduce_group: dist.ProcessGroup | None = None) -> torch.Tensor:
        cfg = self.cfg
        if loss_mask is not None and float(loss_mask.sum()) == 0:
            return x.float()
        xf = x.double()
        mask = None if loss_mask is None else loss_mask.double()
        gs = cfg.group_size
        if cfg.mean_level == "batch":
            mean = self._mean(xf, mask, cfg.mean_leave1out, reduce_group, True).expand_as(xf)
        elif cfg.mean_level == "group":
            mean = torch.zeros_like(xf)
            for i in range(xf.shape[0] // gs):
                sl = slice(i * gs, (i + 1) * gs)
                if gs == 1 and cfg.mean_leave1out:
                    continue
                m = None if mask is None else mask[sl]
                mean[sl] = self._mean(xf[sl], m, cfg.mean_leave1out, None, False).expand_as(xf[sl])
        else:
            mean = torch.zeros_like(xf)
        centered = xf - mean
        if mask is not None:
            centered = centered * mask
        eps = cfg.eps
        if cfg.std_level == "batch":
            std = self._std(xf, mask, mean, cfg.std_unbiased, reduce_group, True).expand_as(xf)
        elif cfg.std_level == "group":
            std = torch.ones_like(xf)
            for i in range(xf.shape[0] // gs):
                sl = slice(i * gs, (i + 1) * gs)
                if gs == 1 and cfg.std_unbiased:
                    continue
                m = None if mask is None else mask[sl]
                std[sl] = self._std(xf[sl], m, mean[sl], cfg.std_unbiased, None, False).expand_as(xf[sl])
        else:
            std = torch.ones_like(xf)
            eps = 0.0
        return (centered / (std + eps)).float()

    @staticmethod
    def _reduce(t: torch.Tensor, group, do: bool) -> torch.Tensor:
        if do and dist.is_initialized():
            if not t.is_cuda and dist.get_backend(group) == "nccl":
                dev = t.cuda()  # NCCL reduces device tensors only
                dist.all_reduce(dev, group=group)
                t.copy_(dev)
            else:
                dist.all_reduce(t, group=group)
        return t

    @classmethod
    def _mean(cls, x, mask, leave1out, group, all_reduce):
        if mask is None:
            n = torch.tensor(float(x.numel()), dtype=x.dtype, device=x.device)
            xm = x
        else:
            n = mask.sum()
            xm = x * mask
        s = xm.sum()
        n = cls._reduce(n.clone(), group, all_reduce)
        s = cls._reduce(s.clone(), group, all_reduce)
        if leave1out:
            if float(n) <= 1:
                return torch.zeros_like(x)
            if mask is None:
                return (s - x) / (n - 1)
            loo = (s - xm) / torch.clamp(n - mask, min=1.0)
            return torch.where(mask > 0, loo, (s / n).expand_as(x))
        if float(n) == 0:
            return torch.zeros((), dtype=x.dtype, device=x.device)
        return s / n

    @classmethod
    def _std(cls, x, mask, mean, unbiased, group, all_reduce):
        if mask is None:
            n = torch.tensor(float(x.numel()), dtype=x.dtype, device=x.device)
            ss = ((x - mean) ** 2).sum()
        else:
            n = mask.sum()
            ss = (((x - mean) * mask) ** 2).sum()
        n = cls._reduce(n.clone(), group, all_reduce)
        ss = cls._reduce(ss.clone(), group, all_reduce)
        if unbiased:
            if float(n) <= 1:
                return torch.ones((), dtype=x.dtype, device=x.device)
            return (ss / (n - 1)).sqrt()
        if float(n) == 0:
            return torch.ones((), dtype=x.dtype, device=x.device)
        return (ss / n).sqrt()


class KLEstimator:
    """k1 / k2 / k3 estimators of KL(π‖π_base) from per-token logprobs, clamped to ±10."""

    def __init__(self, kind: str = "k1", apply_clamp: bool = True):
        if kind not in ("k1", "k2", "k3"):
            raise ValueError(f"unknown KL estimator {kind}")
        self.kind, self.apply_clamp = kind, apply_clamp

    def __call__(self, logp: torch.Tensor, logp_base: torch.Tensor) -> torch.Tensor:
        d = logp.float() - logp_base.float()
        if self.kind == "k1":
            kl = d
        elif self.kind == "k2":
            kl = 0.5 * d * d
        else:
            kl = torch.exp(-d) - 1 + d
        return kl.clamp(-10.0, 10.0) if self.apply_clamp else kl


# --------------------------------------------------------------------------- collectives on containers


def _device_for(group) -> torch.device:
    if dist.is_initialized() and dist.get_backend(group) == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def broadcast_tensor_container(data: Any, src_rank: int = 0, group: dist.ProcessGroup | None = None) -> Any:
    """Broadcasts a (nested) dict/list of tensors and picklable leaves from ``src_rank``
    (a global rank) to every rank of ``group``."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return data
    rank = dist.get_rank()
    dev = _device_for(group)
    if rank == src_rank:
        flat: list[torch.Tensor] = []

        def strip(x):
            if torch.is_tensor(x):
                flat.append(x)
                return ("__tensor__", len(flat) - 1, tuple(x.shape), str(x.dtype).replace("torch.", ""))
            if isinstance(x, dict):
                return {k: strip(v) for k, v in x.items()}
            if isinstance(x, (list, tuple)):
                return type(x)(strip(v) for v in x)
            return x

        meta = [strip(data)]
        dist.broadcast_object_list(meta, src=src_rank, group=group)
        for t in flat:
            dist.broadcast(t.to(dev).contiguous(), src=src_rank, group=group)
        return data
    meta = [None]
    dist.broadcast_object_list(meta, src=src_rank, group=group)
    specs: dict[int, tuple] = {}

    def collect(x):
        if isinstance(x, tuple) and len(x) == 4 and x[0] == "__tensor__":
            specs[x[1]] = (x[2], x[3])
        elif isinstance(x, dict):
            for v in x.values():
                collect(v)
        elif isinstance(x, (list, tuple)):
            for v in x:
                collect(v)

    collect(meta[0])
    tensors = {}
    for i in sorted(specs):
        shape, dt = specs[i]
        t = torch.empty(shape, dtype=getattr(torch, dt), device=dev)
        dist.broadcast(t, src=src_rank, group=group)
        tensors[i] = t

    def rebuild(x):
        if isinstance(x, tuple) and len(x) == 4 and x[0] == "__tensor__":
            return tensors[x[1]]
        if isinstance(x, dict):
            return {k: rebuild(v) for k, v in x.items()}
        if isinstance(x, (list, tuple)):
            return type(x)(rebuild(v) for v in x)
        return x

    return rebuild(meta[0])


def all_gather_tensor_container(data: Any, group: dist.ProcessGroup | None = None) -> list[Any]:
    """Every rank receives the list of all ranks' containers (tensors moved through CPU)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return [data]

    def to_cpu(x):
        if torch.is_tensor(x):
            return x.detach().cpu()
        if isinstance(x, dict):
            return {k: to_cpu(v) for k, v in x.items()}
        if isinstance(x, (list, tuple)):
            return type(x)(to_cpu(v) for v in x)
        return x

    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, to_cpu(data), group=group)
    return out


def cycle_dataloader(dataloader, num_cycles: int | None = None):
    """Endless (or ``num_cycles``-long) iteration, bumping the sampler epoch each pass."""
    epoch = 0
    while num_cycles is None or epoch < num_cycles:
        sampler = getattr(dataloader, "sampler", None)
        # a loader that advances its own epoch (and may have been restored in the middle of one) is left alone
        if sampler is not None and hasattr(sampler, "set_epoch") and not getattr(dataloader, "auto_epoch", False):
            sampler.set_epoch(epoch)
        for batch in dataloader:
            yield batch
        epoch += 1


# ------------------------------------------------------------------ container helpers
# Small conveniences over dicts / lists of tensors that workflow and reward code uses (areal/utils/data.py has
# helpers of the same names; these are written against this package's batch conventions).
def list_of_dict2dict_of_list(items: Sequence[dict[str, Any]]) -> dict[str, list[Any]]:
    """``[{a: 1, b: 2}, {a: 3, b: 4}]`` → ``{a: [1, 3], b: [2, 4]}``; every item must have the same keys."""
    if not items:
        return {}
    keys = list(items[0].keys())
    for it in items:
        if set(it.keys()) != set(keys):
            raise ValueError(f"items have different keys: {sorted(it.keys())} vs {sorted(keys)}")
    return {k: [it[k] for it in items] for k in keys}


def dict_of_list2list_of_dict(d: dict[str, Sequence[Any]]) -> list[dict[str, Any]]:
    """Inverse of :func:`list_of_dict2dict_of_list`; every list must have the same length."""
    if not d:
        return []
    n = {len(v) for v in d.values()}
    if len(n) != 1:
        raise ValueError(f"lists have different lengths: { {k: len(v) for k, v in d.items()} }")
    return [{k: v[i] for k, v in d.items()} for i in range(n.pop())]


def dict_map(fn, d: dict[str, Any]) -> dict[str, Any]:
    return {k: fn(v) for k, v in d.items()}


def tensor_container_to(data: Any, *args, **kwargs) -> Any:
    """``.to(*args, **kwargs)`` on every tensor inside nested dicts / lists / tuples; other leaves pass through."""
    if torch.is_tensor(data):
        return data.to(*args, **kwargs)
    if isinstance(data, dict):
        return {k: tensor_container_to(v, *args, **kwargs) for k, v in data.items()}
    if isinstance(data, (list, tuple)):
        return type(data)(tensor_container_to(v, *args, **kwargs) for v in data)
    return data


def pad_and_stack_tensors_along_first_dim(tensors: Sequence[torch.Tensor], pad_value: float = 0.0) -> torch.Tensor:
    """Stacks tensors whose first dimension differs, padding at the end: ``[n_i, ...]`` → ``[len, max n_i, ...]``."""
    n = max(t.shape[0] for t in tensors)
    out = tensors[0].new_full((len(tensors), n) + tuple(tensors[0].shape[1:]), pad_value)
    for i, t in enumerate(tensors):
        out[i, : t.shape[0]] = t
    return out


def unpad_input(x: torch.Tensor, attention_mask: torch.Tensor):
    """Padded ``[B, L, ...]`` → packed ``[T, ...]`` with the flat indices of the kept positions, ``cu_seqlens``
    (int32) and the longest sequence (the calling convention of variable-length attention)."""
    mask = attention_mask.bool()
    lens = mask.sum(-1).to(torch.int32)
    idx = mask.reshape(-1).nonzero(as_tuple=False).squeeze(-1)
    cu = torch.zeros(lens.numel() + 1, dtype=torch.int32, device=lens.device)
    cu[1:] = lens.cumsum(0)
    flat = x.reshape((-1,) + tuple(x.shape[2:]))
    return flat[idx], idx, cu, int(lens.max()) if lens.numel() else 0


def pad_input(packed: torch.Tensor, indices: torch.Tensor, batch: int, seqlen: int) -> torch.Tensor:
    """Inverse of :func:`unpad_input`: scatters packed rows back into a zero ``[batch, seqlen, ...]`` tensor."""
    out = packed.new_zeros((batch * seqlen,) + tuple(packed.shape[1:]))
    out[indices] = packed
    return out.reshape((batch, seqlen) + tuple(packed.shape[1:]))


def unpack_sequence(x: torch.Tensor, cu_seqlens: torch.Tensor | Sequence[int] | None = None,
                    lens: Sequence[int] | None = None, dim: int = 0) -> list[torch.Tensor]:
    """Cuts a packed tensor into its sequences along ``dim``, by ``cu_seqlens`` or by ``lens``."""
    if lens is None:
        cu = cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else list(cu_seqlens)
        lens = [b - a for a, b in zip(cu[:-1], cu[1:])]
    return list(torch.split(x, [int(n) for n in lens], dim=dim))


def split_batch(data: dict[str, Any], n: int) -> list[dict[str, Any]]:
    """``n`` consecutive parts of a padded batch with sizes as equal as possible (tensors and per-sample lists are
    cut along the batch dimension, everything else is shared)."""
    B = get_batch_size(data)
    if not 1 <= n <= max(B, 1):
        raise ValueError(f"cannot split a batch of {B} into {n} parts")
    sizes = [B // n + (1 if i < B % n else 0) for i in range(n)]
    out, a = [], 0
    for s in sizes:
        out.append({k: (v[a:a + s] if (torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == B) or
                        (isinstance(v, list) and len(v) == B) else v) for k, v in data.items()})
        a += s
    return out


def concat_batch(parts: Sequence[dict[str, Any]], pad_value: float = 0.0) -> dict[str, Any]:
    """Inverse of :func:`split_batch` (sequence dimensions are padded to the longest part)."""
    return concat_padded_tensors(list(parts), pad_value)


def make_dummy_eval_item(template: dict[str, Any]) -> dict[str, Any]:
    """A sample shaped like ``template`` that carries no loss weight: a one-token sequence with an all-zero
    ``loss_mask``. Evaluation batches that do not divide over the data-parallel ranks are topped up with these."""
    out: dict[str, Any] = {}
    for k, v in template.items():
        if torch.is_tensor(v) and v.dim() >= 2:
            z = torch.zeros((1, 1) + tuple(v.shape[2:]), dtype=v.dtype)
            if k == "attention_mask":
                z[:] = 1
            out[k] = z
        elif torch.is_tensor(v) and v.dim() == 1:
            out[k] = torch.zeros(1, dtype=v.dtype)
        elif isinstance(v, list):
            out[k] = [None]
        else:
            out[k] = v
    return out


def broadcast_tensor(t: torch.Tensor | None, src_rank: int = 0, group: dist.ProcessGroup | None = None,
                     device=None) -> torch.Tensor:
    """Broadcasts one tensor whose shape and dtype the receivers do not know (metadata first, then the data)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return t
    meta = [None]
    if dist.get_rank() == src_rank:
        meta = [(tuple(t.shape), t.dtype)]
    dist.broadcast_object_list(meta, src=src_rank, group=group)
    shape, dtype = meta[0]
    dev = device if device is not None else (t.device if t is not None else _device_for(group))
    buf = t.to(dev).contiguous() if dist.get_rank() == src_rank else torch.empty(shape, dtype=dtype, device=dev)
    dist.broadcast(buf, src=src_rank, group=group)
    return buf
