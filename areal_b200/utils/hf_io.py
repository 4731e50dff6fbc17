"""HF-format checkpoint IO: sharded safetensors + ``config.json`` (+ tokenizer files).

Weights are written under HF parameter names, so checkpoints interchange with
``transformers`` and with the reference's savers
(areal/engine/fsdp_engine.py:1627-1666). Loading streams tensors file by file
straight into the model's fused parameters.
"""

from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Iterator

import torch
from safetensors import safe_open
from safetensors.torch import save_file

MAX_SHARD_BYTES = 5 * (1 << 30)


def weight_files(path: str) -> list[Path]:
    """The safetensors files that hold the model's weights: those the index names when there is one, else
    every ``*.safetensors`` file except adapter files (``adapter_model.safetensors`` of a LoRA checkpoint
    sits beside the merged model and is not part of it)."""
    p = Path(path)
    idx = p / "model.safetensors.index.json"
    if idx.exists():
        with open(idx) as f:
            names = sorted(set(json.load(f).get("weight_map", {}).values()))
        files = [p / n for n in names if (p / n).exists()]
        if files:
            return files
    return [f for f in sorted(p.glob("*.safetensors")) if not f.name.startswith("adapter_")]


def remove_weight_files(path: str, tag: str | None = None):
    """Deletes earlier weight files of a checkpoint directory before it is written again, so that files
    of another sharding do not linger (``tag``: only the files of that writer)."""
    p = Path(path)
    if not p.is_dir():
        return
    pat = f"model-{tag}-*.safetensors" if tag else "model*.safetensors"
    for f in p.glob(pat):
        f.unlink(missing_ok=True)
    if not tag:
        (p / "model.safetensors.index.json").unlink(missing_ok=True)


def dequant_fp8_blockwise(w: torch.Tensor, scale_inv: torch.Tensor, block: int = 128,
                          dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``out[i, j] = w[i, j] * scale_inv[i // block, j // block]`` for an e4m3 weight with one fp32 scale per
    ``block x block`` tile (the layout of block-quantised HF checkpoints: ``<name>.weight`` in float8 beside
    ``<name>.weight_scale_inv``). Reference: areal/experimental/models/archon/fp8_checkpoint.py:119-150."""
    M, N = w.shape
    s = scale_inv.float().repeat_interleave(block, 0)[:M].repeat_interleave(block, 1)[:, :N]
    return (w.float() * s).to(dtype)


_FP8 = tuple(getattr(torch, n) for n in ("float8_e4m3fn", "float8_e5m2") if hasattr(torch, n))


def iter_hf_tensors(path: str, dequant_dtype: torch.dtype = torch.bfloat16) -> Iterator[tuple[str, torch.Tensor]]:
    """``(name, tensor)`` of every weight. Block-quantised fp8 weights are returned dequantised (their
    ``*_scale_inv`` companions are consumed here and not yielded); the block size comes from ``config.json``
    (``quantization_config.weight_block_size``, default 128)."""
    files = weight_files(path)
    if not files:
        raise FileNotFoundError(f"no .safetensors files under {path}")
    block = 128
    cfg = Path(path) / "config.json"
    if cfg.exists():
        try:
            q = json.load(open(cfg)).get("quantization_config") or {}
            block = int((q.get("weight_block_size") or [128])[0])
        except (ValueError, TypeError, json.JSONDecodeError):
            pass
    # a weight and its scale may sit in different files: index the scales first
    scale_file: dict[str, Path] = {}
    for f in files:
        with safe_open(str(f), framework="pt", device="cpu") as sf:
            for name in sf.keys():
                if name.endswith("_scale_inv"):
                    scale_file[name] = f
    for f in files:
        with safe_open(str(f), framework="pt", device="cpu") as sf:
            for name in sf.keys():
                if name in scale_file:
                    continue
                t = sf.get_tensor(name)
                if t.dtype in _FP8:
                    sname = name + "_scale_inv"
                    if sname not in scale_file:
                        raise KeyError(f"{name} is stored in {t.dtype} but {sname} is missing")
                    with safe_open(str(scale_file[sname]), framework="pt", device="cpu") as ss:
                        t = dequant_fp8_blockwise(t, ss.get_tensor(sname), block, dequant_dtype)
                yield name, t


def load_hf_weights(model, path: str, strict: bool = True):
    model.load_hf(iter_hf_tensors(path), strict=strict)
    return model


def write_hf_index(path: str):
    """``model.safetensors.index.json`` over every ``*.safetensors`` file of the directory (pipeline stages write
    their own files; the index lets HF loaders find every tensor)."""
    index, total = {}, 0
    files = sorted(Path(path).glob("*.safetensors"))
    for f in files:
        if f.name.startswith("adapter_"):
            continue
        with safe_open(str(f), framework="pt", device="cpu") as sf:
            for name in sf.keys():
                index[name] = f.name
                sl = sf.get_slice(name)
                n = 1
                for d in sl.get_shape():
                    n *= d
                total += n * {"F32": 4, "F64": 8, "I64": 8, "I32": 4}.get(sl.get_dtype(), 2)
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": index}, f, indent=2)


def save_hf_checkpoint(model, model_config, path: str, tokenizer=None, max_shard_bytes: int = MAX_SHARD_BYTES,
                       processor=None, write: bool = True, file_tag: str = "", keep=None):
    """``write=False``: only take part in the collectives of ``model.to_hf()`` (tensor-parallel gathers) without
    touching the directory. ``file_tag`` keeps the files of several writers apart (one per pipeline stage or
    expert-parallel rank: ``model-<tag>-00001-of-0000N.safetensors``; call :func:`write_hf_index` once all of
    them are done). ``keep(name)`` selects the tensors this writer puts down (an expert-parallel rank other than
    the first writes only its experts)."""
    if not write:
        for _ in model.to_hf():
            pass
        return
    os.makedirs(path, exist_ok=True)
    if not file_tag:
        remove_weight_files(path)  # several writers: the caller clears the directory once, before any of them
    shards: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    index: dict[str, str] = {}
    for name, t in model.to_hf():
        if keep is not None and not keep(name):
            continue
        nbytes = t.numel() * t.element_size()
        if shards[-1] and size + nbytes > max_shard_bytes:
            shards.append({})
            size = 0
        shards[-1][name] = t.detach().to("cpu").contiguous().clone()
        size += nbytes
    n = len(shards)
    total = 0
    for i, sh in enumerate(shards):
        if file_tag:
            fname = f"model-{file_tag}-{i + 1:05d}-of-{n:05d}.safetensors"
        else:
            fname = "model.safetensors" if n == 1 else f"model-{i + 1:05d}-of-{n:05d}.safetensors"
        save_file(sh, os.path.join(path, fname), metadata={"format": "pt"})
        for k, v in sh.items():
            index[k] = fname
            total += v.numel() * v.element_size()
    if n > 1 and not file_tag:
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": index}, f, indent=2)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(model_config.to_hf_config(), f, indent=2)
    if tokenizer is not None and hasattr(tokenizer, "save_pretrained"):
        tokenizer.save_pretrained(path)
    if processor is not None and hasattr(processor, "save_pretrained"):
        processor.save_pretrained(path)  # image preprocessing settings of a vision-language checkpoint


def load_hf_tokenizer(path: str, **kwargs):
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(path, **kwargs)


def load_hf_processor_and_tokenizer(path: str, **kwargs):
    """``(processor, tokenizer)`` of a vision-language checkpoint (the processor expands image placeholders and
    produces ``pixel_values`` / ``image_grid_thw``)."""
    from transformers import AutoProcessor

    processor = AutoProcessor.from_pretrained(path, **kwargs)
    return processor, getattr(processor, "tokenizer", None) or load_hf_tokenizer(path, **kwargs)


def chat_template_ids(tokenizer, messages, **kwargs) -> list[int]:
    """Token ids of ``tokenizer.apply_chat_template(messages, tokenize=True, ...)`` as a plain list: depending on
    the ``transformers`` version the call returns a list, a tensor or a ``BatchEncoding`` holding ``input_ids``."""
    out = tokenizer.apply_chat_template(messages, tokenize=True, **kwargs)
    if hasattr(out, "keys") and "input_ids" in out:
        out = out["input_ids"]
    if hasattr(out, "tolist"):
        out = out.tolist()
    out = list(out)
    if out and isinstance(out[0], (list, tuple)):
        out = list(out[0])
    return [int(t) for t in out]
