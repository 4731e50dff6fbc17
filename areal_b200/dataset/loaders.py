"""Local-file record loading shared by the dataset builders."""

from __future__ import annotations

import json
import os
from typing import Any


def load_records(path: str, split: str = "train") -> list[dict[str, Any]]:
    """Reads ``path`` (file or directory). Directories are searched for ``{split}.jsonl|json|parquet``
    (also under ``main/`` or ``data/``) or loaded with ``datasets.load_from_disk``."""
    if os.path.isdir(path):
        for sub in ("", "main", "data", "default"):
            for ext in ("jsonl", "json", "parquet"):
                for name in (f"{split}.{ext}", f"{split}-00000-of-00001.{ext}"):
                    cand = os.path.join(path, sub, name)
                    if os.path.exists(cand):
                        return load_records(cand, split)
        try:
            import datasets

            ds = datasets.load_from_disk(path)
            ds = ds[split] if hasattr(ds, "keys") and split in ds else ds
            return [dict(x) for x in ds]
        except Exception as e:
            raise FileNotFoundError(f"no {split} split found under {path}: {e}") from e
    if path.endswith(".jsonl"):
        with open(path) as f:
            return [json.loads(line) for line in f if line.strip()]
    if path.endswith(".json"):
        with open(path) as f:
            data = json.load(f)
        return data[split] if isinstance(data, dict) and split in data else data
    if path.endswith(".parquet"):
        import pyarrow.parquet as pq

        return pq.read_table(path).to_pylist()
    raise FileNotFoundError(f"unsupported dataset file {path}")


def tokenize_prompt_answer(tokenizer, prompt: str, answer: str, max_length: int | None):
    """SFT sample: loss on the answer tokens (and EOS) only."""
    p = tokenizer.encode(prompt)
    a = tokenizer.encode(answer, add_special_tokens=False)
    eos = [tokenizer.eos_token_id] if getattr(tokenizer, "eos_token_id", None) is not None else []
    ids = p + a + eos
    mask = [0] * len(p) + [1] * (len(a) + len(eos))
    if max_length is not None and len(ids) > max_length:
        return None
    return dict(input_ids=ids, loss_mask=mask)
