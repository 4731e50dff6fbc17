"""Experiment metadata saved next to the logs: config snapshot, git commit of the working tree,
versions of the key packages, launch command. Reference: areal/infra/utils/exp_metadata.py."""

from __future__ import annotations

import dataclasses
import json
import os
import subprocess
import sys
import time


def collect_metadata(config=None) -> dict:
    meta = {"time": time.strftime("%Y-%m-%dT%H:%M:%S"), "argv": list(sys.argv), "python": sys.version.split()[0]}
    try:
        import torch

        meta["torch"] = torch.__version__
        meta["cuda"] = torch.version.cuda
    except Exception:
        pass
    try:
        here = os.path.dirname(os.path.abspath(__file__))
        meta["git_commit"] = subprocess.run(["git", "rev-parse", "HEAD"], cwd=here, capture_output=True, text=True,
                                            timeout=5).stdout.strip() or None
    except Exception:
        meta["git_commit"] = None
    if config is not None:
        meta["config"] = dataclasses.asdict(config) if dataclasses.is_dataclass(config) else config
    return meta


def save_metadata(path: str, config=None) -> str:
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "w") as f:
        json.dump(collect_metadata(config), f, indent=2, default=str)
    return path
