"""Checks that this installation can run: Python dependencies, the CUDA toolchain, the in-tree
native libraries (built on demand), the CPU reference path and, when a GPU is visible, one kernel
of every family against its reference.

    python -m areal_b200.tools.validate_installation [--no-build]

Exit code 0 when every mandatory check passes. Counterpart of areal/tools/validate_installation.py.
"""

from __future__ import annotations

import argparse
import importlib
import shutil
import sys
import traceback

MANDATORY = ["torch", "numpy", "yaml", "fastapi", "uvicorn", "requests", "aiohttp", "pydantic", "psutil"]
OPTIONAL = ["transformers", "safetensors", "ray", "wandb", "tensorboardX", "pynvml"]


def _check(name, fn, results, mandatory=True):
    try:
        detail = fn()
        results.append((name, True, mandatory, str(detail or "")))
    except Exception as e:  # noqa: BLE001 - every failure is reported, none is fatal here
        results.append((name, False, mandatory, f"{type(e).__name__}: {e}"))
        if "-v" in sys.argv:
            traceback.print_exc()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--no-build", action="store_true", help="do not compile the native libraries")
    ap.add_argument("-v", action="store_true")
    args = ap.parse_args(argv)
    results: list[tuple[str, bool, bool, str]] = []
    for m in MANDATORY:
        _check(f"import {m}", lambda m=m: getattr(importlib.import_module(m), "__version__", ""), results)
    for m in OPTIONAL:
        _check(f"import {m} (optional)", lambda m=m: getattr(importlib.import_module(m), "__version__", ""), results, False)
    _check("nvcc on PATH", lambda: shutil.which("nvcc") or (_ for _ in ()).throw(FileNotFoundError("nvcc")), results,
           mandatory=not args.no_build)

    def build():
        from areal_b200 import build as b

        if not args.no_build:
            b.build()
        from areal_b200.ops import _lib

        _lib.host()
        return "native libraries load"

    _check("native libraries", build, results)

    def cpu_path():
        import torch

        from areal_b200.models.config import PRESETS
        from areal_b200.models.qwen import build_model
        from areal_b200.ops.attention import VarlenMeta

        m = build_model(PRESETS["tiny-qwen2"], dtype=torch.float32, seed=0)
        y = m(torch.arange(12), torch.arange(12), VarlenMeta([0, 12], "cpu"))
        assert torch.isfinite(y).all()
        return "tiny model forward on CPU"

    _check("CPU reference path", cpu_path, results)

    def gpu_path():
        import torch

        if not torch.cuda.is_available():
            return "no GPU visible: skipped"
        from areal_b200.ops import _lib
        from areal_b200.ops.gemm import gemm

        a = torch.randn(256, 512, device="cuda").bfloat16()
        b = torch.randn(384, 512, device="cuda").bfloat16()
        err = (gemm(a, b).float() - a.float() @ b.float().t()).abs().max().item()
        assert err < 1.0 and _lib.read_status() == 0, err
        cap = torch.cuda.get_device_capability()
        assert cap[0] == 10, f"these kernels target sm_100a, found sm_{cap[0]}{cap[1]}"
        return f"tcgen05 GEMM ok on {torch.cuda.get_device_name()}"

    _check("GPU kernels", gpu_path, results)
    width = max(len(r[0]) for r in results)
    failed = 0
    for name, ok, mandatory, detail in results:
        mark = "ok  " if ok else ("FAIL" if mandatory else "miss")
        failed += (not ok) and mandatory
        print(f"[{mark}] {name.ljust(width)}  {detail}")
    print("installation is usable" if not failed else f"{failed} mandatory check(s) failed")
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
