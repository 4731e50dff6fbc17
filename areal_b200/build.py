"""Builds the native libraries in-tree.

Two shared objects are produced under ``areal_b200/_native``:

* ``libareal_b200_kernels.so`` – every CUDA kernel (``csrc/*.cu``), compiled by
  nvcc for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``).
* ``libareal_b200_host.so`` – the C++ host runtime (``csrc/host/*.cpp``):
  sequence packer/partitioners and the paged-KV block manager + scheduler.

Both expose a plain C ABI and are loaded with ctypes (see ``ops/_lib.py``), so
no Python headers are needed and the build takes seconds per file.

Run ``python -m areal_b200.build`` (add ``--force`` to rebuild everything).
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "_native"
OBJ = OUT / "obj"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-lineinfo",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
    "-I",
    str(CSRC),
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha256()
    h.update(path.read_bytes())
    for hdr in sorted((CSRC / "common").glob("*")):
        if hdr.suffix in (".h", ".cuh"):
            h.update(hdr.read_bytes())
    h.update(extra.encode())
    return h.hexdigest()


def _compile(cmd: list[str], src: Path, obj: Path, stamp: str, verbose: bool) -> None:
    stamp_file = obj.with_suffix(obj.suffix + ".stamp")
    if obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose and res.stderr.strip():
        print(res.stderr, flush=True)
    stamp_file.write_text(stamp)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> dict[str, Path]:
    OBJ.mkdir(parents=True, exist_ok=True)
    if force:
        for f in OBJ.glob("*"):
            f.unlink()
    nvcc = _nvcc()
    cu_srcs = sorted(CSRC.glob("*.cu")) + sorted((CSRC / "common").glob("*.cu"))
    # selftest.cpp is a standalone sanitizer driver with its own main(), not part of the library
    cpp_srcs = sorted(p for p in (CSRC / "host").glob("*.cpp") if p.name != "selftest.cpp")
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])
    jobs = []
    cu_objs, cpp_objs = [], []
    for src in cu_srcs:
        obj = OBJ / (src.stem + ".o")
        cu_objs.append(obj)
        cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
        jobs.append((cmd, src, obj, _digest(src, " ".join(flags))))
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    for src in cpp_srcs:
        obj = OBJ / (src.stem + ".host.o")
        cpp_objs.append(obj)
        cmd = [cxx, *CXX_FLAGS, "-c", str(src), "-o", str(obj)]
        jobs.append((cmd, src, obj, _digest(src, " ".join(CXX_FLAGS))))
    with ThreadPoolExecutor(max_workers=max(1, (os.cpu_count() or 2))) as ex:
        futs = [ex.submit(_compile, *j, verbose or ptxas_info) for j in jobs]
        for f in futs:
            f.result()
    out = {}
    if cu_objs:
        lib = OUT / "libareal_b200_kernels.so"
        newest = max(o.stat().st_mtime for o in cu_objs)
        if force or not lib.exists() or lib.stat().st_mtime < newest:
            cmd = [nvcc, "-shared", "-o", str(lib), *map(str, cu_objs), "-gencode",
                   "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        out["kernels"] = lib
    if cpp_objs:
        lib = OUT / "libareal_b200_host.so"
        newest = max(o.stat().st_mtime for o in cpp_objs)
        if force or not lib.exists() or lib.stat().st_mtime < newest:
            cmd = [cxx, "-shared", "-o", str(lib), *map(str, cpp_objs), "-pthread"]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        out["host"] = lib
    return out


def main(argv: list[str] | None = None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    libs = build(force="--force" in argv, verbose="-v" in argv, ptxas_info="--ptxas" in argv)
    for k, v in libs.items():
        print(f"{k}: {v}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
