"""ctypes loader for the in-tree native libraries.

The CUDA kernels live in ``_native/libareal_b200_kernels.so`` and the C++ host
runtime in ``_native/libareal_b200_host.so`` (built by ``areal_b200.build``).
Every exported symbol has a plain C signature: raw device pointers, sizes and a
``cudaStream_t``; the wrappers in this package pass ``tensor.data_ptr()`` and the
current torch stream.

On a machine with a GPU a missing kernel library is an error (ops never fall
back silently to PyTorch); on a CPU-only machine the ops use their PyTorch
reference implementation, which is also the numerics oracle of the tests.
"""

from __future__ import annotations

import ctypes
import functools
import os
from pathlib import Path

import torch

_NATIVE = Path(__file__).resolve().parent.parent / "_native"


class NativeLibraryMissing(RuntimeError):
    pass


@functools.lru_cache(maxsize=None)
def kernels() -> ctypes.CDLL:
    path = _NATIVE / "libareal_b200_kernels.so"
    if not path.exists():
        raise NativeLibraryMissing(
            f"{path} not found: run `python -m areal_b200.build` (needs nvcc with sm_100a support)"
        )
    return ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)


@functools.lru_cache(maxsize=None)
def host() -> ctypes.CDLL:
    path = _NATIVE / "libareal_b200_host.so"
    if not path.exists():
        raise NativeLibraryMissing(f"{path} not found: run `python -m areal_b200.build`")
    return ctypes.CDLL(str(path))


def have_host() -> bool:
    try:
        host()
        return True
    except (NativeLibraryMissing, OSError):
        return False


def use_cuda_kernels(*tensors: torch.Tensor) -> bool:
    """True when the op must run on the hand-written kernels.

    That is the case whenever the inputs are CUDA tensors. ``AREAL_B200_FORCE_TORCH=1``
    routes CUDA tensors to the PyTorch reference instead (used by tests that
    compare the two on the same device).
    """
    if not tensors or not all(t.is_cuda for t in tensors if t is not None):
        return False
    if os.environ.get("AREAL_B200_FORCE_TORCH") == "1":
        return False
    lib = kernels()  # raises loudly if the library is missing on a GPU box
    rc = lib.b200_ensure_device(ctypes.c_int(tensors[0].device.index or 0))
    if rc != 0:
        raise RuntimeError(f"b200_ensure_device failed with code {rc}")
    return True


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"areal_b200 native call {what} failed with code {rc}")


_launch_count = 0


def count_launch(n: int = 1) -> None:
    """Counts launches of this library's own kernels (read by the benchmark)."""
    global _launch_count
    _launch_count += n


def launch_count() -> int:
    return _launch_count


def reset_launch_count() -> None:
    global _launch_count
    _launch_count = 0


_fallbacks: dict[str, int] = {}


def count_fallback(op: str) -> None:
    """Records that an op ran on a PyTorch library operator although its inputs were CUDA tensors (a shape
    this library's kernels do not cover). The benchmark reports these counts; zero means every hot op ran on
    the in-tree kernels. The first occurrence of each op is also logged."""
    n = _fallbacks.get(op, 0)
    if n == 0:
        import logging

        logging.getLogger("areal_b200.ops").warning(f"CUDA fallback to a PyTorch operator: {op}")
    _fallbacks[op] = n + 1


def fallback_counts() -> dict[str, int]:
    return dict(_fallbacks)


def read_status() -> int:
    """Synchronises the current stream and returns (and clears) the device status word.

    A non-zero value means a kernel gave up on a bounded wait (see
    ``csrc/common/ptx.cuh`` for the codes).
    """
    lib = kernels()
    lib.b200_read_status.argtypes = [ctypes.c_void_p]
    lib.b200_read_status.restype = ctypes.c_int
    return lib.b200_read_status(stream_ptr())


class DeviceWaitTimeout(RuntimeError):
    """A kernel's bounded wait (mbarrier or peer flag) ran out."""


def raise_on_status() -> None:
    code = read_status()
    if code != 0:
        raise DeviceWaitTimeout(f"device status word = {code}")
