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


class KernelArgumentError(RuntimeError):
    """Checked mode found an argument that would make a kernel read or write outside its buffers."""


def checked() -> bool:
    """Checked mode (``AREAL_B200_CHECKED=1``): before a launch the wrappers validate, on the host, every
    index that the kernel takes from data (positions, cache slots, page tables, expert ids) against the
    extent of the buffer it indexes, and the layout of the operands. Each check costs a device
    synchronisation, so the mode is for tests and debugging; it is skipped while a CUDA graph is captured."""
    if os.environ.get("AREAL_B200_CHECKED") != "1":
        return False
    return not (torch.cuda.is_available() and torch.cuda.is_current_stream_capturing())


_checks_run = 0


def checks_run() -> int:
    return _checks_run


def check_index(site: str, t: torch.Tensor | None, upper: int, lower: int = 0, where: torch.Tensor | None = None,
                allow_negative: bool = False) -> None:
    """Raises unless every element of ``t`` (restricted to ``where``; negative values pass when
    ``allow_negative`` says that the kernel skips them) lies in ``[lower, upper)``."""
    global _checks_run
    if t is None or t.numel() == 0:
        return
    _checks_run += 1
    v = t if where is None else t[where]
    if v.numel() == 0:
        return
    if allow_negative:
        v = v[v >= 0]
        if v.numel() == 0:
            return
    lo, hi = int(v.min()), int(v.max())
    if lo < lower or hi >= upper:
        raise KernelArgumentError(f"{site}: index range [{lo}, {hi}] outside [{lower}, {upper})")


def check_operand(site: str, t: torch.Tensor | None, dtype: torch.dtype | None = None, shape: tuple | None = None,
                  align: int = 16, contiguous: bool = True) -> None:
    """Layout of one kernel operand: dtype, shape (``None`` entries are free), base alignment, contiguity."""
    global _checks_run
    if t is None:
        return
    _checks_run += 1
    if dtype is not None and t.dtype != dtype:
        raise KernelArgumentError(f"{site}: dtype {t.dtype}, expected {dtype}")
    if shape is not None and (t.dim() != len(shape) or any(e is not None and e != a for a, e in zip(t.shape, shape))):
        raise KernelArgumentError(f"{site}: shape {tuple(t.shape)}, expected {shape}")
    if contiguous and not t.is_contiguous():
        raise KernelArgumentError(f"{site}: operand is not contiguous (strides {t.stride()})")
    if align and t.numel() and t.data_ptr() % align:
        raise KernelArgumentError(f"{site}: base address {t.data_ptr():#x} is not {align}-byte aligned")


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
