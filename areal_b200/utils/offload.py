"""Offloadable device buffers on CUDA virtual memory management (``csrc/vmm_offload.cu``).

An :class:`OffloadableBuffer` keeps its virtual address for life; ``offload()`` releases the
physical HBM behind it (optionally parking the contents in pinned host memory) and
``onload()`` maps fresh memory at the same address. Tensors, TMA descriptors, CUDA graphs
and peer tables that point into the buffer therefore survive the cycle, which is what lets
a colocated trainer and rollout engine trade HBM without rebuilding anything.

Counterpart of the reference's use of ``torch_memory_saver`` (areal/utils/offload.py,
areal/engine/fsdp_engine.py ``offload`` / ``onload``). On CPU the buffer is an ordinary
tensor and both calls only flip the state flag.
"""

from __future__ import annotations

import ctypes

import torch

from ..ops import _lib
from ..parallel.symm_mem import tensor_from_ptr


class OffloadableBuffer:
    def __init__(self, nbytes: int, device=None):
        self.nbytes = int(nbytes)
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.ptr = 0
        self.resident = True
        if self.device.type == "cuda":
            lib = _lib.kernels()
            lib.b200_ensure_device(ctypes.c_int(self.device.index or 0))
            lib.b200_vmm_alloc.restype = ctypes.c_void_p
            p = lib.b200_vmm_alloc(ctypes.c_size_t(self.nbytes))
            if not p:
                raise MemoryError(f"b200_vmm_alloc({self.nbytes}) failed")
            self.ptr = int(p)
            self._bytes = tensor_from_ptr(self.ptr, self.nbytes, self.device)
        else:
            self._bytes = torch.zeros(self.nbytes, dtype=torch.uint8)

    def tensor(self, dtype: torch.dtype, shape=None, byte_offset: int = 0) -> torch.Tensor:
        """A view into the buffer; only valid to touch while the buffer is resident."""
        item = torch.empty((), dtype=dtype).element_size()
        if shape is None:
            n = (self.nbytes - byte_offset) // item
            return self._bytes[byte_offset:byte_offset + n * item].view(dtype)
        n = 1
        for d in shape:
            n *= int(d)
        return self._bytes[byte_offset:byte_offset + n * item].view(dtype).view(*shape)

    def offload(self, preserve: bool = True):
        if not self.resident:
            return
        if self.ptr:
            torch.cuda.synchronize(self.device)
            rc = _lib.kernels().b200_vmm_offload(ctypes.c_void_p(self.ptr), ctypes.c_int(int(preserve)))
            _lib.check(rc, "b200_vmm_offload")
        elif not preserve:
            self._bytes.zero_()
        self.resident = False

    def onload(self):
        if self.resident:
            return
        if self.ptr:
            rc = _lib.kernels().b200_vmm_onload(ctypes.c_void_p(self.ptr))
            if rc == -2:
                raise MemoryError("not enough free device memory to bring the buffer back")
            _lib.check(rc, "b200_vmm_onload")
        self.resident = True

    def free(self):
        if self.ptr:
            self._bytes = None
            _lib.kernels().b200_vmm_free(ctypes.c_void_p(self.ptr))
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
