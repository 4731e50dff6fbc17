"""Symmetric memory over NVLink: every rank of a process group allocates the
same buffer, exports it through CUDA IPC and maps the peers' buffers, after
which this library's kernels read and write peer memory directly
(``csrc/symm_comm.cu``, ``csrc/optim.cu``).

``SymmBuffer``   – one allocation per rank + the table of peer pointers.
``SymmBarrier``  – flag barrier in symmetric memory (bounded device-side wait).
``SymmComm``     – all-gather / reduce-scatter / all-reduce / all-to-all on top.

On CPU (gloo) the same interface is backed by ``torch.distributed`` collectives
so host-side logic can be tested without GPUs. The NCCL-based counterparts in
the reference are the FSDP2 / Ulysses / vocab-parallel call sites
(areal/models/fsdp/ulysses.py:153-204).
"""

from __future__ import annotations

import ctypes
from typing import Sequence

import torch
import torch.distributed as dist

from ..ops import _lib


class _RawCudaMemory:
    """Exposes a raw device allocation to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


def tensor_from_ptr(ptr: int, nbytes: int, device) -> torch.Tensor:
    return torch.as_tensor(_RawCudaMemory(ptr, nbytes), device=device)


class SymmBuffer:
    """``nbytes`` of device memory on every rank of ``group`` with peer mappings.

    ``ranks_subset`` limits the exchange to some ranks of the group (the others
    pass ``nbytes=0`` and only learn the pointers, e.g. trainer ranks that write
    into rollout buffers they do not themselves allocate)."""

    def __init__(self, nbytes: int, group: dist.ProcessGroup | None | str = None, device=None):
        # group == "local": a private allocation of this process (no exchange), e.g. the rollout
        # engine's weight buffer, which is exported separately to the trainer ranks
        local = isinstance(group, str) and group == "local"
        self.group = None if local else group
        self.world = dist.get_world_size(group) if (dist.is_initialized() and not local) else 1
        self.rank = dist.get_rank(group) if (dist.is_initialized() and not local) else 0
        self.nbytes = int(nbytes)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.local_ptr = 0
        self.peer_ptrs: list[int] = [0] * self.world
        self._opened: list[int] = []
        lib = _lib.kernels()
        lib.b200_ensure_device(ctypes.c_int(self.device.index or 0))
        lib.b200_symm_alloc.restype = ctypes.c_void_p
        lib.b200_ipc_open_handle.restype = ctypes.c_void_p
        if self.nbytes > 0:
            # 2 MiB granularity keeps the IPC mapping simple and TMA-aligned
            padded = (self.nbytes + (1 << 21) - 1) >> 21 << 21
            p = lib.b200_symm_alloc(ctypes.c_size_t(padded))
            if not p:
                raise MemoryError(f"b200_symm_alloc({padded}) failed")
            self.local_ptr = int(p)
        handle = None
        if self.local_ptr and self.world > 1:
            buf = ctypes.create_string_buffer(64)
            rc = lib.b200_ipc_get_handle(ctypes.c_void_p(self.local_ptr), buf)
            _lib.check(rc, "b200_ipc_get_handle")
            handle = bytes(buf.raw)
        if self.world > 1:
            handles: list = [None] * self.world
            dist.all_gather_object(handles, (handle, self.nbytes), group=self.group)
            self.peer_sizes = [h[1] for h in handles]
            for r, (h, _) in enumerate(handles):
                if r == self.rank:
                    self.peer_ptrs[r] = self.local_ptr
                elif h is not None:
                    p = lib.b200_ipc_open_handle(ctypes.c_char_p(h))
                    if not p:
                        raise RuntimeError(f"could not map the buffer of rank {r}")
                    self.peer_ptrs[r] = int(p)
                    self._opened.append(int(p))
        else:
            self.peer_ptrs[0] = self.local_ptr
            self.peer_sizes = [self.nbytes]
        self._local_bytes = tensor_from_ptr(self.local_ptr, self.nbytes, self.device) \
            if self.local_ptr else None

    def tensor(self, dtype: torch.dtype, numel: int | None = None, byte_offset: int = 0) -> torch.Tensor:
        """View of the local allocation."""
        itemsize = torch.empty((), dtype=dtype).element_size()
        n = (self.nbytes - byte_offset) // itemsize if numel is None else numel
        return self._local_bytes[byte_offset: byte_offset + n * itemsize].view(dtype)

    def ptr_table(self, ranks: Sequence[int] | None = None, byte_offset: int = 0):
        """ctypes array of peer pointers (optionally offset) for the C launchers."""
        ranks = list(range(self.world)) if ranks is None else list(ranks)
        arr = (ctypes.c_void_p * len(ranks))()
        for i, r in enumerate(ranks):
            if not self.peer_ptrs[r]:
                raise RuntimeError(f"rank {r} exported no buffer")
            arr[i] = self.peer_ptrs[r] + byte_offset
        return arr

    def ipc_handle(self) -> bytes:
        """CUDA IPC handle of the local allocation (for processes outside ``group``)."""
        lib = _lib.kernels()
        buf = ctypes.create_string_buffer(64)
        _lib.check(lib.b200_ipc_get_handle(ctypes.c_void_p(self.local_ptr), buf), "b200_ipc_get_handle")
        return bytes(buf.raw)

    def close(self):
        lib = _lib.kernels()
        for p in self._opened:
            lib.b200_ipc_close_handle(ctypes.c_void_p(p))
        self._opened.clear()
        if self.local_ptr:
            self._local_bytes = None
            lib.b200_symm_free(ctypes.c_void_p(self.local_ptr))
            self.local_ptr = 0


def open_ipc_handle(handle: bytes, device_index: int = 0) -> int:
    """Maps another process's allocation; returns the device pointer in this process."""
    lib = _lib.kernels()
    lib.b200_ensure_device(ctypes.c_int(device_index))
    lib.b200_ipc_open_handle.restype = ctypes.c_void_p
    p = lib.b200_ipc_open_handle(ctypes.c_char_p(handle))
    if not p:
        raise RuntimeError("cudaIpcOpenMemHandle failed")
    return int(p)


class SymmBarrier:
    """Device-side barrier among the ranks of ``group`` on the current stream."""

    def __init__(self, group: dist.ProcessGroup | None = None, device=None):
        self.buf = SymmBuffer(256, group, device)
        self.epoch = 0
        self.world, self.rank = self.buf.world, self.buf.rank
        self._table = self.buf.ptr_table()

    def sync(self):
        self.epoch += 1
        lib = _lib.kernels()
        rc = lib.b200_symm_barrier(self._table, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                   ctypes.c_uint(self.epoch), _lib.stream_ptr())
        _lib.check(rc, "b200_symm_barrier")
        _lib.count_launch()

    def next_epochs(self, n: int) -> int:
        """Reserves ``n`` consecutive epochs for a kernel with built-in barriers."""
        first = self.epoch + 1
        self.epoch += n
        return first


class SymmComm:
    """Collectives over peer memory with a staging buffer of ``max_bytes`` per rank."""

    def __init__(self, max_bytes: int, group: dist.ProcessGroup | None = None, device=None):
        self.group = group
        self.stage = SymmBuffer(max_bytes, group, device)
        self.barrier = SymmBarrier(group, device)
        self.world, self.rank = self.stage.world, self.stage.rank
        self.device = self.stage.device
        self._table = self.stage.ptr_table()

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """Returns ``[world * n]``: every rank pushes its shard into all peers' staging buffers."""
        x = x.contiguous()
        nbytes = x.numel() * x.element_size()
        assert nbytes % 16 == 0 and nbytes * self.world <= self.stage.nbytes
        lib = _lib.kernels()
        self.barrier.sync()  # previous readers are done with the staging buffer
        rc = lib.b200_push_all(self._table, ctypes.c_int(self.world), _lib.ptr(x),
                               ctypes.c_longlong(nbytes), ctypes.c_longlong(self.rank * nbytes),
                               _lib.stream_ptr())
        _lib.check(rc, "b200_push_all")
        _lib.count_launch()
        self.barrier.sync()
        return self.stage.tensor(x.dtype, x.numel() * self.world).clone()

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        """``x [world * n]`` on every rank → this rank's summed slice ``[n]`` (pull)."""
        x = x.contiguous()
        nbytes = x.numel() * x.element_size()
        assert nbytes <= self.stage.nbytes and x.numel() % self.world == 0
        n = x.numel() // self.world
        self.barrier.sync()
        self.stage.tensor(x.dtype, x.numel()).copy_(x)
        self.barrier.sync()
        out = torch.empty(n, dtype=x.dtype, device=x.device)
        lib = _lib.kernels()
        rc = lib.b200_pull_reduce(self._table, ctypes.c_int(self.world), ctypes.c_longlong(self.rank * n),
                                  ctypes.c_longlong(n), _lib.ptr(out),
                                  ctypes.c_int(0 if x.dtype == torch.float32 else 1), _lib.stream_ptr())
        _lib.check(rc, "b200_pull_reduce")
        _lib.count_launch()
        return out

    def all_reduce_small(self, x: torch.Tensor) -> torch.Tensor:
        """One-shot all-reduce (sum) of a small fp32 tensor: one kernel, barriers inside."""
        x = x.float().contiguous()
        assert x.numel() * 4 <= self.stage.nbytes
        self.stage.tensor(torch.float32, x.numel()).copy_(x)
        out = torch.empty_like(x)
        lib = _lib.kernels()
        epoch = self.barrier.next_epochs(2)
        rc = lib.b200_allreduce_oneshot_f32(self._table, self.barrier._table, ctypes.c_int(self.rank),
                                            ctypes.c_int(self.world), ctypes.c_uint(epoch),
                                            ctypes.c_longlong(x.numel()), _lib.ptr(out), _lib.stream_ptr())
        _lib.check(rc, "b200_allreduce_oneshot_f32")
        _lib.count_launch()
        return out

    def all_to_all(self, x: torch.Tensor) -> torch.Tensor:
        """Equal-split all-to-all: chunk ``p`` of ``x`` goes to rank ``p``; returns the
        received chunks ordered by source rank."""
        x = x.contiguous()
        nbytes = x.numel() * x.element_size()
        assert x.numel() % self.world == 0 and nbytes <= self.stage.nbytes
        chunk = nbytes // self.world
        assert chunk % 16 == 0
        lib = _lib.kernels()
        self.barrier.sync()
        rc = lib.b200_a2a_push(self._table, ctypes.c_int(self.world), ctypes.c_int(self.rank),
                               _lib.ptr(x), ctypes.c_longlong(chunk), _lib.stream_ptr())
        _lib.check(rc, "b200_a2a_push")
        _lib.count_launch()
        self.barrier.sync()
        return self.stage.tensor(x.dtype, x.numel()).clone().view(x.shape)
