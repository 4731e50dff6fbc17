"""Platform classes: device type, communication backend, visibility env var, memory queries,
NUMA affinity of the current GPU (read through NVML; nothing is ever set on the GPU itself).
Reference: areal/infra/platforms/{platform,cuda,cpu}.py."""

from __future__ import annotations

import os


class Platform:
    device_type = "cpu"
    device_name = "cpu"
    communication_backend = "gloo"
    device_control_env_var = ""
    dispatch_key = "CPU"

    def is_available(self) -> bool:
        return True

    def device_count(self) -> int:
        return 0

    def current_device(self) -> int:
        return 0

    def set_device(self, index: int):
        pass

    def synchronize(self):
        pass

    def memory_info(self) -> tuple[int, int]:
        """(free, total) bytes of the current device."""
        import psutil

        vm = psutil.virtual_memory()
        return vm.available, vm.total

    def clear_memory(self):
        import gc

        gc.collect()

    def set_numa_affinity(self, index: int | None = None) -> list[int]:
        return []


class CpuPlatform(Platform):
    pass


class CudaPlatform(Platform):
    device_type = "cuda"
    device_name = "NVIDIA"
    communication_backend = "nccl"
    device_control_env_var = "CUDA_VISIBLE_DEVICES"
    dispatch_key = "CUDA"

    def is_available(self) -> bool:
        import torch

        return torch.cuda.is_available()

    def device_count(self) -> int:
        import torch

        return torch.cuda.device_count()

    def current_device(self) -> int:
        import torch

        return torch.cuda.current_device()

    def set_device(self, index: int):
        import torch

        torch.cuda.set_device(index)

    def synchronize(self):
        import torch

        torch.cuda.synchronize()

    def memory_info(self) -> tuple[int, int]:
        import torch

        return torch.cuda.mem_get_info()

    def clear_memory(self):
        import gc

        import torch

        gc.collect()
        torch.cuda.empty_cache()

    def set_numa_affinity(self, index: int | None = None) -> list[int]:
        """Pins this process to the CPUs NVML reports as local to the GPU (a host-side scheduling
        hint; the GPU's own settings are only read). Returns the CPU list (empty when unknown)."""
        try:
            import pynvml

            pynvml.nvmlInit()
            idx = self.current_device() if index is None else index
            vis = os.environ.get(self.device_control_env_var)
            phys = int(vis.split(",")[idx]) if vis else idx
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            n_words = (os.cpu_count() + 63) // 64
            mask = pynvml.nvmlDeviceGetCpuAffinity(h, n_words)
            cpus = [w * 64 + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1]
            if cpus:
                os.sched_setaffinity(0, cpus)
            return cpus
        except Exception:
            return []
