"""Device platform description. This package targets NVIDIA B200 (sm_100a) only: there is one
accelerator platform, plus a CPU platform for tests; no vendor dispatch. ``current_platform`` is
resolved lazily on first attribute access (areal/infra/platforms/__init__.py:48-95 in the
reference resolves among CUDA / NPU / CPU)."""

from __future__ import annotations

from .platform import CpuPlatform, CudaPlatform, Platform


class _Lazy:
    _inst: Platform | None = None

    def _get(self) -> Platform:
        if self._inst is None:
            import torch

            type(self)._inst = CudaPlatform() if torch.cuda.is_available() else CpuPlatform()
        return self._inst

    def __getattr__(self, name):
        return getattr(self._get(), name)


current_platform = _Lazy()

__all__ = ["Platform", "CudaPlatform", "CpuPlatform", "current_platform"]
