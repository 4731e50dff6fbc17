import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "multi_gpu: needs more than one CUDA device")
    config.addinivalue_line("markers", "slow: takes more than a few seconds")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        ngpu = torch.cuda.device_count()
        skip_multi = pytest.mark.skip(reason="needs >=2 GPUs")
        for item in items:
            if "multi_gpu" in item.keywords and ngpu < 2:
                item.add_marker(skip_multi)
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords or "multi_gpu" in item.keywords:
            item.add_marker(skip)


def pytest_sessionstart(session):
    # the native libraries are not tracked in git: build them once per session
    from areal_b200 import build as _build

    _build.build()


def free_port() -> int:
    """A TCP port that is free right now (for torchrun rendezvous of tests that may run side by side)."""
    import socket

    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]
