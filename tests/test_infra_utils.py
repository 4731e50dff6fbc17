"""Small infrastructure helpers: distributed lock, async checkpointer, HTTP retry, process tree
termination, network helpers, experiment metadata, platform description."""
import asyncio
import os
import subprocess
import sys
import threading
import time

import pytest
import torch
from torch.distributed import HashStore

from areal_b200.infra.platforms import current_platform
from areal_b200.infra.utils import concurrent, exp_metadata, proc
from areal_b200.infra.utils.http import HTTPRequestError, request_with_retry
from areal_b200.utils import network
from areal_b200.utils.async_checkpoint import AsyncCheckpointer
from areal_b200.utils.lock import DistributedLock


def test_distributed_lock_is_exclusive_and_expires():
    store = HashStore()
    counter = {"v": 0, "max_inside": 0, "inside": 0}

    def worker():
        for _ in range(20):
            with DistributedLock(store, "l"):
                counter["inside"] += 1
                counter["max_inside"] = max(counter["max_inside"], counter["inside"])
                v = counter["v"]
                time.sleep(0.0005)
                counter["v"] = v + 1
                counter["inside"] -= 1

    ts = [threading.Thread(target=worker) for _ in range(4)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert counter["v"] == 80 and counter["max_inside"] == 1
    a = DistributedLock(store, "m", lease_seconds=0.05)
    assert a.acquire(timeout=1)
    b = DistributedLock(store, "m", lease_seconds=5)
    assert not b.acquire(timeout=0.01)
    time.sleep(0.1)  # a's lease ran out without a release (a crashed owner)
    assert b.acquire(timeout=1)


def test_async_checkpointer_writes_atomically(tmp_path):
    ck = AsyncCheckpointer()
    state = {"w": torch.arange(10.0), "step": 3}
    p = str(tmp_path / "c" / "ckpt.pt")
    fut = ck.save(state, p)
    state["w"].zero_()  # the staged copy is what gets written
    fut.result()
    got = torch.load(p)
    assert torch.equal(got["w"], torch.arange(10.0)) and got["step"] == 3
    ck.close()


def test_http_retry_gives_up_with_a_typed_error():
    port = network.find_free_ports(1)[0]
    t0 = time.monotonic()
    with pytest.raises(HTTPRequestError):
        request_with_retry("GET", f"http://127.0.0.1:{port}/x", max_retries=2, backoff=0.01, timeout=0.5)
    assert time.monotonic() - t0 < 5


def test_kill_process_tree_and_wait_for():
    p = subprocess.Popen([sys.executable, "-c", "import subprocess,sys,time; subprocess.Popen([sys.executable,'-c','import time; time.sleep(60)']); time.sleep(60)"])
    time.sleep(0.5)
    n = proc.kill_process_tree(p.pid, timeout=5)
    assert n >= 2
    proc.wait_for(lambda: p.poll() is not None, timeout=5)
    with pytest.raises(TimeoutError):
        proc.wait_for(lambda: False, timeout=0.05, interval=0.01)


def test_network_metadata_platform_and_concurrency(tmp_path):
    ports = network.find_free_ports(3)
    assert len(set(ports)) == 3
    assert network.format_addr("::1", 80) == "[::1]:80" and network.gethostip()
    assert not network.wait_for_port("127.0.0.1", ports[0], timeout=0.2)
    path = exp_metadata.save_metadata(str(tmp_path / "meta.json"), {"a": 1})
    assert os.path.exists(path)
    assert current_platform.device_type in ("cpu", "cuda") and current_platform.memory_info()[1] > 0

    async def f(x):
        await asyncio.sleep(0.001)
        return x * 2

    assert concurrent.run_async_task(f, 4) == 8
    assert asyncio.run(concurrent.gather_with_limit([f(i) for i in range(5)], 2)) == [0, 2, 4, 6, 8]


def test_local_sandbox_runs_limits_and_scores():
    from areal_b200.infra.sandbox import LocalSandbox, code_reward

    sb = LocalSandbox(cpu_seconds=2, memory_mb=512)
    r = sb.run("print(int(input()) * 2)", stdin="21\n")
    assert r.ok and r.stdout.strip() == "42"
    assert not sb.run("raise SystemExit(3)").ok
    r = sb.run("while True: pass", timeout=1.0)
    assert not r.ok
    assert code_reward(sb, "print(int(input()) + 1)", [("1", "2"), ("5", "6"), ("7", "9")]) == pytest.approx(2 / 3)
