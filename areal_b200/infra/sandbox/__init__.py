"""Code-execution sandbox for tool-use rewards.

The reference talks to a remote Daytona sandbox service (areal/infra/sandbox/{_client,runner}.py).
This package has no network dependency: :class:`LocalSandbox` runs the snippet in a fresh
interpreter process with CPU-time / memory / file-size limits, an empty environment, a private
working directory and a wall-clock time-out, and returns stdout / stderr / exit code. It is a
resource fence, not a security boundary against hostile code; deployments that need one put the
same interface in front of a container or remote service (``SandboxClient`` protocol)."""

from __future__ import annotations

import asyncio
import os
import resource
import shutil
import subprocess
import sys
import tempfile
from dataclasses import dataclass
from typing import Protocol


@dataclass
class ExecResult:
    stdout: str
    stderr: str
    exit_code: int
    timed_out: bool = False

    @property
    def ok(self) -> bool:
        return self.exit_code == 0 and not self.timed_out


class SandboxClient(Protocol):
    def run(self, code: str, stdin: str = "", timeout: float = 10.0) -> ExecResult: ...


class LocalSandbox:
    def __init__(self, cpu_seconds: int = 10, memory_mb: int = 1024, max_output: int = 1 << 16, python: str | None = None):
        self.cpu_seconds, self.memory_mb, self.max_output = cpu_seconds, memory_mb, max_output
        self.python = python or sys.executable

    def _limits(self):
        resource.setrlimit(resource.RLIMIT_CPU, (self.cpu_seconds, self.cpu_seconds + 1))
        mem = self.memory_mb << 20
        resource.setrlimit(resource.RLIMIT_AS, (mem, mem))
        resource.setrlimit(resource.RLIMIT_FSIZE, (16 << 20, 16 << 20))
        resource.setrlimit(resource.RLIMIT_NPROC, (64, 64))
        os.setsid()

    def run(self, code: str, stdin: str = "", timeout: float = 10.0) -> ExecResult:
        work = tempfile.mkdtemp(prefix="sandbox_")
        try:
            path = os.path.join(work, "main.py")
            with open(path, "w") as f:
                f.write(code)
            try:
                p = subprocess.run([self.python, "-I", "-S", path], input=stdin, capture_output=True, text=True,
                                   timeout=timeout, cwd=work, env={"PATH": "/usr/bin:/bin", "HOME": work},
                                   preexec_fn=self._limits)
                return ExecResult(p.stdout[:self.max_output], p.stderr[:self.max_output], p.returncode)
            except subprocess.TimeoutExpired as e:
                out = (e.stdout or b"").decode(errors="replace") if isinstance(e.stdout, bytes) else (e.stdout or "")
                return ExecResult(out[:self.max_output], "timed out", -9, timed_out=True)
        finally:
            shutil.rmtree(work, ignore_errors=True)

    async def arun(self, code: str, stdin: str = "", timeout: float = 10.0) -> ExecResult:
        return await asyncio.get_running_loop().run_in_executor(None, self.run, code, stdin, timeout)


def code_reward(sandbox: SandboxClient, code: str, tests: list[tuple[str, str]], timeout: float = 10.0) -> float:
    """Fraction of ``(stdin, expected stdout)`` cases the program passes."""
    if not tests:
        return 0.0
    passed = 0
    for stdin, expected in tests:
        r = sandbox.run(code, stdin, timeout)
        passed += int(r.ok and r.stdout.strip() == expected.strip())
    return passed / len(tests)
