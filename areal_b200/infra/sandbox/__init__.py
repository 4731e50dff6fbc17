"""Code-execution sandbox for tool-use rewards.

The reference talks to a remote Daytona sandbox service (areal/infra/sandbox/{_client,runner}.py).
This package has no network dependency: :class:`LocalSandbox` runs the snippet in a fresh
interpreter process with CPU-time / memory / file-size limits, an empty environment, a private
working directory and a wall-clock time-out, and returns stdout / stderr / exit code. It is a
resource fence, not a security boundary against hostile code; deployments that need one put the
same interface in front of a container or remote service (``SandboxClient`` protocol): ``sandbox/remote.py`` has
an HTTP runner service around any sandbox and the matching client."""

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


class ShellWorkspace:
    """A private working directory that shell commands run in, one after another, with the same resource
    fence as :class:`LocalSandbox` (CPU time, address space, file size, process count, wall clock; each
    command in its own session so a time-out ends the whole process group). State lives in the directory:
    files written by one command are there for the next. ``close()`` (or leaving the ``with`` block)
    removes it. Terminal-style agent tasks use one workspace per episode."""

    def __init__(self, files: dict[str, str] | None = None, cpu_seconds: int = 10, memory_mb: int = 2048,
                 max_output: int = 1 << 14, shell: str = "/bin/bash"):
        self.cpu_seconds, self.memory_mb, self.max_output, self.shell = cpu_seconds, memory_mb, max_output, shell
        self.root = tempfile.mkdtemp(prefix="workspace_")
        for rel, content in (files or {}).items():
            self.write_file(rel, content)

    def _resolve(self, rel: str) -> str:
        path = os.path.realpath(os.path.join(self.root, rel))
        if path != self.root and not path.startswith(self.root + os.sep):
            raise ValueError(f"path {rel!r} leaves the workspace")
        return path

    def write_file(self, rel: str, content: str) -> None:
        path = self._resolve(rel)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, "w") as f:
            f.write(content)

    def read_file(self, rel: str, max_chars: int | None = None) -> str:
        with open(self._resolve(rel)) as f:
            return f.read(max_chars if max_chars is not None else self.max_output)

    def _limits(self):
        resource.setrlimit(resource.RLIMIT_CPU, (self.cpu_seconds, self.cpu_seconds + 1))
        mem = self.memory_mb << 20
        resource.setrlimit(resource.RLIMIT_AS, (mem, mem))
        resource.setrlimit(resource.RLIMIT_FSIZE, (16 << 20, 16 << 20))

    def run(self, command: str, timeout: float = 10.0) -> ExecResult:
        env = {"PATH": "/usr/local/bin:/usr/bin:/bin", "HOME": self.root, "LANG": "C.UTF-8"}
        proc = subprocess.Popen([self.shell, "-c", command], cwd=self.root, env=env, stdin=subprocess.DEVNULL,
                                stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, start_new_session=True,
                                preexec_fn=self._limits)
        try:
            out, err = proc.communicate(timeout=timeout)
            return ExecResult(out[: self.max_output], err[: self.max_output], proc.returncode)
        except subprocess.TimeoutExpired:
            try:
                os.killpg(proc.pid, 9)   # the command's own session: nothing else is in that group
            except ProcessLookupError:
                pass
            out, err = proc.communicate()
            return ExecResult((out or "")[: self.max_output], "timed out", -9, timed_out=True)

    async def arun(self, command: str, timeout: float = 10.0) -> ExecResult:
        return await asyncio.get_running_loop().run_in_executor(None, self.run, command, timeout)

    def close(self) -> None:
        shutil.rmtree(self.root, ignore_errors=True)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
