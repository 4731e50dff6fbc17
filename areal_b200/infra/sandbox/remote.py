"""Code execution on another machine: a small HTTP service around a sandbox and its client.

``create_runner_app(sandbox, token)`` serves ``POST /run {"code", "stdin", "timeout"}`` →
``{"stdout", "stderr", "exit_code", "timed_out"}`` and ``POST /run_batch {"jobs": [...]}`` for several programs
at once (run concurrently up to ``max_parallel``); ``RemoteSandbox(url, token)`` is the matching
:class:`~areal_b200.infra.sandbox.SandboxClient`, so ``code_reward`` and the code-reward function work against a
pool of execution hosts instead of the trainer's own CPUs. The service executes untrusted model output: run it
in a container or VM of its own and give it a token.

Role in the reference: the remote sandbox client and runner of areal/infra/sandbox/{_client,runner}.py (there
against the Daytona service).
"""

from __future__ import annotations

import asyncio
import hmac
from typing import Callable

from fastapi import FastAPI, HTTPException, Request

from . import ExecResult, LocalSandbox, SandboxClient


def create_runner_app(sandbox: SandboxClient | None = None, token: str | None = None, max_parallel: int = 8,
                      max_timeout: float = 60.0):
    app = FastAPI()
    sb = sandbox or LocalSandbox()
    gate = asyncio.Semaphore(max_parallel)
    stats = {"runs": 0, "timeouts": 0, "failures": 0}

    def auth(req: Request):
        if token is None:
            return
        got = req.headers.get("authorization", "")
        if not got.lower().startswith("bearer ") or not hmac.compare_digest(got[7:].strip(), token):
            raise HTTPException(status_code=401, detail="invalid or missing bearer token")

    async def run_one(job: dict) -> dict:
        code = job.get("code")
        if not isinstance(code, str):
            raise HTTPException(status_code=400, detail="`code` must be a string")
        timeout = min(float(job.get("timeout", 10.0)), max_timeout)
        async with gate:
            r: ExecResult = await asyncio.get_running_loop().run_in_executor(
                None, sb.run, code, str(job.get("stdin", "")), timeout)
        stats["runs"] += 1
        stats["timeouts"] += int(r.timed_out)
        stats["failures"] += int(not r.ok)
        return {"stdout": r.stdout, "stderr": r.stderr, "exit_code": r.exit_code, "timed_out": r.timed_out}

    @app.get("/health")
    def health():
        return dict(stats, status="ok")

    @app.post("/run")
    async def run(req: Request):
        auth(req)
        return await run_one(await req.json())

    @app.post("/run_batch")
    async def run_batch(req: Request):
        auth(req)
        jobs = (await req.json()).get("jobs") or []
        return {"results": await asyncio.gather(*[run_one(j) for j in jobs])}

    return app


class RemoteSandbox:
    """Client of :func:`create_runner_app`. ``post(url, body, headers) -> dict`` is the transport (default:
    ``requests`` with the request's own time-out plus a margin). Transport failures come back as a failed
    ``ExecResult`` (exit code -1) rather than an exception: a reward function must not take the rollout down."""

    def __init__(self, url: str, token: str | None = None, post: Callable[[str, dict, dict], dict] | None = None):
        self.url, self.token = url.rstrip("/"), token
        self._post = post or self._requests_post

    @staticmethod
    def _requests_post(url: str, body: dict, headers: dict) -> dict:
        import requests

        r = requests.post(url, json=body, headers=headers, timeout=float(body.get("timeout", 10.0)) + 30.0)
        r.raise_for_status()
        return r.json()

    def _headers(self) -> dict[str, str]:
        return {"Authorization": f"Bearer {self.token}"} if self.token else {}

    @staticmethod
    def _result(d: dict) -> ExecResult:
        return ExecResult(d.get("stdout", ""), d.get("stderr", ""), int(d.get("exit_code", -1)), bool(d.get("timed_out", False)))

    def run(self, code: str, stdin: str = "", timeout: float = 10.0) -> ExecResult:
        try:
            return self._result(self._post(self.url + "/run", {"code": code, "stdin": stdin, "timeout": timeout},
                                           self._headers()))
        except Exception as e:  # noqa: BLE001 - reported as a failed execution
            return ExecResult("", f"sandbox service error: {type(e).__name__}: {e}", -1)

    def run_batch(self, jobs: list[dict]) -> list[ExecResult]:
        try:
            out = self._post(self.url + "/run_batch", {"jobs": jobs, "timeout": max((j.get("timeout", 10.0) for j in jobs),
                                                                                   default=10.0)}, self._headers())
            return [self._result(d) for d in out["results"]]
        except Exception as e:  # noqa: BLE001
            return [ExecResult("", f"sandbox service error: {type(e).__name__}: {e}", -1) for _ in jobs]

    async def arun(self, code: str, stdin: str = "", timeout: float = 10.0) -> ExecResult:
        return await asyncio.get_running_loop().run_in_executor(None, self.run, code, stdin, timeout)
