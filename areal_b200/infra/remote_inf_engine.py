"""Inference engine that talks HTTP to one or more rollout servers.

Use it when the rollout GPUs are separate processes or nodes reached over the network (the
single-node layouts of ``PPOTrainer`` use :class:`~areal_b200.infra.dist_rollout.RemoteRolloutClient`,
which pushes weights over NVLink instead). It implements the whole ``InferenceEngine`` contract:

* **server discovery**: explicit addresses, ``AREAL_LLM_SERVER_ADDRS``, or the name-resolve subtree
  that the servers register under (``names.gen_servers``), waited for up to ``setup_timeout``;
* **routing**: round-robin with request-id affinity, so the turns of one conversation hit the same
  server (and its warm cache);
* **interruptible generation**: one HTTP call is one scheduler request; a reply with finish reason
  ``abort`` (the server was paused for a weight update) carries the tokens produced so far, and the
  loop re-issues prompt + partial output until a stop or the token budget is reached. Every token is
  tagged with the weight version that produced it;
* **control fan-out**: pause / continue / version / memory release to every server, weight updates
  from a checkpoint directory;
* the workflow API (``submit`` / ``wait`` / ``prepare_batch`` ...) through the same
  ``WorkflowExecutor`` as the in-process engine, and ``launch_server`` for a local subprocess.

The wire format is a pluggable backend: :class:`NativeBackend` (this repo's server,
``engine/native_server.py``), :class:`SGLangBackend`, :class:`VLLMBackend`. Counterpart of
areal/infra/remote_inf_engine.py:393-1264, areal/engine/sglang_remote.py:43-298 and
areal/engine/vllm_remote.py:44-253.
"""

from __future__ import annotations

import asyncio
import os
import subprocess
import sys
import time
from collections import OrderedDict
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Any

from ..api.cli_args import InferenceEngineConfig
from ..api.engine_api import InferenceEngine
from ..api.io_struct import (HttpGenerationResult, HttpRequest, LocalInfServerInfo, ModelRequest, ModelResponse,
                             ParamSpec, WeightUpdateMeta)
from ..utils import logging, name_resolve, names
from .utils.http import HTTPRequestError, arequest_with_retry, request_with_retry
from .workflow_context import get_aiohttp_session

logger = logging.getLogger("RemoteInfEngine")

RID_CACHE_SIZE = 16384


# ------------------------------------------------------------------------------ backends


class SGLangBackend:
    """Request builders / reply parser for SGLang-style servers."""

    name = "sglang"

    def build_generation_request(self, req: ModelRequest, input_ids: list[int], max_new_tokens: int) -> HttpRequest:
        g = req.gconfig
        sp = {"top_p": g.top_p, "top_k": g.top_k if g.top_k and g.top_k > 0 else -1, "max_new_tokens": max_new_tokens,
              "temperature": 0.0 if g.greedy else g.temperature, "stop_token_ids": list(g.stop_token_ids or []),
              "ignore_eos": bool(g.ignore_eos), "skip_special_tokens": True,
              "frequency_penalty": getattr(g, "frequency_penalty", 0.0)}
        if g.min_new_tokens:
            sp["min_new_tokens"] = g.min_new_tokens
        if getattr(g, "stop", None):
            sp["stop"] = list(g.stop)
        payload: dict[str, Any] = {"input_ids": input_ids, "sampling_params": sp, "return_logprob": True,
                                   "stream": False, "rid": req.rid}
        if req.image_data:
            payload["image_data"] = req.image_data
        return HttpRequest("/generate", payload)

    def parse_generation_response(self, body: dict[str, Any]) -> tuple[HttpGenerationResult, int | None]:
        meta = body.get("meta_info", {})
        reason = meta.get("finish_reason") or {}
        reason = reason.get("type", "stop") if isinstance(reason, dict) else str(reason)
        pairs = meta.get("output_token_logprobs") or []
        tokens = [int(p[1]) for p in pairs]
        logprobs = [float(p[0]) for p in pairs]
        return HttpGenerationResult(tokens, logprobs, reason), meta.get("version")

    def health(self) -> HttpRequest:
        return HttpRequest("/health", {}, "GET")

    def pause(self) -> HttpRequest:
        return HttpRequest("/pause_generation", {})

    def resume(self) -> HttpRequest:
        return HttpRequest("/continue_generation", {})

    def update_from_disk(self, meta: WeightUpdateMeta) -> HttpRequest:
        return HttpRequest("/update_weights_from_disk", {"model_path": str(meta.path), "allow_interrupt": True})

    def release_memory(self) -> HttpRequest:
        return HttpRequest("/release_memory_occupation", {})

    def resume_memory(self, tags: list[str] | None = None) -> HttpRequest:
        return HttpRequest("/resume_memory_occupation", {"tags": tags} if tags else {})

    def set_version(self, version: int) -> HttpRequest | None:
        return None  # the stock server has no version store; the client tags tokens itself


class NativeBackend(SGLangBackend):
    """This repo's ``engine/native_server.py``: the same generation format, plus a version store."""

    name = "native"

    def update_from_disk(self, meta: WeightUpdateMeta) -> HttpRequest:
        return HttpRequest("/update_weights_from_disk", {"model_path": str(meta.path), "version": meta.version})

    def set_version(self, version: int) -> HttpRequest | None:
        return HttpRequest("/set_version", {"version": int(version)})


class VLLMBackend(SGLangBackend):
    """vLLM's OpenAI-style completions endpoint with token ids in and out."""

    name = "vllm"

    def build_generation_request(self, req: ModelRequest, input_ids: list[int], max_new_tokens: int) -> HttpRequest:
        g = req.gconfig
        payload = {"prompt": input_ids, "top_p": g.top_p, "top_k": g.top_k if g.top_k and g.top_k > 0 else -1,
                   "max_tokens": max_new_tokens, "temperature": 0.0 if g.greedy else g.temperature,
                   "stop_token_ids": list(g.stop_token_ids or []), "ignore_eos": bool(g.ignore_eos),
                   "return_tokens_as_token_ids": True, "logprobs": 0, "stream": False, "request_id": req.rid}
        if g.min_new_tokens:
            payload["min_tokens"] = g.min_new_tokens
        return HttpRequest("/v1/completions", payload)

    def parse_generation_response(self, body: dict[str, Any]) -> tuple[HttpGenerationResult, int | None]:
        choice = body["choices"][0]
        lp = choice.get("logprobs") or {}
        tokens = [int(str(t).split(":")[-1]) for t in lp.get("tokens", [])]  # "token_id:123"
        logprobs = [float(x) for x in lp.get("token_logprobs", [])]
        reason = choice.get("finish_reason") or "stop"
        if reason not in ("stop", "length", "abort"):
            reason = "stop"
        return HttpGenerationResult(tokens, logprobs, reason), None

    def pause(self) -> HttpRequest:
        return HttpRequest("/areal_pause_generation", {})

    def resume(self) -> HttpRequest:
        return HttpRequest("/areal_continue_generation", {})

    def update_from_disk(self, meta: WeightUpdateMeta) -> HttpRequest:
        return HttpRequest("/areal_update_weights", {"model_path": str(meta.path)})

    def release_memory(self) -> HttpRequest:
        return HttpRequest("/sleep", {})

    def resume_memory(self, tags: list[str] | None = None) -> HttpRequest:
        return HttpRequest("/wake_up", {"tags": tags} if tags else {})


BACKENDS = {"native": NativeBackend, "sglang": SGLangBackend, "vllm": VLLMBackend}


# -------------------------------------------------------------------------------- engine


class RemoteInfEngine(InferenceEngine):
    # encoded images travel in the request body; whether the served model takes them is the server's answer
    supports_images = True

    def __init__(self, config: InferenceEngineConfig, backend: Any = None):
        self.config = config
        kind = (config.backend or "native").split(":")[0] if isinstance(config.backend, str) else "native"
        self.backend = backend or BACKENDS.get(kind, NativeBackend)()
        self.addresses: list[str] = []
        self._rr = 0
        self._rid_to_addr: "OrderedDict[str, str]" = OrderedDict()
        self._version = 0
        self._paused = False
        self._executor = None
        self._pool = ThreadPoolExecutor(max_workers=8, thread_name_prefix="remote-inf")
        self._servers: list[LocalInfServerInfo] = []

    # ------------------------------------------------------------ lifecycle
    def initialize(self, addr: str | list[str] | None = None, train_data_parallel_size: int | None = None, **_):
        self.addresses = self._discover(addr)
        self._wait_healthy()
        from .workflow_executor import WorkflowExecutor

        self._executor = WorkflowExecutor(self.config, self).initialize(train_data_parallel_size)
        logger.info(f"connected to {len(self.addresses)} rollout server(s): {self.addresses}")
        return self

    def _discover(self, addr) -> list[str]:
        if addr:
            return [addr] if isinstance(addr, str) else list(addr)
        env = os.environ.get("AREAL_LLM_SERVER_ADDRS")
        if env:
            return [a for a in env.split(",") if a]
        cfg = self.config
        if not (cfg.experiment_name and cfg.trial_name):
            raise ValueError("no server address given: pass addr=, set AREAL_LLM_SERVER_ADDRS, or set "
                             "experiment_name / trial_name so that servers are found through name_resolve")
        root = names.gen_servers(cfg.experiment_name, cfg.trial_name)
        deadline = time.time() + cfg.setup_timeout
        while True:
            found = sorted(set(name_resolve.get_subtree(root)))
            if found:
                return found
            if time.time() > deadline:
                raise TimeoutError(f"no rollout server registered under {root} within {cfg.setup_timeout}s")
            time.sleep(0.5)

    def _wait_healthy(self):
        deadline = time.time() + self.config.setup_timeout
        h = self.backend.health()
        for a in self.addresses:
            while True:
                try:
                    request_with_retry(h.method, f"http://{a}{h.endpoint}", timeout=5.0, max_retries=0)
                    break
                except Exception:  # noqa: BLE001 - keep polling until the deadline
                    if time.time() > deadline:
                        raise TimeoutError(f"rollout server {a} did not become healthy")
                    time.sleep(0.5)

    def destroy(self):
        if self._executor is not None:
            self._executor.destroy()
            self._executor = None
        self.teardown_server()
        self._pool.shutdown(wait=False)

    # -------------------------------------------------------------- routing
    def choose_server(self, rid: str | None = None) -> str:
        if rid is not None and rid in self._rid_to_addr:
            self._rid_to_addr.move_to_end(rid)
            return self._rid_to_addr[rid]
        a = self.addresses[self._rr % len(self.addresses)]
        self._rr += 1
        if rid is not None:
            self._rid_to_addr[rid] = a
            if len(self._rid_to_addr) > RID_CACHE_SIZE:
                self._rid_to_addr.popitem(last=False)
        return a

    # ----------------------------------------------------------- generation
    async def agenerate(self, req: ModelRequest) -> ModelResponse:
        g = req.gconfig
        if g.n_samples != 1:
            raise ValueError("agenerate produces one sample; use n_samples=1 and group at the workflow level")
        max_new = min(g.max_new_tokens, max(g.max_tokens - len(req.input_ids), 0))
        addr = self.choose_server(req.rid)
        session = await get_aiohttp_session()
        t0 = time.perf_counter()
        out_tokens: list[int] = []
        out_logprobs: list[float] = []
        out_versions: list[int] = []
        stop_reason = "length"
        ttft = float("inf")
        while len(out_tokens) < max_new:
            while self._paused:
                await asyncio.sleep(0.01)
            http = self.backend.build_generation_request(req, list(req.input_ids) + out_tokens, max_new - len(out_tokens))
            body = await arequest_with_retry(session, http.method, f"http://{addr}{http.endpoint}", json=http.payload,
                                             timeout=self.config.request_timeout, max_retries=self.config.request_retries)
            res, version = self.backend.parse_generation_response(body)
            if res.output_tokens and ttft == float("inf"):
                ttft = time.perf_counter() - t0
            out_tokens += res.output_tokens
            out_logprobs += res.output_logprobs
            out_versions += [self._version if version is None else int(version)] * len(res.output_tokens)
            stop_reason = res.stop_reason
            if stop_reason != "abort":
                break
            if not res.output_tokens:
                await asyncio.sleep(0.01)  # aborted before prefill: the server is between pause and resume
        if stop_reason == "abort":
            stop_reason = "length"
        return ModelResponse(input_tokens=list(req.input_ids), output_tokens=out_tokens, output_logprobs=out_logprobs,
                             output_versions=out_versions, stop_reason=stop_reason, tokenizer=req.tokenizer,
                             latency=time.perf_counter() - t0, ttft=ttft)

    def generate(self, req: ModelRequest) -> ModelResponse:
        """Blocking form for callers without an event loop: runs one private loop and closes the HTTP
        session that belongs to it (sessions are per loop)."""
        from .workflow_context import close_clients

        async def run():
            try:
                return await self.agenerate(req)
            finally:
                await close_clients()

        return asyncio.run(run())

    # -------------------------------------------------------------- control
    def _fanout(self, http: HttpRequest | None, timeout: float | None = None) -> list[Any]:
        if http is None:
            return []
        timeout = timeout or self.config.request_timeout

        def one(a):
            return request_with_retry(http.method, f"http://{a}{http.endpoint}",
                                      json=http.payload if http.method != "GET" else None, timeout=timeout,
                                      max_retries=self.config.request_retries)

        return list(self._pool.map(one, self.addresses))

    def pause_generation(self):
        self._paused = True
        self._fanout(self.backend.pause())
        if self.config.pause_grace_period > 0:
            time.sleep(self.config.pause_grace_period)

    def continue_generation(self):
        self._fanout(self.backend.resume())
        self._paused = False

    def update_weights_from_disk(self, meta: WeightUpdateMeta) -> Future:
        """Every server loads the checkpoint at ``meta.path``; resolves when all have."""
        def run():
            self._fanout(self.backend.update_from_disk(meta))
            if meta.version is not None:
                self.set_version(meta.version)

        return self._pool.submit(run)

    def update_weights_from_distributed(self, meta: WeightUpdateMeta, param_specs: list[ParamSpec]) -> Future:
        raise NotImplementedError("servers reached over HTTP take weights from disk; device-to-device weight pushes "
                                  "are the job of infra.dist_rollout.RemoteRolloutClient")

    def init_weights_update_group(self, meta: WeightUpdateMeta) -> Future:
        fut: Future = Future()
        fut.set_result(None)
        return fut

    def set_version(self, version: int):
        self._version = int(version)
        self._fanout(self.backend.set_version(version))
        if self._executor is not None:
            self._executor.on_version_changed(version)

    def get_version(self) -> int:
        return self._version

    def offload(self):
        self._fanout(self.backend.release_memory())

    def onload(self, tags: list[str] | None = None):
        self._fanout(self.backend.resume_memory(tags))

    # ---------------------------------------------------------- workflow API
    def submit(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None, group_size=1,
               task_id=None, callback_addr=None, is_eval=False, proxy_addr=None) -> int:
        return self._executor.submit(data, workflow, workflow_kwargs, should_accept_fn, group_size,
                                     task_id=task_id, is_eval=is_eval)

    def wait(self, count: int, timeout: float | None = None, raise_timeout: bool = True):
        return self._executor.wait(count, timeout, raise_timeout)

    def wait_for_task(self, task_id: int, timeout: float | None = None, raise_timeout: bool = True):
        return self._executor.wait_for_task(task_id, timeout, raise_timeout)

    def rollout_batch(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None, group_size=1,
                      is_eval=False):
        return self._executor.rollout_batch(data, workflow, workflow_kwargs, should_accept_fn, group_size,
                                            is_eval=is_eval)

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None,
                      group_size=1, dynamic_bs=False):
        return self._executor.prepare_batch(dataloader, workflow, workflow_kwargs, should_accept_fn,
                                            group_size, dynamic_bs)

    def pause(self):
        self._executor.pause()

    def resume(self):
        self._executor.resume()

    def export_stats(self) -> dict[str, float]:
        return self._executor.export_stats() if self._executor is not None else {}

    # --------------------------------------------------------- local servers
    def launch_server(self, server_args: dict[str, Any]) -> LocalInfServerInfo:
        """Starts ``engine/native_server.py`` as a subprocess with ``--key value`` arguments taken from
        ``server_args`` and waits until it answers ``/health``."""
        from ..utils.network import find_free_ports

        args = dict(server_args)
        host = args.setdefault("host", "127.0.0.1")
        port = int(args.get("port") or find_free_ports(1)[0])
        args["port"] = port
        cmd = [sys.executable, "-m", "areal_b200.engine.native_server"]
        for k, v in args.items():
            flag = "--" + k.replace("_", "-")
            if isinstance(v, bool):
                if v:
                    cmd.append(flag)
            elif v is not None:
                cmd += [flag, str(v)]
        proc = subprocess.Popen(cmd, start_new_session=True)
        info = LocalInfServerInfo(host=host, port=port, process=proc)
        self._servers.append(info)
        deadline = time.time() + self.config.setup_timeout
        while True:
            if proc.poll() is not None:
                raise RuntimeError(f"rollout server exited with code {proc.returncode} during start-up")
            try:
                request_with_retry("GET", f"http://{host}:{port}/health", timeout=2.0, max_retries=0)
                break
            except Exception:  # noqa: BLE001 - not up yet
                if time.time() > deadline:
                    self.teardown_server()
                    raise TimeoutError("rollout server did not start in time")
                time.sleep(0.5)
        self.addresses.append(f"{host}:{port}")
        return info

    def teardown_server(self):
        for info in self._servers:
            p = info.process
            if p is not None and p.poll() is None:
                p.terminate()
                try:
                    p.wait(timeout=10)
                except subprocess.TimeoutExpired:
                    p.kill()
        self._servers.clear()


__all__ = ["RemoteInfEngine", "NativeBackend", "SGLangBackend", "VLLMBackend", "HTTPRequestError"]
