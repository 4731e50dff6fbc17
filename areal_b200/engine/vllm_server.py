"""vLLM as a rollout server for this framework: vLLM's OpenAI-compatible server plus the control routes that
``VLLMBackend`` (``infra/remote_inf_engine.py``) calls.

    python -m areal_b200.engine.vllm_server --model /models/Qwen3-1.7B --port 8100 [any `vllm serve` flag]

Added routes (all POST, JSON):

* ``/areal_pause_generation``     – stop taking new requests and abort the running ones; their clients get the
  tokens produced so far with ``finish_reason: "abort"`` and re-submit prompt + partial output after the update
  (the interruptible-generation loop of ``RemoteInfEngine.agenerate``).
* ``/areal_continue_generation``  – resume.
* ``/areal_update_weights``       – ``{"model_path"}``: every worker reloads the checkpoint under that path (the
  trainer's disk weight update writes one per version), then the prefix cache is dropped: its KV belongs to the
  old weights.
* ``/areal_update_weights_lora``  – ``{"lora_name", "lora_model_path", "lora_int_id"}``: (re)loads an adapter.
* ``/areal_set_version`` / ``/areal_get_version`` – the weight version the trainer last pushed.
* ``/areal_init_weights_update_group``, ``/areal_set_update_weight_meta``, ``/areal_update_weights_xccl`` – answer
  501: external servers take weights through a checkpoint directory here; the collective path is this
  framework's own rollout engine with peer-memory pushes.

The routes only use the engine client's public asynchronous interface (``pause_generation``,
``resume_generation``, ``collective_rpc``, ``reset_prefix_cache``, ``add_lora``), read from
``app.state.engine_client`` like vLLM's own routes, so they can be mounted on any app that provides one
(``attach_areal_routes``); the tests mount them on a stub.

Reference: the vLLM server extension with the same route names, areal/engine/vllm_ext/areal_vllm_server.py and
areal/engine/vllm_ext/vllm_worker_extension.py.
"""

from __future__ import annotations

import inspect
import time
from typing import Any

from fastapi import APIRouter, FastAPI, HTTPException, Request

router = APIRouter()


def _engine(req: Request):
    eng = getattr(req.app.state, "engine_client", None)
    if eng is None:
        raise HTTPException(status_code=503, detail="the engine is not ready")
    return eng


async def _json(req: Request) -> dict:
    return (await req.json()) if await req.body() else {}


@router.post("/areal_pause_generation")
async def pause_generation(req: Request):
    eng = _engine(req)
    t0 = time.perf_counter()
    params = inspect.signature(eng.pause_generation).parameters
    if "mode" in params:
        await eng.pause_generation(mode="abort")
    else:  # older interface: abort unless asked to wait
        await eng.pause_generation(wait_for_inflight_requests=False, clear_cache=False)
    req.app.state.areal_paused = True
    return {"paused": True, "seconds": time.perf_counter() - t0}


@router.post("/areal_continue_generation")
async def continue_generation(req: Request):
    await _engine(req).resume_generation()
    req.app.state.areal_paused = False
    return {"paused": False}


@router.post("/areal_update_weights")
async def update_weights(req: Request):
    eng = _engine(req)
    body = await _json(req)
    path = body.get("model_path")
    if not path:
        raise HTTPException(status_code=400, detail="`model_path` is required")
    t0 = time.perf_counter()
    was_paused = bool(getattr(req.app.state, "areal_paused", False))
    if not was_paused:  # a caller that did not pause first: do it around the reload
        await pause_generation(req)
    try:
        await eng.collective_rpc("reload_weights", kwargs={"weights_path": str(path)})
        await eng.reset_prefix_cache()
    finally:
        if not was_paused:
            await continue_generation(req)
    if body.get("version") is not None:
        req.app.state.areal_version = int(body["version"])
    return {"success": True, "model_path": str(path), "seconds": time.perf_counter() - t0}


@router.post("/areal_update_weights_lora")
async def update_weights_lora(req: Request):
    eng = _engine(req)
    body = await _json(req)
    for k in ("lora_name", "lora_model_path"):
        if not body.get(k):
            raise HTTPException(status_code=400, detail=f"`{k}` is required")
    try:
        from vllm.lora.request import LoRARequest
    except ImportError as e:  # pragma: no cover - vLLM is there whenever this server runs
        raise HTTPException(status_code=501, detail=f"vLLM's LoRA support is not importable: {e}")
    lora = LoRARequest(lora_name=body["lora_name"], lora_int_id=int(body.get("lora_int_id", 1)),
                       lora_path=body["lora_model_path"])
    ok = await eng.add_lora(lora)
    await eng.reset_prefix_cache()
    return {"success": bool(ok) if ok is not None else True, "lora_name": body["lora_name"]}


@router.post("/areal_set_version")
async def set_version(req: Request):
    req.app.state.areal_version = int((await _json(req)).get("version", 0))
    return {"version": req.app.state.areal_version}


@router.post("/areal_get_version")
async def get_version(req: Request):
    return {"version": int(getattr(req.app.state, "areal_version", 0))}


def _collective_only(name: str):
    async def route(req: Request):
        raise HTTPException(status_code=501, detail=f"{name}: weights reach external servers through a checkpoint "
                                                    "directory (/areal_update_weights); there is no collective "
                                                    "weight-update group on this server")

    return route


for _name in ("areal_init_weights_update_group", "areal_set_update_weight_meta", "areal_update_weights_xccl",
              "areal_update_weights_lora_xccl"):
    router.add_api_route("/" + _name, _collective_only(_name), methods=["POST"])


def attach_areal_routes(app: FastAPI) -> FastAPI:
    app.include_router(router)
    if not hasattr(app.state, "areal_version"):
        app.state.areal_version = 0
    return app


def main(argv: list[str] | None = None) -> None:
    """``vllm serve`` with the control routes mounted: vLLM's own argument parser and server loop, with its app
    factory wrapped."""
    import uvloop
    from vllm.entrypoints.openai import api_server
    from vllm.entrypoints.openai.cli_args import make_arg_parser, validate_parsed_serve_args
    from vllm.utils.argparse_utils import FlexibleArgumentParser

    build = api_server.build_app

    def build_with_control_routes(*a: Any, **k: Any) -> FastAPI:
        return attach_areal_routes(build(*a, **k))

    api_server.build_app = build_with_control_routes
    parser = make_arg_parser(FlexibleArgumentParser(description="vLLM rollout server with weight-update control routes"))
    args = parser.parse_args(argv)
    validate_parsed_serve_args(args)
    uvloop.run(api_server.run_server(args))


if __name__ == "__main__":
    main()
