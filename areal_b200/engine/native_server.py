"""HTTP front of the native rollout engine: one process, one GPU, one ``NativeRolloutEngine``.

The wire format of ``/generate`` follows the fields the reference exchanges with its inference
servers (``input_ids``, ``sampling_params{max_new_tokens, temperature, top_p, top_k, stop_token_ids,
ignore_eos, min_new_tokens}``, ``return_logprob``; reply ``meta_info.finish_reason.type`` in
``stop | length | abort`` and ``meta_info.output_token_logprobs`` as ``(logprob, token_id)`` pairs), so
:class:`areal_b200.infra.remote_inf_engine.RemoteInfEngine` drives this server and an SGLang server
through the same request builder. One ``/generate`` call is ONE scheduler request: when generation is
paused for a weight update it returns ``abort`` with the tokens produced so far and the client
re-issues prompt + partial output (interruptible rollout).

    python -m areal_b200.engine.native_server --model-path /models/Qwen3-1.7B --port 30000 \
        --experiment-name exp --trial-name t0 --server-index 0

Role of the reference's server launchers and endpoints: areal/infra/launcher/sglang_server.py,
areal/engine/sglang_remote.py:89-298, areal/engine/vllm_ext/areal_vllm_server.py:164-339.
"""

from __future__ import annotations

import argparse
import asyncio
import os
from typing import Any

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse

from ..api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeRolloutConfig
from ..api.io_struct import WeightUpdateMeta


def _image_processor(engine):
    """The image processor of the served checkpoint, loaded once (``engine.image_processor`` overrides it)."""
    proc = getattr(engine, "image_processor", None)
    if proc is None and getattr(engine.ncfg, "model_path", None):
        from transformers import AutoImageProcessor

        proc = engine.image_processor = AutoImageProcessor.from_pretrained(engine.ncfg.model_path)
    return proc


def create_app(engine) -> FastAPI:
    """FastAPI application around an initialised ``NativeRolloutEngine``."""
    app = FastAPI()

    @app.get("/health")
    async def health():
        return {"status": "ok", "version": engine.get_version(), "paused": engine._paused.is_set()}

    @app.get("/get_model_info")
    async def model_info():
        mc = engine.model_config
        return {"model_type": mc.model_type, "vocab_size": mc.vocab_size, "context_length": engine.ncfg.context_length}

    @app.get("/stats")
    async def stats():
        return engine.export_stats()

    @app.post("/generate")
    async def generate(req: Request):
        body = await req.json()
        sp = body.get("sampling_params", {})
        ids = [int(t) for t in body["input_ids"]]
        temperature = float(sp.get("temperature", 1.0))
        g = GenerationHyperparameters(
            n_samples=1, max_new_tokens=int(sp.get("max_new_tokens", 16)), min_new_tokens=int(sp.get("min_new_tokens", 0)),
            greedy=temperature == 0.0, temperature=temperature if temperature > 0 else 1.0,
            top_p=float(sp.get("top_p", 1.0)), top_k=int(sp.get("top_k", 0) if sp.get("top_k", 0) and sp["top_k"] > 0 else 0),
            stop_token_ids=[int(t) for t in sp.get("stop_token_ids", []) or []], ignore_eos=bool(sp.get("ignore_eos", False)))
        version = engine.get_version()
        if engine._paused.is_set():
            reason, toks, lps = "abort", [], []  # "abort before prefill": nothing was generated
        else:
            try:
                images = None
                if body.get("image_data"):
                    # base64 images, as SGLang's /generate takes them; the server's own image processor (from the
                    # model directory) turns them into pixel rows and patch grids
                    from ..api.io_struct import ModelRequest

                    proc = _image_processor(engine)
                    images = engine._image_inputs(ModelRequest(input_ids=ids, image_data=list(body["image_data"]),
                                                               processor=proc))
                reason, toks, lps = await engine._generate_once(ids, g, g.max_new_tokens, images)
            except (ValueError, NotImplementedError) as e:
                return JSONResponse({"error": str(e)}, status_code=400)
        return {"output_ids": toks,
                "meta_info": {"finish_reason": {"type": reason}, "version": version,
                              "output_token_logprobs": [[float(lp), int(t)] for lp, t in zip(lps, toks)],
                              "prompt_tokens": len(ids), "completion_tokens": len(toks)}}

    @app.post("/pause_generation")
    async def pause():
        await asyncio.get_running_loop().run_in_executor(None, engine.pause_generation)
        return {"success": True}

    @app.post("/continue_generation")
    async def cont():
        engine.continue_generation()
        return {"success": True}

    @app.post("/update_weights_from_disk")
    async def update_from_disk(req: Request):
        body = await req.json()
        meta = WeightUpdateMeta(type="disk", path=body["model_path"], version=body.get("version"))
        loop = asyncio.get_running_loop()
        try:
            await loop.run_in_executor(None, lambda: engine.update_weights_from_disk(meta).result())
        except Exception as e:  # noqa: BLE001 - reported to the caller, the server stays up
            return JSONResponse({"success": False, "message": f"{type(e).__name__}: {e}"}, status_code=500)
        return {"success": True, "version": engine.get_version()}

    @app.post("/set_version")
    async def set_version(req: Request):
        engine.set_version(int((await req.json())["version"]))
        return {"success": True}

    @app.get("/get_version")
    async def get_version():
        return {"version": engine.get_version()}

    @app.post("/release_memory_occupation")
    async def release():
        await asyncio.get_running_loop().run_in_executor(None, engine.offload)
        return {"success": True}

    @app.post("/resume_memory_occupation")
    async def resume():
        await asyncio.get_running_loop().run_in_executor(None, engine.onload)
        return {"success": True}

    return app


def build_engine(args: argparse.Namespace):
    from .rollout_engine import NativeRolloutEngine

    native = NativeRolloutConfig(model_path=args.model_path or "", model_preset=args.model_preset,
                                 context_length=args.context_length, max_num_seqs=args.max_num_seqs,
                                 max_num_batched_tokens=args.max_num_batched_tokens, seed=args.seed,
                                 cuda_graph=not args.disable_cuda_graph, num_kv_blocks=args.num_kv_blocks)
    cfg = InferenceEngineConfig(experiment_name=args.experiment_name, trial_name=args.trial_name,
                                backend="native:d1", native=native)
    eng = NativeRolloutEngine(cfg)
    eng.initialize(**({"device": args.device} if args.device else {}))
    return eng


def parse_args(argv=None) -> argparse.Namespace:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-path", default=None)
    ap.add_argument("--model-preset", default=None)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=0, help="0 = pick a free port")
    ap.add_argument("--context-length", type=int, default=32768)
    ap.add_argument("--max-num-seqs", type=int, default=512)
    ap.add_argument("--max-num-batched-tokens", type=int, default=16384)
    ap.add_argument("--num-kv-blocks", type=int, default=None)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--device", default=None)
    ap.add_argument("--disable-cuda-graph", action="store_true")
    ap.add_argument("--experiment-name", default="")
    ap.add_argument("--trial-name", default="")
    ap.add_argument("--server-index", type=int, default=0)
    ap.add_argument("--name-resolve-root", default=None, help="NFS name-resolve root shared with the trainer")
    return ap.parse_args(argv)


def main(argv=None) -> int:
    import uvicorn

    from ..utils import name_resolve, names
    from ..utils.network import find_free_ports

    args = parse_args(argv)
    if not (args.model_path or args.model_preset):
        raise SystemExit("--model-path or --model-preset is required")
    engine = build_engine(args)
    port = args.port or find_free_ports(1)[0]
    if args.experiment_name and args.trial_name:
        if args.name_resolve_root:
            from ..api.cli_args import NameResolveConfig

            name_resolve.reconfigure(NameResolveConfig(type="nfs", nfs_record_root=args.name_resolve_root))
        # the trainer's RemoteInfEngine discovers servers under this key
        name_resolve.add(names.gen_server(args.experiment_name, args.trial_name, args.server_index),
                         f"{args.host}:{port}", replace=True)
    try:
        uvicorn.run(create_app(engine), host=args.host, port=port, log_level=os.environ.get("AREAL_B200_HTTP_LOG", "warning"))
    finally:
        engine.destroy()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
