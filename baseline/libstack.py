"""Library-stack context numbers for the benchmark shapes. NOT the reference and never reported as such.

The reference cannot be imported on this image (its entry points import hydra, omegaconf, peft, ... which
are not installed), so there is no same-box ratio. What IS installed are the libraries its stack is made
of: vLLM (one of its two rollout backends), HF ``transformers`` model code with flash-attn, PyTorch FSDP2
and the fused ``torch.optim.AdamW``. This module times those libraries, driven directly, on the shapes of
the headline benchmark (Qwen3-1.7B architecture, random weights, synthetic token ids):

* ``rollout``: vLLM generating responses whose lengths are drawn like the benchmark's (groups of 8 sharing a
  prompt, EOS ignored, forced length) on one GPU → generated tokens/s;
* ``train``: HF ``Qwen3ForCausalLM`` under FSDP2 (bf16 compute, fp32 master weights), packed varlen
  micro-batches of 16384 tokens through flash-attn, one no-grad forward (the proximal log-probabilities) plus
  one forward/backward per micro-batch and a fused AdamW step → consumed tokens/s per GPU;
* ``broadcast``: NCCL broadcast of the bf16 weights (3.4 GB) from rank 0 → seconds (N >= 2 only).

``python bench.py --impl libstack [--gpus N]`` prints one JSON line with ``"impl": "libstack"``.
"""

from __future__ import annotations

import json
import os
import sys
import tempfile
import time


def _hf_config_dir(preset: str) -> str:
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from areal_b200.models.config import PRESETS

    d = tempfile.mkdtemp(prefix="libstack_cfg_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(PRESETS[preset].to_hf_config(), f)
    return d


def _lengths(n_groups: int, group: int, prompt, resp, seed=1234):
    import torch

    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n_groups):
        L = int(torch.randint(prompt[0], prompt[1] + 1, (1,), generator=g))
        ids = torch.randint(0, 150000, (L,), generator=g).tolist()
        for _ in range(group):
            out.append((ids, int(torch.randint(resp[0], resp[1] + 1, (1,), generator=g))))
    return out


def rollout_vllm(preset="qwen3-1.7b", n_groups=80, group=8, prompt=(128, 512), resp=(256, 4096)) -> dict:
    """All requests are submitted at once (640 sequences: what one rollout GPU of the benchmark holds in
    flight at staleness 4); the rate is generated tokens over the whole call, tail included."""
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
    from vllm import LLM, SamplingParams

    reqs = _lengths(n_groups, group, prompt, resp)
    llm = LLM(model=_hf_config_dir(preset), skip_tokenizer_init=True, load_format="dummy", dtype="bfloat16",
              seed=0, gpu_memory_utilization=0.85, max_model_len=prompt[1] + resp[1] + 64, max_num_seqs=1024,
              max_num_batched_tokens=32768, enable_prefix_caching=True)
    prompts = [{"prompt_token_ids": ids} for ids, _ in reqs]
    params = [SamplingParams(temperature=1.0, max_tokens=n, min_tokens=n, ignore_eos=True, detokenize=False, logprobs=0)
              for _, n in reqs]
    warm = 16
    llm.generate(prompts[:warm], [SamplingParams(temperature=1.0, max_tokens=64, ignore_eos=True, detokenize=False)] * warm,
                 use_tqdm=False)
    t0 = time.perf_counter()
    outs = llm.generate(prompts, params, use_tqdm=False)
    dt = time.perf_counter() - t0
    gen = sum(len(o.outputs[0].token_ids) for o in outs)
    return {"generated_tokens": gen, "seconds": dt, "generated_tok_s": gen / dt, "sequences": len(reqs),
            "engine": "vLLM " + __import__("vllm").__version__}


def train_hf_fsdp2(preset="qwen3-1.7b", tokens_per_mb=16384, n_mbs=10, steps=3, warmup=2, seq=(384, 4608)) -> dict:
    import torch
    import torch.distributed as dist
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    from transformers import AutoConfig, AutoModelForCausalLM

    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        dist.init_process_group("nccl")
    rank = dist.get_rank()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    cfg = AutoConfig.from_pretrained(_hf_config_dir(preset))
    attn = "flash_attention_2"
    try:
        import flash_attn  # noqa: F401
    except Exception:
        attn = "sdpa"
    with torch.device("cuda"):
        model = AutoModelForCausalLM.from_config(cfg, torch_dtype=torch.float32, attn_implementation=attn)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for layer in model.model.layers:
        fully_shard(layer, mp_policy=mp)
    fully_shard(model, mp_policy=mp)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-6, weight_decay=0.01, fused=True)
    g = torch.Generator().manual_seed(7 + rank)

    def micro_batch():
        ids, pos, total = [], [], 0
        while True:
            L = int(torch.randint(seq[0], seq[1] + 1, (1,), generator=g))
            if total + L > tokens_per_mb:
                break
            ids.append(torch.randint(0, 150000, (L,), generator=g))
            pos.append(torch.arange(L))
            total += L
        return torch.cat(ids)[None].cuda(), torch.cat(pos)[None].cuda()

    mbs = [micro_batch() for _ in range(n_mbs)]
    n_tok = sum(int(i.numel()) for i, _ in mbs)

    def logp_of(ids, pos):
        out = model(input_ids=ids, position_ids=pos, use_cache=False).logits[0, :-1]
        return torch.log_softmax(out.float(), -1).gather(1, ids[0, 1:, None]).squeeze(1)

    def step():
        with torch.no_grad():
            prox = [logp_of(i, p) for i, p in mbs]  # proximal log-probabilities of the decoupled objective
        for (i, p), old in zip(mbs, prox):
            lp = logp_of(i, p)
            ratio = torch.exp(lp - old)
            loss = -(torch.clamp(ratio, 0.8, 1.2) * 0.1).mean() / n_mbs
            loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)

    try:
        for _ in range(warmup):
            step()
    except Exception as e:  # e.g. a flash-attn build without kernels for this GPU
        return {"error": f"{type(e).__name__}: {str(e)[:200]}", "attention": attn}
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    s = float(ms) / 1e3 / steps
    return {"tokens_per_step_per_gpu": n_tok, "seconds_per_step": s, "consumed_tok_s_per_gpu": n_tok / s,
            "attention": attn, "world": dist.get_world_size(),
            "stack": "HF Qwen3ForCausalLM + FSDP2 (bf16 compute, fp32 master) + torch.optim.AdamW(fused)"}


def rollout_ours(preset="qwen3-1.7b", n_groups=80, group=8, prompt=(128, 512), resp=(256, 4096)) -> dict:
    """This repository's rollout engine under the protocol of :func:`rollout_vllm`: the same 640 requests, all
    submitted at once, no weight updates in between, rate over the whole call."""
    import asyncio

    import torch

    from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeRolloutConfig
    from areal_b200.api.io_struct import ModelRequest
    from areal_b200.engine.rollout_engine import NativeRolloutEngine
    from areal_b200.models.config import PRESETS

    reqs = _lengths(n_groups, group, prompt, resp)
    mc = PRESETS[preset]
    ctx = prompt[1] + resp[1] + 64
    kv_per_token = 2 * mc.num_hidden_layers * mc.num_key_value_heads * mc.head_dim * 2
    n_blocks = int(min(120.0, len(reqs) * ctx * 0.75 * kv_per_token / 2**30) * 2**30 / (kv_per_token * 16))
    cfg = InferenceEngineConfig(backend="native:d1", consumer_batch_size=len(reqs), max_concurrent_rollouts=len(reqs),
                                native=NativeRolloutConfig(model_preset=preset, context_length=ctx, max_num_seqs=1024,
                                                           max_num_batched_tokens=32768, kv_block_size=16,
                                                           num_kv_blocks=n_blocks))
    eng = NativeRolloutEngine(cfg)
    eng.initialize()

    async def run(items):
        async def one(ids, n):
            g = GenerationHyperparameters(n_samples=1, max_new_tokens=n, temperature=1.0, ignore_eos=True)
            r = await eng.agenerate(ModelRequest(input_ids=ids, gconfig=g))
            return r.output_len

        return sum(await asyncio.gather(*[one(ids, n) for ids, n in items]))

    asyncio.run(run([(ids, 64) for ids, _ in reqs[:16]]))  # warm-up
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    gen = asyncio.run(run(reqs))
    dt = time.perf_counter() - t0
    eng.destroy()
    torch.cuda.empty_cache()
    return {"generated_tokens": gen, "seconds": dt, "generated_tok_s": gen / dt, "sequences": len(reqs),
            "engine": "areal_b200 NativeRolloutEngine"}


def train_ours(preset="qwen3-1.7b", tokens_per_mb=16384, n_mbs=10, steps=3, warmup=2, seq=(384, 4608)) -> dict:
    """This repository's train engine under the protocol of :func:`train_hf_fsdp2`: the same packed
    micro-batches, one no-grad forward for the proximal log-probabilities, one forward/backward per micro-batch
    with a clipped-ratio loss, one AdamW step."""
    import torch

    from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig
    from areal_b200.engine.train_engine import B200TrainEngine

    cfg = TrainEngineConfig(backend="fsdp:d1", model_preset=preset, init_from_scratch=True, dtype="bfloat16",
                            optimizer=OptimizerConfig(lr=1e-6, weight_decay=0.01, gradient_clipping=1.0),
                            mb_spec=MicroBatchSpec(max_tokens_per_mb=tokens_per_mb))
    eng = B200TrainEngine(cfg)
    eng.create_process_group()
    eng.initialize(None, None)
    g = torch.Generator().manual_seed(7)
    rows, total = [], 0
    while len(rows) < 4096:
        L = int(torch.randint(seq[0], seq[1] + 1, (1,), generator=g))
        if total + L > tokens_per_mb * n_mbs:
            break
        rows.append(torch.randint(0, 150000, (L,), generator=g))
        total += L
    Lmax = max(len(r) for r in rows)
    ids = torch.zeros(len(rows), Lmax, dtype=torch.long)
    mask = torch.zeros(len(rows), Lmax, dtype=torch.bool)
    for i, r in enumerate(rows):
        ids[i, :len(r)] = r
        mask[i, :len(r)] = True
    batch = dict(input_ids=ids, attention_mask=mask, loss_mask=mask.long())

    def step():
        old = eng.forward_batch(batch)  # proximal log-probabilities (no grad)
        b = dict(batch, prox=old)

        def loss_fn(logp, ent, mb):
            ratio = torch.exp(logp - mb["prox"].to(logp.device))
            m = mb["loss_mask"].float()
            return -(torch.clamp(ratio, 0.8, 1.2) * 0.1 * m).sum() / m.sum()

        return eng.train_batch(b, loss_fn, lambda mb: float(mb["loss_mask"].sum()))

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    s = e0.elapsed_time(e1) / 1e3 / steps
    eng.destroy()
    torch.cuda.empty_cache()
    return {"tokens_per_step_per_gpu": total, "seconds_per_step": s, "consumed_tok_s_per_gpu": total / s,
            "stack": "areal_b200 B200TrainEngine (own kernels, flat ZeRO optimizer)"}


def broadcast_nccl(nbytes=3_440_000_000, iters=5) -> dict:
    import torch
    import torch.distributed as dist

    buf = torch.empty(nbytes // 2, dtype=torch.bfloat16, device="cuda")
    for _ in range(2):
        dist.broadcast(buf, src=0)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        dist.broadcast(buf, src=0)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return {"bytes": nbytes, "seconds": float(ms) / 1e3, "ranks": dist.get_world_size()}


def main(n_gpus: int) -> int:
    res: dict = {"impl": "libstack", "n_gpus": n_gpus,
                 "note": "library stack driven directly (vLLM / HF + FSDP2 + flash-attn / NCCL); context for the "
                         "per-role rates of the benchmark line, not the reference and not a reference ratio"}
    rank = int(os.environ.get("RANK", "0"))
    try:
        res["train"] = train_hf_fsdp2()
    except Exception as e:
        res["train"] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
    if n_gpus > 1:
        try:
            res["broadcast"] = broadcast_nccl()
        except Exception as e:
            res["broadcast"] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
    else:
        import gc

        import torch
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
        gc.collect()
        torch.cuda.empty_cache()
        for k in ("RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "LOCAL_RANK"):
            os.environ.pop(k, None)
        # the same two protocols on this repository's engines, for a like-for-like reading
        for key, fn in (("train_ours", train_ours), ("rollout_ours", rollout_ours)):
            try:
                res[key] = fn()
            except Exception as e:
                res[key] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
            gc.collect()
            torch.cuda.empty_cache()
        try:
            res["rollout"] = rollout_vllm()
        except Exception as e:
            res["rollout"] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
    if rank == 0:
        print(json.dumps(res), flush=True)
    return 0
