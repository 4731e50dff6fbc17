#!/usr/bin/env python
"""Headline benchmark: asynchronous GRPO trained tokens/s (and weight-sync latency)
for the Qwen3-1.7B-architecture configuration, random-init weights, synthetic prompts.

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Allocation: N = 1 → rollout and trainer colocated on the GPU (time-shared, generation
overlaps training on separate streams); N ≥ 2 → the first N/2 ranks run the rollout engine
(``native:d{N/2}``) and the last N/2 ranks train (``fsdp:d{N/2}``), i.e. ``d4 + d4`` at N = 8.
Per-GPU work is fixed (weak scaling): 8 prompts x group 8 per GPU, 64 x 8 at N = 8.

One step = wait for a batch (bounded staleness 4) → recompute proximal logprobs →
advantages → decoupled-PPO update (AdamW) → pause rollout, push weights over NVLink,
resume. Generation runs concurrently all the time. ``value`` is timed with CUDA events on
the trainer stream over K steps (max over ranks); ``e2e`` is the wall-clock of K further
steps through the public ``PPOTrainer.train`` API, including the pinned-host → device copy
of every micro-batch and the device → host read of the step's loss / grad-norm.

``--impl reference`` reports why the reference cannot run on this image; ``--impl libstack`` times the
libraries its stack is built from (vLLM, HF + FSDP2 + flash-attn, NCCL) on the same shapes, as context.
``--config 3|4|5`` selects the other benchmark configurations (Ulysses, fp8 + tensor parallel, MoE + expert
parallel); the default is the headline configuration 2.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import time

REFERENCE_UNAVAILABLE = (
    "the reference cannot start on this image: its trainer entry points import hydra and omegaconf "
    "(areal/api/cli_args.py:14-17), its FSDP engine imports peft (areal/engine/fsdp_engine.py:21), and flask, "
    "colorlog, tensordict, torchao, ray, megatron-core, mbridge and SGLang are needed further down; none of them is "
    "installed or in /opt/wheelhouse (pip install of the tree itself also stops at its build backend uv_build). "
    "vLLM, flash-attn and transformers ARE installed: `--impl libstack` times those libraries on the same shapes")


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=2)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference", "libstack"])
    p.add_argument("--config", type=int, default=2, choices=[2, 3, 4, 5],
                   help="benchmark configuration: 2 = Qwen3-1.7B native:dN/2 + fsdp:dN/2 (the headline, default); "
                        "3 = Qwen3-8B rollout dN/2 + trainer Ulysses cN/2; 4 = Qwen2.5-7B block-scaled fp8, trainer "
                        "tp2 x dN/4; 5 = Qwen3-30B-A3B, expert-parallel trainer time-sharing the GPUs with rollout")
    p.add_argument("--model", default=None)
    p.add_argument("--prompts-per-gpu", type=int, default=None)
    p.add_argument("--group", type=int, default=8)
    p.add_argument("--prompt-min", type=int, default=None)
    p.add_argument("--prompt-max", type=int, default=None)
    p.add_argument("--resp-min", type=int, default=None)
    p.add_argument("--resp-max", type=int, default=None)
    p.add_argument("--staleness", type=int, default=4)
    p.add_argument("--max-tokens-per-mb", type=int, default=None)
    p.add_argument("--kv-gb", type=float, default=0.0, help="KV-cache budget per rollout GPU (0 = automatic)")
    p.add_argument("--no-fused-comm-check", action="store_true",
                   help="N >= 2: skip the untimed check of the fused compute+collective kernels")
    p.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (invalidates the result)")
    return p.parse_args()


def synthetic_reward(prompt, completion, prompt_ids, completion_ids, **kw):
    """Seeded deterministic 0/1 function of the response tokens."""
    h = hashlib.blake2b(bytes(str(completion_ids[:64]), "ascii"), digest_size=2).digest()
    return float(h[0] & 1)


def make_workflow_cls():
    import torch

    from areal_b200.workflow.rlvr import RLVRWorkflow

    class SyntheticLengthWorkflow(RLVRWorkflow):
        """EOS is forced at a per-sample length drawn uniformly from [resp_min, resp_max]
        (seeded by the prompt), as the benchmark configuration prescribes."""

        def __init__(self, resp_min: int, resp_max: int, **kw):
            super().__init__(**kw)
            self.resp_min, self.resp_max = resp_min, resp_max
            self._count = 0

        async def arun_episode(self, engine, data):
            self._count += 1
            seed = int.from_bytes(hashlib.blake2b(
                bytes(str((data["input_ids"][:16], self._count)), "ascii"), digest_size=4).digest(), "little")
            g = torch.Generator().manual_seed(seed)
            n_new = int(torch.randint(self.resp_min, self.resp_max + 1, (1,), generator=g))
            saved = self.gconfig
            self.gconfig = saved.new(max_new_tokens=n_new, ignore_eos=True)
            try:
                return await super().arun_episode(engine, data)
            finally:
                self.gconfig = saved

    return SyntheticLengthWorkflow


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                power = float(parts[3])
                clk = float(parts[1])
            except ValueError:
                continue
            if power > 250:  # under load
                sm.append(clk)
            mx.append(float(parts[2]))
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                 parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples_under_load": len(sm)}


_RO_PHASES = {"decode_gpu_wait": "rollout/host_s/wait", "decode_stage": "rollout/host_s/stage",
              "plan": "rollout/host_s/plan", "params": "rollout/host_s/params",
              "commit_deliver": "rollout/host_s/commit_deliver", "prefill": "rollout/host_s/prefill",
              "paused": "rollout/host_s/paused", "idle": "rollout/host_s/idle"}


def role_budget(a: dict, b: dict) -> dict:
    """Per rollout rank: what its engine did between two snapshots of its counters (taken when the first and
    the last batch of the timed window arrived): generated tokens per second and the share of its wall time
    spent in each phase of the engine loop."""
    out = {}
    for g in b:
        if g not in a:
            continue
        d = lambda k: float(b[g].get(k, 0.0)) - float(a[g].get(k, 0.0))
        wall = d("rollout/wall_s")
        if wall <= 0:
            continue
        frac = {name: d(key) / wall for name, key in _RO_PHASES.items()}
        frac["other"] = 1.0 - sum(frac.values())
        out[int(g)] = {"wall_s": wall, "generated_tok_s": d("rollout/generated_tokens") / wall,
                       "decode_steps": d("rollout/engine_steps"),
                       "tokens_per_decode_step": d("rollout/generated_tokens") / max(d("rollout/engine_steps"), 1.0),
                       "prefill_tok_s": d("rollout/prefill_tokens") / max(d("rollout/host_s/prefill"), 1e-9),
                       "prefill_tokens": d("rollout/prefill_tokens"),
                       "resubmitted_context_tokens": d("rollout/reprefill_tokens"),
                       "time_frac": {k: round(v, 4) for k, v in frac.items()}}
    return out


def summarize_roles(roles: list, window_s: float, n_gen: int, n_train: int, trained_tokens: float,
                    steps: int) -> dict:
    ro = {}
    for r in roles:
        ro.update(r["rollout"])
    gen = [v["generated_tok_s"] for v in ro.values()]
    keys = sorted({k for v in ro.values() for k in v["time_frac"]})
    mean_frac = {k: round(sum(v["time_frac"].get(k, 0.0) for v in ro.values()) / max(len(ro), 1), 4) for k in keys}
    wait = [r["phase_s"]["timeperf/rollout"] for r in roles]
    busy = [sum(v for k, v in r["phase_s"].items() if k != "timeperf/rollout") for r in roles]
    return {
        "generated_tok_s_per_rollout_gpu": (sum(gen) / len(gen)) if gen else None,
        "rollout_time_frac": mean_frac,
        "rollout_tokens_per_decode_step": (sum(v["tokens_per_decode_step"] for v in ro.values()) / len(ro)) if ro else None,
        "rollout_prefill_tok_s": (sum(v["prefill_tok_s"] for v in ro.values()) / len(ro)) if ro else None,
        # context tokens of requests re-submitted after a weight update (counted when re-submitted; the pages of a
        # shared prompt are not recomputed) beside the tokens that prefill steps actually computed in the window
        "rollout_prefill_tokens_per_gpu": (sum(v["prefill_tokens"] for v in ro.values()) / len(ro)) if ro else None,
        "rollout_resubmitted_context_tokens_per_gpu":
            (sum(v["resubmitted_context_tokens"] for v in ro.values()) / len(ro)) if ro else None,
        "consumed_tok_s_per_trainer_gpu": trained_tokens / max(sum(busy), 1e-9),
        "trainer_idle_frac": sum(wait) / max(window_s * len(roles), 1e-9),
        "trainer_phase_s_per_step": {k.split("/")[1]: round(sum(r["phase_s"][k] for r in roles) / len(roles) / steps, 4)
                                     for k in roles[0]["phase_s"]},
        "n_rollout_gpus": n_gen, "n_trainer_gpus": n_train,
    }


# Per configuration: model preset, prompts per GPU (weak scaling: the named global batch at N = 8), prompt and
# response length ranges, micro-batch token budget.
CONFIGS = {
    2: dict(model="qwen3-1.7b", prompts_per_gpu=8, prompt=(128, 512), resp=(256, 4096), mb=16384),
    3: dict(model="qwen3-8b", prompts_per_gpu=4, prompt=(512, 512), resp=(1024, 16384), mb=32768),
    4: dict(model="qwen2.5-7b", prompts_per_gpu=4, prompt=(256, 256), resp=(256, 8192), mb=16384),
    5: dict(model="qwen3-30b-a3b", prompts_per_gpu=2, prompt=(512, 512), resp=(512, 8192), mb=16384),
}


def resolve_config(args, N: int) -> dict:
    """Fills unset arguments from the chosen configuration and derives the allocation strings for N GPUs."""
    c = CONFIGS[args.config]
    args.model = args.model or c["model"]
    args.prompts_per_gpu = args.prompts_per_gpu or c["prompts_per_gpu"]
    args.prompt_min = args.prompt_min or c["prompt"][0]
    args.prompt_max = args.prompt_max or c["prompt"][1]
    args.resp_min = args.resp_min or c["resp"][0]
    args.resp_max = args.resp_max or c["resp"][1]
    args.max_tokens_per_mb = args.max_tokens_per_mb or c["mb"]
    half = max(N // 2, 1)
    if args.config == 2:
        n_gen = n_train = N if N == 1 else half
        rollout, actor = f"native:d{n_gen}", f"fsdp:d{n_train}"
    elif args.config == 3:
        # Ulysses sequence parallelism over all trainer GPUs (d1 x c4 at N = 8)
        n_gen = n_train = N if N == 1 else half
        rollout, actor = f"native:d{n_gen}", f"fsdp:d1c{n_train}"
    elif args.config == 4:
        # tensor parallel 2 inside the trainer half (d2 x t2 at N = 8); the rollout engine serves one model per GPU
        if N < 4 or N % 4:
            raise SystemExit("--config 4 needs a multiple of 4 GPUs (trainer tp 2 on one half, rollout on the other)")
        n_gen = n_train = half
        rollout, actor = f"native:d{n_gen}", f"megatron:d{n_train // 2}t2"
    else:
        # every GPU hosts a rollout engine and one expert-parallel trainer rank (time-shared)
        if N < 2:
            raise SystemExit("--config 5 needs at least 2 GPUs (expert parallelism)")
        n_gen = n_train = N
        rollout, actor = f"native:d{N}", f"megatron:d{N}e{N}"
    return dict(n_gen=n_gen, n_train=n_train, rollout=rollout, actor=actor, colocated=(N == 1 or args.config == 5))


def main():
    args = parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    if args.impl == "libstack":
        # context numbers from the installed libraries (vLLM, HF + FSDP2 + flash-attn, NCCL) on the benchmark's
        # shapes: NOT the reference, never a reference ratio (see baseline/libstack.py)
        from baseline import libstack

        return libstack.main(args.gpus)
    import torch
    import torch.distributed as dist

    from areal_b200.api.cli_args import (GenerationHyperparameters, GRPOConfig, InferenceEngineConfig,
                                         MicroBatchSpec, NativeRolloutConfig, NormConfig, OptimizerConfig,
                                         PPOActorConfig, RejectionSamplingConfig, _propagate_names)
    from areal_b200.models.config import PRESETS
    from areal_b200.ops import _lib
    from areal_b200.trainer.rl_trainer import PPOTrainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torchrun for N > 1")
    N = args.gpus
    lay = resolve_config(args, N)
    n_gen, n_train = lay["n_gen"], lay["n_train"]
    group = args.group
    prompts_global = args.prompts_per_gpu * N
    model_over = {"num_hidden_layers": args.layers} if args.layers else {}
    mc = PRESETS[args.model]
    ctx = args.prompt_max + args.resp_max + 64
    kv_per_token = 2 * (args.layers or mc.num_hidden_layers) * mc.num_key_value_heads * mc.head_dim * 2
    per_rollout_seqs = prompts_global * group // n_gen
    inflight = per_rollout_seqs * (args.staleness + 1)
    weights_gb = mc.num_params() * 2 / 2**30
    kv_cap = (70.0 if args.config != 5 else 40.0) if lay["colocated"] else max(150.0 - weights_gb, 20.0) * 0.8
    kv_gb = args.kv_gb or min(kv_cap, inflight * (ctx * 0.75) * kv_per_token / 2**30)
    block = 16
    n_blocks = int(kv_gb * 2**30 / (kv_per_token * block))

    cfg = GRPOConfig(experiment_name="bench", trial_name=f"n{N}")
    cfg.cluster.fileroot = os.environ.get("AREAL_B200_FILEROOT", "/tmp/areal_b200_bench")
    cfg.train_dataset.batch_size = prompts_global
    cfg.train_dataset.shuffle = False
    cfg.gconfig = GenerationHyperparameters(n_samples=group, max_new_tokens=args.resp_max, temperature=1.0)
    cfg.actor = PPOActorConfig(
        experiment_name="bench", trial_name=f"n{N}", backend=lay["actor"], model_preset=args.model,
        model_overrides=model_over, init_from_scratch=True, dtype="bfloat16",
        optimizer=OptimizerConfig(lr=1e-6, weight_decay=0.01, gradient_clipping=1.0),
        mb_spec=MicroBatchSpec(max_tokens_per_mb=args.max_tokens_per_mb), ppo_n_minibatches=1,
        reward_norm=NormConfig(mean_level="group", std_level="group", group_size=group),
        adv_norm=NormConfig(mean_level="batch", std_level="batch"), kl_ctl=0.0, eps_clip=0.2,
        use_decoupled_loss=True, recompute_logprob=True,
        rejection_sampling=RejectionSamplingConfig(level="token", action="mask", metric="ratio", upper=5.0),
        max_new_tokens=args.resp_max)
    cfg.rollout = InferenceEngineConfig(
        backend=lay["rollout"], max_head_offpolicyness=args.staleness,
        max_concurrent_rollouts=prompts_global * (args.staleness + 1),
        native=NativeRolloutConfig(model_preset=args.model, model_overrides=model_over, context_length=ctx,
                                   max_num_seqs=min(1024, inflight), max_num_batched_tokens=32768,
                                   kv_block_size=block, num_kv_blocks=n_blocks))
    if args.config == 4:
        from areal_b200.api.cli_args import FP8EngineConfig

        cfg.actor.megatron.fp8_config = FP8EngineConfig(mode="e4m3", recipe="blockwise")
    if args.config in (3, 5):
        cfg.actor.gradient_checkpointing = True  # 16k-token responses / 48 MoE blocks: recompute block activations
    _propagate_names(cfg)

    g = torch.Generator().manual_seed(1234)
    n_items = prompts_global * (args.warmup + 2 * args.steps + 8)
    dataset = []
    for _ in range(n_items):
        L = int(torch.randint(args.prompt_min, args.prompt_max + 1, (1,), generator=g))
        dataset.append({"input_ids": torch.randint(0, mc.vocab_size, (L,), generator=g).tolist()})

    W, K = args.warmup, args.steps
    total_steps = W + 2 * K
    fused_comm = None
    if N > 1 and not args.no_fused_comm_check:
        # Outside the timed region: the fused compute+collective kernels (GEMM->reduce-scatter, all-gather->GEMM,
        # GEMM->all-to-all, all-to-all->GEMM over NVLink peer memory) checked against NCCL and timed on the N ranks
        # of this very job. The flagship layout (data-parallel rollout + ZeRO trainer) does not call them, so this
        # is where a scaling run shows that they work at N ranks.
        import datetime

        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        if not dist.is_initialized():
            dist.init_process_group(backend="nccl", timeout=datetime.timedelta(seconds=7200))
        from areal_b200.parallel.selfcheck import fused_comm_check

        # M x K x N large enough that the timings are bound by the GPU and the links, not by launches; every
        # per-rank extent stays a multiple of the 128-wide tile up to 8 ranks
        try:
            fused_comm = fused_comm_check(M=16384, K=4096, N=4096, iters=5)
        except (RuntimeError, AssertionError, ValueError) as e:  # same inputs on every rank: all ranks land here
            fused_comm = {"error": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.synchronize()
        dist.barrier()
    trainer = PPOTrainer(cfg, dataset)
    dev = torch.device("cuda", torch.cuda.current_device())
    marks: dict[str, object] = {}
    tok_per_step: list[float] = []
    sync_s: list[float] = []
    sampler = ClockSampler()
    cpu_group = trainer.train_cpu_group

    def fence():
        if dist.is_initialized() and trainer.is_trainer and trainer.actor_engine.world_size > 1:
            dist.barrier(group=cpu_group)
        torch.cuda.synchronize()

    resp_per_step: list[float] = []
    phase_keys = ("timeperf/rollout", "timeperf/recompute_logp", "timeperf/compute_advantage", "timeperf/train_step",
                  "timeperf/update_weights")
    phases: list[dict] = []

    def rollout_snapshot() -> dict:
        """Latest counters of the rollout engine(s) this rank is paired with (its own when colocated)."""
        if trainer.colocated:
            return {trainer.rank: dict(trainer.rollout.export_stats())}
        return {g: dict(st) for g, st in getattr(trainer.rollout_client, "rollout_stats", {}).items()}

    def on_step(step: int, stats: dict):
        tok_per_step.append(stats.get("step/trained_tokens", 0.0))
        resp_per_step.append(stats.get("step/response_tokens", 0.0))
        sync_s.append(stats.get("step/weight_sync_s", 0.0))
        phases.append({k: float(stats.get(k, 0.0)) for k in phase_keys})
        if step == W - 1:
            marks["ro0"] = rollout_snapshot()
        elif step == W + K - 1:
            marks["ro1"] = rollout_snapshot()
        if step == W - 1:
            fence()
            if trainer.rank == (0 if trainer.colocated else trainer.topo.train_ranks[0]):
                sampler.start()
            _lib.reset_launch_count()
            eng = trainer.actor_engine
            eng.h2d_bytes = eng.d2h_bytes = 0
            marks["ev0"] = torch.cuda.Event(enable_timing=True)
            marks["ev0"].record()
        elif step == W + K - 1:
            marks["ev1"] = torch.cuda.Event(enable_timing=True)
            marks["ev1"].record()
            fence()
            marks["launches"] = _lib.launch_count()
            marks["t0"] = time.perf_counter()
            eng = trainer.actor_engine
            eng.h2d_bytes = eng.d2h_bytes = 0
        elif step == W + 2 * K - 1:
            fence()
            marks["t1"] = time.perf_counter()
            eng = trainer.actor_engine
            marks["h2d"], marks["d2h"] = eng.h2d_bytes, eng.d2h_bytes

    WorkflowCls = make_workflow_cls()
    wf_kwargs = dict(resp_min=args.resp_min, resp_max=args.resp_max, reward_fn=synthetic_reward,
                     gconfig=cfg.gconfig, reward_in_process=True)
    try:
        trainer.train(workflow=WorkflowCls, workflow_kwargs=wf_kwargs, max_steps=total_steps, step_callback=on_step)
    finally:
        clocks = sampler.stop() if sampler.proc is not None else None

    result = None
    if trainer.is_trainer:
        dev_ms = marks["ev0"].elapsed_time(marks["ev1"])
        wall_s = marks["t1"] - marks["t0"]
        # ranks of one model-parallel replica (tensor / sequence / pipeline peers) train the same batch: the
        # replica's head counts its tokens
        counts = 1.0 if trainer.actor_engine.is_data_parallel_head() else 0.0
        tok_value = counts * sum(tok_per_step[W:W + K])
        tok_e2e = counts * sum(tok_per_step[W + K:W + 2 * K])
        t = torch.tensor([dev_ms, wall_s, -tok_value, -tok_e2e, max(sync_s[W:]) if sync_s[W:] else 0.0],
                         dtype=torch.float64)
        sums = torch.tensor([tok_value, tok_e2e], dtype=torch.float64)
        if dist.is_initialized() and trainer.actor_engine.world_size > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=cpu_group)
            dist.all_reduce(sums, group=cpu_group)
        head = 0 if trainer.colocated else trainer.topo.train_ranks[0]
        # per-role view: what each rollout GPU did during the timed window, and how the trainer's step splits
        ro = role_budget(marks.get("ro0", {}), marks.get("ro1", {}))
        mine = {"rollout": ro, "phase_s": {k: sum(p[k] for p in phases[W:W + K]) for k in phase_keys},
                "resp_tokens": counts * sum(resp_per_step[W:W + K])}
        roles = [mine]
        if dist.is_initialized() and trainer.actor_engine.world_size > 1:
            roles = [None] * trainer.actor_engine.world_size
            dist.all_gather_object(roles, mine, group=cpu_group)
        if trainer.rank == head:
            dev_ms, wall_s, sync_max = float(t[0]), float(t[1]), float(t[4])
            value = float(sums[0]) / (dev_ms / 1e3)
            e2e = float(sums[1]) / wall_s
            result = {
                "metric": "async-GRPO trained tokens/s (whole job)", "value": value, "unit": "tokens/s",
                "n_gpus": N, "steps": K, "warmup": W, "ms_per_step": dev_ms / K,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic prompts (uniform-random ids), random-init weights",
                "config": {
                    "model": args.model + ("" if not args.layers else f"[layers={args.layers} DEBUG]"),
                    "global_batch": prompts_global * group, "prompts": prompts_global, "group": group,
                    "seq_len": f"prompt U[{args.prompt_min},{args.prompt_max}] + response U[{args.resp_min},{args.resp_max}] (EOS forced)",
                    "parallelism": (f"colocated {lay['rollout']}|{lay['actor']}" if lay["colocated"]
                                    else f"{lay['rollout']}+{lay['actor']}"),
                    "benchmark_config": args.config,
                    "staleness": args.staleness, "max_tokens_per_mb": args.max_tokens_per_mb,
                    "l2": "no explicit flush: every step streams >3.4 GB of weights plus activations, far above the 126 MB L2",
                    "weight_sync_s_max": sync_max,
                },
                "clocks": clocks,
                "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": int(marks["h2d"] / K),
                        "d2h_bytes_per_step": int(marks["d2h"] / K)},
                "gpu_launches": int(marks["launches"]),
                "weight_sync_latency_s": sync_max,
                "token_accounting": "trained tokens = prompt + response tokens of every sequence of the batch "
                                    "(the prompt is part of the forward/backward pass); response_tok_s counts "
                                    "the loss-masked response tokens only",
                "response_tok_s": sum(r["resp_tokens"] for r in roles) / (dev_ms / 1e3),
                "roles": summarize_roles(roles, dev_ms / 1e3, n_gen, n_train, float(sums[0]), K),
                "fallback_ops": _lib.fallback_counts(),
            }
            if fused_comm is not None and "error" in fused_comm:
                result["extra_keys"] = {"fused_comm_ok": False, "fused_comm_error": fused_comm["error"]}
            elif fused_comm is not None:
                fc = fused_comm
                result["extra_keys"] = {
                    "fused_comm_ok": fc["ok"], "fused_comm_max_err": fc["max_err"],
                    "fused_comm_status": fc["status_end"] or fc["status"], "fused_comm_ranks": fc["world"],
                    "fused_comm_shape": fc["shape"],
                    "fused_vs_unfused_ms": {k: [round(fc[f"t_{k}_fused_ms"], 4), round(fc[f"t_{k}_nccl_ms"], 4)]
                                            for k in ("gemm_rs", "ag_gemm", "gemm_a2a", "a2a_gemm")},
                    "fused_frac_of_roofline": {k: round(fc[f"frac_of_roofline_{k}_fused"], 3)
                                               for k in ("gemm_rs", "ag_gemm", "gemm_a2a", "a2a_gemm")},
                    "fused_comm_note": "measured outside the timed region on all ranks of this job; unfused = this "
                                       "library's GEMM + the NCCL collective; roofline = max(FLOPs / measured bf16 "
                                       "peak, NVLink bytes / 770 GB/s)",
                }
    if os.environ.get("AREAL_B200_BENCH_DIAG"):
        # host-side view of the rollout engine (stderr only): scheduler counters and where its loop spent time
        eng = getattr(trainer, "rollout", None)
        inner = getattr(eng, "engine", eng)
        if inner is not None and hasattr(inner, "export_stats"):
            try:
                st = inner.export_stats()
                print("rollout diag: " + json.dumps({k: round(float(v), 3) for k, v in sorted(st.items())}),
                      file=sys.stderr, flush=True)
            except Exception as e:  # diagnostics must never change the run's outcome
                print(f"rollout diag unavailable: {e}", file=sys.stderr)
    trainer.close()
    if result is not None:
        print(json.dumps(result), flush=True)
    if dist.is_initialized():
        try:
            dist.barrier()
        except Exception:
            pass
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
