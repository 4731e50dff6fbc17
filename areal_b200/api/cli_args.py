"""Experiment configuration: dataclasses, YAML loading and ``a.b=c`` overrides.

The field names and defaults are the public configuration surface of the
reference (areal/api/cli_args.py:41-2994), so existing YAML files and
``key=value`` command lines keep working. The loader itself is self-contained
(PyYAML + dataclass introspection): it merges a YAML tree with dotted
overrides, resolves ``${path.to.key}`` interpolations and builds the typed
dataclasses recursively, rejecting unknown keys.
"""

from __future__ import annotations

import argparse
import dataclasses
import getpass
import json
import os
import re
import types
import typing
from dataclasses import asdict, dataclass, field, fields, is_dataclass
from pathlib import Path
from typing import Any, ClassVar, TypeVar

import yaml

MISSING = "???"

PROX_LOGP_METHOD_RECOMPUTE = "recompute"
PROX_LOGP_METHOD_LOGLINEAR = "loglinear"
PROX_LOGP_METHOD_LINEAR = "linear"
PROX_LOGP_METHOD_METRICS = "metrics"
PROX_LOGP_METHOD_ROLLOUT = "rollout"
PROX_LOGP_METHODS = (PROX_LOGP_METHOD_RECOMPUTE, PROX_LOGP_METHOD_LOGLINEAR,
                     PROX_LOGP_METHOD_LINEAR, PROX_LOGP_METHOD_METRICS, PROX_LOGP_METHOD_ROLLOUT)


# --------------------------------------------------------------------------- numerics


@dataclass
class NormConfig:
    """How rewards / advantages are normalised: independent levels for the mean
    and the std (``batch``, ``group`` or ``None``)."""

    mean_level: str | None = "batch"
    mean_leave1out: bool = False
    std_level: str | None = "batch"
    std_unbiased: bool = True
    eps: float = 1e-5
    group_size: int = 1

    def __post_init__(self):
        for name in ("mean_level", "std_level"):
            v = getattr(self, name)
            if v in ("none", "None", "null"):
                setattr(self, name, None)
                v = None
            if v not in ("batch", "group", None):
                raise ValueError(f"{name} must be 'batch', 'group' or None, got {v}")
        if "group" in (self.mean_level, self.std_level) and self.group_size < 1:
            raise ValueError(f"group_size must be positive for group normalization, got {self.group_size}")


@dataclass
class MicroBatchSpec:
    """How a batch is cut into micro-batches: at least ``n_mbs`` pieces, at most
    ``max_tokens_per_mb`` tokens each, sequence counts multiples of ``granularity``."""

    n_mbs: int | None = 1
    granularity: int = 1
    max_tokens_per_mb: int | None = None
    n_mbs_divisor: int = 1
    packing_algorithm: str = "ffd"

    def __post_init__(self):
        if self.packing_algorithm not in ("ffd", "kk"):
            raise ValueError(f"packing_algorithm must be 'ffd' or 'kk', got {self.packing_algorithm}")

    @classmethod
    def new(cls, mb_spec: "MicroBatchSpec", **kwargs) -> "MicroBatchSpec":
        d = dict(n_mbs=mb_spec.n_mbs, granularity=mb_spec.granularity,
                 max_tokens_per_mb=mb_spec.max_tokens_per_mb, n_mbs_divisor=mb_spec.n_mbs_divisor,
                 packing_algorithm=mb_spec.packing_algorithm)
        d.update(kwargs)
        return cls(**d)


@dataclass
class GenerationHyperparameters:
    n_samples: int = 1
    max_new_tokens: int = 16384
    min_new_tokens: int = 0
    max_tokens: int = 32768
    greedy: bool = False
    top_p: float = 1.0
    top_k: int = int(1e8)
    temperature: float = 1.0
    stop_token_ids: list[int] = field(default_factory=list)
    ignore_eos: bool = False
    skip_special_tokens: bool = True
    stop: list[str] | None = None
    frequency_penalty: float = 0.0
    lora_name: str = "default_lora"
    use_beam_search: bool = False

    _OPENAI_UNSUPPORTED_ARGS: ClassVar[set[str]] = {
        "min_new_tokens", "greedy", "top_k", "stop_token_ids", "ignore_eos",
        "skip_special_tokens", "lora_name", "use_beam_search", "max_tokens"}

    def new(self, **kwargs) -> "GenerationHyperparameters":
        d = {f.name: getattr(self, f.name) for f in fields(self)}
        d["stop_token_ids"] = list(d["stop_token_ids"])
        d.update(kwargs)
        return GenerationHyperparameters(**d)

    def to_openai_args_dict(self, exclude_args: list[str] | None = None) -> dict[str, Any]:
        """Arguments accepted by an OpenAI-style completion call."""
        exclude = set(exclude_args or []) | self._OPENAI_UNSUPPORTED_ARGS
        out = {}
        for f in fields(self):
            if f.name in exclude:
                continue
            v = getattr(self, f.name)
            if f.name == "n_samples":
                out["n"] = v
            elif f.name == "max_new_tokens":
                out["max_completion_tokens"] = v
            else:
                out[f.name] = v
        return out


@dataclass
class OptimizerConfig:
    type: str = "adam"
    lr: float = 1e-3
    weight_decay: float = 0.01
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    min_lr_ratio: float = 0.0
    lr_scheduler_type: str = "constant"
    warmup_steps_proportion: float = 0.001
    initial_loss_scale: float = 2 ** 32
    min_loss_scale: float = 1.0
    loss_scale_window: float = 5
    hysteresis: int = 2
    gradient_clipping: float = 1.0

    def __post_init__(self):
        if self.type not in ("adam", "adamw", "sgd", "adam_bf16"):
            raise ValueError(f"unknown optimizer type {self.type}")
        if self.lr_scheduler_type not in ("constant", "linear", "cosine"):
            raise ValueError(f"unknown lr scheduler {self.lr_scheduler_type}")


# --------------------------------------------------------------------------- engines


@dataclass
class FSDPEngineConfig:
    """Sharded data-parallel engine options. ``reshard_after_forward=False``
    keeps a full bf16 replica of the weights on every GPU (180 GB HBM makes this
    the fast default up to ~30B dense parameters); optimizer state and fp32
    master weights are always sharded."""

    wrap_policy: Any = None
    offload_params: bool = False
    memory_efficient_load: bool = False
    per_layer_optim_step: bool = False
    optim_step_prefetch_layers: int = 1
    shard_vision_across_sp: bool = False
    reshard_after_forward: bool = False
    overlap_grad_reduce: bool = True


@dataclass
class ArchonFP8Config:
    mode: str = "disabled"  # disabled | blockwise
    exclude_modules: list[str] = field(default_factory=lambda: ["output"])
    include_experts: bool = False
    use_triton: bool = False


@dataclass
class ArchonEngineConfig:
    attn_type: str = "varlen"
    enable_compile: bool = False
    ac_mode: str = "selective"  # none | full | selective | memory_budget
    selective_ac_option: str = "op"
    ac_memory_budget: float = 0.5
    pp_schedule: str = "Interleaved1F1B"
    pp_layers_per_stage: int | None = None
    pp_first_stage_less_layers: int = 1
    pp_last_stage_less_layers: int = 1
    reshard_after_forward_policy: str = "default"
    fp8_config: ArchonFP8Config = field(default_factory=ArchonFP8Config)
    moe_router_dtype: str = "fp32"
    offload_params: bool = False


@dataclass
class DistributedDataParallelConfig:
    grad_reduce_in_fp32: bool = True
    overlap_grad_reduce: bool = True
    overlap_param_gather: bool = False
    align_param_gather: bool = False
    use_distributed_optimizer: bool = True
    check_for_nan_in_grad: bool = False
    bucket_size: int | None = None
    average_in_collective: bool = False
    fp8_param_gather: bool = False


@dataclass
class FP8EngineConfig:
    mode: str | None = None  # None | e4m3 | hybrid
    recipe: str = "blockwise"  # delayed | tensorwise | mxfp8 | blockwise
    param: bool = False
    margin: int = 0
    amax_history_len: int = 1
    amax_compute_algo: str = "most_recent"
    wgrad: bool = True
    dot_product_attention: bool = False
    multi_head_attention: bool = False
    direct_convert: bool = True


@dataclass
class MegatronEngineConfig:
    wrap_with_ddp: bool = True
    use_torch_fsdp2: bool = False
    use_custom_fsdp: bool = False
    ddp: DistributedDataParallelConfig = field(default_factory=DistributedDataParallelConfig)
    virtual_pipeline_parallel_size: int = 1
    overlap_param_gather_with_optimizer_step: bool = False
    use_precision_aware_optimizer: bool = False
    main_grads_dtype: str = "float32"
    main_params_dtype: str = "float32"
    exp_avg_dtype: str = "float32"
    exp_avg_sq_dtype: str = "float32"
    async_save: bool = False
    use_checkpoint_opt_param_scheduler: bool = True
    use_deterministic_algorithms: bool = False
    recompute_granularity: str | None = "full"
    recompute_method: str | None = "uniform"
    recompute_num_layers: int | None = 1
    distribute_saved_activations: bool | None = None
    recompute_modules: list[str] | None = None
    moe_router_dtype: str | None = "fp32"
    moe_shared_expert_overlap: bool = False
    moe_enable_deepep: bool = False
    moe_token_dispatcher_type: str = "alltoall"
    moe_permute_fusion: bool = False
    fp8_config: FP8EngineConfig | None = None
    # context parallelism of the Megatron-style engine: "allgather" / "p2p" = zig-zag chunks with gathered K/V,
    # "a2a" = Ulysses head exchange (what the FSDP-style engine always uses)
    cp_comm_type: str = "allgather"
    use_sequence_parallel: bool = True
    bridge_type: str = "native"


class SchedulingStrategyType:
    separation = "separation"
    colocation = "colocation"


@dataclass
class SchedulingStrategy:
    type: str = "separation"
    target: str | None = None
    fork: bool = True


@dataclass
class SchedulingSpec:
    cpu: int = 8
    gpu: int = 0
    mem: int = 32
    port_count: int = 2
    image: str = ""
    task_type: str = "worker"
    env_vars: dict[str, str] = field(default_factory=dict)
    cmd: str | None = None
    srun_additional_args: str = "--unbuffered --mpi=pmi2 -K --chdir $PWD"
    additional_bash_cmds: list[str] | None = None
    container_type: str = "apptainer"
    mount: str = "/storage:/storage"
    nodelist: str | None = None
    exclude: str | None = None
    ray_placement_strategy: str = "shared"


def _default_worker_spec() -> tuple[SchedulingSpec, ...]:
    return (SchedulingSpec(cmd="python -m areal_b200.infra.rpc.rpc_server"),)


@dataclass
class TrainEngineConfig:
    experiment_name: str = MISSING
    trial_name: str = MISSING
    path: str = ""
    attn_impl: str = "b200_varlen"
    use_kernels: bool = True
    init_from_scratch: bool = False
    is_critic: bool = False
    temperature: float = 1.0
    mb_spec: MicroBatchSpec = field(default_factory=MicroBatchSpec)
    pad_to_maximum: bool = False
    disable_dropout: bool = False
    gradient_checkpointing: bool = False
    dtype: str = "bfloat16"
    grad_reduce_dtype: str = "float32"
    optimizer: OptimizerConfig | None = None
    weight_update_mode: str = "xccl"
    fsdp: FSDPEngineConfig = field(default_factory=FSDPEngineConfig)
    archon: ArchonEngineConfig = field(default_factory=ArchonEngineConfig)
    megatron: MegatronEngineConfig = field(default_factory=MegatronEngineConfig)
    offload: bool = False
    use_lora: bool = False
    lora_rank: int = 32
    lora_alpha: int = 16
    target_modules: list[str] = field(default_factory=list)
    peft_type: str = "lora"
    enable_tree_training: bool = False
    scheduling_spec: tuple[SchedulingSpec, ...] = field(default_factory=_default_worker_spec)
    backend: str = MISSING
    _version: str = "v1"
    admin_api_key: str = "areal-admin-key"
    log_level: str = "warning"
    request_timeout: float = 3600.0
    setup_timeout: float = 3600.0
    scheduling_strategy: SchedulingStrategy = field(default_factory=SchedulingStrategy)
    # model shape for init_from_scratch without a checkpoint directory (preset name or inline dict)
    model_preset: str | None = None
    model_overrides: dict[str, Any] = field(default_factory=dict)


@dataclass
class RejectionSamplingConfig:
    """Filtering of stale samples by the gap between the proximal and the
    behaviour policy."""

    level: str = "token"  # token | sequence
    action: str = "mask"  # mask | clamp
    metric: str = "ratio"  # ratio | kl_k1 | kl_k2 | kl_k3
    agg: str = "mean"  # sum | mean | max (sequence level)
    upper: float = 5.0
    lower: float | None = None

    def __post_init__(self):
        if self.level not in ("token", "sequence"):
            raise ValueError(f"level must be token|sequence, got {self.level}")
        if self.action not in ("mask", "clamp"):
            raise ValueError(f"action must be mask|clamp, got {self.action}")
        if self.metric not in ("ratio", "kl_k1", "kl_k2", "kl_k3"):
            raise ValueError(f"unknown metric {self.metric}")
        if self.agg not in ("sum", "mean", "max"):
            raise ValueError(f"unknown agg {self.agg}")
        if self.lower is not None and self.lower > self.upper:
            raise ValueError("lower must not exceed upper")
        if self.action == "clamp" and self.metric != "ratio":
            raise ValueError("clamp is only defined for the ratio metric")


@dataclass
class PPOActorConfig(TrainEngineConfig):
    ppo_n_minibatches: int = 4
    eps_clip: float = 0.2
    eps_clip_higher: float | None = None
    c_clip: float | None = None
    m2_threshold: float | None = None
    reward_norm: NormConfig | None = None
    reward_scaling: float = 1.0
    reward_bias: float = 0.0
    reward_clip: float = 20.0
    overlong_reward_penalty: bool = False
    overlong_tokens: int | None = None
    overlong_penalty_factor: float | None = None
    mask_no_eos_with_zero: bool = False
    discount: float = 1.0
    gae_lambda: float = 1.0
    adv_norm: NormConfig | None = None
    kl_ctl: float = 0.1
    kl_estimator: str = "k1"
    use_sapo_loss: bool = False
    sapo_tau_pos: float = 1.0
    sapo_tau_neg: float = 1.05
    recompute_logprob: bool = False
    use_decoupled_loss: bool = False
    rejection_sampling: RejectionSamplingConfig | None = None
    importance_sampling_level: str = "token"
    prox_logp_method: str = PROX_LOGP_METHOD_RECOMPUTE
    log_agent_stats: bool = False
    log_agent_stats_keys: list[str] = field(default_factory=list)
    max_new_tokens: int = 1024

    def __post_init__(self):
        if self.prox_logp_method not in PROX_LOGP_METHODS:
            raise ValueError(f"prox_logp_method must be one of {PROX_LOGP_METHODS}")
        if self.use_sapo_loss and self.use_decoupled_loss:
            raise ValueError("SAPO is incompatible with the decoupled loss")
        if self.importance_sampling_level not in ("token", "sequence"):
            raise ValueError("importance_sampling_level must be token|sequence")
        if self.c_clip is not None and self.c_clip <= 1.0:
            raise ValueError("c_clip must be > 1")

    def should_compute_prox_logp(self) -> bool:
        """Whether an extra forward pass for the proximal policy is needed."""
        if self.use_decoupled_loss:
            return self.prox_logp_method in (PROX_LOGP_METHOD_RECOMPUTE, PROX_LOGP_METHOD_METRICS)
        return self.recompute_logprob


@dataclass
class PPOCriticConfig(TrainEngineConfig):
    ppo_n_minibatches: int = 4
    eps_clip: float = 0.5
    mask_no_eos_with_zero: bool = False


@dataclass
class DPOEngineConfig(TrainEngineConfig):
    beta: float = 0.1
    loss_type: str = "sigmoid"  # sigmoid | ipo


@dataclass
class TeacherConfig(PPOActorConfig):
    rl_loss_weight: float = 1.0
    distill_loss_weight: float = 0.005


# --------------------------------------------------------------------------- rollout


@dataclass
class NativeRolloutConfig:
    """Options of this framework's own rollout engine (paged KV, continuous batching)."""

    model_path: str = ""
    model_preset: str | None = None
    model_overrides: dict[str, Any] = field(default_factory=dict)
    dtype: str = "bfloat16"
    kv_block_size: int = 16
    mem_fraction_static: float = 0.85
    max_num_seqs: int = 512
    max_num_batched_tokens: int = 16384
    context_length: int = 32768
    cuda_graph: bool = True
    cuda_graph_batch_sizes: list[int] = field(
        default_factory=lambda: [1, 2, 4, 8, 16, 32, 48, 64, 96, 128, 160, 192, 224, 256, 320, 384, 448, 512, 640, 768, 1024])
    seed: int = 1
    host: str = "127.0.0.1"
    port: int = 0
    kv_cache_dtype: str = "auto"
    num_kv_blocks: int | None = None
    # samples of one prompt prefill once and read the same (read-only) prompt pages
    prompt_sharing: bool = True
    # graph-captured decode steps draw the next token inside the LM-head GEMM (Gumbel-max in the epilogue); off:
    # logits are written out and the stand-alone sampler runs (always the case with top-k / top-p requests)
    fused_sampling: bool = True


@dataclass
class vLLMConfig:
    model: str = ""
    seed: int = 1
    skip_tokenizer_init: bool = False
    enforce_eager: bool = False
    dtype: str = "bfloat16"
    distributed_executor_backend: str = "mp"
    max_num_seqs: int = 256
    block_size: int = 16
    swap_space: int = 4
    cpu_offload_gb: float = 0
    disable_sliding_window: bool = True
    max_model_len: int | None = 32768
    no_enable_chunked_prefill: bool = False
    no_enable_prefix_caching: bool = True
    gpu_memory_utilization: float = 0.9
    worker_extension_cls: str = "areal_b200.engine.rollout_server.WorkerExtension"
    enable_sleep_mode: bool = False
    uvicorn_log_level: str = "warning"
    enable_lora: bool = False
    max_lora_rank: int = 16
    max_loras: int = 1

    @staticmethod
    def build_args(vllm_config: "vLLMConfig", tp_size: int, pp_size: int, host: str, port: int,
                   dist_init_addr: str | None = None) -> dict[str, Any]:
        d = {k: v for k, v in asdict(vllm_config).items()}
        d.update(tensor_parallel_size=tp_size, pipeline_parallel_size=pp_size, host=host, port=port)
        return d

    @staticmethod
    def build_cmd(vllm_config: "vLLMConfig", tp_size: int, pp_size: int, host: str, port: int,
                  dist_init_addr: str | None = None) -> list[str]:
        args = vLLMConfig.build_args(vllm_config, tp_size, pp_size, host, port, dist_init_addr)
        return ["python", "-m", "areal_b200.engine.rollout_server"] + _args_to_flags(args)


@dataclass
class SGLangConfig:
    model_path: str = ""
    random_seed: int = 1
    skip_tokenizer_init: bool = False
    disable_cuda_graph: bool = False
    disable_radix_cache: bool = True
    disable_cuda_graph_padding: bool = False
    enable_nccl_nvls: bool = False
    disable_outlines_disk_cache: bool = False
    disable_custom_all_reduce: bool = False
    disable_overlap_schedule: bool = False
    enable_mixed_chunk: bool = False
    enable_dp_attention: bool = False
    enable_ep_moe: bool = False
    enable_torch_compile: bool = False
    torch_compile_max_bs: int = 32
    cuda_graph_max_bs: int | None = None
    cuda_graph_bs: list[int] | None = None
    torchao_config: str = ""
    enable_nan_detection: bool = False
    enable_p2p_check: bool = False
    triton_attention_reduce_in_fp32: bool = False
    triton_attention_num_kv_splits: int = 8
    num_continuous_decode_steps: int = 1
    enable_memory_saver: bool = False
    allow_auto_truncate: bool = False
    attention_backend: str | None = "fa3"
    enable_multimodal: bool = False
    sampling_backend: str | None = None
    context_length: int | None = 32768
    mem_fraction_static: float | None = 0.9
    max_running_requests: int | None = None
    chunked_prefill_size: int | None = -1
    max_prefill_tokens: int = 32768
    schedule_policy: str = "lpm"
    schedule_conservativeness: float = 1.0
    cpu_offload_gb: int = 0
    dtype: str = "bfloat16"
    kv_cache_dtype: str = "auto"
    dp_size: int = 1
    ep_size: int = 1
    enable_lora: bool | None = None
    max_lora_rank: int | None = None
    lora_target_modules: list[str] | None = None
    lora_paths: list[str] | None = None
    max_loaded_loras: int = 1
    max_loras_per_batch: int = 1
    lora_backend: str = "triton"
    log_level: str = "warning"
    log_level_http: str | None = "warning"
    log_requests: bool = False
    log_requests_level: int = 0
    show_time_cost: bool = False
    enable_metrics: bool = True
    decode_log_interval: int = 1
    enable_return_routed_experts: bool = False

    @staticmethod
    def build_args(sglang_config: "SGLangConfig", tp_size: int, base_gpu_id: int, host: str | None = None,
                   port: int | None = None, dist_init_addr: str | None = None, n_nodes: int = 1,
                   node_rank: int = 0, pp_size: int = 1) -> dict[str, Any]:
        d = {k: v for k, v in asdict(sglang_config).items()}
        d.update(tp_size=tp_size, pp_size=pp_size, base_gpu_id=base_gpu_id, nnodes=n_nodes,
                 node_rank=node_rank, dist_init_addr=dist_init_addr, host=host, port=port)
        return d

    @staticmethod
    def build_cmd(sglang_config: "SGLangConfig", tp_size: int, base_gpu_id: int, host: str | None = None,
                  port: int | None = None, dist_init_addr: str | None = None, n_nodes: int = 1,
                  node_rank: int = 0, pp_size: int = 1) -> list[str]:
        args = SGLangConfig.build_args(sglang_config, tp_size, base_gpu_id, host, port,
                                       dist_init_addr, n_nodes, node_rank, pp_size)
        return ["python", "-m", "areal_b200.engine.rollout_server"] + _args_to_flags(args)


def _args_to_flags(args: dict[str, Any]) -> list[str]:
    flags: list[str] = []
    for k, v in args.items():
        if v is None or v is False or v == "":
            continue
        name = "--" + k.replace("_", "-")
        if v is True:
            flags.append(name)
        elif isinstance(v, (list, tuple)):
            flags.extend([name, *map(str, v)])
        else:
            flags.extend([name, str(v)])
    return flags


@dataclass
class AgentConfig:
    agent_cls_path: str = ""
    admin_api_key: str = "areal-admin-key"
    scheduling_spec: tuple[SchedulingSpec, ...] = field(
        default_factory=lambda: (SchedulingSpec(gpu=0, cmd="python -m areal_b200.infra.rpc.rpc_server"),))
    mode: str = "inline"  # inline | subproc | online
    tool_call_parser: str = "qwen"
    reasoning_parser: str = "qwen3"
    chat_template_type: str = "hf"
    engine_max_tokens: int | None = None
    turn_discount: float = 1.0
    export_style: str = "individual"  # individual | concat
    subproc_max_workers: int = 4
    session_timeout_seconds: int = 3600
    set_reward_finish_timeout: float = 0.0

    def __post_init__(self):
        if self.mode not in ("inline", "subproc", "online"):
            raise ValueError(f"agent mode must be inline|subproc|online, got {self.mode}")
        if self.export_style not in ("individual", "concat"):
            raise ValueError(f"export_style must be individual|concat, got {self.export_style}")


@dataclass
class InferenceEngineConfig:
    experiment_name: str | None = None
    trial_name: str | None = None
    fileroot: str | None = None
    max_concurrent_rollouts: int | None = None
    queue_size: int | None = None
    consumer_batch_size: int = 1
    max_head_offpolicyness: int = 0
    enable_rollout_tracing: bool = False
    check_trajectory_format: bool = False
    tokenizer_path: str = ""
    dump_to_file: bool = False
    setup_timeout: float = 300.0
    request_timeout: float = 3600
    request_retries: int = 3
    pause_grace_period: float = 0.0
    scheduling_spec: tuple[SchedulingSpec, ...] = field(default_factory=_default_worker_spec)
    backend: str = MISSING
    scheduling_strategy: SchedulingStrategy = field(default_factory=SchedulingStrategy)
    use_lora: bool = False
    agent: AgentConfig = field(default_factory=lambda: AgentConfig(
        agent_cls_path="areal_b200.openai.proxy.online_agent.OnlineAgent"))
    return_routed_experts: bool = False
    _version: str = "v1"
    model: str = "default"
    routing_strategy: str = "round_robin"
    poll_interval: float = 5.0
    admin_api_key: str = "areal-admin-key"
    api_url: str | None = None
    provider_api_key: str | None = None
    native: NativeRolloutConfig = field(default_factory=NativeRolloutConfig)


# --------------------------------------------------------------------------- services


@dataclass
class _Timer:
    experiment_name: str = MISSING
    trial_name: str = MISSING
    fileroot: str = MISSING
    freq_epochs: int | None = None
    freq_steps: int | None = None
    freq_secs: int | None = None


@dataclass
class EvaluatorConfig(_Timer):
    eval_before_train: bool = False


@dataclass
class SaverConfig(_Timer):
    mode: str = "auto"  # auto | sync | async


@dataclass
class RecoverConfig(_Timer):
    mode: str = "disabled"  # disabled | auto | fault | resume | on | off
    retries: int = 3
    no_save_optim: bool = False
    no_load_optim: bool = False


@dataclass
class WandBConfig:
    mode: str = "disabled"
    wandb_base_url: str = ""
    wandb_api_key: str = ""
    entity: str | None = None
    project: str | None = None
    name: str | None = None
    job_type: str | None = None
    group: str | None = None
    notes: str | None = None
    tags: list[str] | None = None
    config: dict | None = None
    id_suffix: str | None = "train"


@dataclass
class SwanlabConfig:
    project: str | None = None
    name: str | None = None
    config: dict | None = None
    logdir: str | None = None
    mode: str | None = "disabled"
    api_key: str | None = None


@dataclass
class TensorBoardConfig:
    path: str | None = None


@dataclass
class TrackioConfig:
    mode: str = "disabled"
    project: str | None = None
    name: str | None = None
    space_id: str | None = None


@dataclass
class StatsLoggerConfig:
    experiment_name: str = MISSING
    trial_name: str = MISSING
    fileroot: str = MISSING
    wandb: WandBConfig = field(default_factory=WandBConfig)
    swanlab: SwanlabConfig = field(default_factory=SwanlabConfig)
    tensorboard: TensorBoardConfig = field(default_factory=TensorBoardConfig)
    trackio: TrackioConfig = field(default_factory=TrackioConfig)


@dataclass
class SessionTracerConfig:
    enabled: bool = False
    flush_threshold: int = 256


@dataclass
class MemoryProfilerConfig:
    profile_steps: list[int] = field(default_factory=lambda: [0, 1])
    max_entries: int = 100000


@dataclass
class PerfTracerConfig:
    experiment_name: str = MISSING
    trial_name: str = MISSING
    fileroot: str = MISSING
    enabled: bool = False
    save_interval: int = 1
    profile_steps: list[int] | None = None
    session_tracer: SessionTracerConfig | None = None


@dataclass
class NameResolveConfig:
    type: str = "nfs"  # memory | nfs | etcd3 | ray
    nfs_record_root: str = "/tmp/areal/name_resolve"
    etcd3_addr: str = "localhost:2379"
    ray_actor_name: str = "ray_kv_store"


@dataclass
class ClusterSpecConfig:
    name_resolve: NameResolveConfig = field(default_factory=NameResolveConfig)
    cluster_name: str = "local"
    fileroot: str = "/tmp/areal/"
    n_nodes: int = 32
    n_gpus_per_node: int = 8


@dataclass
class SchedulerConfig:
    type: str | None = None  # None (SPMD) | local | ray | slurm
    endpoint: str = "http://localhost:8081"
    deploy_mode: str = "separation"
    functioncall_service_domain: str = "http://localhost:8080"
    reward_functioncall_config: dict = field(default_factory=dict)
    reward_model_path: str = ""
    reward_model_service_url: str = "http://localhost:30000/classify"


@dataclass
class _DatasetConfig:
    split: str = "train"
    path: str = MISSING
    type: str = MISSING
    batch_size: int = 1
    shuffle: bool = True
    pin_memory: bool = False
    num_workers: int = 0
    num_dataset_workers: int = 1
    drop_last: bool = True
    max_length: int | None = None
    dataset_kwargs: dict[str, Any] = field(default_factory=dict)
    scheduling_spec: SchedulingSpec | None = field(
        default_factory=lambda: SchedulingSpec(cpu=1, gpu=0, mem=10,
                                               cmd="python -m areal_b200.infra.rpc.rpc_server"))
    setup_timeout: float = 120.0


@dataclass
class TrainDatasetConfig(_DatasetConfig):
    pass


@dataclass
class ValidDatasetConfig(_DatasetConfig):
    split: str = "test"
    shuffle: bool = False
    drop_last: bool = False


@dataclass
class BaseExperimentConfig:
    experiment_name: str = MISSING
    trial_name: str = MISSING
    cluster: ClusterSpecConfig = field(default_factory=ClusterSpecConfig)
    allocation_mode: str = ""
    seed: int = 1
    enable_offload: bool = False
    total_train_epochs: int = 1
    total_train_steps: int | None = None
    total_train_n_seqs: int | None = None
    tokenizer_path: str = ""
    train_dataset: TrainDatasetConfig = field(default_factory=TrainDatasetConfig)
    valid_dataset: ValidDatasetConfig | None = None
    saver: SaverConfig = field(default_factory=SaverConfig)
    evaluator: EvaluatorConfig = field(default_factory=EvaluatorConfig)
    stats_logger: StatsLoggerConfig = field(default_factory=StatsLoggerConfig)
    perf_tracer: PerfTracerConfig | None = None
    memory_profiler: MemoryProfilerConfig | None = None
    recover: RecoverConfig = field(default_factory=RecoverConfig)
    sglang: SGLangConfig = field(default_factory=SGLangConfig)
    vllm: vLLMConfig = field(default_factory=vLLMConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)


@dataclass
class SFTConfig(BaseExperimentConfig):
    actor: TrainEngineConfig = field(default_factory=TrainEngineConfig)
    # legacy alias used by some YAML files
    model: TrainEngineConfig | None = None


@dataclass
class RWConfig(BaseExperimentConfig):
    actor: TrainEngineConfig = field(default_factory=lambda: TrainEngineConfig(is_critic=True))
    model: TrainEngineConfig | None = None


@dataclass
class DPOConfig(BaseExperimentConfig):
    actor: DPOEngineConfig = field(default_factory=DPOEngineConfig)
    ref: DPOEngineConfig | None = None


@dataclass
class PPOConfig(BaseExperimentConfig):
    gconfig: GenerationHyperparameters = field(default_factory=GenerationHyperparameters)
    eval_gconfig: GenerationHyperparameters | None = None
    rollout: InferenceEngineConfig = field(default_factory=InferenceEngineConfig)
    actor: PPOActorConfig = field(default_factory=PPOActorConfig)
    ref: PPOActorConfig | None = None
    critic: PPOCriticConfig | None = None
    teacher: TeacherConfig | None = None
    dynamic_bs: bool = False


@dataclass
class GRPOConfig(PPOConfig):
    pass


# --------------------------------------------------------------------------- loader

ConfigT = TypeVar("ConfigT")
_INTERP = re.compile(r"\$\{([^}]+)\}")


def _parse_scalar(text: str) -> Any:
    try:
        return yaml.safe_load(text)
    except yaml.YAMLError:
        return text


def _set_dotted(tree: dict, dotted: str, value: Any) -> None:
    keys = dotted.split(".")
    cur = tree
    for k in keys[:-1]:
        nxt = cur.get(k)
        if not isinstance(nxt, dict):
            nxt = {}
            cur[k] = nxt
        cur = nxt
    cur[keys[-1]] = value


def _get_dotted(tree: dict, dotted: str) -> Any:
    cur: Any = tree
    for k in dotted.split("."):
        if isinstance(cur, dict) and k in cur:
            cur = cur[k]
        else:
            raise KeyError(dotted)
    return cur


def _resolve(tree: dict) -> dict:
    """Resolves ``${a.b}`` references against the root (nested references allowed)."""

    def res(v, depth=0):
        if depth > 16:
            raise ValueError("interpolation cycle")
        if isinstance(v, dict):
            return {k: res(x, depth) for k, x in v.items()}
        if isinstance(v, list):
            return [res(x, depth) for x in v]
        if isinstance(v, str):
            m = _INTERP.fullmatch(v.strip())
            if m:
                key = m.group(1).strip()
                if key.startswith("oc.env:") or key.startswith("env:"):
                    name, _, dflt = key.split(":", 1)[1].partition(",")
                    return os.environ.get(name.strip(), dflt.strip() or None)
                return res(_get_dotted(tree, key), depth + 1)
            if _INTERP.search(v):
                return _INTERP.sub(lambda mm: str(res("${" + mm.group(1) + "}", depth + 1)), v)
        return v

    return res(tree)


def _strip_optional(tp):
    origin = typing.get_origin(tp)
    if origin in (typing.Union, types.UnionType):
        args = [a for a in typing.get_args(tp) if a is not type(None)]
        return (args[0] if len(args) == 1 else tp), True
    return tp, False


def _build(tp, value, path: str):
    tp, optional = _strip_optional(tp)
    if value is None:
        return None
    origin = typing.get_origin(tp)
    if is_dataclass(tp):
        if is_dataclass(value):
            return value
        if not isinstance(value, dict):
            raise TypeError(f"{path}: expected a mapping for {tp.__name__}, got {type(value).__name__}")
        hints = typing.get_type_hints(tp)
        known = {f.name: f for f in fields(tp)}
        unknown = set(value) - set(known)
        if unknown:
            raise KeyError(f"{path or tp.__name__}: unknown config keys {sorted(unknown)}")
        kwargs = {}
        for name, v in value.items():
            if not known[name].init:
                continue
            kwargs[name] = _build(hints[name], v, f"{path}.{name}" if path else name)
        return tp(**kwargs)
    if origin in (list, tuple):
        args = typing.get_args(tp)
        elem = args[0] if args else Any
        seq = [_build(elem, v, f"{path}[{i}]") for i, v in enumerate(value)] \
            if isinstance(value, (list, tuple)) else [_build(elem, value, path)]
        return tuple(seq) if origin is tuple else seq
    if origin is dict or tp is dict:
        return dict(value)
    if tp is float and isinstance(value, (int, str)) and not isinstance(value, bool):
        return float(value)
    if tp is int and isinstance(value, float) and value.is_integer():
        return int(value)
    if tp is int and isinstance(value, str):
        return int(float(value))
    if tp is bool and isinstance(value, str):
        return value.lower() in ("1", "true", "yes", "on")
    if tp is str and not isinstance(value, str):
        return str(value)
    return value


def to_structured_cfg(cfg: dict, config_cls: type[ConfigT]) -> ConfigT:
    return _build(config_cls, _resolve(cfg), "")


def _propagate_names(cfg) -> None:
    """Copies experiment/trial names and fileroot into sub-configs that left them unset."""
    exp = getattr(cfg, "experiment_name", MISSING)
    trial = getattr(cfg, "trial_name", MISSING)
    root = cfg.cluster.fileroot if hasattr(cfg, "cluster") else MISSING
    for f in fields(cfg):
        sub = getattr(cfg, f.name)
        if is_dataclass(sub):
            for attr, val in (("experiment_name", exp), ("trial_name", trial), ("fileroot", root)):
                if hasattr(sub, attr) and getattr(sub, attr) in (MISSING, None):
                    setattr(sub, attr, val)
            if hasattr(sub, "session_tracer") or hasattr(sub, "wandb"):
                pass


def parse_cli_args(argv: list[str]):
    parser = argparse.ArgumentParser()
    parser.add_argument("--config", required=True, help="path to the YAML experiment config")
    args, overrides = parser.parse_known_args(argv)
    path = Path(args.config).absolute()
    if not path.exists():
        raise FileNotFoundError(path)
    tree = yaml.safe_load(path.read_text()) or {}
    for ov in overrides:
        if "=" not in ov:
            raise ValueError(f"override {ov!r} is not of the form key=value")
        k, v = ov.split("=", 1)
        k = k.lstrip("+")
        _set_dotted(tree, k, _parse_scalar(v))
    return tree, path


def load_expr_config(argv: list[str], config_cls: type[ConfigT]) -> tuple[ConfigT, str]:
    """``--config file.yaml a.b=c ...`` → ``(typed config, config file path)``."""
    tree, path = parse_cli_args(argv)
    cfg = to_structured_cfg(tree, config_cls)
    _propagate_names(cfg)
    from ..utils import name_resolve

    if hasattr(cfg, "cluster"):
        name_resolve.reconfigure(cfg.cluster.name_resolve)
    return cfg, str(path)


def config_to_dict(cfg) -> dict:
    return asdict(cfg)


def conf_as_dict(cfg) -> dict:
    """A configuration (dataclass tree or plain mapping) as nested dicts."""
    return dict(cfg) if isinstance(cfg, dict) else asdict(cfg)


def get_py_cmd(module: str, args: dict[str, Any]) -> list[str]:
    """``python3 -m module --flag value ...`` from a mapping: ``None`` / ``False`` / empty values are left out,
    ``True`` becomes a bare flag, lists become one flag followed by their items; underscores turn into dashes."""
    cmd = ["python3", "-m", module]
    for k, v in args.items():
        if v is None or v is False or v == "" or (isinstance(v, (list, tuple)) and not v):
            continue
        cmd.append("--" + k.replace("_", "-"))
        if v is True:
            continue
        cmd.extend(str(x) for x in v) if isinstance(v, (list, tuple)) else cmd.append(str(v))
    return cmd


def get_log_path(cfg) -> str:
    root = cfg.cluster.fileroot if hasattr(cfg, "cluster") else cfg.fileroot
    path = os.path.join(root, "logs", getpass.getuser(), cfg.experiment_name, cfg.trial_name)
    os.makedirs(path, exist_ok=True)
    return path


def save_config(cfg, log_dir: str) -> str:
    os.makedirs(log_dir, exist_ok=True)
    out = os.path.join(log_dir, "config.yaml")
    with open(out, "w") as f:
        yaml.safe_dump(json.loads(json.dumps(asdict(cfg), default=str)), f, sort_keys=False)
    return out
