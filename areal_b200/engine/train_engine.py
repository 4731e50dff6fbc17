"""The B200 train engine: packed varlen forward/backward on this library's
kernels, flat ZeRO-style sharded optimizer with NVLink peer reduce-scatter /
all-gather, fused LM-head logprobs, weight push to the rollout engine,
HF-safetensors and sharded checkpoints.

It implements the ``TrainEngine`` contract that the reference's FSDP / Archon
engines implement (areal/engine/fsdp_engine.py:219-2256;
areal/experimental/engine/archon_engine.py:147-1533): ``train_batch``,
``forward_batch``, ``eval_batch``, ``update_weights``, ``save`` / ``load``,
``offload`` / ``onload``. It runs on CUDA (bf16, hand-written kernels) and on CPU
(fp32 PyTorch reference ops + gloo), the latter being the functional oracle.
"""

from __future__ import annotations

import dataclasses
import os
import time
from typing import Any, Callable

import torch
import torch.distributed as dist

from ..api.alloc_mode import ModelAllocation, ParallelStrategy
from ..api.cli_args import OptimizerConfig, TrainEngineConfig
from ..api.engine_api import InferenceEngine, TrainEngine
from ..api.io_struct import FinetuneSpec, ParamSpec, SaveLoadMeta, WeightUpdateMeta
from ..models.config import PRESETS, ModelConfig
from ..models.qwen import QwenModel, build_model
from ..ops.attention import VarlenMeta
from ..ops.lm_head import lm_head_logprobs
from ..utils import logging, stats_tracker
from ..utils.data import MicroBatchList, amend_position_ids, split_padded_tensor_dict_into_mb_list
from .flat_params import FlatParams, ShardedAdamW

logger = logging.getLogger("TrainEngine")

DIST_TIMEOUT_S = 7200


def resolve_model_config(cfg: TrainEngineConfig) -> ModelConfig:
    if cfg.path and os.path.exists(os.path.join(cfg.path, "config.json")):
        mc = ModelConfig.from_hf_config(cfg.path)
    elif cfg.model_preset:
        mc = dataclasses.replace(PRESETS[cfg.model_preset])
    else:
        raise ValueError("TrainEngineConfig needs `path` (HF directory) or `model_preset`")
    for k, v in (cfg.model_overrides or {}).items():
        setattr(mc, k, v)
    if cfg.is_critic:
        mc.is_critic = True
        mc.tie_word_embeddings = False
    # fp8 training: the Megatron-style (`megatron.fp8_config.mode`) and the Archon-style
    # (`archon.fp8_config.mode: blockwise`) switches both select the block-scaled e4m3 forward GEMMs
    meg = getattr(cfg.megatron, "fp8_config", None)
    arch = getattr(cfg.archon, "fp8_config", None)
    if (meg is not None and meg.mode) or (arch is not None and getattr(arch, "mode", "disabled") == "blockwise"):
        if meg is not None and meg.mode and meg.recipe not in ("blockwise", "mxfp8"):
            raise ValueError(f"fp8 recipe {meg.recipe!r} is not supported: this engine implements block-wise scaling")
        mc.fp8 = True
    if getattr(cfg, "use_lora", False):
        if cfg.peft_type != "lora":
            raise ValueError(f"peft_type {cfg.peft_type!r} is not supported (only 'lora')")
        mc.lora_rank, mc.lora_alpha = int(cfg.lora_rank), float(cfg.lora_alpha)
        mc.lora_targets = list(cfg.target_modules or [])
    return mc


class _PinnedStager:
    """Host→device staging through two reusable pinned arenas instead of one ``cudaHostAlloc`` per tensor."""

    def __init__(self, device, nbytes: int = 8 << 20):
        self.device = device
        self.arenas = [torch.empty(nbytes, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
        self.events = [None, None]
        self.cur, self.off = 0, 0

    def begin(self):
        self.cur ^= 1
        ev = self.events[self.cur]
        if ev is not None:
            ev.synchronize()  # the copies issued from this arena two micro-batches ago
        self.off = 0

    def to_device(self, t: torch.Tensor) -> torch.Tensor:
        t = t.contiguous()
        n = t.numel() * t.element_size()
        start = (self.off + 255) // 256 * 256
        if start + n > self.arenas[self.cur].numel():
            if self.off == 0:  # nothing issued from this arena yet: grow it
                self.arenas[self.cur] = torch.empty(max(2 * self.arenas[self.cur].numel(), start + n), dtype=torch.uint8,
                                                    pin_memory=True)
            else:  # rare: fall back to a one-off pinned copy rather than disturb copies in flight
                return t.pin_memory().to(self.device, non_blocking=True)
        view = self.arenas[self.cur][start:start + n].view(t.dtype).view(t.shape)
        view.copy_(t)
        self.off = start + n
        return view.to(self.device, non_blocking=True)

    def end(self):
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self.events[self.cur] = ev


def _resolve_fn(fn):
    """A loss or weight function given by import path (a controller or a service sent it from another process)."""
    if isinstance(fn, str):
        from ..utils.dynamic_import import import_from_string

        return import_from_string(fn)
    return fn


class B200TrainEngine(TrainEngine):
    def __init__(self, config: TrainEngineConfig):
        self.config = config
        self.optimizer_config: OptimizerConfig | None = config.optimizer
        self.model: QwenModel | None = None
        self.flat: FlatParams | None = None
        self.optimizer: ShardedAdamW | None = None
        self.model_config: ModelConfig | None = None
        self._version = 0
        self._initialized = False
        self._own_pg = False
        self.rank = 0
        self.world_size = 1
        self._dp_group = None
        self._cpu_group = None
        self.parallel = ParallelStrategy()
        self.rollout_engine: InferenceEngine | None = None
        self.weight_update_meta: WeightUpdateMeta | None = None
        self._rollout_tables = None
        self._offloaded: dict[str, torch.Tensor] | None = None
        self.is_critic = config.is_critic
        # bytes moved host→device (pinned staging) and device→host, for the benchmark report
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # ------------------------------------------------------------ process groups
    def create_process_group(self, parallel_strategy: ParallelStrategy | None = None,
                             ranks: list[int] | None = None, backend: str | None = None, groups=None):
        """Builds the data-parallel group over ``ranks`` (default: the whole world).
        ``torch.distributed`` is initialised from the torchrun environment if needed.
        ``groups=(dp_group, cpu_group)`` reuses groups another engine already created (group
        creation is collective over the whole world, so engines that only some ranks own must
        not create their own)."""
        use_cuda = torch.cuda.is_available() and self.config.dtype != "float32_cpu"
        if not dist.is_initialized() and "RANK" in os.environ:
            backend = backend or ("nccl" if use_cuda else "gloo")
            if use_cuda:
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
            import datetime

            dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=DIST_TIMEOUT_S))
            self._own_pg = True
        if parallel_strategy is None and self.config.backend not in (None, "", "???"):
            parallel_strategy = ModelAllocation.from_str(self.config.backend).parallel
        self.parallel = parallel_strategy or ParallelStrategy()
        self.mesh = None
        self.pctx = None
        ps = self.parallel
        model_parallel = ps.tp_size * ps.cp_size * ps.pp_size * ps.ep_size * getattr(ps, "etp_size", 1) > 1
        if model_parallel:
            assert dist.is_initialized(), "tensor / sequence / pipeline parallelism needs torch.distributed"
            from ..parallel.context import build_mesh

            self.rank = dist.get_rank()
            world = dist.get_world_size()
            ranks = list(range(world)) if ranks is None else list(ranks)
            self.train_ranks = ranks
            dp = len(ranks) // (ps.tp_size * ps.cp_size * ps.pp_size)
            # context_parallel_size is Ulysses sequence parallelism for this engine family
            self.mesh = build_mesh(ranks, dp=dp, sp=ps.cp_size, tp=ps.tp_size, pp=ps.pp_size, ep=ps.ep_size,
                                   etp=getattr(ps, "etp_size", 1))
            self.pctx = self.mesh.ctx
            if ps.pp_size > 1:
                # schedule and virtual stages: `archon.pp_schedule` for the Archon-style backend, 1F1B otherwise;
                # `megatron.virtual_pipeline_parallel_size` chunks per rank select the interleaved order
                from ..parallel.pipeline import canonical_schedule, placement_of

                family = (self.config.backend or "").split(":")[0]
                vpp = max(int(getattr(self.config.megatron, "virtual_pipeline_parallel_size", 1) or 1), 1)
                name = os.environ.get("AREAL_B200_PP_SCHEDULE") or (
                    self.config.archon.pp_schedule if family == "archon" else ("Interleaved1F1B" if vpp > 1 else "1F1B"))
                self._pp_placement = placement_of(name)
                if self._pp_placement == "v":
                    vpp = 2  # the V-shaped placement is defined for two chunks per rank
                    self.pctx.extras["pp_placement"] = "v"
                self._pp_schedule = canonical_schedule(name, vpp)
                self._vpp = vpp
                if self._pp_schedule == "zero_bubble":
                    from ..ops import wgrad_defer

                    wgrad_defer.arm()  # linear layers get the backward that can park its weight-gradient GEMM
                self.pctx.extras["vpp"] = vpp
            if ps.cp_size > 1 and self.config.backend.split(":")[0] == "megatron" and \
                    getattr(self.config.megatron, "cp_comm_type", "a2a") in ("allgather", "p2p"):
                self.pctx.extras["cp_mode"] = "zigzag"
            # parameters are sharded (ZeRO) over dp x sp: those ranks hold the same weights
            self._dp_group = self.mesh.shard_group
            self._cpu_group = self.mesh.cpu_shard_group
            self._data_group = self.mesh.dp_group
            self.world_size = self.mesh.shard_size
            self.dp_rank = self.mesh.shard_rank
            self._data_rank, self._data_size = self.mesh.dp_rank, self.mesh.dp_size
            self._mp_group = self.mesh.mp_group
            # checkpoint coordination spans every train rank (tp / pp / ep peers write their own tensors); the
            # second group serves writes on a background thread
            self._all_cpu_group = dist.new_group(ranks, backend="gloo")
            self._async_ckpt_group = dist.new_group(ranks, backend="gloo")
        elif dist.is_initialized():
            self.rank = dist.get_rank()
            world = dist.get_world_size()
            ranks = list(range(world)) if ranks is None else list(ranks)
            self.train_ranks = ranks
            if groups is not None:
                self._dp_group, self._cpu_group = groups
                self._async_ckpt_group = None
            else:
                self._async_ckpt_group = dist.new_group(ranks, backend="gloo")
                if ranks == list(range(world)):
                    self._dp_group = dist.group.WORLD
                else:
                    self._dp_group = dist.new_group(ranks)
                self._cpu_group = dist.new_group(ranks, backend="gloo") if dist.get_backend() != "gloo" \
                    else self._dp_group
            self._all_cpu_group = self._cpu_group
            self.world_size = len(ranks)
            self.dp_rank = ranks.index(self.rank) if self.rank in ranks else -1
        else:
            self._all_cpu_group = self._async_ckpt_group = None
            self.train_ranks = [0]
            self.world_size, self.dp_rank = 1, 0
        self.device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")

    @property
    def data_parallel_group(self):
        """Ranks that receive DIFFERENT data. (Parameters are sharded over a possibly larger
        group that also spans the Ulysses ranks: ``self._dp_group``.)"""
        return self._data_group if self.mesh is not None else self._dp_group

    @property
    def data_parallel_rank(self) -> int:
        return self._data_rank if self.mesh is not None else self.dp_rank

    @property
    def data_parallel_world_size(self) -> int:
        return self._data_size if self.mesh is not None else self.world_size

    @property
    def context_and_model_parallel_group(self):
        """Ranks that must be fed the same batch (tp x sp x pp of one data-parallel replica)."""
        return getattr(self, "_mp_group", None)

    @property
    def cpu_group(self):
        return self._cpu_group

    def is_data_parallel_head(self) -> bool:
        if self.mesh is None:
            return True
        c = self.pctx
        return c.tp_rank == 0 and c.sp_rank == 0 and self.mesh.pp_rank == 0

    def current_data_parallel_head(self) -> int:
        if self.mesh is None:
            return self.rank
        ps = self.parallel
        i = self.train_ranks.index(self.rank)
        mp = ps.tp_size * ps.cp_size
        return self.train_ranks[(i % (mp * self._data_size)) // mp * mp]

    # ----------------------------------------------------------------- init
    def initialize(self, addr: str | None = None, ft_spec: FinetuneSpec | None = None, *args, **kwargs):
        if not hasattr(self, "device"):
            self.create_process_group()
        cfg = self.config
        if getattr(cfg.megatron, "use_deterministic_algorithms", False):
            from ..utils.determinism import set_deterministic_algorithms

            set_deterministic_algorithms(True)
        self.model_config = resolve_model_config(cfg)
        dtype = torch.float32 if self.device.type == "cpu" else getattr(torch, cfg.dtype)
        t0 = time.perf_counter()
        seed = kwargs.get("seed", 0)
        pctx = self.pctx
        if pctx is not None:
            mc = self.model_config
            widest = max(mc.q_size + 2 * mc.kv_size, 2 * mc.intermediate_size) // max(pctx.tp_size, 1)
            max_tok = int(self.config.mb_spec.max_tokens_per_mb or 32768) + 1024
            pctx.enable_fused(max_tok, mc.hidden_size, widest, self.device)
        self.model = build_model(self.model_config, dtype=dtype, device=self.device,
                                 seed=seed if (cfg.init_from_scratch or not cfg.path) else None, pctx=pctx)
        if cfg.path and not cfg.init_from_scratch:
            from ..utils.hf_io import load_hf_weights

            load_hf_weights(self.model, cfg.path)
        family = (cfg.backend or "").split(":")[0]
        if family == "archon" and cfg.archon.ac_mode != "none" and self.optimizer_config is not None:
            # the Archon-style options: none | full | selective (layer- or op-level) | memory_budget
            from ..models.activation_checkpoint import apply_activation_checkpointing

            apply_activation_checkpointing(self.model, cfg.archon.ac_mode, cfg.archon.selective_ac_option,
                                           cfg.archon.ac_memory_budget)
        elif cfg.gradient_checkpointing:
            self.model.checkpoint_every = 1
        if self.model_config.is_vl:
            if cfg.enable_tree_training or (pctx is not None and pctx.extras.get("cp_mode") == "zigzag"):
                raise NotImplementedError("vision-language models train packed, under data / Ulysses parallelism")
            self.model.shard_vision = bool(cfg.fsdp.shard_vision_across_sp)
        tp = pctx.tp_size if pctx is not None else 1
        rep_first = None
        if tp > 1:
            from ..parallel.tensor_parallel import is_tp_replicated

            rep_first = is_tp_replicated
        # experts that differ between ranks (expert parallelism and / or expert tensor parallelism) live apart
        ep = (pctx.ep_size * pctx.etp_size) if pctx is not None else 1
        is_expert = (lambda n: n.endswith(("mlp.gate_up", "mlp.down")) and ".mlp." in n and
                     dict(self.model.named_parameters())[n].dim() == 3)
        self.flat_base = None
        if self.model_config.lora_rank:
            # adapters train, the base model is frozen: the base weights keep a flat buffer of their own
            # (no gradients, no optimizer state; it is what the rollout engine and checkpoints read) and
            # `self.flat` — the buffer the optimizer shards — holds the adapters only
            from ..models.lora import is_lora_param

            assert ep == 1, "LoRA training does not combine with expert parallelism"
            for n, p_ in self.model.named_parameters():
                if not is_lora_param(n):
                    p_.requires_grad_(False)
            self.flat_base = FlatParams(self.model, self._dp_group, with_grads=False, replicated_first=rep_first,
                                        select=lambda n: not is_lora_param(n))
            self.flat = FlatParams(self.model, self._dp_group, with_grads=self.optimizer_config is not None,
                                   replicated_first=rep_first, select=is_lora_param)
        else:
            self.flat = FlatParams(self.model, self._dp_group, with_grads=self.optimizer_config is not None,
                                   replicated_first=rep_first,
                                   select=(lambda n: not is_expert(n)) if ep > 1 else None)
        self.flat_experts = None
        if ep > 1:
            # expert weights differ across the ep group: they are reduced only over the ranks that hold
            # the same experts, and live in a flat buffer (and optimizer) of their own
            edp = self.mesh.edp_group if self.mesh.edp_size > 1 else "local"
            self.flat_experts = FlatParams(self.model, edp, with_grads=self.optimizer_config is not None,
                                           select=is_expert)
            if self.device.type == "cuda" and pctx.ep_size > 1:
                from ..parallel.expert_parallel import EPGroupState

                mc = self.model_config
                cap = int((self.config.mb_spec.max_tokens_per_mb or 32768) * mc.num_experts_per_tok * 2)
                pctx.extras["ep_state"] = EPGroupState(pctx.ep_group, mc.num_experts, mc.hidden_size, cap, self.device)
        if self.optimizer_config is not None:
            total = ft_spec.total_train_steps if ft_spec is not None else 1
            fs = cfg.fsdp
            self.optimizer = ShardedAdamW(self.flat, self.optimizer_config, total_steps=total,
                                          tp_group=pctx.tp_group if tp > 1 else None,
                                          host_state=bool(getattr(fs, "per_layer_optim_step", False)),
                                          prefetch=int(getattr(fs, "optim_step_prefetch_layers", 1)))
            if self.flat_experts is not None:
                self.optimizer.partner = ShardedAdamW(self.flat_experts, self.optimizer_config, total_steps=total)
                # the ranks whose expert parameters differ from this rank's: the expert-parallel group times the
                # expert-tensor-parallel group
                self.optimizer.partner_group = pctx.extras.get("emp_group", pctx.ep_group)
            balanced = [l.mlp for l in getattr(self.model, "layers", []) if getattr(l.mlp, "load_acc", None) is not None]
            if balanced:
                # aux-loss-free balancing: one bias update per optimizer step, from the token counts of every rank
                # that holds the layer (data / sequence / tensor parallel peers routed other tokens)
                groups = []
                if self.mesh is not None:
                    if self.mesh.shard_size > 1:
                        groups.append(self.mesh.shard_group)
                    if pctx.tp_size > 1:
                        groups.append(pctx.tp_group)
                elif dist.is_initialized() and self.world_size > 1:
                    groups.append(self._dp_group)
                for m in balanced:
                    m.defer_bias_update = True
                self.optimizer.pre_step_hooks.append(lambda: [m.update_expert_bias(groups) for m in balanced])
            if pctx is not None and pctx.pp_size > 1:
                self.optimizer.norm_groups.append(pctx.pp_group)
                if self.optimizer.partner is not None:
                    # the experts of other pipeline stages count in the global gradient norm as well
                    self.optimizer.partner.norm_groups.append(pctx.pp_group)
                if self.model_config.tie_word_embeddings and not self.is_critic and self.model.embed is not None \
                        and self.model.embed.requires_grad and pctx.last_stage_rank != 0:
                    # (frozen under LoRA: nothing to sum; V-shaped placement: embedding and head share one copy)
                    self.optimizer.pre_step_hooks.append(self._sum_tied_embedding_grads)
                    if not self.model.first_stage:
                        # both copies apply the summed gradient; the first stage's copy counts in the norm
                        off = next(o for n_, p_, o, _ in self.flat.entries if p_ is self.model.embed)
                        self.optimizer.norm_exclude.append((off, self.model.embed.numel()))
        self.ft_spec = ft_spec
        self._initialized = True
        logger.info(f"engine initialised: {self.model_config.num_params() / 1e9:.2f}B params, "
                    f"dp={self.world_size}, device={self.device}, {time.perf_counter() - t0:.1f}s")
        return self

    def _sum_tied_embedding_grads(self):
        """First and last pipeline stage each hold a copy of the tied embedding / head matrix; both
        apply the sum of the two gradients so the copies stay identical."""
        dist.all_reduce(self.model.embed.main_grad, group=self.pctx.pp_tie_group)

    def destroy(self):
        self.model = None
        self.optimizer = None
        if self.device.type == "cuda" if hasattr(self, "device") else False:
            torch.cuda.synchronize(self.device)
        for name in ("flat", "flat_base", "flat_experts"):
            f = getattr(self, name, None)
            if f is not None:
                f.close()
            setattr(self, name, None)
        if self._own_pg and dist.is_initialized():
            dist.destroy_process_group()

    def train(self, mode: bool = True):
        if self.model is not None:
            self.model.train(mode)
        return self

    def set_version(self, version: int):
        self._version = version

    def get_version(self) -> int:
        return self._version

    # ----------------------------------------------------------- micro-batches
    def _prepare_mb_list(self, input_: dict[str, Any]) -> MicroBatchList:
        input_ = {k: v for k, v in input_.items()}
        if "attention_mask" not in input_ and "cu_seqlens" in input_:
            from ..utils.data import unpack_to_padded

            input_ = unpack_to_padded(input_)
        spec = self.config.mb_spec
        if self.pctx is not None and self.pctx.pp_size > 1:
            # a pipeline fills only with enough micro-batches (2 x stages for the 1F1B family); the interleaved
            # order moves them through the chunks in groups of `stages`
            from ..api.cli_args import MicroBatchSpec
            from ..parallel.pipeline import min_micro_batches

            pp = self.pctx.pp_size
            need = min_micro_batches(self._pp_schedule, pp, self._vpp)
            n_seq = int(input_["attention_mask"].shape[0]) // max(spec.granularity, 1)
            need = min(need, max(n_seq // pp * pp, pp) if self._vpp > 1 else max(n_seq, 1))
            div = spec.n_mbs_divisor * pp if (self._vpp > 1 and spec.n_mbs_divisor % pp) else spec.n_mbs_divisor
            spec = MicroBatchSpec.new(spec, n_mbs=max(spec.n_mbs or 1, need), n_mbs_divisor=div)
        mb_list = split_padded_tensor_dict_into_mb_list(
            input_, spec,
            group=self._cpu_group if (dist.is_initialized() and self.world_size > 1) else None)
        return mb_list

    def _mb_to_device(self, mb: dict[str, Any]) -> tuple[dict[str, Any], VarlenMeta]:
        cu_cpu = mb["cu_seqlens"].cpu()
        meta = VarlenMeta(cu_cpu.tolist(), self.device)
        out = {}
        cuda = self.device.type == "cuda"
        if cuda:
            # one pinned arena per micro-batch in flight (two alternate): the tensors of a micro-batch are laid
            # out in it and copied asynchronously; an arena is reused once the copies issued from it have finished
            if getattr(self, "_stager", None) is None:
                self._stager = _PinnedStager(self.device)
            self._stager.begin()
        for k, v in mb.items():
            if torch.is_tensor(v):
                if cuda and not v.is_cuda:
                    self.h2d_bytes += v.numel() * v.element_size()
                    out[k] = self._stager.to_device(v)
                else:
                    out[k] = v.to(self.device, non_blocking=True)
            else:
                out[k] = v
        if cuda:
            self._stager.end()
        out = amend_position_ids(out)
        out["cu_seqlens"] = meta.cu_seqlens
        return out, meta

    def _forward_mb(self, mb: dict[str, Any], meta: VarlenMeta, need_entropy: bool = True, stage_input=None,
                    chunk: int | None = None):
        """Returns ``(logprobs [T], entropy [T])`` in next-token form, or values for a critic. A
        pipeline stage other than the last returns ``((x, res), None)`` instead."""
        ids = mb["input_ids"]
        pctx = self.pctx
        if pctx is None or (pctx.seq_shards == 1 and pctx.pp_size == 1):
            if self.config.enable_tree_training and not self.is_critic:
                return self._forward_mb_tree(mb, meta)
            hidden = self.model(ids, mb["position_ids"], meta, **self._vision_inputs(mb))
            if self.is_critic:
                return self.model.values(hidden), None
            labels = torch.roll(ids, shifts=-1, dims=0)
            logp, ent = lm_head_logprobs(hidden, self.model.output_weight(), labels,
                                         self.config.temperature)
            return logp, ent
        return self._forward_mb_parallel(mb, meta, stage_input, chunk)

    def _vision_inputs(self, mb: dict[str, Any]) -> dict[str, Any]:
        """Pixel rows and patch grids of the micro-batch's images, concatenated in sequence order.
        ``multi_modal_input`` holds one dict per sequence (what the image processor returned for it, empty for
        a text-only sample), as areal/workflow/vision_rlvr.py of the reference stores it in a trajectory."""
        mm = mb.get("multi_modal_input")
        if not mm or not self.model_config.is_vl:
            if mm and any(d and d.get("pixel_values") is not None for d in mm):
                raise NotImplementedError(f"{self.model_config.model_type} is a text-only model: the batch has images")
            return {}
        pix = [torch.as_tensor(d["pixel_values"]) for d in mm if d and d.get("pixel_values") is not None]
        grid = [torch.as_tensor(d["image_grid_thw"]).view(-1, 3) for d in mm
                if d and d.get("pixel_values") is not None]
        if not pix:
            return {}
        pv = torch.cat(pix, 0)
        if self.device.type == "cuda" and not pv.is_cuda:
            pv = pv.pin_memory()
            self.h2d_bytes += pv.numel() * pv.element_size()
        return {"pixel_values": pv.to(self.device, non_blocking=True), "image_grid_thw": torch.cat(grid, 0)}

    def _forward_mb_tree(self, mb: dict[str, Any], meta: VarlenMeta):
        """Tree training: the micro-batch's sequences are merged into prefix tries, every distinct
        token (trie node) runs through the trunk once under the ancestor mask, and the LM head runs
        once per trie edge: the log-probability of node ``c``'s token given the path to its parent.
        Position ``i`` of a sequence then reads the value of the node at position ``i + 1``; the last
        position of every sequence has no label and yields zeros (the loss mask excludes it, as it
        excludes the rolled-in label of the packed layout). Same outputs as the packed path within
        floating-point reordering. Reference: areal/models/tree_attn/{tree.py:273,functional.py}."""
        from ..ops.tree_attn import TreeMeta, build_packed_tree, tree_attention

        ids = mb["input_ids"]
        cu = meta.cu_cpu.tolist()
        flat_ids = ids.tolist()
        tree = build_packed_tree([flat_ids[a:b] for a, b in zip(cu[:-1], cu[1:])])
        dev = ids.device
        tmeta = TreeMeta(tree, dev) if dev.type == "cuda" else None
        hidden = self.model(tree.tokens.to(dev), tree.position_ids.to(dev), meta,
                            attn_fn=lambda q, k, v, _m: tree_attention(q, k, v, tree, tmeta))
        parent = tree.parent.clamp(min=0).to(dev)  # roots: a dummy row, never read back
        logp_n, ent_n = lm_head_logprobs(hidden.index_select(0, parent), self.model.output_weight(),
                                         tree.tokens.to(dev), self.config.temperature)
        nxt, has = [], []
        for path in tree.seq_nodes:
            nxt.extend(path[1:] + [0])
            has.extend([1.0] * (len(path) - 1) + [0.0])
        nxt = torch.tensor(nxt, dtype=torch.long, device=dev)
        has = torch.tensor(has, dtype=logp_n.dtype, device=dev)
        stats_tracker.scalar(**{"tree/node_ratio": tree.num_nodes / max(len(flat_ids), 1)})
        return logp_n.index_select(0, nxt) * has, ent_n.index_select(0, nxt) * has

    def _forward_mb_parallel(self, mb: dict[str, Any], meta: VarlenMeta, stage_input=None, chunk: int | None = None):
        """Tensor- and/or Ulysses-parallel forward. Every rank of the model-parallel group holds the
        same micro-batch; the packed tokens are padded to a multiple of the shard count, each
        Ulysses rank takes its contiguous slice (tensor parallelism shards further inside the
        model) and the per-token outputs are re-assembled so the loss sees the whole micro-batch."""
        from ..parallel.tensor_parallel import gather_seq_replicated

        pctx = self.pctx
        if pctx.extras.get("cp_mode") == "zigzag" and pctx.sp_size > 1:
            return self._forward_mb_zigzag(mb, meta, stage_input)
        ids, pos = mb["input_ids"], mb["position_ids"]
        T = ids.shape[0]
        align = pctx.seq_shards * (128 if ids.is_cuda else 1)
        Tp = (T + align - 1) // align * align
        labels = torch.roll(ids, shifts=-1, dims=0)
        if Tp != T:
            pad = Tp - T
            ids = torch.cat([ids, ids.new_zeros(pad)])
            pos = torch.cat([pos, torch.arange(pad, device=pos.device, dtype=pos.dtype)])
            labels = torch.cat([labels, labels.new_zeros(pad)])
            meta = VarlenMeta(list(meta.cu_cpu.tolist()) + [Tp], self.device)  # the padding is one more sequence
        S, r = pctx.sp_size, pctx.sp_rank
        n = Tp // S
        sl = slice(r * n, (r + 1) * n)
        if S > 1:
            pctx.extras["full_positions"] = pos.to(torch.int32)  # for RoPE after the fused sequence→head exchange
        if self.model_config.is_vl:
            # image features and the per-token rotary table are built for the whole micro-batch, then sliced
            hidden = self.model(ids, pos, meta, seq_slice=sl, stage_input=stage_input, **self._vision_inputs(mb))
        else:
            kw = {} if chunk is None else {"chunk": chunk}
            hidden = self.model(ids[sl], pos[sl], meta, stage_input=stage_input, **kw)  # [n, H]: this Ulysses shard
        if pctx.pp_size > 1 and (not pctx.is_last_stage or (chunk is not None and chunk != self.model.vpp - 1)):
            return hidden, None  # (x, res) for the next (virtual) stage
        if self.is_critic:
            out, ent = self.model.values(hidden), None
        else:
            tp = pctx.tp_size
            vloc = self.model.output_weight().shape[0]
            out, ent = lm_head_logprobs(hidden, self.model.output_weight(), labels[sl], self.config.temperature,
                                        tp_group=pctx.tp_group if tp > 1 else None,
                                        vocab_start=pctx.tp_rank * vloc if tp > 1 else 0,
                                        tp_fused=pctx.tp_fused if tp > 1 else None)
        if S > 1:
            out = gather_seq_replicated(out, pctx.sp_fused)
            ent = gather_seq_replicated(ent, pctx.sp_fused) if ent is not None else None
        return out[:T], (ent[:T] if ent is not None else None)

    def _forward_mb_zigzag(self, mb: dict[str, Any], meta: VarlenMeta, stage_input=None):
        """Context-parallel forward with zig-zag chunks: every sequence is padded to a multiple of
        ``2 * cp * 128`` tokens and cut into ``2 * cp`` chunks, rank ``r`` holds chunks ``r`` and
        ``2cp - 1 - r`` (balanced causal work); attention gathers K/V over the group, everything else
        is token-local. Unlike the head exchange this does not limit ``cp`` by the number of kv heads.
        Outputs are gathered back and un-padded, so the loss sees the micro-batch in packed order.
        Reference: areal/engine/megatron_utils/packed_context_parallel.py:14-185."""
        from ..parallel.context_parallel import CPLayout, cp_attention
        from ..parallel.tensor_parallel import gather_seq_replicated

        pctx = self.pctx
        assert pctx.tp_size == 1 and pctx.pp_size == 1, "zig-zag context parallelism combines with data parallelism"
        ids, pos = mb["input_ids"], mb["position_ids"]
        cu = meta.cu_cpu.tolist()
        seqlens = [b - a for a, b in zip(cu[:-1], cu[1:])]
        lay = CPLayout(seqlens, pctx.sp_size, pctx.sp_rank, device=ids.device)
        labels = torch.roll(ids, shifts=-1, dims=0)
        ids_l, pos_l, lab_l = (lay.split(lay.pad_packed(t)) for t in (ids, pos, labels))
        hidden = self.model(ids_l, pos_l, meta,
                            attn_fn=lambda q, k, v, _m: cp_attention(q, k, v, lay, pctx.sp_group))
        if self.is_critic:
            out, ent = self.model.values(hidden), None
        else:
            out, ent = lm_head_logprobs(hidden, self.model.output_weight(), lab_l, self.config.temperature)
        keep = torch.cat([torch.arange(int(lay.full_cu[s]), int(lay.full_cu[s]) + L) for s, L in enumerate(seqlens)])
        index = lay.gather_to_seq.to(out.device)[keep.to(out.device)]  # packed token -> row of the rank-major gather

        def back(t):
            return gather_seq_replicated(t, pctx.sp_fused).index_select(0, index)

        return back(out), (back(ent) if ent is not None else None)

    # ---------------------------------------------------------------- pipeline
    def _stage_shapes(self, T: int):
        """Shape of the activations that travel between stages for a micro-batch of ``T`` tokens."""
        pctx = self.pctx
        align = pctx.seq_shards * (128 if self.device.type == "cuda" else 1)
        Tp = (T + align - 1) // align * align
        return (Tp // pctx.seq_shards, self.model_config.hidden_size)

    def _pipeline_forward_backward(self, mbs, scales, loss_fn, forward_only: bool = False, collect=None):
        """Runs the micro-batches through this rank's pipeline chunks following the configured schedule
        (``parallel/pipeline.py``: GPipe, 1F1B, interleaved 1F1B over virtual stages) with asynchronous
        point-to-point transfers. Every stage of a replica holds the same micro-batch list, so activation
        shapes are known without a handshake. Returns the scaled losses (last stage) or zeros (other stages;
        the caller broadcasts statistics).
        Reference: areal/engine/megatron_engine.py:882 (mcore schedules) and
        areal/experimental/models/archon/pipeline_parallel.py:48-82,349-494."""
        from ..parallel.pipeline import PipelineRunner

        pctx = self.pctx
        V = self._vpp
        dtype = next(self.model.parameters()).dtype
        runner = PipelineRunner(pctx.extras["pp_links"], pctx.pp_rank, pctx.pp_size, V,
                                "gpipe" if forward_only and V == 1 else self._pp_schedule, dtype, self.device,
                                placement=getattr(self, "_pp_placement", "interleaved"))
        staged: dict[int, tuple] = {}

        def on_device(i):
            if i not in staged:
                staged[i] = self._mb_to_device(mbs[i])
            return staged[i]

        def forward(i, c, stage_in):
            dev_mb, meta = on_device(i)
            out, ent = self._forward_mb(dev_mb, meta, stage_input=stage_in, chunk=c if V > 1 else None)
            return out if ent is None and isinstance(out, tuple) else (out, ent)

        def finish(i, outs):
            out, ent = outs
            dev_mb, meta = on_device(i)
            if collect is not None:
                collect(i, out, ent, dev_mb, meta)
                return None
            loss = loss_fn(out, dev_mb) if self.is_critic else loss_fn(out, ent, dev_mb)
            return loss * scales[i]

        results = runner.run(len(mbs), forward, finish, lambda i: self._stage_shapes(int(mbs[i]["cu_seqlens"][-1])),
                             forward_only=forward_only)
        zero = torch.zeros((), device=self.device)
        return [results[i] if (i in results and results[i] is not None) else zero for i in range(len(mbs))]

    # ------------------------------------------------------------------ train
    def optimizer_zero_grad(self):
        self.flat.zero_grad()

    def optimizer_step(self) -> dict[str, float]:
        return self.optimizer.step()

    def lr_scheduler_step(self):
        self.optimizer.sched_step += 1
        if self.optimizer.partner is not None:
            # the expert-weight optimizer follows the same schedule
            self.optimizer.partner.sched_step = self.optimizer.sched_step

    def train_batch(self, input_: dict[str, Any], loss_fn: Callable, loss_weight_fn: Callable) -> dict[str, float]:
        """One optimizer step over ``input_`` (this rank's share of the batch), split into
        micro-batches. ``loss_fn(logprobs, entropy, mb) -> scalar`` (``loss_fn(values, mb)``
        for critics); ``loss_weight_fn(mb) -> weight`` (e.g. the number of loss tokens).
        The total loss is the weight-averaged loss over all micro-batches of all ranks."""
        assert self.optimizer is not None, "engine was created without an optimizer"
        loss_fn, loss_weight_fn = _resolve_fn(loss_fn), _resolve_fn(loss_weight_fn)
        self.model.train()
        mb_list = self._prepare_mb_list(input_)
        weights = [float(loss_weight_fn(mb)) for mb in mb_list.mbs]
        total = torch.tensor([sum(weights)], dtype=torch.float64)
        if dist.is_initialized() and self.world_size > 1:
            dist.all_reduce(total, group=self._cpu_group)
        total_w = float(total)
        if self.pctx is not None:
            total_w /= self.pctx.sp_size  # Ulysses ranks of one replica counted the same micro-batches
        assert total_w > 0, "total loss weight must be positive"
        losses = []
        if self.pctx is not None and self.pctx.pp_size > 1:
            losses = self._pipeline_forward_backward(mb_list.mbs, [w / total_w for w in weights], loss_fn)
        else:
            for mb, w in zip(mb_list.mbs, weights):
                dev_mb, meta = self._mb_to_device(mb)
                out, ent = self._forward_mb(dev_mb, meta)
                loss = loss_fn(out, dev_mb) if self.is_critic else loss_fn(out, ent, dev_mb)
                (loss * (w / total_w)).backward()
                losses.append(loss.detach() * (w / total_w))
        stats = self.optimizer.step()
        self.lr_scheduler_step()
        stats["loss"] = float(torch.stack(losses).sum()) if losses else 0.0
        if self.pctx is not None and self.pctx.pp_size > 1:
            t = torch.tensor([stats["loss"]], dtype=torch.float32, device=self.device)
            dist.all_reduce(t, group=self.pctx.pp_group)  # only the last stage holds a non-zero loss
            stats["loss"] = float(t)
        self.d2h_bytes += 12  # grad-norm, skip flag, loss
        stats["n_mbs"] = float(len(mb_list))
        return stats

    @torch.no_grad()
    def eval_batch(self, input_: dict[str, Any], loss_fn: Callable, loss_weight_fn: Callable):
        loss_fn, loss_weight_fn = _resolve_fn(loss_fn), _resolve_fn(loss_weight_fn)
        self.model.eval()
        mb_list = self._prepare_mb_list(input_)
        weights = [float(loss_weight_fn(mb)) for mb in mb_list.mbs]
        acc = torch.zeros(2, dtype=torch.float64)
        for mb, w in zip(mb_list.mbs, weights):
            if w <= 0:
                continue  # nothing to score (padding samples of a batch that did not divide over the ranks)
            dev_mb, meta = self._mb_to_device(mb)
            out, ent = self._forward_mb(dev_mb, meta)
            loss = loss_fn(out, dev_mb) if self.is_critic else loss_fn(out, ent, dev_mb)
            acc[0] += float(loss) * w
            acc[1] += w
        if dist.is_initialized() and self.world_size > 1:
            dist.all_reduce(acc, group=self._cpu_group)
        return float(acc[0] / acc[1].clamp(min=1e-12))

    @torch.no_grad()
    def forward_batch(self, input_: dict[str, Any], output_seqlens=None, aggregate_fn=None,
                      return_entropy: bool = False):
        """Per-token outputs for every sample, padded back to ``[B, L]`` in input order:
        next-token logprobs (position t holds log π(x[t+1] | x[≤t])) or values for a critic."""
        self.model.eval()
        mb_list = self._prepare_mb_list(input_)
        B, L = input_["attention_mask"].shape
        result = torch.zeros(B, L, dtype=torch.float32)
        ent_result = torch.zeros(B, L, dtype=torch.float32) if return_entropy else None
        row = 0
        pp = self.pctx is not None and self.pctx.pp_size > 1
        staged = {}
        if pp:
            self._pipeline_forward_backward(mb_list.mbs, [1.0] * len(mb_list.mbs), None, forward_only=True,
                                            collect=lambda i, o, e, m, mt: staged.__setitem__(i, (o, e, mt)))
        # the micro-batches run back to back on the device; their outputs cross to the host in ONE copy at the
        # end (a read per micro-batch would put a host synchronisation between every two forwards)
        outs, ents, metas = [], [], []
        for i_mb, mb in enumerate(mb_list.mbs):
            if pp:
                if not self.pctx.is_last_stage:
                    continue
                out, ent, meta = staged[i_mb]
            else:
                dev_mb, meta = self._mb_to_device(mb)
                out, ent = self._forward_mb(dev_mb, meta)
            outs.append(out.float())
            ents.append(ent.float() if (ent is not None and return_entropy) else None)
            metas.append(meta)
        if outs:
            flat = torch.cat(outs)
            self.d2h_bytes += flat.numel() * 4
            flat = flat.cpu()
            eflat = torch.cat(ents).cpu() if (return_entropy and all(e is not None for e in ents)) else None
            base = 0
            for out, meta in zip(outs, metas):
                cu = meta.cu_cpu
                for i in range(len(cu) - 1):
                    src = mb_list.forward_indices[row]
                    a, b = base + int(cu[i]), base + int(cu[i + 1])
                    result[src, :b - a] = flat[a:b]
                    if eflat is not None:
                        ent_result[src, :b - a] = eflat[a:b]
                    if not self.is_critic and b > a:
                        # a sequence's last position has no next token: what the packed computation put there
                        # belongs to its neighbour in the micro-batch, so it is cleared
                        result[src, b - a - 1] = 0.0
                        if eflat is not None:
                            ent_result[src, b - a - 1] = 0.0
                    row += 1
                base += out.shape[0]
        if pp:
            # the last stage holds the outputs: hand them to every stage of the replica
            src = dist.get_global_rank(self.pctx.pp_group, self.pctx.last_stage_rank)
            for t in ([result] + ([ent_result] if return_entropy else [])):
                dev = t.to(self.device)
                dist.broadcast(dev, src=src, group=self.pctx.pp_group)
                t.copy_(dev.cpu())
        if return_entropy:
            return result, ent_result
        return result

    def forward_backward_batch(self, mb_list, process_output_fn, forward_only: bool = False):
        outs = []
        for mb in mb_list.mbs:
            dev_mb, meta = self._mb_to_device(mb)
            with torch.set_grad_enabled(not forward_only):
                out, ent = self._forward_mb(dev_mb, meta)
                res = process_output_fn(out, dev_mb)
            if not forward_only and res is not None:
                res.backward()
            outs.append(res.detach() if torch.is_tensor(res) else res)
        return outs

    # -------------------------------------------------------------- weight sync
    def connect_engine(self, engine: InferenceEngine, meta: WeightUpdateMeta):
        """Registers the rollout engine that receives this engine's weights."""
        self.rollout_engine = engine
        self.weight_update_meta = meta
        if meta.type == "p2p" and hasattr(engine, "register_trainer"):
            engine.register_trainer(self)

    def update_weights(self, meta: WeightUpdateMeta | None = None):
        """Pushes the current weights to the connected rollout engine and bumps its version."""
        meta = meta or self.weight_update_meta
        assert self.rollout_engine is not None, "connect_engine() has not been called"
        t0 = time.perf_counter()
        if meta.type == "disk":
            # one directory per version (`weight_update_v{N}`), the previous one removed once the servers
            # have loaded the new weights
            vdir = meta.path
            if meta.version is not None and not os.path.basename(vdir.rstrip("/")).startswith("weight_update_v"):
                vdir = os.path.join(vdir, f"weight_update_v{meta.version}")  # `with_version` already names it
            self.save(SaveLoadMeta(path=vdir, weight_format="hf", with_optim=False))
            if dist.is_initialized() and self.world_size > 1:
                dist.barrier(group=self._cpu_group)
            if self.dp_rank == 0:
                self.rollout_engine.update_weights_from_disk(dataclasses.replace(meta, path=vdir)).result()
                prev = getattr(self, "_last_weight_dir", None)
                if prev and prev != vdir and os.path.isdir(prev):
                    import shutil

                    shutil.rmtree(prev, ignore_errors=True)
                self._last_weight_dir = vdir
        else:
            self.rollout_engine.pause_generation()
            with self._merged_weights():
                self.rollout_engine.receive_weights(self, version=meta.version)
            self.rollout_engine.continue_generation()
        if meta.version is not None:
            self.rollout_engine.set_version(meta.version)
        dt = time.perf_counter() - t0
        stats_tracker.scalar(**{"timeperf/update_weights": dt})
        return dt

    @property
    def weight_flat(self) -> FlatParams:
        """The flat buffer with the model's (base) weights: what rollout engines and checkpoints read."""
        return self.flat_base if self.flat_base is not None else self.flat

    def _merged_weights(self):
        """Context in which the base weights include the adapters' product (no-op without LoRA)."""
        if self.flat_base is None:
            import contextlib

            return contextlib.nullcontext()
        from ..models.lora import merged

        return merged(self.model)

    def get_param_specs(self, weight_chunked_mem_mb: int = 1024) -> list[list[ParamSpec]]:
        limit = weight_chunked_mem_mb * (1 << 20)
        groups, cur, size = [], [], 0
        for name, t in self.model.to_hf():
            spec = ParamSpec(name=name, shape=tuple(t.shape), dtype=str(t.dtype).replace("torch.", ""))
            if cur and size + spec.size > limit:
                groups.append(cur)
                cur, size = [], 0
            cur.append(spec)
            size += spec.size
        if cur:
            groups.append(cur)
        return groups

    # ------------------------------------------------------------- checkpoints
    def save(self, meta: SaveLoadMeta):
        from ..utils.hf_io import save_hf_checkpoint

        os.makedirs(meta.path, exist_ok=True)
        if meta.weight_format == "hf":
            pctx = self.pctx
            pp = pctx.pp_size if pctx is not None else 1
            ep = pctx.ep_size if pctx is not None else 1
            # savers: the first data-parallel replica; under expert parallelism the first expert-parallel block
            # (its ranks hold different experts: the first writes everything it has, the others their experts)
            saver = self.mesh.edp_rank == 0 if ep > 1 else self.dp_rank == 0
            if saver:
                # with LoRA: the merged model (loadable by any HF consumer, and by the rollout engine's
                # disk update) plus the adapter alone in the PEFT layout.
                # One writer per pipeline stage and expert-parallel rank (tensor- / sequence-parallel peers only
                # take part in the gathers); writers use their own files and the first one indexes them afterwards
                if ep > 1:
                    # every expert-parallel rank of the block holds experts nobody else in it has; the ranks that
                    # hold slices of the same experts gather them, and the first of them writes
                    writer = pctx.etp_rank == 0
                else:
                    writer = pctx is None or (pctx.tp_rank == 0 and pctx.sp_rank == 0)
                tag = (f"stage{self.mesh.pp_rank + 1:02d}of{pp:02d}" if pp > 1 else "") + \
                      (f"ep{pctx.ep_rank + 1:02d}of{ep:02d}" if ep > 1 else "")
                keep = (lambda name: ".mlp.experts." in name) if (ep > 1 and pctx.ep_rank > 0) else None
                if pp > 1 or ep > 1:
                    # several writers: the indexing rank clears earlier weight files, then everyone starts
                    from ..utils.hf_io import remove_weight_files

                    if writer and self.mesh.pp_rank == 0 and (ep == 1 or pctx.ep_rank == 0):
                        remove_weight_files(meta.path)
                    if pp > 1:
                        dist.barrier(group=pctx.pp_group)
                    if ep > 1:
                        dist.barrier(group=pctx.ep_group)
                    if pp > 1 and ep > 1:
                        dist.barrier(group=pctx.pp_group)
                with self._merged_weights():
                    save_hf_checkpoint(self.model, self.model_config, meta.path, tokenizer=meta.tokenizer,
                                       processor=meta.processor, write=writer, file_tag=tag, keep=keep)
                if pp > 1 or ep > 1:
                    from ..utils.hf_io import write_hf_index

                    if pp > 1:
                        dist.barrier(group=pctx.pp_group)
                    if ep > 1:
                        dist.barrier(group=pctx.ep_group)
                    if pp > 1 and ep > 1:
                        dist.barrier(group=pctx.pp_group)
                    if writer and self.mesh.pp_rank == 0 and (ep == 1 or pctx.ep_rank == 0):
                        write_hf_index(meta.path)
                if self.flat_base is not None:
                    from ..models.lora import save_adapter

                    save_adapter(self.model, self.model_config, meta.path, base_model_path=self.config.path or "",
                                 gather_group=pctx.pp_group if pp > 1 else None, write=writer)
        elif meta.weight_format == "dcp":
            # torch.distributed.checkpoint: named tensors, every rank writes the part of its own flat shard
            from ..utils.dcp_state import save_engine

            self.wait_for_checkpoint()
            ex = self._ckpt_executor() if (getattr(meta, "async_save", False) and
                                           (self._async_ckpt_group is not None or not dist.is_initialized())) else None
            group = self._async_ckpt_group if ex is not None else self._all_cpu_group
            self._pending_ckpt = save_engine(self, meta.path, with_optim=meta.with_optim, process_group=group,
                                             executor=ex)
            if meta.with_optim:
                self._save_rng(meta.path)
            return
        else:
            raise ValueError(f"unknown weight format {meta.weight_format}")
        if meta.with_optim and self.optimizer is not None:
            # beside HF weights the optimizer state goes into a DCP sub-directory (named, reshardable, one
            # writer per distinct shard under every parallel layout)
            from ..utils.dcp_state import save_engine

            save_engine(self, os.path.join(meta.path, "optimizer"), with_optim=True, with_model=False,
                        process_group=self._all_cpu_group)
            self._save_rng(meta.path)
        if dist.is_initialized() and self.world_size > 1:
            dist.barrier(group=self._cpu_group)

    def _save_rng(self, path: str):
        # a checkpoint with optimizer state is one a run resumes from: it also carries every rank's generators
        from ..utils.rng_state import save_rng_state

        save_rng_state(path, self.rank, self.world_size, self.device)

    def _load_rng(self, path: str):
        from ..utils.rng_state import load_rng_state

        load_rng_state(path, self.rank, self.world_size, self.device)

    def _ckpt_executor(self):
        from concurrent.futures import ThreadPoolExecutor

        if getattr(self, "_ckpt_pool", None) is None:
            self._ckpt_pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="dcp-save")
        return self._ckpt_pool

    def wait_for_checkpoint(self):
        """Blocks until a checkpoint write that runs in the background has finished (and re-raises its error)."""
        f = getattr(self, "_pending_ckpt", None)
        self._pending_ckpt = None
        if f is not None:
            f.result()

    def load(self, meta: SaveLoadMeta):
        from ..utils.hf_io import load_hf_weights

        if meta.weight_format == "hf":
            if self.flat_base is not None and os.path.exists(os.path.join(meta.path, "adapter_model.safetensors")):
                # a LoRA checkpoint: the base model stays as loaded at initialisation, the adapter resumes
                from ..models.lora import load_adapter

                load_adapter(self.model, meta.path)
            else:
                load_hf_weights(self.model, meta.path)
        elif meta.weight_format == "dcp":
            from ..utils.dcp_state import load_engine

            self.wait_for_checkpoint()
            load_engine(self, meta.path, with_optim=meta.with_optim, process_group=self._all_cpu_group)
            if meta.with_optim:
                self._load_rng(meta.path)
            return
        else:
            raise ValueError(f"unknown weight format {meta.weight_format}")
        if self.optimizer is not None:
            self.optimizer.refresh_master()
            if self.optimizer.partner is not None:
                self.optimizer.partner.refresh_master()
            if meta.with_optim:
                from ..utils.dcp_state import load_engine

                load_engine(self, os.path.join(meta.path, "optimizer"), with_optim=True, with_model=False,
                            process_group=self._all_cpu_group)
                self._load_rng(meta.path)

    # ----------------------------------------------------------------- offload
    def offload(self):
        """Moves optimizer state to pinned host memory (colocated train/rollout time-sharing)."""
        if self.optimizer is None or self._offloaded is not None:
            return
        self._offloaded = {}
        names = ("shard_grad",) if self.optimizer.host_state else ("master", "exp_avg", "exp_avg_sq", "shard_grad")
        for name in names:
            t = getattr(self.optimizer, name)
            host = torch.empty(t.shape, dtype=t.dtype, pin_memory=self.device.type == "cuda")
            host.copy_(t)
            self._offloaded[name] = host
            setattr(self.optimizer, name, torch.empty(0, dtype=t.dtype, device=self.device))
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    def onload(self):
        if self._offloaded is None:
            return
        for name, host in self._offloaded.items():
            setattr(self.optimizer, name, host.to(self.device, non_blocking=True))
        self._offloaded = None

    def export_stats(self) -> dict[str, float]:
        return stats_tracker.export_all(reduce_group=self._cpu_group)

