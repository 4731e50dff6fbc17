"""Plain data records exchanged between workflows, engines and controllers.

Field names follow the reference so that workflows written against it keep
working (areal/api/io_struct.py:27-417): requests / responses carry token ids,
per-token logprobs and the *policy version of every generated token*;
``WeightUpdateMeta`` describes how weights travel from trainer to rollout.
"""

from __future__ import annotations

import enum
import os
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Literal

from .cli_args import GenerationHyperparameters


@dataclass
class ModelRequest:
    rid: str = field(default_factory=lambda: str(uuid.uuid4()))
    input_ids: list[int] = field(default_factory=list)
    gconfig: GenerationHyperparameters = field(default_factory=GenerationHyperparameters)
    metadata: dict[str, Any] = field(default_factory=dict)
    tokenizer: Any = None
    image_data: list[Any] | None = None
    processor: Any = None
    vision_msg_vllm: list[Any] | None = None

    def copy(self) -> "ModelRequest":
        return ModelRequest(rid=self.rid, input_ids=list(self.input_ids),
                            gconfig=self.gconfig.new(), metadata=dict(self.metadata),
                            tokenizer=self.tokenizer, image_data=self.image_data,
                            processor=self.processor, vision_msg_vllm=self.vision_msg_vllm)


@dataclass
class ModelResponse:
    input_tokens: list[int] = field(default_factory=list)
    output_tokens: list[int] = field(default_factory=list)
    output_logprobs: list[float] = field(default_factory=list)
    output_versions: list[int] = field(default_factory=list)
    stop_reason: Literal["length", "stop", "tool_calls", "abort", "interrupt"] = "stop"
    routed_experts: Any = None
    tokenizer: Any = None
    input_images: list[Any] = field(default_factory=list)
    latency: float = float("inf")
    ttft: float = float("inf")
    itl: list[float] = field(default_factory=list)

    @property
    def input_len(self) -> int:
        return len(self.input_tokens)

    @property
    def output_len(self) -> int:
        return len(self.output_tokens)


@dataclass
class FinetuneSpec:
    total_train_epochs: int
    dataset_size: int
    train_batch_size: int

    @property
    def total_train_steps(self) -> int:
        return self.total_train_epochs * self.steps_per_epoch

    @property
    def steps_per_epoch(self) -> int:
        return max(self.dataset_size // max(self.train_batch_size, 1), 1)


@dataclass
class ParamSpec:
    name: str
    shape: tuple
    dtype: str

    @property
    def size(self) -> int:
        import numpy as np

        width = {"bfloat16": 2, "float16": 2, "float32": 4, "float8_e4m3fn": 1, "int32": 4}
        return int(np.prod(self.shape)) * width.get(self.dtype.replace("torch.", ""), 2)


class WeightUpdateType(str, enum.Enum):
    disk = "disk"
    xccl = "xccl"  # collective broadcast (NCCL) from trainer rank 0
    p2p = "p2p"    # direct peer-memory writes into the rollout engine's weight buffers
    awex = "awex"


@dataclass
class WeightUpdateMeta:
    type: str = "p2p"
    path: str | None = None
    alloc_mode: Any = None
    nccl_master_address: str = "127.0.0.1"
    nccl_master_port: int = 29500
    nccl_group_name: str = "update_weight_group"
    weight_chunked_mem_mb: int = 1024
    use_lora: bool = False
    lora_name: str = ""
    version: int | None = None

    def with_version(self, version: int) -> "WeightUpdateMeta":
        import copy

        m = copy.copy(self)
        m.version = version
        if m.type == "disk" and m.path is not None:
            base = m.path.rstrip("/")
            if os.path.basename(base).startswith("weight_update_v"):
                base = os.path.dirname(base)
            m.path = os.path.join(base, f"weight_update_v{version}")
        return m

    @classmethod
    def from_disk(cls, experiment_name: str, trial_name: str, file_root: str,
                  name: str = "default", use_lora: bool = False) -> "WeightUpdateMeta":
        from ..utils.saver import Saver

        path = os.path.join(Saver.get_model_save_root(experiment_name, trial_name, file_root, name),
                            "weight_update")
        return cls(type="disk", path=path, use_lora=use_lora)

    @classmethod
    def from_fsdp_xccl(cls, alloc_mode=None, nccl_group_name="update_weight_group",
                       weight_chunked_mem_mb=1024) -> "WeightUpdateMeta":
        return cls(type="xccl", alloc_mode=alloc_mode, nccl_group_name=nccl_group_name,
                   weight_chunked_mem_mb=weight_chunked_mem_mb)

    from_megatron_xccl = from_fsdp_xccl

    @classmethod
    def from_p2p(cls, weight_chunked_mem_mb=1024) -> "WeightUpdateMeta":
        return cls(type="p2p", weight_chunked_mem_mb=weight_chunked_mem_mb)


@dataclass
class HttpRequest:
    endpoint: str
    payload: dict[str, Any]
    method: str = "POST"


@dataclass
class HttpGenerationResult:
    output_tokens: list[int]
    output_logprobs: list[float]
    stop_reason: str
    routed_experts: Any = None


@dataclass
class WeightUpdateRequests:
    requests: list[HttpRequest]


@dataclass
class SaveLoadMeta:
    path: str
    weight_format: str = "hf"  # hf | dcp
    with_optim: bool = False
    tokenizer: Any = None
    processor: Any = None
    base_model_path: str | None = None
    naive_distributed: bool = False
    async_save: bool = False  # dcp: stage to host memory, write on a background thread


@dataclass
class RolloutStat:
    accepted: int = 0
    enqueued: int = 0
    rejected: int = 0
    running: int = 0


@dataclass
class StepInfo:
    epoch: int
    epoch_step: int
    global_step: int
    steps_per_epoch: int

    def next(self) -> "StepInfo":
        last = self.epoch_step == self.steps_per_epoch - 1
        return StepInfo(epoch=self.epoch + int(last), epoch_step=0 if last else self.epoch_step + 1,
                        global_step=self.global_step + 1, steps_per_epoch=self.steps_per_epoch)


@dataclass
class LocalInfServerInfo:
    host: str
    port: int
    process: Any = None


@dataclass
class DeviceRuntimeInfo:
    """Memory of the current device in ``unit`` (GB / MB / KB): allocated and reserved by the caching allocator, used
    on the device by anyone, and its capacity."""
    mem_allocated: float = 0.0
    mem_reserved: float = 0.0
    mem_used: float = 0.0
    mem_total: float = 0.0
    unit: str = "GB"
    ts: float = field(default_factory=time.time)

    @classmethod
    def get_current(cls, unit: str = "GB") -> "DeviceRuntimeInfo":
        import torch

        div = {"GB": 1024 ** 3, "MB": 1024 ** 2, "KB": 1024}.get(unit)
        if div is None:
            raise ValueError(f"unsupported unit {unit!r}: GB, MB or KB")
        if not torch.cuda.is_available():
            return cls(unit=unit)
        free, total = torch.cuda.mem_get_info()
        return cls(mem_allocated=torch.cuda.memory_allocated() / div, mem_reserved=torch.cuda.memory_reserved() / div,
                   mem_used=(total - free) / div, mem_total=total / div, unit=unit)

    def log(self, label: str = "") -> str:
        return (f"{label}{' ' if label else ''}memory [{self.unit}]: allocated {self.mem_allocated:.2f}, reserved "
                f"{self.mem_reserved:.2f}, used on device {self.mem_used:.2f} of {self.mem_total:.2f}")


def get_versioned_lora_name(lora_name: str, version: int) -> str:
    """Name under which version ``version`` of an adapter is registered with an inference server."""
    return f"{lora_name}-v{version}"


_IMAGE_MAGIC = (("iVBOR", "image/png"), ("/9j/", "image/jpeg"), ("R0lGOD", "image/gif"), ("UklGR", "image/webp"),
                ("Qk", "image/bmp"))


def detect_image_mime(base64_data: str) -> str:
    """MIME type of a base64-encoded image, from the encoding of its magic bytes (JPEG when unknown)."""
    for prefix, mime in _IMAGE_MAGIC:
        if base64_data.startswith(prefix):
            return mime
    return "image/jpeg"
