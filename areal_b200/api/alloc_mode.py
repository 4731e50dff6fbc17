"""Allocation-mode mini-language: which backend runs on how many GPUs and how
they are parallelised.

Accepted strings (same surface as the reference grammar,
areal/api/alloc_mode.py:594-638):

* ``fsdp:d4``, ``megatron:d2p2t2c2e4``, ``archon:d2t2``, ``sglang:d4t2``, ``vllm:d2p2``
* named components ``fsdp[actor]:d4``
* disaggregation ``sglang:d4+fsdp:d4`` (``+``), colocation ``fsdp[actor]:d4|fsdp[ref]:d4``
  (``|`` binds tighter than ``+``)
* hybrid MoE ``megatron:(attn:d1p12t4|ffn:d1p12e4)``

The parser is a small hand-written tokenizer + recursive descent; it needs no
parser generator at run time.
"""

from __future__ import annotations

import enum
import math
import re
from dataclasses import dataclass, field
from typing import Literal

INFER_BACKENDS = ("sglang", "vllm", "native")
TRAIN_BACKENDS = ("fsdp", "megatron", "archon")


class AllocationValidationError(Exception):
    """The string parsed but describes an impossible allocation."""


class InvalidAllocationModeError(Exception):
    """Kept for callers that catch the legacy exception type."""


class SchedulingStrategyType(str, enum.Enum):
    separation = "separation"
    colocation = "colocation"


@dataclass
class SchedulingStrategy:
    type: SchedulingStrategyType = SchedulingStrategyType.separation
    target: str | None = None

    def __post_init__(self):
        if isinstance(self.type, str) and not isinstance(self.type, SchedulingStrategyType):
            self.type = SchedulingStrategyType(self.type)


@dataclass
class ParallelStrategy:
    """tp / pp / dp / cp / ep / etp sizes. ``world_size = dp * cp * tp * pp``
    (expert dims fold into the same ranks)."""

    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    context_parallel_size: int = 1
    expert_parallel_size: int = 1
    expert_tensor_parallel_size: int = 1

    def __post_init__(self):
        if self.expert_parallel_size > 1:
            emp = (self.pipeline_parallel_size * self.expert_tensor_parallel_size
                   * self.expert_parallel_size)
            self.expert_model_parallel_size = emp
            if self.world_size % emp != 0:
                raise AssertionError(
                    f"Expert model parallel size {emp} cannot divide world size {self.world_size}.")

    @property
    def world_size(self) -> int:
        return (self.data_parallel_size * self.context_parallel_size
                * self.tensor_parallel_size * self.pipeline_parallel_size)

    @property
    def expert_data_parallel_size(self) -> int:
        emp = getattr(self, "expert_model_parallel_size", None)
        return self.data_parallel_size if emp is None else self.world_size // emp

    tp_size = property(lambda self: self.tensor_parallel_size)
    pp_size = property(lambda self: self.pipeline_parallel_size)
    dp_size = property(lambda self: self.data_parallel_size)
    cp_size = property(lambda self: self.context_parallel_size)
    ep_size = property(lambda self: self.expert_parallel_size)
    etp_size = property(lambda self: self.expert_tensor_parallel_size)
    edp_size = property(lambda self: self.expert_data_parallel_size)

    def __str__(self):
        parts = [f"tp={self.tp_size}", f"pp={self.pp_size}", f"dp={self.dp_size}"]
        if self.cp_size > 1:
            parts.append(f"cp={self.cp_size}")
        if self.ep_size > 1:
            parts.append(f"ep={self.ep_size}")
            if self.etp_size != 1:
                parts.append(f"ep_tp={self.etp_size}")
        return f"Parallel({','.join(parts)})"

    @staticmethod
    def parallelism_eq(a, b) -> bool:
        return all(getattr(a, f) == getattr(b, f) for f in (
            "tensor_parallel_size", "pipeline_parallel_size", "data_parallel_size",
            "context_parallel_size", "expert_parallel_size", "expert_tensor_parallel_size"))


@dataclass
class FSDPParallelStrategy(ParallelStrategy):
    pass


@dataclass
class MegatronParallelStrategy(ParallelStrategy):
    virtual_pipeline_parallel_size: int = 1
    use_sequence_parallel: bool = False

    def __post_init__(self):
        super().__post_init__()
        if self.virtual_pipeline_parallel_size <= 1:
            self.virtual_pipeline_parallel_size = 1
        elif self.pipeline_parallel_size <= 1:
            raise AllocationValidationError(
                "Virtual pipeline parallelism requires pipeline_parallel_size > 1.")

    @staticmethod
    def parallelism_eq(a, b) -> bool:
        return ParallelStrategy.parallelism_eq(a, b) and (
            a.virtual_pipeline_parallel_size == b.virtual_pipeline_parallel_size)


@dataclass
class ModelAllocation:
    backend: Literal["fsdp", "megatron", "archon", "vllm", "sglang", "native"]
    name: str | None
    parallel: ParallelStrategy
    scheduling_strategy: SchedulingStrategy = field(default_factory=SchedulingStrategy)

    def __post_init__(self):
        if self.backend == "fsdp" and (self.parallel.pp_size > 1 or self.parallel.ep_size > 1):
            raise AllocationValidationError(
                "FSDP backend only supports data/tensor/context parallelism. "
                f"Got strategy: {self.parallel}")

    @property
    def is_inference(self) -> bool:
        return self.backend in INFER_BACKENDS

    @property
    def world_size(self) -> int:
        return self.parallel.world_size

    @classmethod
    def from_str(cls, spec: str, name: str | None = None,
                 scheduling_strategy: SchedulingStrategy | None = None) -> "ModelAllocation":
        """Parses exactly one ``backend:dims`` component."""
        allocs = _Parser(spec).parse()
        if len(allocs) != 1:
            raise AllocationValidationError(
                f"Expected a single component, got {len(allocs)} in {spec!r}; "
                "give each engine its own backend string.")
        a = allocs[0]
        if name is not None:
            a.name = name
        if scheduling_strategy is not None:
            a.scheduling_strategy = scheduling_strategy
        return a


class AllocationMode:
    """A full expression: one or more components joined by ``+`` / ``|``."""

    def __init__(self, allocations: list[ModelAllocation]):
        self.allocations = allocations

    @classmethod
    def from_str(cls, expr: str) -> "AllocationMode":
        return cls(_Parser(expr).parse())

    def __len__(self):
        return len(self.allocations)

    def __getitem__(self, name: str) -> ModelAllocation:
        for a in self.allocations:
            if a.name == name:
                return a
        raise KeyError(name)

    def _first(self, inference: bool) -> ModelAllocation | None:
        for a in self.allocations:
            if a.is_inference == inference:
                return a
        return None

    @property
    def gen(self) -> ParallelStrategy | None:
        a = self._first(True)
        return a.parallel if a else None

    @property
    def train(self) -> ParallelStrategy | None:
        a = self._first(False)
        return a.parallel if a else None

    @property
    def gen_backend(self) -> str | None:
        a = self._first(True)
        return a.backend if a else None

    @property
    def train_backend(self) -> str | None:
        a = self._first(False)
        return a.backend if a else None

    @property
    def gen_instance_size(self) -> int:
        g = self.gen
        return g.tp_size * g.pp_size if g else 0

    @property
    def world_size(self) -> int:
        """GPUs needed: colocated components share their anchor's devices."""
        return sum(a.world_size for a in self.allocations
                   if a.scheduling_strategy.type == SchedulingStrategyType.separation)


_TOKEN = re.compile(r"\s*(?:(?P<name>[A-Za-z_][A-Za-z0-9_]*)|(?P<num>[0-9]+)|(?P<sym>[+|:\[\]()]))")

_HINT = ("Hints: separate backends from dimensions with a colon, e.g. 'sglang:d4+fsdp:d4'; "
         "hybrid MoE looks like 'megatron:(attn:d1p12t4|ffn:d1p12e4)'.")


class _Parser:
    def __init__(self, text: str):
        self.text = text
        self.toks: list[tuple[str, str]] = []
        pos = 0
        text_s = text.strip()
        while pos < len(text_s):
            m = _TOKEN.match(text_s, pos)
            if not m:
                raise ValueError(f"Parsing error at {text_s[pos:]!r} in {text!r}\n{_HINT}")
            pos = m.end()
            if m.group("name") is not None:
                self.toks.append(("name", m.group("name")))
            elif m.group("num") is not None:
                self.toks.append(("num", m.group("num")))
            else:
                self.toks.append(("sym", m.group("sym")))
        self.i = 0
        self.names: set[str] = set()

    # token helpers
    def _peek(self, k=0):
        return self.toks[self.i + k] if self.i + k < len(self.toks) else ("eof", "")

    def _eat(self, kind=None, val=None):
        t = self._peek()
        if (kind and t[0] != kind) or (val is not None and t[1] != val):
            raise ValueError(f"Parsing error: expected {val or kind}, got {t[1]!r} in {self.text!r}\n{_HINT}")
        self.i += 1
        return t

    def parse(self) -> list[ModelAllocation]:
        if not self.toks:
            raise ValueError(f"Parsing error: empty allocation mode\n{_HINT}")
        groups = [self._colocate_group()]
        while self._peek() == ("sym", "+"):
            self._eat()
            groups.append(self._colocate_group())
        if self._peek()[0] != "eof":
            raise ValueError(f"Parsing error: unexpected {self._peek()[1]!r} in {self.text!r}\n{_HINT}")
        allocs = [a for g in groups for a in g]
        if len(allocs) >= 3:
            unnamed = [a for a in allocs if a.name is None]
            if unnamed:
                raise AllocationValidationError(
                    "When using 3+ components, all must have names. "
                    f"Found {len(unnamed)} unnamed components.")
        return allocs

    def _colocate_group(self) -> list[ModelAllocation]:
        first = self._single()
        group = [first]
        while self._peek() == ("sym", "|"):
            self._eat()
            nxt = self._single()
            if nxt.name is None:
                raise AllocationValidationError("Components in colocation group must have names")
            if nxt.world_size != first.world_size:
                raise AllocationValidationError(
                    "Colocated components must have matching world sizes. "
                    f"'{first.name}' has {first.world_size}, '{nxt.name}' has {nxt.world_size}.")
            nxt.scheduling_strategy = SchedulingStrategy(SchedulingStrategyType.colocation, first.name)
            group.append(nxt)
        return group

    def _register(self, name):
        if name is not None:
            if name in self.names:
                raise AllocationValidationError(f"Duplicate component name: {name}")
            self.names.add(name)

    def _single(self) -> ModelAllocation:
        t = self._peek()
        if t == ("sym", "["):
            raise AllocationValidationError(
                "Backend must be explicitly specified. Got a named component without a backend "
                "prefix. Use e.g. 'fsdp[actor]:d4', 'megatron[actor]:d4t2p2'.")
        if t == ("sym", "(") or (t[0] == "name" and t[1] == "attn"):
            raise AllocationValidationError(
                "Backend must be explicitly specified for hybrid MoE parallelism. "
                "Use e.g. 'megatron:(attn:d1p12t4|ffn:d1p12e4)'.")
        if t[0] != "name":
            raise ValueError(f"Parsing error: unexpected {t[1]!r} in {self.text!r}\n{_HINT}")
        word = t[1]
        if word not in INFER_BACKENDS + TRAIN_BACKENDS:
            if re.fullmatch(r"([dtpce][1-9][0-9]*)+", word):
                raise AllocationValidationError(
                    "Backend must be explicitly specified. Got bare parallelism dimensions "
                    "without a backend prefix. Use e.g. 'fsdp:d4', 'megatron:d4t2p2', 'sglang:d4'.")
            raise ValueError(f"Parsing error: unknown backend {word!r} in {self.text!r}\n{_HINT}")
        self._eat()
        name = None
        if self._peek() == ("sym", "["):
            self._eat()
            name = self._eat("name")[1]
            self._eat("sym", "]")
        self._eat("sym", ":")
        infer = word in INFER_BACKENDS
        nt = self._peek()
        if not infer and (nt == ("sym", "(") or (nt[0] == "name" and nt[1] == "attn")):
            strategy = self._hybrid()
        else:
            dims = self._dims("dtp" if infer else "dtpce")
            strategy = ParallelStrategy(
                tensor_parallel_size=dims.get("t", 1), pipeline_parallel_size=dims.get("p", 1),
                data_parallel_size=dims.get("d", 1), context_parallel_size=dims.get("c", 1),
                expert_parallel_size=dims.get("e", 1))
        self._register(name)
        return ModelAllocation(word, name, strategy, SchedulingStrategy())

    def _dims(self, allowed: str) -> dict[str, int]:
        """Dimension run such as ``d4p2t2``; the tokenizer sees it as one name."""
        t = self._eat("name")
        word = t[1]
        # a run like d4 may be split as name 'd4' only; numbers inside names are kept
        m = re.fullmatch(r"((?:[a-z][0-9]+)+)", word)
        if not m:
            raise ValueError(f"Parsing error: bad dimension spec {word!r} in {self.text!r}\n{_HINT}")
        out: dict[str, int] = {}
        for k, v in re.findall(r"([a-z])([0-9]+)", word):
            if k not in allowed:
                raise ValueError(
                    f"Parsing error: dimension {k!r} not allowed here ({allowed}) in {self.text!r}\n{_HINT}")
            if v.startswith("0"):
                raise ValueError(f"Parsing error: sizes must be positive in {self.text!r}\n{_HINT}")
            out[k] = int(v)
        return out

    def _hybrid(self) -> ParallelStrategy:
        paren = self._peek() == ("sym", "(")
        if paren:
            self._eat()
        self._eat("name", "attn")
        self._eat("sym", ":")
        attn = self._dims("cdtp")
        self._eat("sym", "|")
        self._eat("name", "ffn")
        self._eat("sym", ":")
        ffn = self._dims("detp")
        if paren:
            self._eat("sym", ")")
        a_d, a_t, a_p, a_c = attn.get("d", 1), attn.get("t", 1), attn.get("p", 1), attn.get("c", 1)
        f_p = ffn.get("p", a_p)
        if f_p != a_p:
            raise AllocationValidationError(
                "Pipeline parallel size for attention and FFN modules must be identical. "
                f"Got attention: {a_p}, FFN: {f_p}.")
        f_t, f_e = ffn.get("t", 1), ffn.get("e", 1)
        attn_ws = a_d * a_t * a_p * a_c
        f_d = ffn.get("d")
        if f_d is None:
            non_dp = f_e * f_t * f_p
            if attn_ws % non_dp:
                raise AllocationValidationError(
                    f"Cannot derive expert dp: attn world_size ({attn_ws}) is not divisible by "
                    f"ffn ep*tp*pp ({non_dp}).")
            f_d = attn_ws // non_dp
        ffn_ws = math.prod([f_d, f_p, f_t, f_e])
        if attn_ws != ffn_ws:
            raise InvalidAllocationModeError(
                "World size for expert modules and attention modules must be identical. "
                f"Got attention: {attn_ws}, expert: {ffn_ws}.")
        return ParallelStrategy(tensor_parallel_size=a_t, pipeline_parallel_size=a_p,
                                data_parallel_size=a_d, context_parallel_size=a_c,
                                expert_parallel_size=f_e, expert_tensor_parallel_size=f_t)
