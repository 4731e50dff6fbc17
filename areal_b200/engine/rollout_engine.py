"""In-process rollout engine: continuous batching over a paged KV cache on this
library's kernels, with interruptible generation and in-place weight updates.

The reference has no inference engine of its own — it drives external SGLang /
vLLM servers through HTTP (areal/infra/remote_inf_engine.py:719-884,
areal/engine/sglang_remote.py). This engine provides the same behaviour behind
the ``InferenceEngine`` contract:

* ``agenerate`` returns token ids, per-token logprobs and the *policy version of
  every generated token*; if generation is paused for a weight update the
  in-flight request is aborted inside the scheduler and transparently resumed
  with everything generated so far, so one response can span several versions;
* ``pause_generation`` / ``continue_generation`` / ``receive_weights`` /
  ``update_weights_from_disk`` / ``set_version``;
* ``submit`` / ``wait`` / ``prepare_batch`` / ``rollout_batch`` through the
  workflow executor (bounded staleness).

A background thread runs the engine loop: plan (C++ scheduler) → prefill or
decode step (model on the current CUDA stream) → fused sampling → commit.
"""

from __future__ import annotations

import asyncio
import collections
import ctypes
import hashlib
import os
import dataclasses
import threading
import time
from concurrent.futures import Future
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from ..api.cli_args import InferenceEngineConfig, NativeRolloutConfig
from ..api.engine_api import InferenceEngine
from ..api.io_struct import ModelRequest, ModelResponse, ParamSpec, WeightUpdateMeta
from ..models.config import PRESETS, ModelConfig
from ..models.qwen import build_model
from ..ops import _lib
from ..ops.attention import VarlenMeta
from ..ops.lm_head import lm_head_sample, new_sampling_rng
from ..ops.rollout_ops import sample
from ..utils import logging
from .flat_params import FlatParams

logger = logging.getLogger("RolloutEngine")

_REASONS = {1: "stop", 2: "length", 3: "abort"}


class _PlanHeader(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("n_seqs", ctypes.c_int32), ("n_tokens", ctypes.c_int32),
                ("max_seq_len", ctypes.c_int32), ("n_copies", ctypes.c_int32), ("pad", ctypes.c_int32)]


class PagedScheduler:
    """ctypes façade of ``csrc/host/rollout_scheduler.cpp``."""

    def __init__(self, num_blocks, block_size, max_num_seqs, max_batched_tokens, max_blocks_per_seq):
        self.lib = _lib.host()
        self.lib.b200_sched_create.restype = ctypes.c_void_p
        self.lib.b200_sched_add.restype = ctypes.c_int64
        self.lib.b200_sched_add_shared.restype = ctypes.c_int64
        self.lib.b200_sched_pop_finished.restype = ctypes.c_int64
        self.h = ctypes.c_void_p(self.lib.b200_sched_create(num_blocks, block_size, max_num_seqs,
                                                            max_batched_tokens, max_blocks_per_seq))
        self.max_num_seqs, self.max_blocks_per_seq = max_num_seqs, max_blocks_per_seq
        self.block_size = block_size
        cap = max(max_batched_tokens, max_num_seqs)
        # the plan lands in pinned host memory (when CUDA is there), so a step's inputs go to the
        # device straight from the arrays the C++ scheduler filled; numpy views share the storage
        pin = torch.cuda.is_available()
        mk = lambda n, dt: torch.zeros(n, dtype=dt, pin_memory=pin)
        self.t_tokens, self.t_positions = mk(cap, torch.int32), mk(cap, torch.int32)
        self.t_slots, self.t_seq_lens = mk(cap, torch.int64), mk(max_num_seqs, torch.int32)
        self.t_block_table = mk(max_num_seqs * max_blocks_per_seq, torch.int32)
        self.seq_ids = np.zeros(max_num_seqs, dtype=np.int64)
        self.cu = np.zeros(max_num_seqs + 1, dtype=np.int32)
        self.copy_pairs = np.zeros(2 * max_num_seqs, dtype=np.int32)  # (src page, dst page) of prompt forks
        self.tokens, self.positions = self.t_tokens.numpy(), self.t_positions.numpy()
        self.slots, self.seq_lens = self.t_slots.numpy(), self.t_seq_lens.numpy()
        self.block_table = self.t_block_table.numpy()
        self.hdr = _PlanHeader()

    @staticmethod
    def _p(a):
        return a.ctypes.data_as(ctypes.c_void_p)

    def add(self, prompt, max_new, min_new, stop_ids, ignore_eos, share_len: int = 0) -> int:
        """``share_len``: how many leading tokens the other samples of the same group also start with (0: the
        whole prompt). A request re-submitted with prompt + partial output passes the original prompt's length,
        so the group keeps sharing its prompt pages."""
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        s = np.ascontiguousarray(stop_ids, dtype=np.int32)
        return int(self.lib.b200_sched_add_shared(self.h, self._p(p), ctypes.c_int(len(p)), ctypes.c_int(max_new),
                                                  ctypes.c_int(min_new), self._p(s), ctypes.c_int(len(s)),
                                                  ctypes.c_int(int(ignore_eos)), ctypes.c_int(int(share_len))))

    def plan(self) -> int:
        return self.lib.b200_sched_plan(self.h, ctypes.byref(self.hdr), self._p(self.seq_ids), self._p(self.cu),
                                        self._p(self.tokens), self._p(self.positions), self._p(self.slots),
                                        self._p(self.seq_lens), self._p(self.block_table), self._p(self.copy_pairs))

    def commit(self, sampled: np.ndarray, logprobs: np.ndarray) -> int:
        return self.lib.b200_sched_commit(self.h, self._p(np.ascontiguousarray(sampled, dtype=np.int32)),
                                          self._p(np.ascontiguousarray(logprobs, dtype=np.float32)),
                                          ctypes.c_int(len(sampled)))

    def abort_all(self) -> int:
        return self.lib.b200_sched_abort_all(self.h)

    def abort(self, rid: int) -> int:
        return self.lib.b200_sched_abort(self.h, ctypes.c_int64(rid))

    def pop_finished(self):
        reason, n = ctypes.c_int32(0), ctypes.c_int32(0)
        rid = self.lib.b200_sched_pop_finished(self.h, ctypes.byref(reason), ctypes.byref(n))
        if rid == 0:
            return None
        toks = np.zeros(max(n.value, 1), dtype=np.int32)
        lps = np.zeros(max(n.value, 1), dtype=np.float32)
        got = self.lib.b200_sched_take_output(self.h, ctypes.c_int64(rid), self._p(toks), self._p(lps),
                                              ctypes.c_int(len(toks)))
        return int(rid), _REASONS.get(reason.value, "stop"), toks[:got].tolist(), lps[:got].tolist()

    def stats(self) -> dict[str, int]:
        a = np.zeros(8, dtype=np.int64)
        self.lib.b200_sched_stats(self.h, self._p(a))
        return dict(waiting=int(a[0]), running=int(a[1]), free_blocks=int(a[2]), preemptions=int(a[3]),
                    live=int(a[4]), prompt_forks=int(a[5]), shared_pages=int(a[6]), dedup_pages=int(a[7]))

    def set_prompt_sharing(self, on: bool):
        self.lib.b200_sched_set_prompt_sharing(self.h, ctypes.c_int(int(on)))

    def close(self):
        if self.h:
            self.lib.b200_sched_destroy(self.h)
            self.h = None


class _DecodeGraphs:
    """CUDA graphs of one full decode step (28-odd layers, LM head, sampler) for a set of padded
    batch sizes. All graphs read the same static input tensors and share one memory pool, so a
    step is: copy the scheduler's plan into the static inputs, replay, read tokens + logprobs.
    Weights (flat buffer) and KV pages keep their addresses, so weight updates need no re-capture."""

    def __init__(self, engine: "NativeRolloutEngine", batch_sizes: list[int]):
        self.e = engine
        dev = engine.device
        mb = engine.sched.max_blocks_per_seq
        self.sizes = sorted({b for b in batch_sizes if b <= engine.ncfg.max_num_seqs} | {engine.ncfg.max_num_seqs})
        maxb = self.sizes[-1]
        self.ids = torch.zeros(maxb, dtype=torch.int32, device=dev)
        self.pos = torch.zeros(maxb, dtype=torch.int32, device=dev)
        self.slots = torch.full((maxb,), -1, dtype=torch.int64, device=dev)
        self.seq_lens = torch.zeros(maxb, dtype=torch.int32, device=dev)
        self.bt = torch.zeros((maxb, mb), dtype=torch.int32, device=dev)
        self.temp = torch.ones(maxb, dtype=torch.float32, device=dev)
        self.u = torch.zeros(maxb, dtype=torch.float32, device=dev)
        pctx = getattr(engine.model, "pctx", None)
        self.fused_sampling = bool(getattr(engine.ncfg, "fused_sampling", True)) and \
            (pctx is None or pctx.tp_size == 1) and engine.model_config.hidden_size % 8 == 0
        self.rng_state = new_sampling_rng(engine.ncfg.seed, dev)
        pin = dict(pin_memory=True)
        self.h_pad_slots = torch.full((maxb,), -1, dtype=torch.int64, **pin)
        self.h_pad_lens = torch.zeros(maxb, dtype=torch.int32, **pin)
        self.h_temp = torch.ones(maxb, dtype=torch.float32, **pin)
        self.h_tok = torch.zeros(maxb, dtype=torch.int32, **pin)
        self.h_lp = torch.zeros(maxb, dtype=torch.float32, **pin)
        self.graphs: dict[int, tuple[torch.cuda.CUDAGraph, torch.Tensor, torch.Tensor]] = {}
        self.pool = None
        self.prev_n = 0
        self._last_temps = None

    def _forward(self, b: int):
        e = self.e
        hidden = e.model.decode(self.ids[:b], self.pos[:b], e.kv_caches, self.bt[:b], self.seq_lens[:b],
                                self.slots[:b], max_seq_len=e.ncfg.context_length)
        if self.fused_sampling:
            # the token is drawn in the LM-head GEMM's epilogue: no [B, V] logits, no separate sampler pass
            return lm_head_sample(hidden, e.model.output_weight(), self.temp[:b], self.rng_state)
        logits = e.model.logits(hidden, out_dtype=torch.float32)
        return sample(logits, self.temp[:b], None, None, self.u[:b])

    def capture_all(self, stream):
        with torch.cuda.stream(stream), torch.no_grad():
            for b in reversed(self.sizes):  # largest first: the shared pool is sized once
                self._forward(b)  # warm-up outside capture (kernel attributes, workspace)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, pool=self.pool, stream=stream, capture_error_mode="thread_local"):
                    toks, lps = self._forward(b)
                if self.pool is None:
                    self.pool = g.pool()
                self.graphs[b] = (g, toks, lps)
            torch.cuda.synchronize()

    def bucket(self, n: int) -> int | None:
        for b in self.sizes:
            if b >= n:
                return b if b in self.graphs else None
        return None

    def run(self, n: int, b: int, sched: "PagedScheduler", temps: list[float], rng) -> tuple[np.ndarray, np.ndarray]:
        ts0 = time.perf_counter()
        mb = sched.max_blocks_per_seq
        # inputs go to the device straight from the scheduler's pinned plan arrays
        self.ids[:n].copy_(sched.t_tokens[:n], non_blocking=True)
        self.pos[:n].copy_(sched.t_positions[:n], non_blocking=True)
        self.slots[:n].copy_(sched.t_slots[:n], non_blocking=True)
        self.seq_lens[:n].copy_(sched.t_seq_lens[:n], non_blocking=True)
        self.bt[:n].copy_(sched.t_block_table[: n * mb].view(n, mb), non_blocking=True)
        if self.prev_n > n:  # rows used by the previous step but not by this one become padding
            self.slots[n:self.prev_n].copy_(self.h_pad_slots[n:self.prev_n], non_blocking=True)
            self.seq_lens[n:self.prev_n].copy_(self.h_pad_lens[n:self.prev_n], non_blocking=True)
        if temps != self._last_temps:
            self.h_temp[:n] = torch.tensor(temps, dtype=torch.float32)
            self.temp[:n].copy_(self.h_temp[:n], non_blocking=True)
            self._last_temps = temps
        if not self.fused_sampling:
            self.u[:b].uniform_(generator=rng)
        self.prev_n = n
        g, toks, lps = self.graphs[b]
        g.replay()
        self.h_tok[:n].copy_(toks[:n], non_blocking=True)
        self.h_lp[:n].copy_(lps[:n], non_blocking=True)
        ts1 = time.perf_counter()
        torch.cuda.current_stream().synchronize()
        ts2 = time.perf_counter()
        self.e._phase_s["stage"] += ts1 - ts0
        self.e._phase_s["wait"] += ts2 - ts1
        _lib.count_launch(self.e.launches_per_decode)
        return self.h_tok[:n].numpy(), self.h_lp[:n].numpy()


def stop_string_cut(tokens: list[int], tokenizer, stops: list[str], skip_special_tokens: bool = True) -> int | None:
    """Number of leading tokens to keep so that the decoded text ends with the first completed stop string
    (``None``: no stop string occurs). Stop strings are matched on text, and a string can end inside a token or
    span several, so the cut is the shortest prefix whose decoding contains one: found by bisection, as
    containment is monotone in the prefix length. The engine applies it after generation (tokens past the cut
    were computed and are dropped); stop *token ids* end generation inside the scheduler at no such cost."""
    if not tokens or not stops:
        return None
    has = lambda n: any(s in tokenizer.decode(tokens[:n], skip_special_tokens=skip_special_tokens) for s in stops if s)
    if not has(len(tokens)):
        return None
    lo, hi = 1, len(tokens)
    while lo < hi:
        mid = (lo + hi) // 2
        if has(mid):
            hi = mid
        else:
            lo = mid + 1
    return lo


class NativeRolloutEngine(InferenceEngine):
    def __init__(self, config: InferenceEngineConfig):
        self.config = config
        self.ncfg: NativeRolloutConfig = config.native
        self.model = None
        self.flat: FlatParams | None = None
        self.sched: PagedScheduler | None = None
        self._version = 0
        self._paused = threading.Event()
        self._stop = threading.Event()
        self._wake = threading.Condition()
        self._thread: threading.Thread | None = None
        self._pending: dict[int, tuple[asyncio.AbstractEventLoop, asyncio.Future, dict]] = {}
        self._params: dict[int, tuple[float, int, float, float]] = {}  # temperature, top-k, top-p, frequency penalty
        self._hist: dict[int, collections.Counter] = {}  # requests with a frequency penalty: counts of their output tokens
        # vision-language requests: rid → pixel rows, patch grids, position triples of the prompt and the offset
        # of the positions that follow it
        self._mm: dict[int, dict[str, Any]] = {}
        # vision tower outputs by image content, valid for the current weights: the samples of a group (and a
        # request re-submitted after an interruption that did not change the weights) share one tower pass
        self._vis_cache: "collections.OrderedDict[bytes, tuple]" = collections.OrderedDict()
        self._vis_cache_max = 64
        self.vision_tower_images = 0  # images that went through the tower (cache misses)
        self._lock = threading.Lock()
        self._executor = None
        self._gen_tokens = 0
        self._steps = 0
        self._step_error: BaseException | None = None
        self.device = None
        self._idle = threading.Event()
        self._idle.set()
        self._step_lock = threading.Lock()
        self.weight_pusher = None  # (WeightPusher, cpu group) when a colocated trainer is model-parallel
        # host seconds spent in the phases of decode steps (plan / parameter lookup / stage+replay+sync / commit)
        self._phase_s = {"plan": 0.0, "params": 0.0, "run": 0.0, "commit_deliver": 0.0, "stage": 0.0, "wait": 0.0,
                         "prefill": 0.0, "paused": 0.0, "idle": 0.0}
        self._prefill_tokens = 0     # tokens that went through prefill steps
        self._reprefill_tokens = 0   # of those, context re-computed for requests interrupted by a weight update
        self._t_start = time.perf_counter()

    # ------------------------------------------------------------------ setup
    def initialize(self, engine_id: str | None = None, train_data_parallel_size: int | None = None,
                   device=None, model=None, **kwargs):
        ncfg = self.ncfg
        use_cuda = torch.cuda.is_available()
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu"))
        if ncfg.model_path:
            mc = ModelConfig.from_hf_config(ncfg.model_path)
        elif ncfg.model_preset:
            mc = dataclasses.replace(PRESETS[ncfg.model_preset])
        else:
            raise ValueError("NativeRolloutConfig needs model_path or model_preset")
        for k, v in (ncfg.model_overrides or {}).items():
            setattr(mc, k, v)
        self.model_config = mc
        dtype = torch.float32 if self.device.type == "cpu" else getattr(torch, ncfg.dtype)
        self.model = build_model(mc, dtype=dtype, device=self.device, seed=ncfg.seed)
        if ncfg.model_path:
            from ..utils.hf_io import load_hf_weights

            load_hf_weights(self.model, ncfg.model_path)
        self.model.eval()
        for p in self.model.parameters():
            p.requires_grad_(False)
        # weights live in one flat buffer with the trainer's layout: weight sync is a flat copy
        self.flat = FlatParams(self.model, kwargs.get("weight_group", "local"), with_grads=False)
        bs = ncfg.kv_block_size
        max_blocks_per_seq = (ncfg.context_length + bs - 1) // bs
        nblocks = ncfg.num_kv_blocks or self._auto_num_blocks(mc, dtype, bs)
        self.kv_caches = self._alloc_kv(nblocks, dtype)
        self.sched = PagedScheduler(nblocks, bs, ncfg.max_num_seqs, ncfg.max_num_batched_tokens,
                                    max_blocks_per_seq)
        # Hybrid models: per-sequence state of the linear-attention layers, addressed by a slot that a
        # request keeps from its first prefill until it finishes. Prompts are not shared (a shared page
        # says nothing about the recurrent state) and decode steps run eagerly.
        self.hybrid_state = None
        self._state_slot: dict[int, int] = {}
        self._free_state_slots: list[int] = []
        if mc.has_recurrent_state:
            if mc.is_hybrid:
                from ..models.qwen3_5 import HybridState as State
            else:
                from ..models.lightning import LightningState as State

            self.hybrid_state = State(mc, ncfg.max_num_seqs, dtype, self.device)
            self._free_state_slots = list(range(ncfg.max_num_seqs - 1, -1, -1))
        # prompts are shared by token ids: two prompts with equal ids but different images must not share pages
        self.sched.set_prompt_sharing(bool(getattr(ncfg, "prompt_sharing", True)) and not mc.has_recurrent_state
                                      and not mc.is_vl)
        # The engine thread shares the interpreter with trainer / workflow threads; CPython hands the GIL over
        # every 5 ms by default, which is half a decode step. A shorter interval keeps the step loop's short
        # host phases from queueing behind another thread's Python.
        import sys as _sys

        want = float(os.environ.get("AREAL_B200_SWITCH_INTERVAL", "0.0005"))
        if want > 0 and _sys.getswitchinterval() > want:
            _sys.setswitchinterval(want)
        self._rng = torch.Generator(device=self.device).manual_seed(ncfg.seed)
        self._graphs = None
        self.launches_per_decode = 0
        if (self.device.type == "cuda" and ncfg.cuda_graph and not mc.has_recurrent_state and not mc.is_vl
                and not mc.is_mla
                and _lib.use_cuda_kernels(next(self.model.parameters()))):
            self._capture_graphs()
        self._thread = threading.Thread(target=self._loop, name="rollout-engine", daemon=True)
        self._thread.start()
        from ..infra.workflow_executor import WorkflowExecutor

        self._executor = WorkflowExecutor(self.config, self)
        self._executor.initialize(train_data_parallel_size=train_data_parallel_size)
        logger.info(f"rollout engine ready on {self.device}: {nblocks} KV pages of {bs} tokens")
        return self

    def _alloc_kv(self, nblocks: int, dtype):
        """Paged K/V caches, one pair per layer (None for linear-attention layers of a hybrid model)."""
        mc, bs = self.model_config, self.ncfg.kv_block_size
        mk = lambda: torch.zeros(nblocks, mc.num_key_value_heads, bs, mc.head_dim, dtype=dtype, device=self.device)
        return [(mk(), mk()) if mc.layer_type(i) == "full_attention" else None for i in range(mc.num_hidden_layers)]

    def _state_slots_of(self, seq_ids: list[int]):
        """Slots of these requests in the hybrid state (assigned on first sight, freed when they finish)."""
        out = []
        for r in seq_ids:
            slot = self._state_slot.get(r)
            if slot is None:
                slot = self._state_slot[r] = self._free_state_slots.pop()
            out.append(slot)
        return torch.tensor(out, dtype=torch.long, device=self.device)

    def _capture_graphs(self):
        t0 = time.perf_counter()
        if getattr(self, "_graph_stream", None) is None:
            self._graph_stream = torch.cuda.Stream(self.device, priority=-1)
        graphs = _DecodeGraphs(self, list(self.ncfg.cuda_graph_batch_sizes))
        before = _lib.launch_count()
        with torch.cuda.stream(self._graph_stream), torch.no_grad():
            graphs._forward(graphs.sizes[0])
        self.launches_per_decode = _lib.launch_count() - before
        graphs.capture_all(self._graph_stream)
        self._graphs = graphs
        logger.info(f"captured decode graphs for batch sizes {graphs.sizes} in {time.perf_counter() - t0:.1f}s "
                    f"({self.launches_per_decode} kernels per step)")

    def _auto_num_blocks(self, mc: ModelConfig, dtype, bs: int) -> int:
        per_block = 2 * mc.num_hidden_layers * bs * mc.num_key_value_heads * mc.head_dim * \
            torch.empty((), dtype=dtype).element_size()
        if self.device.type == "cuda":
            free, total = torch.cuda.mem_get_info(self.device)
            budget = int(free * self.ncfg.mem_fraction_static)
        else:
            budget = 256 << 20
        need = self.ncfg.max_num_seqs * ((self.ncfg.context_length + bs - 1) // bs)
        return max(16, min(budget // per_block, need))

    def destroy(self):
        self._stop.set()
        with self._wake:
            self._wake.notify_all()
        if self._thread is not None:
            self._thread.join(timeout=10)
        if self._executor is not None:
            self._executor.destroy()
        if self.sched is not None:
            self.sched.close()
        self.kv_caches = None
        self.model = None

    # ------------------------------------------------------------- engine loop
    def _loop(self):
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        stream = None
        if self.device.type == "cuda":
            stream = self._graph_stream if self._graphs is not None else torch.cuda.Stream(self.device, priority=-1)
        while not self._stop.is_set():
            try:
                if self._paused.is_set():
                    self._idle.set()
                    tp = time.perf_counter()
                    time.sleep(0.0005)
                    self._phase_s["paused"] += time.perf_counter() - tp
                    continue
                self._idle.clear()
                with self._step_lock:
                    if self._paused.is_set():
                        continue
                    if stream is not None:
                        with torch.cuda.stream(stream):
                            worked = self._step()
                    else:
                        worked = self._step()
                if not worked:
                    self._idle.set()
                    tp = time.perf_counter()
                    with self._wake:
                        self._wake.wait(timeout=0.002)
                    self._phase_s["idle"] += time.perf_counter() - tp
            except BaseException as e:  # surface engine failures to every waiter
                logger.error(f"rollout engine loop failed: {type(e).__name__}: {e}")
                self._step_error = e
                self._fail_all(e)
                self._idle.set()
                return
        self._idle.set()

    @torch.no_grad()
    def _step(self) -> bool:
        s = self.sched
        tp0 = time.perf_counter()
        kind = s.plan()
        self._phase_s["plan"] += time.perf_counter() - tp0
        if s.hdr.n_copies > 0:
            self._copy_pages(s.copy_pairs[: 2 * s.hdr.n_copies])
        if kind == 0:
            self._deliver()
            return False
        n, T = s.hdr.n_seqs, s.hdr.n_tokens
        dev = self.device
        if kind != 1 and self._graphs is not None:
            t0 = time.perf_counter()
            seq_ids = s.seq_ids[:n].tolist()
            with self._lock:
                pr = [self._params.get(r, (1.0, 0, 1.0, 0.0)) for r in seq_ids]
            b = self._graphs.bucket(n)
            if b is not None and not any(p[1] > 0 or p[2] < 1.0 or p[3] for p in pr):
                t1 = time.perf_counter()
                toks, lps = self._graphs.run(n, b, s, [p[0] for p in pr], self._rng)
                t2 = time.perf_counter()
                s.commit(toks, lps)
                self._gen_tokens += n
                self._steps += 1
                self._deliver()
                t3 = time.perf_counter()
                tm = self._phase_s
                tm["params"] += t1 - t0
                tm["run"] += t2 - t1
                tm["commit_deliver"] += t3 - t2
                return True
        t_slow = time.perf_counter()
        ids = torch.from_numpy(s.tokens[:T].copy()).to(dev, non_blocking=True)
        pos = torch.from_numpy(s.positions[:T].copy()).to(dev, non_blocking=True)
        slots = torch.from_numpy(s.slots[:T].copy()).to(dev, non_blocking=True)
        seq_ids = s.seq_ids[:n].tolist()
        if kind == 1:
            cu = s.cu[: n + 1].copy()
            meta = VarlenMeta(cu.tolist(), dev)
            extra = dict(hybrid_state=self.hybrid_state, state_slots=self._state_slots_of(seq_ids)) \
                if self.hybrid_state is not None else {}
            if self.model_config.is_vl:
                extra.update(self._vision_prefill_inputs(ids, seq_ids, cu))
                pos = torch.arange(T, dtype=torch.int32, device=dev) if "rope" in extra else pos
            hidden = self.model.prefill(ids, pos, meta, self.kv_caches, slots, **extra)
            last = torch.from_numpy((cu[1:] - 1).astype(np.int64)).to(dev)
            hidden = hidden.index_select(0, last)
        else:
            seq_lens = torch.from_numpy(s.seq_lens[:n].copy()).to(dev, non_blocking=True)
            bt = torch.from_numpy(s.block_table[: n * s.max_blocks_per_seq].copy()).view(n, -1)
            nb = (int(s.hdr.max_seq_len) + self.ncfg.kv_block_size - 1) // self.ncfg.kv_block_size
            bt = bt[:, :max(nb, 1)].contiguous().to(dev, non_blocking=True)
            extra = dict(hybrid_state=self.hybrid_state, state_slots=self._state_slots_of(seq_ids)) \
                if self.hybrid_state is not None else {}
            if self._mm:
                # text after an image continues from the largest grid coordinate, not from the token count
                with self._lock:
                    delta = [self._mm[r]["delta"] if r in self._mm else 0 for r in seq_ids]
                pos = pos + torch.tensor(delta, dtype=pos.dtype, device=dev)
            hidden = self.model.decode(ids, pos, self.kv_caches, bt, seq_lens, slots,
                                       max_seq_len=int(s.hdr.max_seq_len), **extra)
        logits = self.model.logits(hidden, out_dtype=torch.float32)
        with self._lock:
            pr = [self._params.get(r, (1.0, 0, 1.0, 0.0)) for r in seq_ids]
        temp = torch.tensor([p[0] for p in pr], dtype=torch.float32, device=dev)
        need_k = any(p[1] > 0 for p in pr)
        need_p = any(p[2] < 1.0 for p in pr)
        top_k = torch.tensor([p[1] for p in pr], dtype=torch.int32, device=dev) if need_k else None
        top_p = torch.tensor([p[2] for p in pr], dtype=torch.float32, device=dev) if need_p else None
        penalised = [(i, r, p[3]) for i, (r, p) in enumerate(zip(seq_ids, pr)) if p[3]]
        for i, r, pen in penalised:
            # frequency penalty: every earlier occurrence of a token in this request's output lowers its logit
            with self._lock:
                seen = dict(self._hist.get(r) or {})
            if seen:
                idx = torch.tensor(list(seen.keys()), dtype=torch.long, device=dev)
                cnt = torch.tensor(list(seen.values()), dtype=logits.dtype, device=dev)
                logits[i, idx] -= pen * cnt
        u = torch.rand(n, device=dev, generator=self._rng, dtype=torch.float32)
        toks, lps = sample(logits, temp, top_k, top_p, u)
        toks_h = toks.cpu().numpy()
        with self._lock:
            for i, r, _ in penalised:
                if r in self._hist:
                    self._hist[r][int(toks_h[i])] += 1
        s.commit(toks_h, lps.cpu().numpy())
        self._gen_tokens += n
        self._steps += 1
        self._deliver()
        if kind == 1:
            self._prefill_tokens += T
            self._phase_s["prefill"] += time.perf_counter() - t_slow
        else:
            self._phase_s["run"] += time.perf_counter() - t_slow  # an eager decode step (no graph for this batch)
        return True

    def _vision_prefill_inputs(self, ids: torch.Tensor, seq_ids: list[int], cu: np.ndarray) -> dict[str, Any]:
        """Embeddings with image features and the per-token rotary table of a prefill plan; empty when no
        sequence of the plan has images (the ordinary tables then serve: the three axes agree on text)."""
        from ..models.qwen_vl import mrope_tables

        with self._lock:
            mms = [self._mm.get(r) for r in seq_ids]
        if not any(mms):
            return {}
        pos3, keyed = [], []
        for i, mm in enumerate(mms):
            n = int(cu[i + 1] - cu[i])
            if mm is None:
                pos3.append(torch.arange(n)[None].expand(3, -1))
            else:
                assert mm["pos3"].shape[1] == n, "an image prompt is prefilled whole"
                pos3.append(mm["pos3"])
                keyed.append(mm)
        # the tower runs once per distinct image set of the plan that is not cached yet
        todo = {}
        for mm in keyed:
            if mm["key"] not in self._vis_cache:
                todo.setdefault(mm["key"], mm)
        if todo:
            tm = list(todo.values())
            f, deep = self.model.visual(torch.cat([m["pixel_values"] for m in tm], 0),
                                        torch.cat([m["image_grid_thw"] for m in tm], 0), return_deepstack=True)
            unit, o = self.model.visual.unit, 0
            for m in tm:
                k = int(m["image_grid_thw"].prod(-1).sum()) // unit
                self._vis_cache[m["key"]] = (f[o:o + k], [d[o:o + k] for d in deep])
                self.vision_tower_images += int(m["image_grid_thw"].shape[0])
                o += k
        got = []
        for mm in keyed:
            self._vis_cache.move_to_end(mm["key"])
            got.append(self._vis_cache[mm["key"]])
        while len(self._vis_cache) > self._vis_cache_max:
            self._vis_cache.popitem(last=False)
        feats = torch.cat([g[0] for g in got], 0)
        deep = [torch.cat([g[1][j] for g in got], 0) for j in range(len(got[0][1]))]
        mc = self.model_config
        pos3 = torch.cat(pos3, 1).to(self.device)
        x, adds = self.model.embed_inputs(ids.long(), features=(feats, deep))
        return dict(embeds=x, layer_adds=adds,
                    rope=mrope_tables(pos3, mc.rotary_dim, mc.rope_theta, mc.mrope_section, mc.mrope_interleaved))

    @property
    def supports_images(self) -> bool:
        return self.model_config is not None and self.model_config.is_vl

    def _image_inputs(self, req: ModelRequest) -> dict[str, torch.Tensor] | None:
        """``pixel_values`` / ``image_grid_thw`` of a request: taken from ``metadata["multi_modal_input"]``
        when the caller already ran the processor, else computed from ``image_data`` (base64-encoded images)
        with the request's processor."""
        mm = req.metadata.get("multi_modal_input") if req.metadata else None
        if isinstance(mm, (list, tuple)):
            mm = mm[0] if mm else None
        if not mm and not req.image_data:
            return None
        if not self.supports_images:
            raise NotImplementedError(f"{self.model_config.model_type} is a text-only model: it cannot serve images")
        if not mm:
            import base64
            import io

            from PIL import Image

            if req.processor is None:
                raise ValueError("a request with image_data needs its processor (or precomputed multi_modal_input)")
            images = [Image.open(io.BytesIO(base64.b64decode(b))) if isinstance(b, (str, bytes)) else b
                      for b in req.image_data]
            ip = getattr(req.processor, "image_processor", req.processor)
            mm = ip(images=images, return_tensors="pt")
        return dict(pixel_values=torch.as_tensor(mm["pixel_values"]),
                    image_grid_thw=torch.as_tensor(mm["image_grid_thw"]).view(-1, 3))

    def _copy_pages(self, pairs: np.ndarray):
        """Private copies of the page holding a shared prompt's last positions (prompt forks)."""
        idx = torch.from_numpy(pairs.reshape(-1, 2).astype(np.int64)).to(self.device)
        src, dst = idx[:, 0], idx[:, 1]
        for pair in self.kv_caches:
            if pair is None:
                continue
            kc, vc = pair
            kc.index_copy_(0, dst, kc.index_select(0, src))
            vc.index_copy_(0, dst, vc.index_select(0, src))

    def _deliver(self):
        while True:
            item = self.sched.pop_finished()
            if item is None:
                return
            rid, reason, toks, lps = item
            slot = self._state_slot.pop(rid, None)
            if slot is not None:
                self._free_state_slots.append(slot)
            with self._lock:
                entry = self._pending.pop(rid, None)
                self._params.pop(rid, None)
                self._hist.pop(rid, None)
                self._mm.pop(rid, None)
            if entry is None:
                continue
            loop, fut, _ = entry
            loop.call_soon_threadsafe(_set_result, fut, (reason, toks, lps))

    def _fail_all(self, e: BaseException):
        with self._lock:
            entries = list(self._pending.values())
            self._pending.clear()
        for loop, fut, _ in entries:
            loop.call_soon_threadsafe(_set_exception, fut, e)

    # --------------------------------------------------------------- generate
    async def _generate_once(self, input_ids: list[int], g, max_new: int, images=None, share_len: int = 0,
                             history: list[int] | None = None):
        if self._step_error is not None:
            raise RuntimeError("rollout engine stopped") from self._step_error
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        stop = list(g.stop_token_ids or [])
        temp = 0.0 if g.greedy else float(g.temperature)
        top_k = int(g.top_k) if 0 < int(g.top_k) < self.model_config.vocab_size else 0
        mm_state = None
        if images is not None:
            from ..models.qwen_vl import mrope_position_ids

            pos3, deltas = mrope_position_ids(input_ids, [0, len(input_ids)], images["image_grid_thw"].tolist(),
                                              self.model_config)
            h = hashlib.blake2b(digest_size=16)
            h.update(images["pixel_values"].contiguous().numpy().tobytes())
            h.update(images["image_grid_thw"].contiguous().numpy().tobytes())
            mm_state = dict(images, pos3=pos3, delta=int(deltas[0]), key=h.digest())
        with self._lock:
            rid = self.sched.add(input_ids, max_new, int(g.min_new_tokens), stop, bool(g.ignore_eos), share_len)
            if rid < 0:
                raise ValueError(f"prompt of {len(input_ids)} tokens does not fit the rollout engine")
            self._pending[rid] = (loop, fut, {})
            self._params[rid] = (temp, top_k, float(g.top_p), float(g.frequency_penalty or 0.0))
            if g.frequency_penalty:
                self._hist[rid] = collections.Counter(history or [])
            if mm_state is not None:
                self._mm[rid] = mm_state
        with self._wake:
            self._wake.notify_all()
        return await fut

    async def agenerate(self, req: ModelRequest) -> ModelResponse:
        g = req.gconfig
        if g.n_samples != 1:
            raise ValueError("agenerate produces one sample; use n_samples=1 and group at the workflow level")
        if g.use_beam_search:
            raise NotImplementedError("the native rollout engine samples; it has no beam search")
        if g.stop and (req.tokenizer or getattr(self, "tokenizer", None)) is None:
            raise ValueError("stop strings need a tokenizer (ModelRequest.tokenizer or the engine's)")
        max_new = min(g.max_new_tokens, max(g.max_tokens - len(req.input_ids), 0))
        images = self._image_inputs(req)
        t0 = time.perf_counter()
        out_tokens: list[int] = []
        out_logprobs: list[float] = []
        out_versions: list[int] = []
        stop_reason = "length"
        ttft = float("inf")
        while len(out_tokens) < max_new:
            while self._paused.is_set():
                await asyncio.sleep(0.001)
            version = self._version
            if out_tokens:
                self._reprefill_tokens += len(req.input_ids) + len(out_tokens)
            reason, toks, lps = await self._generate_once(list(req.input_ids) + out_tokens, g,
                                                          max_new - len(out_tokens), images,
                                                          share_len=len(req.input_ids), history=out_tokens)
            if toks and ttft == float("inf"):
                ttft = time.perf_counter() - t0
            out_tokens += toks
            out_logprobs += lps
            out_versions += [version] * len(toks)
            stop_reason = reason
            if reason != "abort":
                break
        if stop_reason == "abort":
            stop_reason = "length"
        if g.stop:
            keep = stop_string_cut(out_tokens, req.tokenizer or getattr(self, "tokenizer", None), g.stop,
                                   bool(getattr(g, "skip_special_tokens", True)))
            if keep is not None:
                out_tokens, out_logprobs, out_versions = out_tokens[:keep], out_logprobs[:keep], out_versions[:keep]
                stop_reason = "stop"
        return ModelResponse(input_tokens=list(req.input_ids), output_tokens=out_tokens,
                             output_logprobs=out_logprobs, output_versions=out_versions,
                             stop_reason=stop_reason, tokenizer=req.tokenizer,
                             latency=time.perf_counter() - t0, ttft=ttft)

    # ------------------------------------------------------ pause / weights
    def pause_generation(self):
        """Stops the engine loop after the current step and aborts in-flight requests;
        their callers keep the partial output and resume after ``continue_generation``."""
        self._paused.set()
        # no engine step is in flight once the step lock is ours
        with self._step_lock:
            with self._lock:
                self.sched.abort_all()
            self._deliver()
            self._vis_cache.clear()  # a pause precedes every weight update: cached tower outputs go stale

    def continue_generation(self):
        self._paused.clear()
        with self._wake:
            self._wake.notify_all()

    def receive_weights(self, trainer, version: int | None = None):
        """Copies the trainer's flat bf16 weights into this engine's flat buffer. Both sides
        use the same model class, hence the same layout, so this is one device copy (a peer
        copy over NVLink when the two engines sit on different GPUs)."""
        with self._step_lock:
            self._vis_cache.clear()
        if self.weight_pusher is not None:
            # a model-parallel trainer on the same GPUs: every trainer rank stores its share of a re-sharding
            # plan into every rank's rollout buffer (peer memory). All engines pause before anyone writes and
            # resume only after every write has landed.
            pusher, group = self.weight_pusher
            dist.barrier(group=group)
            pusher.push()
            torch.cuda.current_stream(self.device).synchronize()
            dist.barrier(group=group)
            if version is not None:
                self._version = version
            return
        src = getattr(trainer, "weight_flat", trainer.flat).flat
        dst = self.flat.flat
        assert src.numel() >= dst.numel() or dst.numel() >= src.numel()
        n = min(src.numel(), dst.numel())
        if src.dtype == dst.dtype:
            dst[:n].copy_(src[:n], non_blocking=True)
        else:
            dst[:n].copy_(src[:n].to(dst.dtype))
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        if version is not None:
            self._version = version

    def update_weights_from_disk(self, meta: WeightUpdateMeta) -> Future:
        fut: Future = Future()
        try:
            from ..utils.hf_io import load_hf_weights

            self.pause_generation()
            load_hf_weights(self.model, meta.path)
            if meta.version is not None:
                self._version = meta.version
            self.continue_generation()
            fut.set_result(None)
        except BaseException as e:
            fut.set_exception(e)
        return fut

    def update_weights_from_distributed(self, meta: WeightUpdateMeta, param_specs: list[ParamSpec]) -> Future:
        fut: Future = Future()
        fut.set_result(None)
        return fut

    def init_weights_update_group(self, meta: WeightUpdateMeta) -> Future:
        fut: Future = Future()
        fut.set_result(None)
        return fut

    def set_version(self, version: int):
        self._version = version
        if self._executor is not None:
            self._executor.on_version_changed(version)

    def get_version(self) -> int:
        return self._version

    # ---------------------------------------------------------- workflow API
    def submit(self, data, workflow=None, workflow_kwargs=None, should_accept_fn=None, group_size=1,
               task_id=None, callback_addr=None, is_eval=False, proxy_addr=None) -> int:
        return self._executor.submit(data, workflow, workflow_kwargs, should_accept_fn, group_size,
                                     task_id=task_id, is_eval=is_eval)

    def wait(self, count: int, timeout: float | None = None, raise_timeout: bool = True):
        return self._executor.wait(count, timeout, raise_timeout)

    def wait_for_task(self, task_id: int, timeout: float | None = None, raise_timeout: bool = True):
        return self._executor.wait_for_task(task_id, timeout, raise_timeout)

    def poll_task(self, task_id: int):
        return self._executor.poll_task(task_id)

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

    def offload(self):
        """Releases the KV cache (colocated time-sharing with the trainer)."""
        self.pause_generation()
        self._graphs = None  # the captured graphs point into the cache that is being released
        self.kv_caches = None
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    def onload(self, tags: list[str] | None = None):
        if self.kv_caches is None:
            mc, bs = self.model_config, self.ncfg.kv_block_size
            dtype = next(self.model.parameters()).dtype
            nblocks = self.sched.stats()["free_blocks"]
            self.kv_caches = self._alloc_kv(nblocks, dtype)
            if (self.device.type == "cuda" and self.ncfg.cuda_graph and not self.model_config.has_recurrent_state
                    and not self.model_config.is_vl and not self.model_config.is_mla
                    and _lib.use_cuda_kernels(next(self.model.parameters()))):
                self._capture_graphs()
        self.continue_generation()

    def export_stats(self) -> dict[str, float]:
        st = {f"rollout/{k}": float(v) for k, v in self.sched.stats().items()}
        st["rollout/generated_tokens"] = float(self._gen_tokens)
        st["rollout/engine_steps"] = float(self._steps)
        st["rollout/prefill_tokens"] = float(self._prefill_tokens)
        st["rollout/reprefill_tokens"] = float(self._reprefill_tokens)
        st["rollout/wall_s"] = time.perf_counter() - self._t_start
        for k, v in self._phase_s.items():
            st[f"rollout/host_s/{k}"] = v
        if self._executor is not None:
            st.update(self._executor.export_stats())
        return st


def _set_result(fut: asyncio.Future, value):
    if not fut.done():
        fut.set_result(value)


def _set_exception(fut: asyncio.Future, e: BaseException):
    if not fut.done():
        fut.set_exception(e)
