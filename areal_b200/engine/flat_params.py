"""Flat parameter / gradient storage and the sharded AdamW that runs on it.

All parameters of a model live in ONE bf16 buffer (each parameter a view at a
128-byte aligned offset) and all fp32 main gradients in a second buffer of the
same layout. On CUDA both are symmetric-memory allocations, so

* GEMM wgrad epilogues accumulate straight into ``param.main_grad`` (fp32);
* the optimizer step is two kernels (``csrc/optim.cu``): a reduce-scatter that
  pulls this rank's gradient slice from every data-parallel peer over NVLink
  while computing its squared norm, and an AdamW that clips, updates the fp32
  master shard and stores the new bf16 weights into every peer's parameter
  buffer (the all-gather);
* trainer→rollout weight sync is a peer copy of the same flat layout.

With 180 GB of HBM the bf16 weights are replicated (no per-layer all-gather in
forward/backward) while fp32 master weights and Adam moments are sharded —
ZeRO-2 style. On CPU the same algorithm runs with ``torch.distributed``
collectives, which is the oracle for the CUDA path and what the gloo tests use.

Reference counterparts: FSDP2 sharding + fused AdamW + grad-norm clipping
(areal/engine/fsdp_utils/__init__.py:62-106, grad.py:89-281, fsdp_engine.py:682-713).
"""

from __future__ import annotations

import ctypes
import math

import torch
import torch.distributed as dist

from ..api.cli_args import OptimizerConfig
from ..ops import _lib
from ..parallel.symm_mem import SymmBarrier, SymmBuffer

_ALIGN = 64  # elements: 128 bytes in bf16, 256 in fp32


class FlatParams:
    def __init__(self, model: torch.nn.Module, dp_group: dist.ProcessGroup | None, with_grads: bool = True,
                 replicated_first=None, select=None):
        """``replicated_first(name) -> bool`` marks parameters that are replicated over a
        tensor-parallel group; they are laid out first, so ``flat[:rep_numel]`` is one contiguous
        region (their gradients need one extra all-reduce over that group)."""
        # ``select(name) -> bool`` restricts the buffer to some parameters (e.g. expert weights, which
        # are reduced over a different group than the rest of the model)
        params = [p for n, p in model.named_parameters() if select is None or select(n)]
        assert params, "model has no parameters"
        self.model = model
        self.device = params[0].device
        self.dtype = params[0].dtype
        local = isinstance(dp_group, str) and dp_group == "local"
        self.dp_group = dp_group
        self.dp_world = dist.get_world_size(dp_group) if (dist.is_initialized() and not local) else 1
        self.dp_rank = dist.get_rank(dp_group) if (dist.is_initialized() and not local) else 0
        self.entries: list[tuple[str, torch.nn.Parameter, int, int]] = []
        off = 0
        seen: dict[int, int] = {}
        named = [(n, p) for n, p in model.named_parameters() if select is None or select(n)]
        self.rep_numel = 0
        if replicated_first is not None:
            named = [x for x in named if replicated_first(x[0])] + [x for x in named if not replicated_first(x[0])]
        for name, p in named:
            if replicated_first is not None and not replicated_first(name) and self.rep_numel == 0:
                self.rep_numel = off
            if id(p) in seen:
                continue
            seen[id(p)] = off
            self.entries.append((name, p, off, p.numel()))
            off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        # shard boundaries must be multiples of 4 elements for the vector kernels
        quantum = self.dp_world * _ALIGN
        self.numel = (off + quantum - 1) // quantum * quantum
        self.shard_numel = self.numel // self.dp_world
        self.shard_offset = self.dp_rank * self.shard_numel
        self.cuda = self.device.type == "cuda"
        itemsize = torch.empty((), dtype=self.dtype).element_size()
        if self.cuda:
            self.param_buf = SymmBuffer(self.numel * itemsize, dp_group, self.device)
            self.flat = self.param_buf.tensor(self.dtype, self.numel)
            if with_grads:
                self.grad_buf = SymmBuffer(self.numel * 4, dp_group, self.device)
                self.main_grad = self.grad_buf.tensor(torch.float32, self.numel)
                self.barrier = SymmBarrier(dp_group, self.device)
        else:
            self.flat = torch.zeros(self.numel, dtype=self.dtype)
            self.main_grad = torch.zeros(self.numel, dtype=torch.float32) if with_grads else None
        with torch.no_grad():
            for name, p, o, n in self.entries:
                view = self.flat[o:o + n].view(p.shape)
                view.copy_(p.data)
                p.data = view
                if with_grads:
                    p.main_grad = self.main_grad[o:o + n].view(p.shape)
        self.with_grads = with_grads

    def close(self):
        """Returns the device buffers of a single-rank instance to the driver (the parameters must no
        longer be used). Buffers shared with peers over CUDA IPC are left to process exit: freeing memory
        that another process still has mapped is undefined, and a teardown barrier could hang on a dead rank."""
        if not self.cuda or self.dp_world > 1:
            return
        for _, p, _, _ in self.entries:
            p.data = torch.empty(0, dtype=p.dtype, device=self.device)
            if hasattr(p, "main_grad"):
                del p.main_grad
        self.flat = None
        self.main_grad = None
        for name in ("param_buf", "grad_buf"):
            buf = getattr(self, name, None)
            if buf is not None:
                buf.close()
                setattr(self, name, None)
        bar = getattr(self, "barrier", None)
        if bar is not None:
            bar.buf.close()
            self.barrier = None

    def zero_grad(self):
        if self.with_grads:
            self.main_grad.zero_()
        for _, p, _, _ in self.entries:
            p.grad = None

    def collect_autograd_grads(self):
        """Adds gradients that autograd produced (norm weights, biases, router, CPU path)
        into the fp32 main-grad buffer; GEMM weights were already accumulated there."""
        for _, p, _, _ in self.entries:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(torch.float32))
                p.grad = None

    def named_offsets(self) -> dict[str, tuple[int, int, tuple]]:
        return {name: (o, n, tuple(p.shape)) for name, p, o, n in self.entries}


def lr_at(step: int, total_steps: int, cfg: OptimizerConfig) -> float:
    """Warm-up followed by constant / linear / cosine decay to ``min_lr_ratio``."""
    warm = int(cfg.warmup_steps_proportion * max(total_steps, 1))
    if warm > 0 and step < warm:
        return cfg.lr * (step + 1) / warm
    if cfg.lr_scheduler_type == "constant" or total_steps <= warm:
        return cfg.lr
    frac = min(max((step - warm) / max(total_steps - warm, 1), 0.0), 1.0)
    lo = cfg.min_lr_ratio
    if cfg.lr_scheduler_type == "linear":
        return cfg.lr * (lo + (1 - lo) * (1 - frac))
    return cfg.lr * (lo + (1 - lo) * 0.5 * (1 + math.cos(math.pi * frac)))


class ShardedAdamW:
    """Optimizer over the rank's shard of the flat buffers. ``cfg.type`` selects the rule:

    * ``adam`` / ``adamw``: AdamW with an fp32 master copy and fp32 moments;
    * ``adam_bf16``: AdamW with bf16 moments and, instead of a master copy, a bf16 Kahan compensation
      buffer that carries the rounding error of every weight update (``self.master`` is that buffer);
      the counterpart of the reference's AnyPrecisionAdamW (areal/engine/fsdp_utils/optimizer.py);
    * ``sgd``: plain SGD with coupled weight decay on an fp32 master copy."""

    def __init__(self, flat: FlatParams, cfg: OptimizerConfig, total_steps: int = 1, tp_group=None,
                 tp_full_grad: tuple[str, ...] = ("score",), host_state: bool = False, prefetch: int = 1,
                 chunk_numel: int = 1 << 24):
        """``tp_group``: tensor-parallel group over which the gradients of the replicated region
        (``flat.rep_numel``) are summed before the data-parallel reduction; parameters named in
        ``tp_full_grad`` already hold the full gradient on every tp rank."""
        self.flat = flat
        self.cfg = cfg
        self.tp_group = tp_group
        self.tp_size = dist.get_world_size(tp_group) if (tp_group is not None and dist.is_initialized()) else 1
        self.tp_full_grad = tp_full_grad
        self.partner: "ShardedAdamW | None" = None  # a second optimizer (expert weights) clipped by the same norm
        self.partner_group = None        # group over which the partner's parameters are disjoint (ep group)
        self.norm_groups: list = []      # further groups that hold disjoint parameters (pipeline stages)
        self.pre_step_hooks: list = []   # run after the autograd gradients were collected
        # flat ranges (offset, numel) whose gradient another rank of a norm group also holds and counts (the
        # last pipeline stage's copy of a tied embedding): left out of this rank's share of the squared norm
        self.norm_exclude: list[tuple[int, int]] = []
        self.total_steps = total_steps
        self.step_count = 0  # optimizer steps taken (bias correction)
        self.sched_step = 0  # scheduler position
        n, o = flat.shard_numel, flat.shard_offset
        dev = flat.device
        self.kind = {"adam": "adamw", "adamw": "adamw"}.get(cfg.type, cfg.type)
        # host_state: master weights and moments live in pinned host memory and stream through the GPU
        # in chunks during the step (H2D of chunk i+1 and D2H of chunk i-1 overlap the update of chunk
        # i on separate streams); the counterpart of the reference's PerLayerOptimWrapper
        # (areal/engine/fsdp_utils/optimizer.py:324-633), chunked by flat offset instead of by layer
        self.host_state = bool(host_state) and flat.cuda
        if self.host_state and self.kind != "adamw":
            raise ValueError("host-resident optimizer state requires optimizer type 'adam'")
        self._chunk = max(int(chunk_numel) // 4 * 4, 4)
        self._slots = max(int(prefetch), 0) + 2
        if self.kind == "adam_bf16":
            assert flat.dtype == torch.bfloat16, "adam_bf16 keeps its state in the weights' bf16"
            self.master = torch.zeros(n, dtype=torch.bfloat16, device=dev)  # Kahan compensation
            self.exp_avg = torch.zeros(n, dtype=torch.bfloat16, device=dev)
            self.exp_avg_sq = torch.zeros(n, dtype=torch.bfloat16, device=dev)
        elif self.host_state:
            self.master = torch.empty(n, dtype=torch.float32, pin_memory=True)
            self.master.copy_(flat.flat[o:o + n].to(torch.float32))
            self.exp_avg = torch.zeros(n, dtype=torch.float32, pin_memory=True)
            self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, pin_memory=True)
            c = min(self._chunk, max(n, 4))
            self._stage = [[torch.empty(c, dtype=torch.float32, device=dev) for _ in range(3)]
                           for _ in range(self._slots)]
            self._h2d, self._d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        else:
            self.master = flat.flat[o:o + n].to(torch.float32).clone()
            m = 0 if self.kind == "sgd" else n
            self.exp_avg = torch.zeros(m, dtype=torch.float32, device=dev)
            self.exp_avg_sq = torch.zeros(m, dtype=torch.float32, device=dev)
        self.shard_grad = torch.zeros(n, dtype=torch.float32, device=dev)
        if flat.cuda:
            self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
            self._skipped = torch.zeros(1, dtype=torch.int32, device=dev)
            self._grad_table = flat.grad_buf.ptr_table()
            self._param_table = flat.param_buf.ptr_table()
        self.extra_param_tables: list = []  # rollout buffers that mirror the weights

    @property
    def lr(self) -> float:
        return lr_at(self.sched_step, self.total_steps, self.cfg)

    def refresh_master(self):
        """Re-reads the master shard from the (re)loaded bf16 weights."""
        n, o = self.flat.shard_numel, self.flat.shard_offset
        if self.kind == "adam_bf16":
            self.master.zero_()
        else:
            self.master.copy_(self.flat.flat[o:o + n].to(torch.float32))

    def step(self, grad_scale: float = 1.0) -> dict[str, float]:
        self.flat.collect_autograd_grads()
        for hook in self.pre_step_hooks:
            hook()
        if self.tp_size > 1 and self.flat.rep_numel > 0:
            for name, p, _, _ in self.flat.entries:
                if name.endswith(self.tp_full_grad):
                    p.main_grad.div_(self.tp_size)
            dist.all_reduce(self.flat.main_grad[:self.flat.rep_numel], group=self.tp_group)
        partner = self.partner
        if partner is not None:
            partner.flat.collect_autograd_grads()
        # phase 1: reduce gradients over the data-parallel group(s), squared norm of every part
        nsq = self._reduce(grad_scale)
        if partner is not None:
            pn = partner._reduce(grad_scale)
            if self.partner_group is not None:
                dist.all_reduce(pn, group=self.partner_group)  # the partner's parameters differ across this group
            nsq.add_(pn)
            pn.copy_(nsq)
        # phase 2: clip by the global norm, AdamW, publish the new weights
        out = self._update(nsq)
        if partner is not None:
            partner._update(pn)
            partner.flat.zero_grad()
        self.flat.zero_grad()
        return out

    def _reduce(self, grad_scale: float) -> torch.Tensor:
        return self._reduce_cuda(grad_scale) if self.flat.cuda else self._reduce_torch(grad_scale)

    def _update(self, nsq: torch.Tensor) -> dict[str, float]:
        return self._update_cuda() if self.flat.cuda else self._update_torch(nsq)

    # ---------------------------------------------------------------- CUDA
    def _reduce_cuda(self, grad_scale: float) -> torch.Tensor:
        f, cfg = self.flat, self.cfg
        lib = _lib.kernels()
        world = f.dp_world
        if world > 1:
            f.barrier.sync()  # every peer finished writing its gradients
        self._norm.zero_()
        rc = lib.b200_reduce_scatter_sumsq(self._grad_table, ctypes.c_int(world),
                                           ctypes.c_longlong(f.shard_offset),
                                           ctypes.c_longlong(f.shard_numel), ctypes.c_float(grad_scale),
                                           _lib.ptr(self.shard_grad), _lib.ptr(self._norm),
                                           _lib.stream_ptr())
        _lib.check(rc, "b200_reduce_scatter_sumsq")
        self._dedup_replicated_norm(self._norm)
        if world > 1:
            dist.all_reduce(self._norm, group=f.dp_group)
        if self.tp_size > 1:
            dist.all_reduce(self._norm, group=self.tp_group)
        for g in self.norm_groups:
            dist.all_reduce(self._norm, group=g)
        _lib.count_launch()
        return self._norm

    def _update_cuda(self) -> dict[str, float]:
        """Consumes ``self._norm`` (the global squared gradient norm, on the device)."""
        f, cfg = self.flat, self.cfg
        lib = _lib.kernels()
        world = f.dp_world
        t = self.step_count + 1
        lr = self.lr
        self._skipped.zero_()
        tail = (self._param_table, ctypes.c_int(world), ctypes.c_longlong(f.shard_offset),
                ctypes.c_longlong(f.shard_numel), _lib.ptr(self._norm), ctypes.c_float(lr))
        adam_hp = (ctypes.c_float(cfg.beta1), ctypes.c_float(cfg.beta2), ctypes.c_float(cfg.eps),
                   ctypes.c_float(cfg.weight_decay), ctypes.c_float(1 - cfg.beta1 ** t),
                   ctypes.c_float(1 - cfg.beta2 ** t), ctypes.c_float(cfg.gradient_clipping),
                   _lib.ptr(self._skipped), _lib.stream_ptr())
        if self.host_state:
            rc = self._update_streamed(lib, lr, adam_hp)
        elif self.kind == "sgd":
            rc = lib.b200_sgd_bcast(_lib.ptr(self.master), _lib.ptr(self.shard_grad), *tail,
                                    ctypes.c_float(cfg.weight_decay), ctypes.c_float(cfg.gradient_clipping),
                                    _lib.ptr(self._skipped), _lib.stream_ptr())
        elif self.kind == "adam_bf16":
            w_local = f.flat[f.shard_offset: f.shard_offset + f.shard_numel]
            rc = lib.b200_adamw_bf16_bcast(_lib.ptr(w_local), _lib.ptr(self.master), _lib.ptr(self.exp_avg),
                                           _lib.ptr(self.exp_avg_sq), _lib.ptr(self.shard_grad), *tail, *adam_hp)
        else:
            rc = lib.b200_adamw_bcast(_lib.ptr(self.master), _lib.ptr(self.exp_avg), _lib.ptr(self.exp_avg_sq),
                                      _lib.ptr(self.shard_grad), *tail, *adam_hp)
        _lib.check(rc, "optimizer update kernel")
        if not self.host_state:
            _lib.count_launch()
        if world > 1:
            f.barrier.sync()  # all shards of the new weights have landed everywhere
        vals = torch.cat([self._norm, self._skipped.float()]).tolist()
        ok = vals[1] == 0 and math.isfinite(vals[0])
        if ok:
            self.step_count = t
        return dict(grad_norm=math.sqrt(vals[0]) if vals[0] >= 0 else float("nan"),
                    update_successful=float(ok), lr=lr)

    def _update_streamed(self, lib, lr: float, adam_hp) -> int:
        """AdamW over host-resident state: chunk ``i`` is updated on the current stream while chunk
        ``i+1..`` loads and chunk ``i-1`` stores on two copy streams; a staging slot is reloaded only
        after its previous contents were written back."""
        f = self.flat
        n, chunk, slots = f.shard_numel, self._chunk, self._slots
        spans = [(s, min(chunk, n - s)) for s in range(0, n, chunk)]
        host = (self.master, self.exp_avg, self.exp_avg_sq)
        cur = torch.cuda.current_stream(f.device)
        loaded = [torch.cuda.Event() for _ in spans]
        stored = [torch.cuda.Event() for _ in spans]

        def load(i):
            s, m = spans[i]
            with torch.cuda.stream(self._h2d):
                for dst, src in zip(self._stage[i % slots], host):
                    dst[:m].copy_(src[s:s + m], non_blocking=True)
                loaded[i].record(self._h2d)

        self._h2d.wait_stream(cur)  # the staging buffers' previous users are done
        for i in range(min(slots - 1, len(spans))):
            load(i)
        rc = 0
        for i, (s, m) in enumerate(spans):
            st = self._stage[i % slots]
            cur.wait_event(loaded[i])
            rc = lib.b200_adamw_bcast(_lib.ptr(st[0]), _lib.ptr(st[1]), _lib.ptr(st[2]),
                                      _lib.ptr(self.shard_grad[s:s + m]), self._param_table, ctypes.c_int(f.dp_world),
                                      ctypes.c_longlong(f.shard_offset + s), ctypes.c_longlong(m),
                                      _lib.ptr(self._norm), ctypes.c_float(lr), *adam_hp)
            if rc != 0:
                break
            _lib.count_launch()
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(self._d2h):
                self._d2h.wait_event(done)
                for src, dst in zip(st, host):
                    dst[s:s + m].copy_(src[:m], non_blocking=True)
                stored[i].record(self._d2h)
            nxt = i + slots - 1
            if nxt < len(spans):
                if nxt - slots >= 0:
                    self._h2d.wait_event(stored[nxt - slots])  # that slot's write-back has finished
                load(nxt)
        cur.wait_stream(self._d2h)
        cur.wait_stream(self._h2d)
        return rc

    def _dedup_replicated_norm(self, nsq: torch.Tensor):
        """The squared norm is summed over the tp group afterwards; entries of the replicated
        region would count ``tp`` times, so keep only ``1/tp`` of their share here. Ranges in
        ``norm_exclude`` are counted by another rank and dropped entirely."""
        f = self.flat
        for off, n in self.norm_exclude:
            lo, hi = max(off, f.shard_offset), min(off + n, f.shard_offset + f.shard_numel)
            if hi > lo:
                part = (self.shard_grad[lo - f.shard_offset: hi - f.shard_offset].double() ** 2).sum().float()
                assert self.tp_size == 1 or lo >= f.rep_numel, "excluded ranges lie outside the tp-replicated region"
                nsq.sub_(part)
        if self.tp_size <= 1:
            return
        a, b = f.shard_offset, min(f.shard_offset + f.shard_numel, f.rep_numel)
        if b > a:
            rep = (self.shard_grad[:b - a].double() ** 2).sum().float()
            nsq.sub_(rep * (self.tp_size - 1) / self.tp_size)

    # --------------------------------------------------------------- torch
    def _reduce_torch(self, grad_scale: float) -> torch.Tensor:
        f, cfg = self.flat, self.cfg
        g = f.main_grad
        if f.dp_world > 1:
            dist.all_reduce(g, group=f.dp_group)
        o, n = f.shard_offset, f.shard_numel
        self.shard_grad.copy_(g[o:o + n] * grad_scale)
        nsq = (self.shard_grad.double() ** 2).sum().float().reshape(1)
        self._dedup_replicated_norm(nsq)
        if f.dp_world > 1:
            dist.all_reduce(nsq, group=f.dp_group)
        if self.tp_size > 1:
            dist.all_reduce(nsq, group=self.tp_group)
        for g in self.norm_groups:
            dist.all_reduce(nsq, group=g)
        return nsq

    def _update_torch(self, nsq: torch.Tensor) -> dict[str, float]:
        f, cfg = self.flat, self.cfg
        o, n = f.shard_offset, f.shard_numel
        norm = float(nsq.sqrt())
        lr = self.lr
        if not math.isfinite(norm):
            return dict(grad_norm=norm, update_successful=0.0, lr=lr)
        coef = min(1.0, cfg.gradient_clipping / (norm + 1e-6)) if cfg.gradient_clipping > 0 else 1.0
        t = self.step_count + 1
        gk = self.shard_grad * coef
        if self.kind == "sgd":
            self.master.sub_(lr * (gk + cfg.weight_decay * self.master))
            new = self.master.to(f.dtype)
        elif self.kind == "adam_bf16":
            w = f.flat[o:o + n].float()
            mk = cfg.beta1 * self.exp_avg.float() + (1 - cfg.beta1) * gk
            vk = cfg.beta2 * self.exp_avg_sq.float() + (1 - cfg.beta2) * gk * gk
            denom = vk.sqrt() / math.sqrt(1 - cfg.beta2 ** t) + cfg.eps
            c = self.master.float() - lr * cfg.weight_decay * w - (lr / (1 - cfg.beta1 ** t)) * mk / denom
            new = (w + c).to(f.dtype)
            self.exp_avg.copy_(mk)
            self.exp_avg_sq.copy_(vk)
            self.master.copy_(c + (w - new.float()))
        else:
            self.exp_avg.mul_(cfg.beta1).add_(gk, alpha=1 - cfg.beta1)
            self.exp_avg_sq.mul_(cfg.beta2).addcmul_(gk, gk, value=1 - cfg.beta2)
            denom = self.exp_avg_sq.sqrt() / math.sqrt(1 - cfg.beta2 ** t) + cfg.eps
            self.master.mul_(1 - lr * cfg.weight_decay).addcdiv_(self.exp_avg, denom,
                                                                 value=-lr / (1 - cfg.beta1 ** t))
            new = self.master.to(f.dtype)
        if f.dp_world > 1:
            parts = [torch.empty_like(new) for _ in range(f.dp_world)]
            dist.all_gather(parts, new, group=f.dp_group)
            f.flat.copy_(torch.cat(parts))
        else:
            f.flat[o:o + n].copy_(new)
        self.step_count = t
        return dict(grad_norm=norm, update_successful=1.0, lr=lr)

    # ------------------------------------------------------------ checkpoint
    def state_dict(self) -> dict:
        return dict(master=self.master, exp_avg=self.exp_avg, exp_avg_sq=self.exp_avg_sq,
                    step_count=self.step_count, sched_step=self.sched_step,
                    shard_offset=self.flat.shard_offset, shard_numel=self.flat.shard_numel,
                    dp_world=self.flat.dp_world)

    def load_state_dict(self, s: dict):
        if s["dp_world"] != self.flat.dp_world or s["shard_numel"] != self.flat.shard_numel:
            raise ValueError("optimizer shards were saved with a different data-parallel size")
        self.master.copy_(s["master"])
        self.exp_avg.copy_(s["exp_avg"])
        self.exp_avg_sq.copy_(s["exp_avg_sq"])
        self.step_count, self.sched_step = s["step_count"], s["sched_step"]
