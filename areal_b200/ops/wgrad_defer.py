"""Deferred weight gradients: the two halves of a linear layer's backward pass, run at different times.

The backward of ``y = x @ w.T`` is an input-gradient GEMM (``dx = dy @ w``), which the previous pipeline
stage is waiting for, and a weight-gradient GEMM (``dw = dy.T @ x``), which nobody waits for until the
optimizer step. Zero-bubble pipeline schedules run the first at once (action ``B``) and park the second
(action ``W``) until the stage would otherwise idle. While a :class:`WgradQueue` is active (``with
queue.collect():`` around the backward call), the linear autograd functions push their weight-gradient GEMM
as a closure instead of running it; ``queue.run()`` executes them later, accumulating into the parameter's
fp32 ``main_grad`` (the engine's flat gradient buffer) or its ``.grad``.

The active queue is process-global, not thread-local: for CUDA tensors autograd runs backward nodes on its
device worker thread, which must see the queue that the training thread activated. One training step runs
at a time per process.

The parked closure keeps the layer input and the output gradient alive until it runs: that memory is the
price of the schedule (bounded by the number of ``B`` actions a stage runs ahead of its ``W`` actions).

Role in the reference: the backward split of torch.distributed.pipelining's zero-bubble schedules
(``stage_backward_input`` / ``stage_backward_weight``) selected by areal/experimental/models/archon/
pipeline_parallel.py:48-82.
"""

from __future__ import annotations

from contextlib import contextmanager
from typing import Callable

import torch

_active: "WgradQueue | None" = None
_armed = False


def arm(on: bool = True) -> None:
    """Tells the linear ops that some backward passes of this process will run under a queue. On CPU the
    plain ``F.linear`` has no hook for the split, so an armed process routes CPU linears through the
    splittable autograd function as well."""
    global _armed
    _armed = bool(on)


def armed() -> bool:
    return _armed


def active() -> "WgradQueue | None":
    return _active


def accumulate(w: torch.Tensor, dw: torch.Tensor) -> None:
    """Adds a weight gradient where the engine collects it."""
    main = getattr(w, "main_grad", None)
    if main is not None:
        main.add_(dw.to(main.dtype))
    elif w.grad is None:
        w.grad = dw.to(w.dtype)
    else:
        w.grad.add_(dw.to(w.dtype))


class WgradQueue:
    def __init__(self):
        self.pending: list[Callable[[], None]] = []

    def push(self, fn: Callable[[], None]) -> None:
        self.pending.append(fn)

    @contextmanager
    def collect(self):
        global _active
        prev, _active = _active, self
        try:
            yield self
        finally:
            _active = prev

    @torch.no_grad()
    def run(self) -> int:
        """Runs and drops every parked weight-gradient product; returns how many there were."""
        todo, self.pending = self.pending, []
        for fn in todo:
            fn()
        return len(todo)

    def __len__(self) -> int:
        return len(self.pending)


class SplitLinear(torch.autograd.Function):
    """``x @ w.T + bias`` on PyTorch operators with the splittable backward (any device; the tcgen05 path has
    the same hook inside its own autograd function)."""

    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        return torch.nn.functional.linear(x, w, bias)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = dy @ w
        if ctx.needs_input_grad[1]:
            x2, dy2 = x.reshape(-1, x.shape[-1]), dy.reshape(-1, dy.shape[-1])
            q = _active
            if q is not None and w.is_leaf:
                q.push(lambda: accumulate(w, dy2.t() @ x2))
            else:
                dw = dy2.t() @ x2
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.reshape(-1, dy.shape[-1]).sum(0)
        return dx, dw, db
