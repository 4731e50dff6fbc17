"""Pipeline-parallel schedules and the executor that runs them over asynchronous point-to-point.

A schedule is, per pipeline rank, an ordered list of actions ``("F" | "B" | "W", micro_batch, chunk)``;
``chunk`` selects one of the rank's ``V`` model chunks (virtual stages: chunk ``v`` of rank ``p`` is virtual
stage ``v * P + p``). Four schedules are built here:

* ``gpipe``: every forward, then every backward (activations of all micro-batches stay alive);
* ``1f1b``: ``P - 1 - p`` warm-up forwards, then one forward / one backward alternating, then the
  remaining backwards; at most ``P - p`` micro-batches are alive on rank ``p``;
* ``interleaved_1f1b``: the same idea over virtual stages, which divides the bubble by ``V``;
* ``zero_bubble``: the backward pass is split. ``B`` computes only the input gradients (what the previous
  stage waits for) and parks every linear layer's weight-gradient GEMM (``ops/wgrad_defer.py``); ``W`` runs
  the parked GEMMs of one micro-batch. Forwards and ``B`` keep the (interleaved) 1F1B order and its
  activation bound, and each rank's ``W`` actions are placed by a list scheduler wherever the rank would
  otherwise wait for a neighbour (the ZB-H1 construction, extended to virtual stages).

Every rank can build every rank's list, so :func:`simulate` replays a whole pipeline on the host and reports
makespan, bubble fraction and the peak number of live activations (used by the tests and the docs).

Transport. Activations flow p → p+1 and gradients p+1 → p (with virtual stages also P-1 → 0 and back).
Each *direction* of each neighbour pair has its own two-rank process group, i.e. its own NCCL communicator
and stream: a group carries one ordered stream of messages one way, sender and receiver enumerate it in the
same order (both follow the schedule), so plain ``isend`` / ``irecv`` can never wait on each other in a
cycle and no send has to be grouped with a receive. Sends are never waited for before the end of the step,
so a stage goes on computing while its output travels. ``x`` and the residual stream travel as two
messages; nothing is stacked or cloned.

Two NCCL facts shape the executor. (1) Creating a communicator blocks the host until the peer creates it
too, so every link is opened by a one-element handshake in a fixed ring order before the first step, not
lazily in the middle of a schedule. (2) A receive posted ahead of time is a kernel that spins on the device
until the peer sends; any device-wide synchronisation on this rank (a ``cudaMalloc`` of the caching
allocator, the first load of a kernel's module) then waits for the peer, and in the steady state of 1F1B the
peer's send can in turn wait for this rank: a cycle. Receives are therefore posted ahead only on CPU (gloo,
where they are host-side requests); on CUDA a receive is posted when its action starts.

Reference: areal/experimental/models/archon/pipeline_parallel.py:48-82 (``build_pipeline_schedule``:
1F1B, Interleaved1F1B, zero-bubble variants) and :349-494, options areal/api/cli_args.py:537-700; Megatron's
schedules behind areal/engine/megatron_engine.py:882.

Placement. With the interleaved placement chunk ``v`` of rank ``p`` is virtual stage ``v * P + p`` (activations
always flow to the next rank, and from the last rank back to the first). ``ZBVZeroBubble`` uses the V-shaped
placement instead (two chunks per rank): chunk 0 of rank ``p`` is stage ``p``, chunk 1 is stage ``2P - 1 - p``, so
activations run down the ranks and back up, the first rank holds the embedding AND the head / loss (a tied
embedding needs no second copy), the turn-around on the last rank is a local hand-over, and every rank holds the
same amount of live activations (the reference puts the last stage on rank 0 the same way,
areal/experimental/engine/archon_engine.py:930-938). Its schedule comes from a list scheduler as well
(:func:`_v_schedules`): the first rank keeps at most ``P`` micro-batches in flight, which bounds every rank's
live activations by ``2P`` chunks (``P`` stages' worth, the 1F1B peak), and weight-gradient work fills the gaps.
The chunks going back up send activations to the PREVIOUS rank and gradients to the NEXT, over two more one-way
groups per neighbour pair.
"""

from __future__ import annotations

import contextlib
import functools
from dataclasses import dataclass, field
from typing import Any, Callable

import torch
import torch.distributed as dist

from ..ops.wgrad_defer import WgradQueue

Action = tuple[str, int, int]  # kind, micro-batch, chunk

_ALIASES = {
    "gpipe": "gpipe", "1f1b": "1f1b", "interleaved1f1b": "interleaved_1f1b", "interleaved_1f1b": "interleaved_1f1b",
    "interleavedzerobubble": "zero_bubble", "zbvzerobubble": "zero_bubble", "zerobubble": "zero_bubble",
    "zb1p": "zero_bubble", "zbh1": "zero_bubble", "zero_bubble": "zero_bubble", "zbv": "zero_bubble",
}


_V_PLACED = {"zbvzerobubble", "zbv"}


def placement_of(name: str) -> str:
    """``"v"`` for the schedules that place their two chunks per rank in a V over the ranks, else
    ``"interleaved"``."""
    return "v" if str(name).replace("-", "").replace("_", "").replace(" ", "").lower() in _V_PLACED else "interleaved"


def stage_of(rank: int, chunk: int, P: int, placement: str = "interleaved") -> int:
    if placement == "v":
        return rank if chunk == 0 else 2 * P - 1 - rank
    return chunk * P + rank


def rank_of(stage: int, P: int, placement: str = "interleaved") -> int:
    if placement == "v":
        return stage if stage < P else 2 * P - 1 - stage
    return stage % P


def canonical_schedule(name: str, virtual: int) -> str:
    key = _ALIASES.get(str(name).replace("-", "").replace(" ", "").lower())
    if key is None:
        raise ValueError(f"unknown pipeline schedule {name!r}; known: GPipe, 1F1B, Interleaved1F1B, "
                         f"InterleavedZeroBubble / ZBVZeroBubble")
    if key == "interleaved_1f1b" and virtual == 1:
        return "1f1b"  # one chunk per rank: the interleaved order degenerates to plain 1F1B
    if key not in ("interleaved_1f1b", "zero_bubble") and virtual > 1:
        raise ValueError(f"schedule {name!r} runs one model chunk per rank; virtual stages need Interleaved1F1B")
    return key


def build_schedule(name: str, pp_size: int, n_mbs: int, rank: int, virtual: int = 1,
                   forward_only: bool = False, placement: str = "interleaved") -> list[Action]:
    """The action list of pipeline rank ``rank``."""
    P, M, V = pp_size, n_mbs, virtual
    kind = canonical_schedule(name, V)
    if placement == "v":
        import os

        if V != 2 or (kind != "zero_bubble" and not forward_only):
            raise ValueError("the V-shaped placement runs two chunks per rank under the zero-bubble schedule")
        slack = float(os.environ.get("AREAL_B200_PP_ZB_SLACK", "0"))
        return list(_v_schedules(P, M, slack, forward_only)[rank])
    if forward_only:
        if V == 1:
            return [("F", m, 0) for m in range(M)]
        return [("F",) + _virtual_to_mb_chunk(k, P, V, True) for k in range(M * V)]
    if kind == "zero_bubble":
        import os

        # extra micro-batches of activation memory the list scheduler may use beyond the 1F1B bound (0 = same
        # memory as 1F1B; every unit lets weight-gradient work slide later and shortens the step a little more)
        slack = float(os.environ.get("AREAL_B200_PP_ZB_SLACK", "0"))
        return _zero_bubble_schedules(P, M, V, slack)[rank]
    if kind == "gpipe":
        return [("F", m, 0) for m in range(M)] + [("B", m, 0) for m in range(M)]
    if kind == "1f1b":
        warm = min(P - 1 - rank, M)
        acts: list[Action] = [("F", m, 0) for m in range(warm)]
        for i in range(M - warm):
            acts.append(("F", warm + i, 0))
            acts.append(("B", i, 0))
        acts += [("B", m, 0) for m in range(M - warm, M)]
        return acts
    # interleaved 1F1B: micro-batches advance in groups of P through the chunks
    if M % P != 0:
        raise ValueError(f"Interleaved1F1B needs a micro-batch count that is a multiple of the pipeline size "
                         f"(got {M} micro-batches, {P} stages)")
    total = M * V
    warm = min((P - 1 - rank) * 2 + (V - 1) * P, total)
    acts = [("F",) + _virtual_to_mb_chunk(k, P, V, True) for k in range(warm)]
    for i in range(total - warm):
        acts.append(("F",) + _virtual_to_mb_chunk(warm + i, P, V, True))
        acts.append(("B",) + _virtual_to_mb_chunk(i, P, V, False))
    acts += [("B",) + _virtual_to_mb_chunk(k, P, V, False) for k in range(total - warm, total)]
    return acts


PARKED_WEIGHT = 0.5  # memory of a micro-batch between B and W, as a share of its memory between F and B


@functools.lru_cache(maxsize=64)
def _zero_bubble_schedules(P: int, M: int, V: int, slack: float = 0.0) -> tuple[tuple[Action, ...], ...]:
    """Action lists of all ranks for the split-backward schedule, by list scheduling on the host.

    Every rank keeps the forward order and the ``B`` order of (interleaved) 1F1B, so the messages of every
    link keep their order. A micro-batch holds its activations from ``F`` to ``B`` and, from ``B`` to ``W``,
    what the parked products keep (layer inputs and output gradients, counted as ``PARKED_WEIGHT`` of a full
    set); a rank starts a forward only if that sum stays within ``cap`` afterwards, the live-activation bound of
    (interleaved) 1F1B, so the schedule needs no more memory than 1F1B. Time is
    simulated with unit costs for F, B and W. A free rank takes, in this order: the next ``B`` if its
    gradient has arrived; the next ``F`` if its input has arrived and the cap allows; a parked ``W``. Only
    when none applies does it wait for the next arrival. W actions therefore land exactly where 1F1B idles:
    while the first gradients travel back and during the cool-down."""
    if V > 1 and M % P != 0:
        raise ValueError(f"virtual stages need a micro-batch count that is a multiple of the pipeline size "
                         f"(got {M} micro-batches, {P} stages)")
    total = M * V
    order_f = [_virtual_to_mb_chunk(k, P, V, True) if V > 1 else (k, 0) for k in range(total)]
    order_b = [_virtual_to_mb_chunk(k, P, V, False) if V > 1 else (k, 0) for k in range(total)]
    cap = [(min((P - 1 - r) * 2 + (V - 1) * P, total) + 1 if V > 1 else min(P - r, M)) + slack for r in range(P)]
    last_vs = P * V - 1
    done: dict[tuple[str, int, int], float] = {}
    nf, nb, nw = [0] * P, [0] * P, [0] * P
    parked: list[list[tuple[int, int]]] = [[] for _ in range(P)]
    free = [0.0] * P
    acts: list[list[Action]] = [[] for _ in range(P)]
    n_left = 3 * total * P
    now = 0.0
    while n_left:
        progressed = False
        for r in range(P):
            if free[r] > now:
                continue
            choice = None
            if nb[r] < total:
                mb, c = order_b[nb[r]]
                vs = c * P + r
                dep = ("F", mb, vs) if vs == last_vs else ("B", mb, vs + 1)
                if done.get(dep, float("inf")) <= now:
                    choice = ("B", mb, c)
            if choice is None and nf[r] < total and (nf[r] - nb[r]) + PARKED_WEIGHT * (nb[r] - nw[r]) + 1 <= cap[r]:
                mb, c = order_f[nf[r]]
                vs = c * P + r
                if vs == 0 or done.get(("F", mb, vs - 1), float("inf")) <= now:
                    choice = ("F", mb, c)
            if choice is None and parked[r]:
                choice = ("W",) + parked[r][0]
            if choice is None:
                continue
            kind, mb, c = choice
            if kind == "F":
                nf[r] += 1
            elif kind == "B":
                nb[r] += 1
                parked[r].append((mb, c))
            else:
                nw[r] += 1
                parked[r].pop(0)
            free[r] = now + 1.0
            done[(kind, mb, c * P + r)] = free[r]
            acts[r].append(choice)
            n_left -= 1
            progressed = True
        if n_left and not progressed:  # nobody can start anything at this instant: go to the next completion
            later = [t for t in free if t > now]
            if not later:
                raise RuntimeError(f"zero-bubble list scheduling stalled (P={P}, M={M}, V={V})")
            now = min(later)
    return tuple(tuple(a) for a in acts)


@functools.lru_cache(maxsize=64)
def _v_schedules(P: int, M: int, slack: float = 0.0, forward_only: bool = False) -> tuple[tuple[Action, ...], ...]:
    """Action lists of all ranks for the V-shaped placement (chunk 0 of rank ``p`` = stage ``p``, chunk 1 = stage
    ``2P - 1 - p``), by list scheduling with unit costs.

    Every rank runs the forwards of a chunk in micro-batch order and its backwards likewise, so every one-way
    link carries its messages in one order on both ends. A free rank takes, in this order: a backward whose
    gradient has arrived (the older micro-batch first); the forward of its returning chunk (stages ``P..2P-1``:
    these finish micro-batches); the forward of its outgoing chunk; a parked weight-gradient product. Memory: the
    first rank admits a new micro-batch only while fewer than ``P (+ slack)`` are in flight, which bounds the live
    activations of EVERY rank by ``2 (P + slack)`` chunks; a forward also waits (and weight-gradient work runs
    first) while live activations plus ``PARKED_WEIGHT`` per parked product would pass that bound."""
    last = 2 * P - 1
    cap = 2 * (P + slack)
    done: dict[tuple[str, int, int], float] = {}
    nf = [[0, 0] for _ in range(P)]
    nb = [[0, 0] for _ in range(P)]
    parked: list[list[tuple[int, int]]] = [[] for _ in range(P)]
    free = [0.0] * P
    acts: list[list[Action]] = [[] for _ in range(P)]
    n_left = (2 * M if forward_only else 6 * M) * P
    now = 0.0
    stage = lambda r, c: r if c == 0 else last - r
    while n_left:
        progressed = False
        for r in range(P):
            if free[r] > now:
                continue
            choice = None
            if not forward_only:
                ready = []
                for c in (0, 1):
                    if nb[r][c] < M:
                        mb, st = nb[r][c], stage(r, c)
                        dep = ("F", mb, st) if st == last else ("B", mb, st + 1)
                        if done.get(dep, float("inf")) <= now:
                            ready.append((mb, c))
                if ready:
                    mb, c = min(ready)
                    choice = ("B", mb, c)
            if choice is None:
                live = (nf[r][0] - nb[r][0]) + (nf[r][1] - nb[r][1])
                room = forward_only or live + PARKED_WEIGHT * len(parked[r]) + 1 <= cap
                for c in (1, 0):
                    if nf[r][c] >= M or not room:
                        continue
                    mb, st = nf[r][c], stage(r, c)
                    if st == 0:
                        if not forward_only and nf[0][0] - nb[0][0] >= P + slack:
                            continue  # the first rank keeps at most P (+ slack) micro-batches in flight
                    elif done.get(("F", mb, st - 1), float("inf")) > now:
                        continue
                    choice = ("F", mb, c)
                    break
            if choice is None and parked[r]:
                choice = ("W",) + parked[r][0]
            if choice is None:
                continue
            kind, mb, c = choice
            if kind == "F":
                nf[r][c] += 1
            elif kind == "B":
                nb[r][c] += 1
                parked[r].append((mb, c))
            else:
                parked[r].pop(0)
            free[r] = now + 1.0
            done[(kind, mb, stage(r, c))] = free[r]
            acts[r].append(choice)
            n_left -= 1
            progressed = True
        if n_left and not progressed:
            later = [t for t in free if t > now]
            if not later:
                raise RuntimeError(f"V-placement list scheduling stalled (P={P}, M={M})")
            now = min(later)
    return tuple(tuple(a) for a in acts)


def _virtual_to_mb_chunk(k: int, P: int, V: int, forward: bool) -> tuple[int, int]:
    """Micro-batch and chunk of the ``k``-th forward (backward) of a rank under the interleaved order."""
    group, r = divmod(k, P * V)
    c = r // P
    return group * P + r % P, (c if forward else V - 1 - c)


def min_micro_batches(name: str, pp_size: int, virtual: int = 1) -> int:
    """Micro-batches below which the pipeline cannot fill: ``2 * pp`` for the 1F1B family (the reference's
    ``min_n_mbs``), rounded up to a multiple of ``pp`` for the interleaved order."""
    kind = canonical_schedule(name, virtual)
    return pp_size if kind == "gpipe" else 2 * pp_size  # zero_bubble included


@dataclass
class SimResult:
    makespan: float
    busy: list[float]
    bubble_fraction: float
    peak_live: list[int]
    order: list[tuple[int, Action, float, float]] = field(default_factory=list)


def simulate(name: str, pp_size: int, n_mbs: int, virtual: int = 1, f_cost: float = 1.0, b_cost: float = 2.0,
             comm_cost: float = 0.0, w_cost: float | None = None, placement: str | None = None) -> SimResult:
    """Replays the schedule of every rank with per-chunk costs ``f_cost / V`` and ``b_cost / V``: an action
    starts when the rank is free and its input has arrived. In a split-backward schedule ``W`` costs
    ``w_cost / V`` (default: half of ``b_cost``) and ``B`` the rest. Raises if the schedules deadlock."""
    P, V = pp_size, virtual
    placement = placement or placement_of(name)
    acts = [build_schedule(name, P, n_mbs, r, V, placement=placement) for r in range(P)]
    split = any(a[0] == "W" for a in acts[0])
    w_cost = (b_cost / 2 if w_cost is None else w_cost) if split else 0.0
    costs = {"F": f_cost / V, "B": (b_cost - w_cost) / V, "W": w_cost / V}
    ptr = [0] * P
    free = [0.0] * P
    done: dict[tuple[str, int, int], float] = {}  # (kind, mb, virtual stage) -> finish time
    live = [0] * P
    peak = [0] * P
    busy = [0.0] * P
    order = []
    last_vs = P * V - 1
    remaining = sum(len(a) for a in acts)
    while remaining:
        progressed = False
        for r in range(P):
            while ptr[r] < len(acts[r]):
                kind, mb, c = acts[r][ptr[r]]
                vs = stage_of(r, c, P, placement)
                if kind == "F":
                    dep = None if vs == 0 else ("F", mb, vs - 1)
                elif kind == "B":
                    dep = ("F", mb, vs) if vs == last_vs else ("B", mb, vs + 1)
                else:
                    dep = ("B", mb, vs)
                if dep is not None and dep not in done:
                    break
                ready = 0.0 if dep is None else done[dep] + (comm_cost if rank_of(dep[2], P, placement) != r else 0.0)
                start = max(free[r], ready)
                cost = costs[kind]
                free[r] = start + cost
                busy[r] += cost
                done[(kind, mb, vs)] = free[r]
                live[r] += {"F": 1, "B": -1, "W": 0}[kind]
                peak[r] = max(peak[r], live[r])
                order.append((r, (kind, mb, c), start, free[r]))
                ptr[r] += 1
                remaining -= 1
                progressed = True
        if not progressed:
            raise RuntimeError(f"pipeline schedule {name} deadlocks at {[a[p] if p < len(a) else None for a, p in zip(acts, ptr)]}")
    makespan = max(free)
    return SimResult(makespan, busy, 1.0 - sum(busy) / (P * makespan), peak, order)


# --------------------------------------------------------------------------- transport


@dataclass
class PipelineLinks:
    """The directed two-rank groups of one pipeline column. ``fwd_next``: this rank → next stage (activations
    out), ``fwd_prev``: previous stage → this rank (activations in), ``bwd_next`` / ``bwd_prev``: the gradient
    streams the other way. ``prev`` / ``next`` are global ranks (with virtual stages the ring closes: the first
    rank's ``prev`` is the last rank)."""
    prev: int | None = None
    next: int | None = None
    fwd_prev: Any = None
    fwd_next: Any = None
    bwd_prev: Any = None
    bwd_next: Any = None
    # the V-shaped placement's returning chunks: activations next → this → prev, gradients prev → this → next
    vfwd_next: Any = None
    vfwd_prev: Any = None
    vbwd_prev: Any = None
    vbwd_next: Any = None


class _Pending:
    """Handles of transfers in flight (the tensors stay referenced until the transfer has finished)."""

    def __init__(self):
        self.items: list[tuple[Any, tuple]] = []

    def add(self, work, *tensors):
        self.items.append((work, tensors))

    def wait_all(self):
        for work, _ in self.items:
            work.wait()
        self.items.clear()


class PipelineRunner:
    """Runs one optimizer step's micro-batches through this rank's chunks following a schedule.

    ``forward(mb_index, chunk, stage_input) -> outputs``: runs the chunk; returns ``(x, res)`` when the
    chunk is not the last virtual stage, else whatever ``finish`` needs. ``finish(mb_index, outputs) ->
    scalar loss | None`` (last virtual stage only; ``None`` in forward-only runs). ``shape_of(mb_index)``:
    shape of the activations travelling between stages for that micro-batch."""

    def __init__(self, links: PipelineLinks, pp_rank: int, pp_size: int, virtual: int, schedule: str,
                 dtype: torch.dtype, device: torch.device, placement: str = "interleaved"):
        self.links, self.rank, self.P, self.V = links, pp_rank, pp_size, virtual
        self.schedule, self.placement = schedule, placement
        self.dtype, self.device = dtype, device
        import os

        self.prefetch = (device.type != "cuda") if os.environ.get("AREAL_B200_PP_PREFETCH") is None \
            else os.environ["AREAL_B200_PP_PREFETCH"] == "1"
        flag = "opened_v" if placement == "v" else "opened"
        if not getattr(links, flag, False):
            self._open_links()
            setattr(links, flag, True)

    def _open_links(self):
        """One element over every link this rank uses, in ring order (edge i joins stage i and stage i + 1):
        both ends of an edge reach it as their next step, so the blocking communicator set-up of NCCL happens
        here, pairwise and in a chain, and never inside a schedule."""
        L, P = self.links, self.P
        token = torch.zeros(1, dtype=self.dtype, device=self.device)
        edges = []  # (edge index, [(group, i_send)])
        if self.placement == "v":  # no ring-closing edge; the two extra streams of every neighbour pair
            if self.rank < P - 1:
                edges.append((self.rank, [(L.fwd_next, True, L.next), (L.bwd_next, False, L.next),
                                          (L.vfwd_next, False, L.next), (L.vbwd_next, True, L.next)]))
            if self.rank > 0:
                edges.append((self.rank - 1, [(L.fwd_prev, False, L.prev), (L.bwd_prev, True, L.prev),
                                              (L.vfwd_prev, True, L.prev), (L.vbwd_prev, False, L.prev)]))
        else:
            if self.rank < P - 1 or self.V > 1:
                edges.append((self.rank, [(L.fwd_next, True, L.next), (L.bwd_next, False, L.next)]))
            if self.rank > 0 or self.V > 1:
                edges.append(((self.rank - 1) % P, [(L.fwd_prev, False, L.prev), (L.bwd_prev, True, L.prev)]))
        for _, ops in sorted(edges, key=lambda e: e[0]):
            for group, sending, peer in ops:
                if sending:
                    dist.send(token, dst=peer, group=group)
                else:
                    dist.recv(token, src=peer, group=group)
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()

    # -- which virtual stage talks to whom
    def _vs(self, chunk: int) -> int:
        return stage_of(self.rank, chunk, self.P, self.placement)

    def _fwd_route(self, chunk: int):
        """``(source, destination)`` of a chunk's forward: ``None`` (first / last stage), ``"local"`` (the other
        chunk of this rank) or ``(peer rank, group)``. Gradients travel the same edges the other way
        (:meth:`_bwd_route`)."""
        L, P, r = self.links, self.P, self.rank
        if self.placement == "v":
            if chunk == 0:
                return (None if r == 0 else (L.prev, L.fwd_prev)), ("local" if r == P - 1 else (L.next, L.fwd_next))
            return ("local" if r == P - 1 else (L.next, L.vfwd_next)), (None if r == 0 else (L.prev, L.vfwd_prev))
        return (None if self._is_first(chunk) else (L.prev, L.fwd_prev)), \
            (None if self._is_last(chunk) else (L.next, L.fwd_next))

    def _bwd_route(self, chunk: int):
        """``(where the output gradient comes from, where the input gradient goes)``."""
        L, P, r = self.links, self.P, self.rank
        if self.placement == "v":
            if chunk == 0:
                return ("local" if r == P - 1 else (L.next, L.bwd_next)), (None if r == 0 else (L.prev, L.bwd_prev))
            return (None if r == 0 else (L.prev, L.vbwd_prev)), ("local" if r == P - 1 else (L.next, L.vbwd_next))
        return (None if self._is_last(chunk) else (L.next, L.bwd_next)), \
            (None if self._is_first(chunk) else (L.prev, L.bwd_prev))

    def _is_first(self, chunk: int) -> bool:
        return self._vs(chunk) == 0

    def _is_last(self, chunk: int) -> bool:
        return self._vs(chunk) == self.P * self.V - 1

    def _recv(self, shape, src: int, group) -> tuple[list, list[torch.Tensor]]:
        bufs = [torch.empty(shape, dtype=self.dtype, device=self.device) for _ in range(2)]
        works = [dist.irecv(b, src=src, group=group) for b in bufs]
        return works, bufs

    def run(self, n_mbs: int, forward: Callable, finish: Callable, shape_of: Callable,
            forward_only: bool = False) -> dict[int, Any]:
        L = self.links
        acts = build_schedule(self.schedule, self.P, n_mbs, self.rank, self.V, forward_only=forward_only,
                              placement=self.placement)
        handed_f: dict[int, tuple] = {}  # micro-batch -> activations handed from this rank's chunk 0 to its chunk 1
        handed_b: dict[int, tuple] = {}  # micro-batch -> gradients handed back
        sends = _Pending()
        posted: dict[int, tuple[list, list[torch.Tensor]]] = {}  # action index -> receive in flight
        saved: dict[tuple[int, int], tuple] = {}  # (mb, chunk) -> (stage input, outputs, loss)
        results: dict[int, Any] = {}
        split = any(a[0] == "W" for a in acts)
        parked: dict[tuple[int, int], WgradQueue] = {}  # (mb, chunk) -> weight-gradient products of its B action

        def post(i: int):
            if i >= len(acts) or i in posted:
                return
            kind, mb, c = acts[i]
            src = self._fwd_route(c)[0] if kind == "F" else (self._bwd_route(c)[0] if kind == "B" else None)
            if isinstance(src, tuple):
                posted[i] = self._recv(shape_of(mb), src[0], src[1])

        import os as _os
        import sys as _sys

        debug = _os.environ.get("AREAL_B200_PP_DEBUG") == "1"

        def note(msg):
            if debug:
                print(f"[pp rank {self.rank}] {msg}", file=_sys.stderr, flush=True)

        post(0)
        for i, (kind, mb, c) in enumerate(acts):
            note(f"action {i}: {kind} mb={mb} chunk={c}: posting receives")
            post(i)
            if self.prefetch:
                post(i + 1)  # the next action's input travels while this one computes
            got = posted.pop(i, None)
            if got is not None:
                for w in got[0]:
                    w.wait()
                note(f"action {i}: input received")
            if kind == "F":
                stage_in = None
                src, dst = self._fwd_route(c)
                if got is not None or src == "local":
                    x_in, r_in = handed_f.pop(mb) if src == "local" else got[1]
                    if not forward_only:
                        x_in.requires_grad_(True)
                        r_in.requires_grad_(True)
                    stage_in = (x_in, r_in)
                with torch.set_grad_enabled(not forward_only):
                    out = forward(mb, c, stage_in)
                if not self._is_last(c):
                    x, res = out
                    res = res if res is not None else torch.zeros_like(x)
                    xs, rs = x.detach(), res.detach()
                    if dst == "local":
                        handed_f[mb] = (xs, rs)  # the turn of the V: this rank's other chunk is the next stage
                    else:
                        sends.add(dist.isend(xs, dst=dst[0], group=dst[1]), xs)
                        sends.add(dist.isend(rs, dst=dst[0], group=dst[1]), rs)
                    if not forward_only:
                        saved[(mb, c)] = (stage_in, (x, res), None)
                else:
                    with torch.set_grad_enabled(not forward_only):
                        loss = finish(mb, out)
                    results[mb] = loss.detach() if torch.is_tensor(loss) else loss
                    if not forward_only:
                        saved[(mb, c)] = (stage_in, None, loss)
            elif kind == "W":
                parked.pop((mb, c)).run()
            else:
                stage_in, outs, loss = saved.pop((mb, c))
                queue = None
                if split:
                    # input gradients now; the linear layers park their weight-gradient GEMMs for the W action
                    queue = parked[(mb, c)] = WgradQueue()
                with (queue.collect() if queue is not None else contextlib.nullcontext()):
                    gsrc, gdst = self._bwd_route(c)
                    if self._is_last(c):
                        loss.backward()
                    else:
                        gx, gr = handed_b.pop(mb) if gsrc == "local" else got[1]
                        torch.autograd.backward([outs[0], outs[1]], [gx, gr])
                if not self._is_first(c):
                    x_in, r_in = stage_in
                    gx = x_in.grad if x_in.grad is not None else torch.zeros_like(x_in)
                    gr = r_in.grad if r_in.grad is not None else torch.zeros_like(r_in)
                    if gdst == "local":
                        handed_b[mb] = (gx, gr)
                    else:
                        sends.add(dist.isend(gx, dst=gdst[0], group=gdst[1]), gx)
                        sends.add(dist.isend(gr, dst=gdst[0], group=gdst[1]), gr)
        note("all actions issued: waiting for sends")
        sends.wait_all()
        note("step done")
        assert not saved and not posted and not parked and not handed_f and not handed_b
        return results
