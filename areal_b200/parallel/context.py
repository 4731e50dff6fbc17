"""Model-parallel context handed to the model: tensor-parallel and Ulysses
sequence-parallel groups plus the symmetric-memory state of the fused
GEMM+collective kernels.

Rank order inside one pipeline stage is ``[dp][sp][tp]`` with ``tp`` innermost, the
same nesting as the reference's device meshes (areal/engine/fsdp_utils/parallel.py:86-123,
areal/api/alloc_mode.py:32-160).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist


def partition_layers(costs, stages: int, first_extra: float = 0.0, last_extra: float = 0.0) -> list[tuple[int, int]]:
    """Min-max contiguous partition of ``costs`` into ``stages`` non-empty ranges (dynamic program
    over prefix sums; ties keep the earlier cut, so every rank derives the same split). Reference:
    areal/engine/megatron_utils/pipeline_parallel.py:17-160."""
    n = len(costs)
    if stages > n:
        raise ValueError(f"{stages} pipeline stages need at least as many layers (got {n})")
    pre = [0.0]
    for c in costs:
        pre.append(pre[-1] + float(c))

    def seg(a, b, k):  # cost of layers [a, b) as stage k
        return pre[b] - pre[a] + (first_extra if k == 0 else 0.0) + (last_extra if k == stages - 1 else 0.0)

    inf = float("inf")
    best = [[inf] * (n + 1) for _ in range(stages + 1)]  # best[k][b]: first k stages cover [0, b)
    cut = [[0] * (n + 1) for _ in range(stages + 1)]
    best[0][0] = 0.0
    for k in range(1, stages + 1):
        for b in range(k, n - (stages - k) + 1):
            for a in range(k - 1, b):
                if best[k - 1][a] == inf:
                    continue
                v = max(best[k - 1][a], seg(a, b, k - 1))
                if v < best[k][b] - 1e-12:
                    best[k][b], cut[k][b] = v, a
    out, b = [], n
    for k in range(stages, 0, -1):
        a = cut[k][b]
        out.append((a, b))
        b = a
    return out[::-1]


@dataclass
class ParallelContext:
    tp_group: Any = None
    tp_rank: int = 0
    tp_size: int = 1
    sp_group: Any = None
    sp_rank: int = 0
    sp_size: int = 1
    ep_group: Any = None
    ep_rank: int = 0
    ep_size: int = 1
    # expert tensor parallelism: the ranks that hold slices (of the intermediate dimension) of the same experts
    etp_group: Any = None
    etp_rank: int = 0
    etp_size: int = 1
    pp_group: Any = None
    pp_rank: int = 0
    pp_size: int = 1
    pp_prev: int | None = None   # global ranks of the neighbouring stages
    pp_next: int | None = None
    pp_tie_group: Any = None     # first + last stage (tied embedding / LM-head gradients)

    def layer_range(self, num_layers: int, layer_costs=None, first_extra: float = 0.0,
                    last_extra: float = 0.0) -> tuple[int, int]:
        """This stage's contiguous block range: the split that minimises the most expensive stage,
        where the first stage also pays ``first_extra`` (embedding) and the last ``last_extra``
        (final norm, LM head and loss), in the units of ``layer_costs`` (default: one per block)."""
        return partition_layers(layer_costs or [1.0] * num_layers, self.pp_size, first_extra, last_extra)[self.pp_rank]

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def last_stage_rank(self) -> int:
        """Pipeline rank that holds the last (virtual) stage: the last rank, or, when the two chunks of every rank
        are placed in a V over the ranks, the first."""
        return 0 if self.extras.get("pp_placement") == "v" else self.pp_size - 1

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.last_stage_rank
    # FusedCommContext of the tp group (CUDA only; None ⇒ NCCL / gloo collectives)
    tp_fused: Any = None
    sp_fused: Any = None
    extras: dict = field(default_factory=dict)

    @property
    def seq_shards(self) -> int:
        """Number of ways the packed token dimension is split between blocks."""
        return self.tp_size * self.sp_size

    def enable_fused(self, max_tokens: int, hidden: int, widest: int, device=None):
        """Creates the communication state of the tp / sp groups. On CUDA this allocates the
        symmetric staging buffers of the fused kernels (``max_tokens`` rows of the widest
        activation); on CPU the same object only carries group, rank and size."""
        from .fused_linear import FusedCommContext

        nbytes = max_tokens * max(hidden, widest) * 2
        if self.tp_size > 1 and self.tp_fused is None:
            self.tp_fused = FusedCommContext(self.tp_group, nbytes, device)
        if self.sp_size > 1 and self.sp_fused is None:
            self.sp_fused = FusedCommContext(self.sp_group, nbytes, device)


@dataclass
class MeshGroups:
    dp_group: Any
    dp_rank: int
    dp_size: int
    # ranks that hold the same parameter shard and see different data: dp x sp
    shard_group: Any
    shard_rank: int
    shard_size: int
    ctx: ParallelContext
    pp_rank: int = 0
    pp_size: int = 1
    pp_prev: int | None = None
    pp_next: int | None = None
    cpu_shard_group: Any = None
    mp_group: Any = None  # every rank of one data-parallel replica (tp x sp x pp): they share a batch
    mp_rank: int = 0
    # expert parallelism: ep groups are blocks of consecutive ranks of a pipeline stage (tensor-parallel index
    # fastest); ranks with the same position in different blocks hold the same experts (expert-data-parallel group)
    edp_group: Any = None
    edp_rank: int = 0
    edp_size: int = 1


def build_mesh(ranks: list[int], dp: int, sp: int = 1, tp: int = 1, pp: int = 1, cpu_groups: bool = True,
               ep: int = 1, etp: int = 1) -> MeshGroups:
    """Creates every group of a ``pp x dp x sp x tp`` mesh over ``ranks``. Collective over the
    WHOLE world (``dist.new_group`` semantics): every process must call it with the same arguments,
    whether or not it belongs to ``ranks``."""
    assert len(ranks) == dp * sp * tp * pp, (len(ranks), dp, sp, tp, pp)
    me = dist.get_rank() if dist.is_initialized() else 0
    backend_is_gloo = (not dist.is_initialized()) or dist.get_backend() == "gloo"

    def coord(i):
        t = i % tp
        s = (i // tp) % sp
        d = (i // (tp * sp)) % dp
        p = i // (tp * sp * dp)
        return p, d, s, t

    def make(sel):
        """One group per distinct key; returns this rank's group, its index inside and the size."""
        buckets: dict[Any, list[int]] = {}
        for i, r in enumerate(ranks):
            buckets.setdefault(sel(*coord(i)), []).append(r)
        mine = (None, 0, 1)
        for key in sorted(buckets):
            members = buckets[key]
            g = dist.new_group(members) if dist.is_initialized() else None  # size-1 groups too: None would mean WORLD
            if me in members:
                mine = (g, members.index(me), len(members))
        return mine

    tp_g = make(lambda p, d, s, t: (p, d, s))
    sp_g = make(lambda p, d, s, t: (p, d, t))
    dp_g = make(lambda p, d, s, t: (p, s, t))
    sh_g = make(lambda p, d, s, t: (p, t))
    mp_g = make(lambda p, d, s, t: d)
    pp_g = make(lambda p, d, s, t: (d, s, t))
    # Expert parallelism runs over the dp x sp x tp ranks of a pipeline stage, numbered with the tensor-parallel
    # index fastest (q): every one of them holds different tokens at a mixture layer (under tensor parallelism the
    # activations between the two halves of a block are sharded by sequence), so any block of ranks can exchange
    # tokens for experts. ``ep = tp`` is the hybrid layout "attention tensor-parallel, experts expert-parallel on the
    # same GPUs"; with ``tp = 1`` the groups are blocks of the dp x sp ranks. With expert tensor parallelism the
    # block of ``ep * etp`` ranks factors with the etp index fastest: ``etp`` consecutive ranks hold slices of the
    # same experts (they gather their tokens, apply their slice and reduce), and the ranks with the same slice index
    # form the expert-parallel group.
    emp = ep * etp
    assert (dp * sp * tp) % emp == 0, "ep x etp must divide dp x sp x tp"
    assert etp == 1 or tp % etp == 0, "an expert-tensor-parallel group lies inside a tensor-parallel group"
    assert tp == 1 or emp == 1 or emp % tp == 0, \
        "under tensor parallelism the ranks sharing a set of experts are whole tensor-parallel groups (e x etp a multiple of t)"
    qof = lambda d, s, t: (d * sp + s) * tp + t
    ep_g = make(lambda p, d, s, t: (p, qof(d, s, t) // emp, qof(d, s, t) % etp)) if ep > 1 else (None, 0, 1)
    etp_g = make(lambda p, d, s, t: (p, qof(d, s, t) // etp)) if etp > 1 else (None, 0, 1)
    emp_g = make(lambda p, d, s, t: (p, qof(d, s, t) // emp)) if emp > 1 else (None, 0, 1)
    edp_g = make(lambda p, d, s, t: (p, qof(d, s, t) % emp)) if emp > 1 else (None, 0, 1)
    tie_g = (None, 0, 1)
    if pp > 1 and dist.is_initialized():
        stride = dp * sp * tp
        for j in range(stride):
            pair = [ranks[j], ranks[j + (pp - 1) * stride]]
            g = dist.new_group(pair)
            if me in pair:
                tie_g = (g, pair.index(me), 2)
    # pipeline transport: one two-rank group per direction of every neighbour pair (the pair that closes the
    # ring serves virtual stages), so each group carries one ordered one-way stream of messages
    links = None
    if pp > 1 and dist.is_initialized():
        from .pipeline import PipelineLinks

        stride = dp * sp * tp
        for j in range(stride):
            col = [ranks[j + k * stride] for k in range(pp)]
            edges = []
            for i in range(pp):
                pair = [col[i], col[(i + 1) % pp]]
                # activations down, gradients up, and the same again for chunks placed on the way back up (V shape)
                edges.append(tuple(dist.new_group(pair) for _ in range(4)))
            if me in col:
                i = col.index(me)
                links = PipelineLinks(prev=col[i - 1], next=col[(i + 1) % pp], fwd_prev=edges[i - 1][0],
                                      bwd_prev=edges[i - 1][1], fwd_next=edges[i][0], bwd_next=edges[i][1],
                                      vfwd_prev=edges[i - 1][2], vbwd_prev=edges[i - 1][3],
                                      vfwd_next=edges[i][2], vbwd_next=edges[i][3])
    cpu_sh = (None, 0, 1)
    if cpu_groups and dist.is_initialized() and not backend_is_gloo:
        buckets: dict[Any, list[int]] = {}
        for i, r in enumerate(ranks):
            p, d, s, t = coord(i)
            buckets.setdefault((p, t), []).append(r)
        for key in sorted(buckets):
            g = dist.new_group(buckets[key], backend="gloo")
            if me in buckets[key]:
                cpu_sh = (g, 0, 0)
    ctx = ParallelContext(tp_group=tp_g[0], tp_rank=tp_g[1], tp_size=tp_g[2],
                          sp_group=sp_g[0], sp_rank=sp_g[1], sp_size=sp_g[2])
    mesh = MeshGroups(dp_group=dp_g[0], dp_rank=dp_g[1], dp_size=dp_g[2], shard_group=sh_g[0], shard_rank=sh_g[1],
                      shard_size=sh_g[2], ctx=ctx, pp_size=pp,
                      cpu_shard_group=cpu_sh[0] if not backend_is_gloo else sh_g[0],
                      mp_group=mp_g[0], mp_rank=mp_g[1])
    if me in ranks:
        i = ranks.index(me)
        p, d, s, t = coord(i)
        mesh.pp_rank = p
        stride = dp * sp * tp
        mesh.pp_prev = ranks[i - stride] if p > 0 else None
        mesh.pp_next = ranks[i + stride] if p < pp - 1 else None
        ctx.pp_group, ctx.pp_rank, ctx.pp_size = pp_g[0], p, pp
        ctx.pp_prev, ctx.pp_next = mesh.pp_prev, mesh.pp_next
        ctx.pp_tie_group = tie_g[0]
        ctx.extras["pp_links"] = links
    if ep > 1:
        ctx.ep_group, ctx.ep_rank, ctx.ep_size = ep_g
    if etp > 1:
        ctx.etp_group, ctx.etp_rank, ctx.etp_size = etp_g
    if emp > 1:
        mesh.edp_group, mesh.edp_rank, mesh.edp_size = edp_g
        ctx.extras["emp_group"] = emp_g[0]  # every rank whose expert parameters differ from this rank's
    return mesh
