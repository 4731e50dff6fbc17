"""Activation checkpointing policies.

A policy marks, per transformer block, what is recomputed in the backward pass instead of kept:

* ``none``: nothing;
* ``full``: every block keeps only its inputs (``x``, residual) and is recomputed whole;
* ``selective`` with an integer option ``N``: every ``N``-th block is recomputed whole, the others keep
  their activations (layer-selective);
* ``selective`` with option ``op``: every block keeps the activations of its attention half and recomputes
  its MLP half (gate/up projection, SwiGLU, down projection or the routed experts) from the post-attention
  normalised input. The MLP's intermediates (``[T, 2I]`` and ``[T, I]``) are the largest tensors of a block;
  attention, whose recomputation would repeat the quadratic part, is kept (op-selective);
* ``memory_budget`` with a budget ``b`` in ``[0, 1]``: ``b = 1`` keeps everything, ``b = 0`` recomputes every
  block; in between the first ``round((1 - b) * L)`` blocks are recomputed whole (the early blocks' activations
  live longest, so recomputing them first frees the most memory-time).

Reference: areal/experimental/models/archon/activation_checkpoint.py:37-270 (``ac_mode`` none / full /
selective / memory_budget, ``selective_ac_option``, ``ac_memory_budget``; areal/api/cli_args.py ArchonEngineConfig)
and the ``gradient_checkpointing`` switch of the FSDP engine, which means ``full``.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class ACPolicy:
    full_layers: set[int] = field(default_factory=set)  # local block indices recomputed whole
    mlp_only: bool = False                               # other blocks recompute their MLP half

    @property
    def active(self) -> bool:
        return bool(self.full_layers) or self.mlp_only


def make_policy(n_layers: int, mode: str = "none", option: str | int = "op", budget: float = 0.5) -> ACPolicy:
    mode = (mode or "none").lower()
    if mode == "none":
        return ACPolicy()
    if mode == "full":
        return ACPolicy(full_layers=set(range(n_layers)))
    if mode == "selective":
        if str(option).lower() == "op":
            return ACPolicy(mlp_only=True)
        try:
            n = int(option)
        except (TypeError, ValueError) as e:
            raise ValueError(f"selective_ac_option must be 'op' or a positive integer, got {option!r}") from e
        if n <= 0:
            raise ValueError(f"selective_ac_option must be positive, got {n}")
        return ACPolicy(full_layers={i for i in range(n_layers) if i % n == 0})
    if mode == "memory_budget":
        if not 0.0 <= float(budget) <= 1.0:
            raise ValueError(f"ac_memory_budget must lie in [0, 1], got {budget}")
        return ACPolicy(full_layers=set(range(int(round((1.0 - float(budget)) * n_layers)))))
    raise ValueError(f"unknown activation checkpointing mode {mode!r} (none | full | selective | memory_budget)")


def apply_activation_checkpointing(model, mode: str = "none", option: str | int = "op", budget: float = 0.5) -> ACPolicy:
    """Installs the policy on a ``QwenModel`` (its forward consults ``model.ac_policy``)."""
    policy = make_policy(len(model.layers), mode, option, budget)
    model.ac_policy = policy
    model.checkpoint_every = 0
    return policy
