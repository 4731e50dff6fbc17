"""Per-session store of interactions with reward back-propagation.

``set_reward`` attaches a reward to one interaction (default: the last one);
``apply_reward_discount`` propagates rewards backwards through the conversation
(``r_parent += discount * r_child``, children found by token-prefix matching);
``export`` returns either every interaction as its own training sample
(``individual``) or only the leaves of the conversation tree, whose token
sequences already contain their ancestors (``concat``)
(role of areal/experimental/openai/cache.py).
"""

from __future__ import annotations

from collections import OrderedDict

from .types import InteractionWithTokenLogpReward


class InteractionCache(OrderedDict):
    def __init__(self):
        super().__init__()
        self._discount_applied = False

    def add(self, inter: InteractionWithTokenLogpReward):
        self[inter.interaction_id] = inter

    @property
    def last_interaction_id(self) -> str | None:
        return next(reversed(self)) if self else None

    def set_reward(self, interaction_id: str | None, reward: float):
        if interaction_id is None:
            interaction_id = self.last_interaction_id
        if interaction_id is None or interaction_id not in self:
            raise KeyError(f"unknown interaction {interaction_id!r}")
        self[interaction_id].reward = float(reward)

    def set_last_reward(self, reward: float):
        self.set_reward(None, reward)

    def _link_parents(self):
        items = list(self.values())
        for i, it in enumerate(items):
            it.parent = None
            best = None
            for cand in items[:i]:
                if cand.is_prefix_of(it) and (best is None or cand.input_len >= best.input_len):
                    best = cand
            it.parent = best

    def apply_reward_discount(self, turn_discount: float = 1.0):
        """Walks the interactions from last to first; an interaction without its own reward
        starts from 0, and every interaction passes ``discount * reward`` up to its parent."""
        if self._discount_applied:
            return
        self._link_parents()
        items = list(self.values())
        for it in items:
            if it.reward is None:
                it.reward = 0.0
        for it in reversed(items):
            if it.parent is not None:
                it.parent.reward += turn_discount * it.reward
        self._discount_applied = True

    def export(self, style: str = "individual", turn_discount: float = 1.0) -> dict[str, InteractionWithTokenLogpReward]:
        self.apply_reward_discount(turn_discount)
        if style == "individual":
            return dict(self)
        if style == "concat":
            parents = {id(it.parent) for it in self.values() if it.parent is not None}
            return {k: v for k, v in self.items() if id(v) not in parents}
        raise ValueError(f"unknown export style {style!r}")
