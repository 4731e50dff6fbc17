"""Rollout workflow contracts (areal/api/workflow_api.py:14-115 in the reference).

A ``RolloutWorkflow`` turns one dataset item into one trajectory batch by talking
to an ``InferenceEngine``; returning ``None`` rejects the sample. Anything with an
``async run(data, **extra_kwargs)`` method (an "agent workflow") is also accepted
and is driven through the OpenAI-compatible proxy.
"""

from __future__ import annotations

import abc
from typing import TYPE_CHECKING, Any, Protocol, Union, runtime_checkable

if TYPE_CHECKING:
    from .engine_api import InferenceEngine


class RolloutWorkflow(abc.ABC):
    @abc.abstractmethod
    async def arun_episode(self, engine: "InferenceEngine", data: dict[str, Any]) -> dict[str, Any] | None:
        """Runs one episode. Returns a padded tensor dict (``input_ids``, ``attention_mask``,
        ``loss_mask``, ``logprobs``, ``versions``, ``rewards`` …), a dict of recorded
        interactions, or ``None`` to reject the sample."""
        raise NotImplementedError


@runtime_checkable
class AgentWorkflow(Protocol):
    async def run(self, data: dict[str, Any], **extra_kwargs: Any) -> Any:
        """Agent entry point; ``extra_kwargs`` carries ``base_url`` / ``api_key`` /
        ``http_client`` of the OpenAI-compatible proxy. Returns the reward (float or
        ``{interaction_id: reward}``)."""
        ...


WorkflowLike = Union[RolloutWorkflow, type, str, AgentWorkflow]
