"""One recorded LLM interaction of an agent: the request messages, the completion and,
for training, the exact token ids, behaviour logprobs and policy versions
(role of areal/experimental/openai/types.py:36-143)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from ..api.io_struct import ModelResponse


@dataclass
class InteractionWithTokenLogpReward:
    interaction_id: str = ""
    messages: list[dict[str, Any]] = field(default_factory=list)
    completion: Any = None  # the OpenAI-style response object / dict handed back to the agent
    model_response: ModelResponse | None = None
    reward: float | None = None
    parent: "InteractionWithTokenLogpReward | None" = None
    output_message: dict[str, Any] | None = None
    chat_template_type: str = "hf"
    created_at: float = 0.0
    # image prompts: the processor's pixel tensors of this interaction's prompt ({} for text)
    multi_modal_input: dict[str, Any] = field(default_factory=dict)

    @property
    def input_len(self) -> int:
        return self.model_response.input_len if self.model_response else 0

    def is_prefix_of(self, other: "InteractionWithTokenLogpReward") -> bool:
        """True when ``other``'s prompt tokens start with this interaction's full token sequence."""
        if self.model_response is None or other.model_response is None:
            return False
        mine = self.model_response.input_tokens + self.model_response.output_tokens
        theirs = other.model_response.input_tokens
        return len(theirs) >= len(mine) and theirs[: len(mine)] == mine

    def to_tensor_dict(self) -> dict[str, torch.Tensor]:
        r = self.model_response
        assert r is not None, "interaction has no model response"
        seq = r.input_tokens + r.output_tokens
        n_in, n_out = r.input_len, r.output_len
        # when this interaction extends its parent, the parent's output tokens are also trained on
        loss_mask = [0] * n_in + [1] * n_out
        logprobs = [0.0] * n_in + list(r.output_logprobs)
        versions = [-1] * n_in + list(r.output_versions)
        out = dict(
            input_ids=torch.tensor(seq, dtype=torch.int32).unsqueeze(0),
            attention_mask=torch.ones(1, len(seq), dtype=torch.bool),
            loss_mask=torch.tensor(loss_mask, dtype=torch.int32).unsqueeze(0),
            logprobs=torch.tensor(logprobs, dtype=torch.float32).unsqueeze(0),
            versions=torch.tensor(versions, dtype=torch.int32).unsqueeze(0),
            rewards=torch.tensor([float(self.reward or 0.0)], dtype=torch.float32),
        )
        if self.multi_modal_input:
            out["multi_modal_input"] = [self.multi_modal_input]
        return out
