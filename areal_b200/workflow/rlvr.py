"""Single-turn RL-with-verifiable-rewards workflow.

One episode = one prompt → one sampled completion → one scalar reward. The
trajectory carries per-token behaviour logprobs and the policy version that
produced each token (prompt positions: logprob 0, version −1, loss_mask 0),
the layout the trainer expects (areal/workflow/rlvr.py:49-178 in the reference).
"""

from __future__ import annotations

import asyncio
import uuid
from typing import Any, Callable

import torch

from ..api.cli_args import GenerationHyperparameters
from ..api.io_struct import ModelRequest
from ..api.reward_api import AsyncRewardWrapper
from ..api.workflow_api import RolloutWorkflow
from ..utils import stats_tracker


def default_get_input_ids(data: dict[str, Any], tokenizer, enable_thinking: bool = False) -> list[int]:
    if "input_ids" in data:
        ids = data["input_ids"]
        return ids.tolist() if torch.is_tensor(ids) else list(ids)
    if tokenizer is None:
        raise ValueError("data has no input_ids and no tokenizer was given")
    if "messages" in data:
        from ..utils.hf_io import chat_template_ids

        return chat_template_ids(tokenizer, data["messages"], add_generation_prompt=True, enable_thinking=enable_thinking)
    return list(tokenizer.encode(data["prompt"]))


def default_data_extract_prompt_fn(data: dict[str, Any]):
    """The prompt of a dataset item as chat messages (``messages``) or, for pre-tokenised items, its ids."""
    return data["messages"] if "messages" in data else data.get("input_ids", data.get("prompt"))


default_get_input_ids_fn = default_get_input_ids  # the name the reference uses


class RLVRWorkflow(RolloutWorkflow):
    def __init__(self, reward_fn: Callable[..., float] | str, gconfig: GenerationHyperparameters,
                 tokenizer=None, enable_thinking: bool = False, get_input_ids_fn: Callable | None = None,
                 reward_in_process: bool = False, reward_timeout: float = 15.0):
        if isinstance(reward_fn, str):
            from ..utils.dynamic_import import import_from_string

            reward_fn = import_from_string(reward_fn)
        self.reward_fn = reward_fn
        self.gconfig = gconfig.new(n_samples=1)
        self.tokenizer = tokenizer
        self.enable_thinking = enable_thinking
        self.get_input_ids_fn = get_input_ids_fn or default_get_input_ids
        self._async_reward = None if (reward_in_process or asyncio.iscoroutinefunction(reward_fn)) \
            else AsyncRewardWrapper(reward_fn, timeout_seconds=reward_timeout)
        self._in_process = reward_in_process

    async def _reward(self, prompt, completion, prompt_ids, completion_ids, data) -> float:
        extra = {k: v for k, v in data.items() if k not in ("input_ids", "messages", "prompt")}
        if asyncio.iscoroutinefunction(self.reward_fn):
            return float(await self.reward_fn(prompt, completion, prompt_ids, completion_ids, **extra))
        if self._in_process:
            return float(self.reward_fn(prompt, completion, prompt_ids, completion_ids, **extra))
        return await self._async_reward(prompt, completion, prompt_ids, completion_ids, **extra)

    async def arun_episode(self, engine, data: dict[str, Any]) -> dict[str, Any] | None:
        prompt_ids = self.get_input_ids_fn(data, self.tokenizer, self.enable_thinking) \
            if self.get_input_ids_fn is default_get_input_ids else self.get_input_ids_fn(data)
        req = ModelRequest(rid=uuid.uuid4().hex, input_ids=prompt_ids, gconfig=self.gconfig,
                           tokenizer=self.tokenizer)
        resp = await engine.agenerate(req)
        prompt_str = completion_str = None
        if self.tokenizer is not None:
            prompt_str = self.tokenizer.decode(prompt_ids)
            completion_str = self.tokenizer.decode(resp.output_tokens)
        reward = await self._reward(prompt_str, completion_str, resp.input_tokens, resp.output_tokens, data)
        stats_tracker.get("rollout").scalar(reward=reward, gen_len=float(resp.output_len))
        seq = resp.input_tokens + resp.output_tokens
        n_in, n_out = resp.input_len, resp.output_len
        return dict(
            input_ids=torch.tensor(seq, dtype=torch.int32).unsqueeze(0),
            attention_mask=torch.ones(1, len(seq), dtype=torch.bool),
            loss_mask=torch.tensor([0] * n_in + [1] * n_out, dtype=torch.int32).unsqueeze(0),
            logprobs=torch.tensor([0.0] * n_in + resp.output_logprobs, dtype=torch.float32).unsqueeze(0),
            versions=torch.tensor([-1] * n_in + resp.output_versions, dtype=torch.int32).unsqueeze(0),
            rewards=torch.tensor([float(reward)], dtype=torch.float32),
            seq_no_eos_mask=torch.tensor([resp.stop_reason == "length"], dtype=torch.bool),
        )
