"""Multi-attempt workflow: keep generating until the reward is positive or ``max_turns`` is
reached; after a wrong answer a fixed "try again" user turn is appended in token space (so no
decode / re-encode drift), and the final reward is discounted by ``turn_discount`` per extra
turn. Behaviour of areal/workflow/multi_turn.py:19-140 in the reference.
"""

from __future__ import annotations

import uuid
from typing import Any, Callable

import torch

from ..api.cli_args import GenerationHyperparameters
from ..api.io_struct import ModelRequest
from ..api.reward_api import AsyncRewardWrapper
from ..api.workflow_api import RolloutWorkflow
from ..infra import workflow_context
from ..utils import stats_tracker
from ..utils.hf_io import chat_template_ids

RETRY_TEXT = ("Your answer is either wrong or not parsable to the reward function. You may misunderstand the original "
              "question. Please carefully read the original question, check the previous errors, and try to answer it again.")


class MultiTurnWorkflow(RolloutWorkflow):
    def __init__(self, reward_fn: Callable[..., Any], gconfig: GenerationHyperparameters, tokenizer, max_turns: int,
                 turn_discount: float, reward_in_process: bool = False):
        if max_turns <= 0:
            raise ValueError("max_turns must be positive")
        if not (0.0 < turn_discount <= 1.0):
            raise ValueError("turn_discount must be in (0, 1].")
        self.reward_fn = reward_fn
        self.gconfig = gconfig.new_with_stop_and_pad_token_ids(tokenizer) \
            if hasattr(gconfig, "new_with_stop_and_pad_token_ids") else gconfig
        self.tokenizer = tokenizer
        self.max_turns, self.turn_discount = max_turns, turn_discount
        self._reward = reward_fn if reward_in_process else AsyncRewardWrapper(reward_fn)
        self._in_process = reward_in_process
        # tokens of the retry turn = template(assistant msg + retry user msg) minus template(assistant msg)
        base = [{"role": "assistant", "content": "some random message."}]
        s1 = chat_template_ids(tokenizer, base)
        s2 = chat_template_ids(tokenizer, base + [{"role": "user", "content": RETRY_TEXT}], add_generation_prompt=True)
        self.multi_turn_prompt_ids = s2[len(s1):]

    async def arun_episode(self, engine, data: dict[str, Any]):
        seq, logprobs, loss_mask, versions = [], [], [], []
        input_ids = chat_template_ids(self.tokenizer, data["messages"], add_generation_prompt=True)
        t, reward, discount = 0, 0.0, 1.0
        eos = getattr(self.tokenizer, "eos_token_id", None)
        while reward == 0.0 and t < self.max_turns:
            resp = await engine.agenerate(ModelRequest(rid=uuid.uuid4().hex, input_ids=input_ids,
                                                       gconfig=self.gconfig.new(n_samples=1), tokenizer=self.tokenizer))
            prompt_str = self.tokenizer.decode(input_ids)
            completion_str = self.tokenizer.decode(resp.output_tokens)
            extra = {k: v for k, v in data.items() if k != "messages"}
            if self._in_process:
                reward = float(self.reward_fn(prompt_str, completion_str, resp.input_tokens, resp.output_tokens, **extra))
            else:
                reward = float(await self._reward(prompt_str, completion_str, resp.input_tokens, resp.output_tokens, **extra))
            new_in = len(resp.input_tokens) - len(seq)
            assert len(seq) == 0 or resp.input_tokens[:len(seq)] == seq, "the conversation prefix changed between turns"
            seq += resp.input_tokens[len(resp.input_tokens) - new_in:] + resp.output_tokens
            logprobs += [0.0] * new_in + resp.output_logprobs
            loss_mask += [0] * new_in + [1] * resp.output_len
            versions += [-1] * new_in + resp.output_versions
            t += 1
            if reward == 0.0 and t < self.max_turns:
                input_ids = input_ids + resp.output_tokens
                if resp.output_tokens and eos is not None and resp.output_tokens[-1] != eos:
                    input_ids = input_ids + [eos]
                input_ids = input_ids + self.multi_turn_prompt_ids
                discount *= self.turn_discount
        reward = float(reward * discount)
        stats_tracker.get(workflow_context.stat_scope()).scalar(reward=reward, num_turns=t)
        res = dict(input_ids=torch.tensor(seq, dtype=torch.int32), logprobs=torch.tensor(logprobs, dtype=torch.float32),
                   loss_mask=torch.tensor(loss_mask, dtype=torch.int32), versions=torch.tensor(versions, dtype=torch.int32),
                   attention_mask=torch.ones(len(seq), dtype=torch.bool))
        out = {k: v.unsqueeze(0) for k, v in res.items()}
        out["rewards"] = torch.tensor([reward], dtype=torch.float32)
        return out
