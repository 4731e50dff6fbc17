"""Multi-turn and vision workflows against scripted engines and a toy tokenizer."""
import asyncio

import pytest
import torch

from areal_b200.api.cli_args import GenerationHyperparameters
from areal_b200.api.io_struct import ModelResponse
from areal_b200.infra import workflow_context
from areal_b200.workflow.multi_turn import MultiTurnWorkflow
from areal_b200.workflow.vision_rlvr import VisionRLVRWorkflow, image_to_base64


class ToyTokenizer:
    """Every word is a token; chat turns are wrapped as <role> ... <end>."""
    eos_token_id = 1
    pad_token_id = 0

    def __init__(self):
        self.vocab = {"<pad>": 0, "<end>": 1, "<gen>": 2}

    def _id(self, w):
        return self.vocab.setdefault(w, len(self.vocab))

    def encode(self, text):
        return [self._id(w) for w in text.split()]

    def decode(self, ids):
        inv = {v: k for k, v in self.vocab.items()}
        return " ".join(inv[i] for i in ids)

    def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=False, **kw):
        out = []
        for m in messages:
            out += [self._id(f"<{m['role']}>")] + self.encode(m["content"]) + [1]
        if add_generation_prompt:
            out.append(2)
        return out if tokenize else self.decode(out)


class ScriptedEngine:
    def __init__(self, tok, answers):
        self.tok, self.answers, self.requests = tok, list(answers), []

    async def agenerate(self, req):
        self.requests.append(list(req.input_ids))
        out = self.tok.encode(self.answers.pop(0)) + [1]
        return ModelResponse(input_tokens=list(req.input_ids), output_tokens=out, output_logprobs=[-0.5] * len(out),
                             output_versions=[3] * len(out), stop_reason="stop")


def reward_fn(prompt, completion, prompt_ids, completion_ids, answer=None, **kw):
    return 1.0 if answer in completion else 0.0


def test_multi_turn_retries_until_correct_and_discounts():
    tok = ToyTokenizer()
    eng = ScriptedEngine(tok, ["it is 5", "it is 7", "never used"])
    wf = MultiTurnWorkflow(reward_fn, GenerationHyperparameters(max_new_tokens=16), tok, max_turns=3, turn_discount=0.5,
                           reward_in_process=True)
    data = {"messages": [{"role": "user", "content": "what is 3 plus 4"}], "answer": "7"}
    with workflow_context.scope(task_id=1):
        traj = asyncio.run(wf.arun_episode(eng, data))
    assert len(eng.requests) == 2
    # the second request is the first conversation + the answer + the retry turn, token for token
    first, second = eng.requests
    assert second[:len(first)] == first and second[-len(wf.multi_turn_prompt_ids):] == wf.multi_turn_prompt_ids
    assert float(traj["rewards"]) == 0.5
    L = traj["input_ids"].shape[1]
    assert traj["loss_mask"].shape == (1, L) and traj["logprobs"].shape == (1, L)
    # only generated tokens carry loss, logprobs and versions
    n_gen = len(tok.encode("it is 5")) + 1 + len(tok.encode("it is 7")) + 1
    assert int(traj["loss_mask"].sum()) == n_gen
    assert (traj["versions"][traj["loss_mask"] == 1] == 3).all() and (traj["versions"][traj["loss_mask"] == 0] == -1).all()


def test_multi_turn_rejects_bad_arguments():
    tok = ToyTokenizer()
    with pytest.raises(ValueError):
        MultiTurnWorkflow(reward_fn, GenerationHyperparameters(), tok, max_turns=0, turn_discount=0.5)
    with pytest.raises(ValueError):
        MultiTurnWorkflow(reward_fn, GenerationHyperparameters(), tok, max_turns=2, turn_discount=1.5)


class ToyProcessor:
    def __init__(self, tok):
        self.tok = tok

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True):
        return self.tok.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt)

    def __call__(self, images=None, text=None, padding=False, return_tensors="pt"):
        ids = torch.tensor([self.tok.encode(text)])
        out = {"input_ids": ids, "attention_mask": torch.ones_like(ids)}
        if images:
            out["pixel_values"] = torch.zeros(len(images), 3, 4, 4)
        return out


def test_vision_workflow_passes_images_and_keeps_processor_outputs():
    tok = ToyTokenizer()
    eng = ScriptedEngine(tok, ["two cats"])
    eng.supports_images = True
    wf = VisionRLVRWorkflow(reward_fn, GenerationHyperparameters(max_new_tokens=8), tok, ToyProcessor(tok),
                            reward_in_process=True)
    png = b"\\x89PNG fake"
    traj = asyncio.run(wf.arun_episode(eng, {"messages": [{"role": "user", "content": "how many"}], "images": [png],
                                             "answer": "two"}))
    assert float(traj["rewards"]) == 1.0
    assert traj["multi_modal_input"][0]["pixel_values"].shape[0] == 1
    assert image_to_base64(png)
    text_only = ScriptedEngine(tok, ["x"])
    with pytest.raises(NotImplementedError):
        asyncio.run(wf.arun_episode(text_only, {"messages": [{"role": "user", "content": "q"}], "images": [png]}))
