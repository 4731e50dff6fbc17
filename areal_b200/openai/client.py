"""OpenAI-style client that talks to an in-process ``InferenceEngine`` and records every
completion with its token ids, logprobs and policy versions.

    client = ArealOpenAI(engine, tokenizer)
    resp = await client.chat.completions.create(messages=[...], max_completion_tokens=256)
    client.set_reward(resp.id, 1.0)
    batch = client.export_interactions(style="individual")

Agents written against ``openai.AsyncOpenAI`` work unchanged when handed this
object (or, out of process, the proxy's ``base_url``)
(role of areal/experimental/openai/client.py:1212 ``ArealOpenAI``).
"""

from __future__ import annotations

import re
import time
import uuid
from types import SimpleNamespace
from typing import Any

from ..api.cli_args import GenerationHyperparameters
from ..api.io_struct import ModelRequest
from .cache import InteractionCache
from .tool_call_parser import parse_reasoning, parse_tool_calls
from .types import InteractionWithTokenLogpReward


def _ns(d: Any) -> Any:
    if isinstance(d, dict):
        return SimpleNamespace(**{k: _ns(v) for k, v in d.items()})
    if isinstance(d, list):
        return [_ns(x) for x in d]
    return d


def build_chat_completion(cid: str, model: str, content: str, tool_calls: list, finish_reason: str,
                          n_prompt: int, n_completion: int, reasoning: str | None = None) -> dict[str, Any]:
    msg: dict[str, Any] = {"role": "assistant", "content": content}
    if tool_calls:
        msg["tool_calls"] = tool_calls
    if reasoning is not None:
        msg["reasoning_content"] = reasoning
    return {"id": cid, "object": "chat.completion", "created": int(time.time()), "model": model,
            "choices": [{"index": 0, "message": msg, "finish_reason": finish_reason, "logprobs": None}],
            "usage": {"prompt_tokens": n_prompt, "completion_tokens": n_completion,
                      "total_tokens": n_prompt + n_completion}}


class _ChatCompletions:
    def __init__(self, client: "ArealOpenAI"):
        self._c = client

    async def create(self, *, messages: list[dict[str, Any]], model: str = "default", tools=None,
                     max_completion_tokens: int | None = None, max_tokens: int | None = None,
                     temperature: float | None = None, top_p: float | None = None, stop=None, n: int = 1,
                     extra_body: dict | None = None, **kwargs):
        return await self._c._complete(messages, model=model, tools=tools,
                                       max_new=max_completion_tokens or max_tokens, temperature=temperature,
                                       top_p=top_p, stop=stop, as_dict=False)


class _Responses:
    def __init__(self, client: "ArealOpenAI"):
        self._c = client

    async def create(self, *, input: Any, model: str = "default", instructions: str | None = None,
                     max_output_tokens: int | None = None, temperature: float | None = None, **kwargs):
        messages = [{"role": "user", "content": input}] if isinstance(input, str) else list(input)
        if instructions:
            messages = [{"role": "system", "content": instructions}] + messages
        comp = await self._c._complete(messages, model=model, tools=kwargs.get("tools"), max_new=max_output_tokens,
                                       temperature=temperature, top_p=None, stop=None, as_dict=True)
        text = comp["choices"][0]["message"]["content"]
        return _ns({"id": comp["id"], "object": "response", "model": model, "output_text": text,
                    "output": [{"type": "message", "role": "assistant",
                                "content": [{"type": "output_text", "text": text}]}],
                    "usage": {"input_tokens": comp["usage"]["prompt_tokens"],
                              "output_tokens": comp["usage"]["completion_tokens"]}})


_DATA_URI = re.compile(r"^data:image/[a-zA-Z0-9.+-]+;base64,(.+)$", re.DOTALL)


def extract_images(messages: list[dict[str, Any]]) -> tuple[list[str], list[dict[str, Any]]]:
    """``image_url`` content parts of chat messages → ``(image_data, messages_for_template)``: the base64
    payloads (data URIs stripped to their payload, other URLs kept as they are) in order of appearance, and the
    messages with every such part replaced by ``{"type": "image"}``, which is what a vision-language chat
    template turns into its image placeholder. Reference: areal/experimental/openai/client.py:151-237."""
    images, out = [], []
    for m in messages:
        c = m.get("content")
        if not isinstance(c, list):
            out.append(m)
            continue
        parts = []
        for part in c:
            if isinstance(part, dict) and part.get("type") == "image_url":
                url = part.get("image_url")
                url = url.get("url") if isinstance(url, dict) else url
                hit = _DATA_URI.match(url or "")
                images.append(hit.group(1) if hit else url)
                parts.append({"type": "image"})
            else:
                parts.append(part)
        out.append(dict(m, content=parts))
    return images, out


class ArealOpenAI:
    def __init__(self, engine, tokenizer, gconfig: GenerationHyperparameters | None = None,
                 tool_call_parser: str = "qwen", reasoning_parser: str | None = None,
                 chat_template_type: str = "hf", engine_max_tokens: int | None = None, processor=None):
        """``processor``: the HF processor of a vision-language model. With it, image prompts are expanded to
        their placeholder tokens and pixel tensors here (what the in-process rollout engine and the train engine
        need); without it the encoded images travel as ``image_data`` and the serving side expands them."""
        self.engine, self.tokenizer = engine, tokenizer
        self.processor = processor
        self.gconfig = gconfig or GenerationHyperparameters()
        self.reasoning_parser = reasoning_parser
        self.chat_template_type = chat_template_type
        self.engine_max_tokens = engine_max_tokens
        self.cache = InteractionCache()
        self.chat = SimpleNamespace(completions=_ChatCompletions(self))
        self.responses = _Responses(self)

    def _tokenize(self, messages, tools):
        kw = {"tools": tools} if tools else {}
        from ..utils.hf_io import chat_template_ids

        return chat_template_ids(self.tokenizer, messages, add_generation_prompt=True, **kw)

    def _process_images(self, messages, image_data, tools):
        """Chat template as text, then the processor on text + decoded images: token ids with the image
        placeholders expanded to one token per merged patch, and the pixel tensors."""
        import base64
        import io

        from PIL import Image

        kw = {"tools": tools} if tools else {}
        text = self.processor.apply_chat_template(messages, tokenize=False, add_generation_prompt=True, **kw)
        images = []
        for b in image_data:
            try:
                images.append(Image.open(io.BytesIO(base64.b64decode(b, validate=True))))
            except Exception as e:
                raise ValueError("image_url must carry a base64 data URI (remote URLs are not fetched)") from e
        proc = self.processor(text=[text], images=images, padding=False, return_tensors="pt")
        mm = {k: v for k, v in proc.items() if k not in ("input_ids", "attention_mask")}
        return proc["input_ids"][0].tolist(), mm

    async def _complete(self, messages, model, tools, max_new, temperature, top_p, stop, as_dict):
        g = self.gconfig.new(n_samples=1)
        if max_new is not None:
            g.max_new_tokens = int(max_new)
        if temperature is not None:
            g.temperature = float(temperature)
            g.greedy = temperature == 0
        if top_p is not None:
            g.top_p = float(top_p)
        if stop:
            g.stop = [stop] if isinstance(stop, str) else list(stop)
        eos = getattr(self.tokenizer, "eos_token_id", None)
        if eos is not None and eos not in g.stop_token_ids:
            g.stop_token_ids = list(g.stop_token_ids) + [eos]
        image_data, tmpl_messages = extract_images(messages)
        mm: dict[str, Any] = {}
        if image_data and self.processor is not None:
            ids, mm = self._process_images(tmpl_messages, image_data, tools)
        else:
            ids = self._tokenize(tmpl_messages if image_data else messages, tools)
        if self.engine_max_tokens is not None:
            g.max_new_tokens = max(min(g.max_new_tokens, self.engine_max_tokens - len(ids)), 1)
        resp = await self.engine.agenerate(ModelRequest(
            rid=uuid.uuid4().hex, input_ids=ids, gconfig=g, tokenizer=self.tokenizer,
            image_data=image_data or None, processor=self.processor,
            metadata={"multi_modal_input": [mm]} if mm else {}))
        out = resp.output_tokens
        if eos is not None and out and out[-1] == eos:
            text = self.tokenizer.decode(out[:-1])
        else:
            text = self.tokenizer.decode(out)
        reasoning = None
        if self.reasoning_parser:
            reasoning, text = parse_reasoning(text)
        content, calls = parse_tool_calls(text, tools)
        finish = "tool_calls" if calls else ("stop" if resp.stop_reason == "stop" else "length")
        cid = f"chatcmpl-{uuid.uuid4().hex[:24]}"
        comp = build_chat_completion(cid, model, content, calls, finish, resp.input_len, resp.output_len, reasoning)
        self.cache.add(InteractionWithTokenLogpReward(
            interaction_id=cid, messages=list(messages), completion=comp, model_response=resp,
            output_message=comp["choices"][0]["message"], chat_template_type=self.chat_template_type,
            created_at=time.time(), multi_modal_input=mm))
        return comp if as_dict else _ns(comp)

    # ------------------------------------------------------------- rewards / export
    def get_interaction(self, interaction_id: str) -> InteractionWithTokenLogpReward:
        return self.cache[interaction_id]

    def set_reward(self, interaction_id: str | None, reward: float):
        self.cache.set_reward(interaction_id, reward)

    def set_last_reward(self, reward: float):
        self.cache.set_last_reward(reward)

    def apply_reward_discount(self, turn_discount: float = 1.0):
        self.cache.apply_reward_discount(turn_discount)

    def export_interactions(self, style: str = "individual", turn_discount: float = 1.0):
        return self.cache.export(style, turn_discount)
