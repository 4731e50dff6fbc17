"""Math agents on the OpenAI chat-completions protocol: single turn, multi-turn with retry feedback,
and a calculator tool user.

Each agent has ``async run(data, **extra)`` with ``data = {"messages": [...], "answer": str}`` and
returns the reward: a float for the last completion, or ``{completion_id: reward}`` when several
completions of one episode are rewarded individually. The chat client comes from ``extra["client"]``
(the engine-bound :class:`~areal_b200.openai.client.ArealOpenAI` of the inline / subproc workflow
modes) or is built from ``extra["base_url"]`` / ``extra["api_key"]`` with the ``openai`` package when
the agent runs against the proxy server (online mode; that package is optional).

The tool agent runs its own function-calling loop (``tools=`` in the request, ``tool`` messages with
the results) instead of depending on an agent SDK, so it works with nothing but the protocol.

Reference behaviour: areal/workflow/openai/math_agent.py (MathAgent :27, MultiTurnMathAgent :50,
MathToolAgent :134), areal/workflow/openai_agent/math_agent.py, areal/workflow/langchain/math_agent.py.
"""

from __future__ import annotations

import json
import math
import os
from typing import Any

from ...reward.math_parser import extract_answer, math_equal

RETRY_PROMPT = ("Your answer is either wrong or not parsable to the reward function. You may misunderstand the "
                "original question. Please carefully read the original question, check the previous errors, and "
                "try to answer it again.")


def math_reward_fn(completions: str | None, answer: str) -> float:
    """1.0 when the completion's final answer (last ``\\boxed{}`` / ``####`` / number) equals ``answer``."""
    if not completions:
        return 0.0
    ref = extract_answer(answer) or answer
    return float(math_equal(extract_answer(completions), ref))


def _client(extra: dict[str, Any]):
    client = extra.get("client")
    if client is not None:
        return client
    try:
        from openai import AsyncOpenAI
    except ImportError as e:  # pragma: no cover - optional dependency
        raise RuntimeError("running an agent against a base_url needs the `openai` package; "
                           "inline / subproc workflow modes pass an engine-bound client instead") from e
    return AsyncOpenAI(base_url=extra.get("base_url") or os.getenv("OPENAI_BASE_URL"),
                       api_key=extra.get("api_key") or os.getenv("OPENAI_API_KEY"),
                       http_client=extra.get("http_client"), max_retries=0)


def _get(obj, key, default=None):
    return obj.get(key, default) if isinstance(obj, dict) else getattr(obj, key, default)


def _message_dict(message) -> dict[str, Any]:
    """Assistant message of a completion as a plain dict that can go back into ``messages``."""
    if hasattr(message, "model_dump"):
        return message.model_dump(exclude_none=True)
    out = {"role": "assistant", "content": _get(message, "content") or ""}
    calls = _get(message, "tool_calls")
    if calls:
        out["tool_calls"] = [c if isinstance(c, dict) else
                             {"id": c.id, "type": "function",
                              "function": {"name": c.function.name, "arguments": c.function.arguments}} for c in calls]
    return out


class MathAgent:
    """One completion, rewarded by answer match."""

    def __init__(self, **sampling):
        self.sampling = {k: v for k, v in sampling.items() if k not in ("max_tokens", "max_turns")}

    async def run(self, data: dict, **extra):
        comp = await _client(extra).chat.completions.create(messages=data["messages"], model="default",
                                                            **self.sampling)
        return math_reward_fn(_get(comp.choices[0].message, "content"), data["answer"])


class MultiTurnMathAgent:
    """Up to ``max_turns`` attempts; after a wrong answer the user asks to try again. Every attempt is
    rewarded on its own (the workflow discounts earlier turns when exporting)."""

    def __init__(self, max_turns: int = 8, **sampling):
        self.max_turns = max_turns
        self.sampling = {k: v for k, v in sampling.items() if k != "max_tokens"}

    async def run(self, data: dict, **extra):
        client = _client(extra)
        messages = list(data["messages"])
        rewards: dict[str, float] = {}
        for _ in range(self.max_turns):
            comp = await client.chat.completions.create(messages=messages, model="default", **self.sampling)
            message = comp.choices[0].message
            messages.append(_message_dict(message))
            reward = math_reward_fn(_get(message, "content"), data["answer"])
            rewards[comp.id] = reward
            if reward == 1.0:
                break
            messages.append({"role": "user", "content": RETRY_PROMPT})
        return rewards


def _sqrt(a: float) -> float:
    if a < 0:
        raise ValueError("cannot take the square root of a negative number")
    return math.sqrt(a)


def _divide(a: float, b: float) -> float:
    if b == 0:
        raise ValueError("division by zero")
    return a / b


_FUNCS = {"add": lambda a, b: a + b, "subtract": lambda a, b: a - b, "multiply": lambda a, b: a * b,
          "divide": _divide, "power": lambda a, b: a ** b, "sqrt": _sqrt}


def _tool(name: str, doc: str, params: tuple[str, ...]) -> dict[str, Any]:
    return {"type": "function", "function": {
        "name": name, "description": doc,
        "parameters": {"type": "object", "properties": {p: {"type": "number"} for p in params},
                       "required": list(params)}}}


CALCULATOR_TOOLS = [_tool("add", "Add two numbers.", ("a", "b")), _tool("subtract", "Subtract b from a.", ("a", "b")),
                    _tool("multiply", "Multiply two numbers.", ("a", "b")), _tool("divide", "Divide a by b.", ("a", "b")),
                    _tool("power", "Raise a to the power of b.", ("a", "b")),
                    _tool("sqrt", "Square root of a.", ("a",))]

TOOL_INSTRUCTIONS = ("Answer the user's math questions using the available calculator tools. Don't give the answer "
                     "directly, you must use tools to do the mathematical calculation.")


def call_tool(name: str, arguments: str | dict) -> str:
    """Result of one tool call as the string that goes into the ``tool`` message (errors included:
    the model sees them and can correct itself)."""
    try:
        args = json.loads(arguments) if isinstance(arguments, str) else dict(arguments)
        return repr(float(_FUNCS[name](**{k: float(v) for k, v in args.items()})))
    except Exception as e:  # noqa: BLE001 - any failure is reported back to the model
        return f"error: {type(e).__name__}: {e}"


class MathToolAgent:
    """Calculator user: completions may request tool calls; the agent executes them, appends the results
    and asks again until the model answers in plain text (or ``max_turns`` requests were made). The
    reward is that of the final answer."""

    def __init__(self, max_turns: int = 8, **sampling):
        self.max_turns = max_turns
        self.sampling = {k: v for k, v in sampling.items() if k != "max_tokens"}

    async def run(self, data: dict, **extra):
        client = _client(extra)
        messages = [{"role": "system", "content": TOOL_INSTRUCTIONS}] + list(data["messages"])
        final = None
        for _ in range(self.max_turns):
            comp = await client.chat.completions.create(messages=messages, model="default", tools=CALCULATOR_TOOLS,
                                                        **self.sampling)
            message = comp.choices[0].message
            messages.append(_message_dict(message))
            calls = _get(message, "tool_calls") or []
            if not calls:
                final = _get(message, "content")
                break
            for c in calls:
                fn = _get(c, "function")
                messages.append({"role": "tool", "tool_call_id": _get(c, "id"),
                                 "content": call_tool(_get(fn, "name"), _get(fn, "arguments"))})
        return math_reward_fn(final, data["answer"])
