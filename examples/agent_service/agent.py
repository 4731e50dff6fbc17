"""A conversational agent for the agent service: answers through any OpenAI-compatible chat endpoint (the rollout
proxy of a training job, an inference gateway, an external provider) and may call a calculator tool.

The service's worker instantiates ``ChatAgent`` once and calls ``run(data, base_url=, api_key=)`` per request;
``data`` is what the gateway's ``/v1/responses`` route hands over: the new ``input`` messages and the conversation's
``history`` (kept by the gateway, so any worker can serve any turn of a conversation it is bound to).
Reference: examples/agent_service/agent.py (an agent SDK behind the same service; that SDK is not installed here)."""

from __future__ import annotations

import ast
import json
import operator
import re

_OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.Div: operator.truediv,
        ast.Pow: operator.pow, ast.USub: operator.neg, ast.Mod: operator.mod, ast.FloorDiv: operator.floordiv}


def calculate(expr: str) -> str:
    """Arithmetic on numbers only (no names, calls or attribute access)."""

    def ev(node):
        if isinstance(node, ast.Constant) and isinstance(node.value, (int, float)):
            return node.value
        if isinstance(node, ast.BinOp) and type(node.op) in _OPS:
            a, b = ev(node.left), ev(node.right)
            if isinstance(node.op, ast.Pow) and abs(b) > 64:
                raise ValueError("exponent too large")
            return _OPS[type(node.op)](a, b)
        if isinstance(node, ast.UnaryOp) and type(node.op) in _OPS:
            return _OPS[type(node.op)](ev(node.operand))
        raise ValueError("only arithmetic is allowed")

    try:
        return str(ev(ast.parse(expr.strip(), mode="eval").body))
    except Exception as e:  # the model sees the error and may try again
        return f"error: {e}"


SYSTEM = ("You are a helpful assistant. For arithmetic write <calc>EXPRESSION</calc> and wait: the result comes back "
          "as <result>VALUE</result>. Give the final answer in plain text.")


class ChatAgent:
    def __init__(self, model: str = "default", max_tool_rounds: int = 4, temperature: float = 0.7,
                 max_tokens: int = 512, post=None):
        self.model, self.max_tool_rounds = model, max_tool_rounds
        self.temperature, self.max_tokens = temperature, max_tokens
        self._post = post  # tests hand in a function; otherwise HTTP

    def _chat(self, base_url: str, api_key: str | None, messages: list[dict]) -> str:
        body = {"model": self.model, "messages": messages, "temperature": self.temperature,
                "max_tokens": self.max_tokens}
        if self._post is not None:
            out = self._post(base_url.rstrip("/") + "/chat/completions", body)
        else:
            from areal_b200.infra.utils.http import request_with_retry

            headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
            out = request_with_retry("POST", base_url.rstrip("/") + "/chat/completions", json=body, headers=headers,
                                     max_retries=2, timeout=600).json()
        return out["choices"][0]["message"]["content"] or ""

    async def run(self, data: dict, base_url: str | None = None, api_key: str | None = None) -> dict:
        if not base_url:
            raise ValueError("the agent service was started without a chat endpoint (`--base-url`)")
        messages = [{"role": "system", "content": SYSTEM}] + list(data.get("history", [])) + list(data["input"])
        calls = 0
        for _ in range(self.max_tool_rounds + 1):
            text = self._chat(base_url, api_key, messages)
            m = re.search(r"<calc>(.*?)</calc>", text, flags=re.S)
            if m is None or calls == self.max_tool_rounds:
                return {"output_text": text.strip(), "tool_calls": calls}
            calls += 1
            messages.append({"role": "assistant", "content": text[:m.end()]})
            messages.append({"role": "user", "content": f"<result>{calculate(m.group(1))}</result>"})
        return {"output_text": text.strip(), "tool_calls": calls}


def main():
    """Prints what to pass to the service (`agent=` of ``create_gateway_app``)."""
    print(json.dumps({"agent": "examples.agent_service.agent.ChatAgent", "tools": ["calc"]}))


if __name__ == "__main__":
    main()
