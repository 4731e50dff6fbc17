"""Extraction of tool calls and reasoning text from raw completions
(Qwen / Hermes style ``<tool_call>{json}</tool_call>`` blocks and ``<think>`` sections;
role of areal/experimental/openai/tool_call_parser.py)."""

from __future__ import annotations

import json
import re
import uuid
from typing import Any

_TOOL = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)
_THINK = re.compile(r"<think>(.*?)</think>", re.S)


def parse_reasoning(text: str) -> tuple[str | None, str]:
    """Returns ``(reasoning, remainder)``; an unterminated ``<think>`` consumes the rest."""
    m = _THINK.search(text)
    if m:
        return m.group(1).strip(), (text[: m.start()] + text[m.end():]).strip()
    if "<think>" in text:
        head, _, tail = text.partition("<think>")
        return tail.strip(), head.strip()
    return None, text


def parse_tool_calls(text: str, tools: list[dict[str, Any]] | None = None) -> tuple[str, list[dict[str, Any]]]:
    """Returns ``(content without tool blocks, tool_calls in OpenAI format)``. Calls naming a
    function that is not in ``tools`` (when given) are dropped, as are malformed JSON bodies."""
    allowed = None
    if tools:
        allowed = {t.get("function", t).get("name") for t in tools}
    calls = []
    for m in _TOOL.finditer(text):
        try:
            body = json.loads(m.group(1))
        except json.JSONDecodeError:
            continue
        name = body.get("name")
        if not name or (allowed is not None and name not in allowed):
            continue
        args = body.get("arguments", body.get("parameters", {}))
        calls.append({"id": f"call_{uuid.uuid4().hex[:24]}", "type": "function",
                      "function": {"name": name, "arguments": args if isinstance(args, str) else json.dumps(args)}})
    content = _TOOL.sub("", text).strip()
    return content, calls
