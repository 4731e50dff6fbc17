"""Terminal tasks: the policy works in a shell until the task's checks pass.

A task is ``{"instruction": str, "files": {path: content}, "checks": [shell command, ...]}``. Every episode
gets a fresh :class:`~areal_b200.infra.sandbox.ShellWorkspace` holding the task's files; the policy calls
``bash(command)``, ``write_file(path, content)`` and ``read_file(path)`` within ``max_turns`` requests and
ends the episode with a plain-text message. The reward is the fraction of check commands that exit 0 in
the final workspace (``all_or_nothing=True``: 1.0 only if every check passes).

Reference behaviour: examples/terminal_bench/{agent/camel_terminal_agent.py,
workflow/camel_rlvr_workflow.py, train.py} (an agent with shell tools inside a task container, rewarded by
the task's test script; every completion of the episode is a training sample).
"""

from __future__ import annotations

import json
from typing import Any

from ...infra.sandbox import ShellWorkspace
from .math_agent import _client, _get, _message_dict
from .search_agent import _tool

TERMINAL_INSTRUCTIONS = (
    "You are working in a Linux shell inside the task's directory. Use the `bash` tool to run commands, "
    "`write_file` to create or replace a file and `read_file` to look at one. Work step by step; when the "
    "task is done, reply with a short summary and no tool call.")

TERMINAL_TOOLS = [
    _tool("bash", "Run a shell command in the task directory; returns exit code, stdout and stderr.",
          {"command": "string"}),
    _tool("write_file", "Write text to a file (relative path), replacing it if it exists.",
          {"path": "string", "content": "string"}),
    _tool("read_file", "Return the content of a file (relative path).", {"path": "string"}),
]


def run_terminal_tool(ws: ShellWorkspace, name: str, arguments: str | dict, timeout: float = 10.0) -> str:
    try:
        args = json.loads(arguments) if isinstance(arguments, str) else dict(arguments)
        if name == "bash":
            r = ws.run(str(args["command"]), timeout)
            head = "timed out" if r.timed_out else f"exit code {r.exit_code}"
            return f"{head}\nstdout:\n{r.stdout}\nstderr:\n{r.stderr}"
        if name == "write_file":
            ws.write_file(str(args["path"]), str(args["content"]))
            return "ok"
        if name == "read_file":
            return ws.read_file(str(args["path"]))
        return f"error: unknown tool {name!r}"
    except Exception as e:  # noqa: BLE001 - reported back to the model
        return f"error: {type(e).__name__}: {e}"


def score_checks(ws: ShellWorkspace, checks: list[str], timeout: float = 20.0, all_or_nothing: bool = False) -> float:
    if not checks:
        return 0.0
    passed = sum(ws.run(c, timeout).ok for c in checks)
    return float(passed == len(checks)) if all_or_nothing else passed / len(checks)


class TerminalAgent:
    def __init__(self, max_turns: int = 12, command_timeout: float = 10.0, check_timeout: float = 20.0,
                 all_or_nothing: bool = False, workspace_kwargs: dict[str, Any] | None = None, **sampling):
        self.max_turns, self.command_timeout, self.check_timeout = max_turns, command_timeout, check_timeout
        self.all_or_nothing = all_or_nothing
        self.workspace_kwargs = dict(workspace_kwargs or {})
        self.sampling = {k: v for k, v in sampling.items() if k != "max_tokens"}

    async def run(self, data: dict, **extra) -> float:
        client = _client(extra)
        messages = [{"role": "system", "content": TERMINAL_INSTRUCTIONS}] + list(
            data.get("messages") or [{"role": "user", "content": data["instruction"]}])
        with ShellWorkspace(files=data.get("files"), **self.workspace_kwargs) as ws:
            for _ in range(self.max_turns):
                comp = await client.chat.completions.create(messages=messages, model="default",
                                                            tools=TERMINAL_TOOLS, **self.sampling)
                message = comp.choices[0].message
                messages.append(_message_dict(message))
                calls = _get(message, "tool_calls") or []
                if not calls:
                    break
                for c in calls:
                    fn = _get(c, "function")
                    messages.append({"role": "tool", "tool_call_id": _get(c, "id"),
                                     "content": run_terminal_tool(ws, _get(fn, "name"), _get(fn, "arguments"),
                                                                  self.command_timeout)})
            return score_checks(ws, list(data.get("checks") or []), self.check_timeout, self.all_or_nothing)
