"""Reward for program-synthesis prompts: run the generated program against the task's input/output cases
in the sandbox (role of examples/sandbox_daytona/reward_example.py in the reference, with the local
resource-fenced sandbox instead of a remote service; any ``SandboxClient`` can be passed).

The program is taken from the last fenced code block of the completion (```` ```python ... ``` ````), or the
whole completion when it has none. ``tests`` is a list of ``{"input": str, "output": str}`` (or pairs); the
reward is the fraction of cases whose stdout matches, or 0/1 with ``all_or_nothing``.
"""

from __future__ import annotations

import re

from ..infra.sandbox import LocalSandbox, SandboxClient, code_reward

_FENCE = re.compile(r"```(?:python|py)?\s*\n(.*?)```", re.S)
_default_sandbox: LocalSandbox | None = None


def extract_program(completion: str | None) -> str:
    blocks = _FENCE.findall(completion or "")
    return (blocks[-1] if blocks else (completion or "")).strip()


def code_reward_fn(prompt, completions, prompt_ids, completion_ids, tests=None, timeout: float = 5.0,
                   all_or_nothing: bool = False, sandbox: SandboxClient | None = None, **kwargs) -> float:
    global _default_sandbox
    program = extract_program(completions)
    if not program or not tests:
        return 0.0
    if sandbox is None:
        if _default_sandbox is None:
            _default_sandbox = LocalSandbox()
        sandbox = _default_sandbox
    cases = [(t["input"], t["output"]) if isinstance(t, dict) else (t[0], t[1]) for t in tests]
    score = code_reward(sandbox, program, cases, timeout)
    return float(score == 1.0) if all_or_nothing else score
