"""Reward for the Countdown numbers game: reach ``target`` with +, -, *, / over the given numbers, each used
exactly once; the solution goes into ``<answer>…</answer>``.

Scores follow examples/countdown/reward_score.py of the reference: 0 without an answer tag, ``format_score``
(0.1) for a tagged expression that uses the wrong numbers, does not parse or misses the target, 1 for a
correct one. The expression is evaluated by a small recursive-descent parser over exact fractions (no
``eval``), so ``8 / 3 * 3`` counts as 8.
"""

from __future__ import annotations

import re
from fractions import Fraction

_ANSWER = re.compile(r"<answer>(.*?)</answer>", re.DOTALL)
_TOKEN = re.compile(r"\s*(\d+|[-+*/()])")


def extract_answer(text: str) -> str | None:
    """The last ``<answer>`` block of the completion (text after an ``=`` sign is dropped)."""
    hits = _ANSWER.findall(text)
    if not hits:
        return None
    return hits[-1].split("=")[0].strip()


def tokenize(expr: str) -> list[str] | None:
    out, i = [], 0
    expr = expr.rstrip()
    while i < len(expr):
        m = _TOKEN.match(expr, i)
        if m is None:
            return None
        out.append(m.group(1))
        i = m.end()
    return out


def evaluate(expr: str) -> Fraction | None:
    """Value of an arithmetic expression over non-negative integers, or None when it is malformed or divides
    by zero. Grammar: sum := prod (('+'|'-') prod)*; prod := atom (('*'|'/') atom)*; atom := int | '(' sum ')' |
    '-' atom."""
    toks = tokenize(expr)
    if not toks:
        return None
    pos = 0

    def atom():
        nonlocal pos
        if pos >= len(toks):
            raise ValueError
        t = toks[pos]
        pos += 1
        if t == "(":
            v = total()
            if pos >= len(toks) or toks[pos] != ")":
                raise ValueError
            pos += 1
            return v
        if t == "-":
            return -atom()
        if t.isdigit():
            return Fraction(int(t))
        raise ValueError

    def prod():
        nonlocal pos
        v = atom()
        while pos < len(toks) and toks[pos] in "*/":
            op = toks[pos]
            pos += 1
            r = atom()
            v = v * r if op == "*" else v / r
        return v

    def total():
        nonlocal pos
        v = prod()
        while pos < len(toks) and toks[pos] in "+-":
            op = toks[pos]
            pos += 1
            r = prod()
            v = v + r if op == "+" else v - r
        return v

    try:
        v = total()
        return v if pos == len(toks) else None
    except (ValueError, ZeroDivisionError):
        return None


def uses_numbers(expr: str, numbers: list[int]) -> bool:
    return sorted(int(n) for n in re.findall(r"\d+", expr)) == sorted(int(n) for n in numbers)


def countdown_score(completion: str, target: int, numbers: list[int], format_score: float = 0.1,
                    score: float = 1.0) -> float:
    expr = extract_answer(completion)
    if expr is None:
        return 0.0
    if not uses_numbers(expr, numbers):
        return format_score
    v = evaluate(expr)
    return score if v is not None and v == target else format_score


def countdown_reward_fn(prompt, completions, prompt_ids, completion_ids, target=None, numbers=None, **kwargs) -> float:
    return countdown_score(completions, int(target), list(numbers))
