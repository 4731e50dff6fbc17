"""Countdown numbers game prompts (role of examples/countdown/countdown.py in the reference).

``generate`` makes solvable puzzles offline: it draws the numbers, combines them with random operations into
an expression whose value is a positive integer, and asks for that value. ``rl`` reads such a file (one JSON
object per line with ``numbers`` and ``target``) into prompts for the RLVR workflow.
"""

from __future__ import annotations

import json
import os
import random
from fractions import Fraction

from .loaders import load_records

PROMPT = ("Using the numbers {numbers}, create an equation that equals {target}. You can use basic arithmetic "
          "operations (+, -, *, /) and each number can only be used once. Show your work in <think> </think> tags. "
          "And return the final answer in <answer> </answer> tags, for example <answer> (1 + 2) / 3 </answer>.")


def random_puzzle(rng: random.Random, n_numbers: int = 4, max_number: int = 50, max_target: int = 999):
    """``(numbers, target, solution)`` with ``solution`` an expression over all numbers that equals ``target``."""
    while True:
        nums = [rng.randint(1, max_number) for _ in range(n_numbers)]
        pool = [(Fraction(n), str(n)) for n in nums]
        ok = True
        while len(pool) > 1:
            a = pool.pop(rng.randrange(len(pool)))
            b = pool.pop(rng.randrange(len(pool)))
            op = rng.choice("+-*/")
            if op == "/" and b[0] == 0:
                ok = False
                break
            v = {"+": a[0] + b[0], "-": a[0] - b[0], "*": a[0] * b[0], "/": a[0] / b[0] if b[0] else None}[op]
            pool.append((v, f"({a[1]} {op} {b[1]})"))
        if not ok:
            continue
        v, expr = pool[0]
        if v.denominator == 1 and 0 < v <= max_target:
            return nums, int(v), expr


def generate(path: str, n: int, seed: int = 0, **kw) -> str:
    """Writes ``n`` puzzles to ``path`` (jsonl) and returns the path."""
    rng = random.Random(seed)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        for _ in range(n):
            nums, target, sol = random_puzzle(rng, **kw)
            f.write(json.dumps({"numbers": nums, "target": target, "solution": sol}) + "\n")
    return path


def rl(path, split="train", tokenizer=None, max_length=None, processor=None, **kw):
    out = []
    for r in load_records(path, split):
        text = PROMPT.format(numbers=r["numbers"], target=r["target"])
        out.append(dict(messages=[{"role": "user", "content": text}], numbers=list(r["numbers"]),
                        target=int(r["target"])))
    return out


BUILDERS = {("countdown", "rl"): rl}
