"""Prompts for the tool-using agent examples.

* ``qa`` (paths containing ``qa``: HotpotQA / NQ / TriviaQA style files): records with ``question`` and
  ``answer`` or ``answers`` become ``{"messages", "answer"}`` with the gold answers as a list.
* ``code`` (paths containing ``code``: MBPP / APPS style files): records ``{"question" | "prompt", "tests":
  [{"input", "output"}]}`` become ``{"messages", "tests"}`` for the sandbox reward (``reward/code.py``).
* ``terminal`` (paths containing ``terminal``): records ``{"instruction", "files", "checks"}`` become
  ``{"messages", "instruction", "files", "checks"}`` for :class:`~areal_b200.workflow.agents.TerminalAgent`.
* ``desk`` (paths containing ``desk``): service-desk task records (``workflow/agents/service_desk_agent.py``); a
  path of the form ``generate:desk:<n>:<seed>`` generates them instead of reading a file.

Role in the reference: the dataset preparation inside examples/search_agent/tongyi_deepresearch/train.py
and examples/terminal_bench/train.py.
"""
from .loaders import load_records


def qa_rl(path, split="train", tokenizer=None, max_length=None, **kw):
    out = []
    for r in load_records(path, split):
        answers = r.get("answers", r.get("answer"))
        if answers is None:
            continue
        answers = [answers] if isinstance(answers, str) else [str(a) for a in answers]
        if tokenizer is not None and max_length is not None and len(tokenizer.encode(r["question"])) > max_length:
            continue
        out.append(dict(messages=[{"role": "user", "content": r["question"]}], answer=answers))
    return out


CODE_SUFFIX = ("\nWrite a Python program that reads from standard input and writes the answer to standard output. "
               "Put the program in one ```python code block.")


def code_rl(path, split="train", tokenizer=None, max_length=None, **kw):
    out = []
    for r in load_records(path, split):
        q = r.get("question") or r.get("prompt")
        if not q or not r.get("tests"):
            continue
        if tokenizer is not None and max_length is not None and len(tokenizer.encode(q)) > max_length:
            continue
        out.append(dict(messages=[{"role": "user", "content": q + CODE_SUFFIX}], tests=list(r["tests"])))
    return out


def terminal_rl(path, split="train", tokenizer=None, max_length=None, **kw):
    out = []
    for r in load_records(path, split):
        if not r.get("checks"):
            continue  # a task without checks cannot be rewarded
        out.append(dict(messages=[{"role": "user", "content": r["instruction"]}], instruction=r["instruction"],
                        files=dict(r.get("files") or {}), checks=list(r["checks"])))
    return out


def desk_rl(path, split="train", tokenizer=None, max_length=None, **kw):
    if str(path).startswith("generate:desk"):
        from ..workflow.agents.service_desk_agent import make_desk_tasks

        parts = str(path).split(":")
        n = int(parts[2]) if len(parts) > 2 else 256
        seed = int(parts[3]) if len(parts) > 3 else 0
        return make_desk_tasks(n, seed + (0 if split == "train" else 1_000_003))
    out = []
    for r in load_records(path, split):
        if "db" not in r or "opening" not in r:
            continue
        out.append(dict(r, messages=r.get("messages") or [{"role": "user", "content": r["opening"]}]))
    return out


BUILDERS = {("qa", "rl"): qa_rl, ("terminal", "rl"): terminal_rl, ("code", "rl"): code_rl, ("desk", "rl"): desk_rl}
